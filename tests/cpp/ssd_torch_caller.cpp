// Plays the part of the tch-rs caller in C++: everything goes through the C entry points a Rust binding would declare
// (atg_ssd_scan / atg_ssd_state_update with torch::Tensor* handles), then `loss.backward()` runs through the autograd node.
// Checks, on a small bf16 problem of the tensor-core family and an fp32 one of the exact family:
//   1. y, final_state and every input gradient against the operator's defining recurrence evaluated step by step in
//      fp64 on the CPU with libtorch's own autograd (gates: bf16 2e-2 max-abs scaled by max(1, max|ref|) and 1e-2 mean-rel;
//      fp32 1e-4 of max|ref|);
//   2. forward + backward captured into a CUDA graph on a side stream and replayed (what the reference's PPO update does
//      with its model, trading_bots/src/torch/train/update.rs:206-328) gives bit-identical results to the eager calls;
//   3. the single-step entry point against the same recurrence;
//   4. an invalid call reports through the error slot instead of throwing across the C boundary.
// Exit code 0 iff every check passes.  Needs a CUDA device.
#include <ATen/cuda/CUDAGraph.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/torch.h>

#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

extern "C" {
typedef at::Tensor* tensor;
void atg_ssd_scan(tensor* out__, tensor x, tensor dt, tensor a, tensor b, tensor c, tensor d, tensor z, tensor init_state,
                  tensor dt_bias, int64_t chunk, int dt_softplus, int algo);
void atg_ssd_state_update(tensor* out__, tensor state, tensor x, tensor dt, tensor a, tensor b, tensor c, tensor d, tensor z,
                          tensor dt_bias, int dt_softplus);
char* ssd_torch_get_and_reset_last_err();
}

namespace {
using torch::Tensor;
int failures = 0;

// `sum_gate`: dA and ddt_bias in bf16 mode are sums over every token of terms that mostly cancel, so the per-token bf16
// error adds up like a random walk; they are gated at 6e-2 of the largest reference entry instead.
void check(const std::string& name, const Tensor& got, const Tensor& ref, bool bf16, bool sum_gate = false) {
  Tensor g = got.detach().to(torch::kCPU, torch::kDouble), r = ref.detach().to(torch::kCPU, torch::kDouble);
  const double max_abs = (g - r).abs().max().item<double>(), ref_max = r.abs().max().item<double>();
  const double mean_rel = (g - r).abs().mean().item<double>() / (r.abs().mean().item<double>() + 1e-300);
  bool ok = torch::isfinite(g).all().item<bool>();
  if (bf16 && sum_gate) ok = ok && max_abs <= 6e-2 * ref_max;
  else if (bf16) ok = ok && max_abs <= 2e-2 * std::max(1.0, ref_max) && mean_rel <= 1e-2;
  else ok = ok && max_abs <= 1e-4 * ref_max;
  std::printf("%-28s max-abs %.3e (max|ref| %.3e)  mean-rel %.3e  %s\n", name.c_str(), max_abs, ref_max, mean_rel, ok ? "ok" : "FAIL");
  if (!ok) ++failures;
}
void expect(const std::string& name, bool ok) {
  std::printf("%-28s %s\n", name.c_str(), ok ? "ok" : "FAIL");
  if (!ok) ++failures;
}

struct Inputs {
  Tensor x, dt, A, B, C, D, z, init, bias;   // leaves on the GPU
  std::vector<Tensor*> all() { return {&x, &dt, &A, &B, &C, &D, &z, &init, &bias}; }
};
const char* NAMES[] = {"dx", "ddt", "dA", "dB", "dC", "dD", "dz", "dinit", "ddt_bias"};

// The defining recurrence, one step at a time, fp64 on the CPU (differentiable through libtorch's autograd).
std::pair<Tensor, Tensor> recurrence(const Inputs& in, int64_t G) {
  const int64_t L = in.x.size(1), H = in.x.size(2);
  Tensor S = in.init;
  std::vector<Tensor> ys;
  for (int64_t t = 0; t < L; ++t) {
    Tensor dtv = torch::softplus(in.dt.select(1, t) + in.bias);                       // [B,H]
    Tensor a = torch::exp(dtv * in.A);                                                // [B,H]
    Tensor xt = in.x.select(1, t);                                                    // [B,H,P]
    Tensor Bt = in.B.select(1, t).repeat_interleave(H / G, 1), Ct = in.C.select(1, t).repeat_interleave(H / G, 1);   // [B,H,N]
    S = a.unsqueeze(-1).unsqueeze(-1) * S + (dtv.unsqueeze(-1) * xt).unsqueeze(-1) * Bt.unsqueeze(2);
    Tensor yt = (S * Ct.unsqueeze(2)).sum(-1) + in.D.unsqueeze(-1) * xt;
    ys.push_back(yt * torch::silu(in.z.select(1, t)));
  }
  return {torch::stack(ys, 1), S};
}

Inputs make_inputs(int64_t Bn, int64_t L, int64_t H, int64_t P, int64_t N, int64_t G, torch::Dtype st) {
  torch::manual_seed(1234);
  auto dev = torch::Device(torch::kCUDA, 0);
  auto seq = [&](std::vector<int64_t> s, double scale) { return (scale * torch::randn(s)).to(st).to(dev).requires_grad_(true); };
  auto par = [&](Tensor t) { return t.to(torch::kFloat).to(dev).requires_grad_(true); };
  Inputs in;
  in.x = seq({Bn, L, H, P}, 1.0);
  in.dt = seq({Bn, L, H}, 0.5);
  in.B = seq({Bn, L, G, N}, 1.0);
  in.C = seq({Bn, L, G, N}, 1.0);
  in.z = seq({Bn, L, H, P}, 1.0);
  in.A = par(-torch::exp(torch::rand({H}) * 2.0));
  in.D = par(torch::ones({H}) + 0.1 * torch::randn({H}));
  in.bias = par(torch::randn({H}) - 3.0);
  in.init = par(0.5 * torch::randn({Bn, H, P, N}));
  return in;
}

void run_case(const char* title, torch::Dtype st, int64_t Bn, int64_t L, int64_t H, int64_t P, int64_t N, int64_t G, int64_t chunk,
              int algo) {
  std::printf("== %s\n", title);
  const bool bf16 = st == torch::kBFloat16;
  Inputs in = make_inputs(Bn, L, H, P, N, G, st);
  Tensor wy = torch::randn({Bn, L, H, P}).to(st).to(in.x.device()), wf = torch::randn({Bn, H, P, N}).to(in.x.device());

  // reference: the same rounded inputs, fp64, CPU
  Inputs rin;
  {
    auto src = in.all();
    auto dst = rin.all();
    for (size_t i = 0; i < src.size(); ++i) *dst[i] = src[i]->detach().to(torch::kCPU, torch::kDouble).requires_grad_(true);
  }
  auto [ry, rfin] = recurrence(rin, G);
  ((ry * wy.to(torch::kCPU, torch::kDouble)).sum() + (rfin * wf.to(torch::kCPU, torch::kDouble)).sum()).backward();

  // the operator, through the C entry point
  Tensor y, fin;
  std::vector<Tensor> eager;
  auto leaves = in.all();
  auto rleaves = rin.all();
  {
    tensor out[2] = {nullptr, nullptr};
    atg_ssd_scan(out, &in.x, &in.dt, &in.A, &in.B, &in.C, &in.D, &in.z, &in.init, &in.bias, chunk, 1, algo);
    char* err = ssd_torch_get_and_reset_last_err();
    if (err) { std::printf("atg_ssd_scan failed: %s\n", err); std::free(err); ++failures; return; }
    Tensor ya = *out[0], fa = *out[1];   // attached to the autograd graph; dropped at the end of this block
    delete out[0]; delete out[1];
    ((ya.to(torch::kFloat) * wy.to(torch::kFloat)).sum() + (fa * wf).sum()).backward();
    y = ya.detach();
    fin = fa.detach();
  }
  check("y", y, ry, bf16);
  check("final_state", fin, rfin, bf16);
  for (size_t i = 0; i < leaves.size(); ++i) {
    expect(std::string(NAMES[i]) + " defined", leaves[i]->grad().defined());
    if (!leaves[i]->grad().defined()) return;
    check(NAMES[i], leaves[i]->grad(), rleaves[i]->grad(), bf16, i == 2 || i == 8);
    eager.push_back(leaves[i]->grad().clone());
  }

  // The same forward + backward captured on a side stream and replayed.  The leaves of the captured graph are made on
  // that stream (their gradient accumulators then belong to it), with static gradient buffers that the replay adds into.
  {
    c10::cuda::CUDAStream side = c10::cuda::getStreamFromPool(false, 0);
    torch::cuda::synchronize();
    c10::cuda::CUDAStreamGuard guard(side);
    Inputs gin;
    auto gleaves = gin.all();
    for (size_t i = 0; i < leaves.size(); ++i) {
      *gleaves[i] = leaves[i]->detach().clone().requires_grad_(true);
      gleaves[i]->mutable_grad() = torch::zeros_like(*gleaves[i]);
    }
    Tensor wyf = wy.to(torch::kFloat);
    side.synchronize();
    at::cuda::CUDAGraph graph;
    Tensor gy, gfin;
    graph.capture_begin();
    {
      tensor o[2] = {nullptr, nullptr};
      atg_ssd_scan(o, &gin.x, &gin.dt, &gin.A, &gin.B, &gin.C, &gin.D, &gin.z, &gin.init, &gin.bias, chunk, 1, algo);
      char* e = ssd_torch_get_and_reset_last_err();
      if (e) { std::printf("capture failed: %s\n", e); std::free(e); ++failures; graph.capture_end(); return; }
      Tensor ya = *o[0], fa = *o[1];
      delete o[0]; delete o[1];
      ((ya.to(torch::kFloat) * wyf).sum() + (fa * wf).sum()).backward();
      gy = ya.detach();
      gfin = fa.detach();
    }
    graph.capture_end();
    for (int rep = 0; rep < 2; ++rep) {
      for (Tensor* t : gleaves) t->mutable_grad().zero_();
      graph.replay();
      side.synchronize();
    }
    bool same = torch::equal(gy, y) && torch::equal(gfin, fin);
    for (size_t i = 0; i < leaves.size(); ++i) same = same && torch::equal(gleaves[i]->grad(), eager[i]);
    expect("graph replay == eager", same);
  }
}

void run_step_case() {
  std::printf("== single step, bf16\n");
  const int64_t S = 64, H = 4, P = 32, N = 64, G = 1;
  Inputs in = make_inputs(S, 3, H, P, N, G, torch::kBFloat16);
  torch::NoGradGuard ng;
  Tensor state = in.init.detach().clone();
  Inputs rin;
  {
    auto src = in.all();
    auto dst = rin.all();
    for (size_t i = 0; i < src.size(); ++i) *dst[i] = src[i]->detach().to(torch::kCPU, torch::kDouble);
  }
  auto [ry, rfin] = recurrence(rin, G);
  Tensor y;
  for (int64_t t = 0; t < 3; ++t) {
    Tensor xt = in.x.detach().select(1, t).contiguous(), dtt = in.dt.detach().select(1, t).contiguous(),
           Bt = in.B.detach().select(1, t).contiguous(), Ct = in.C.detach().select(1, t).contiguous(),
           zt = in.z.detach().select(1, t).contiguous(), A = in.A.detach(), D = in.D.detach(), bias = in.bias.detach();
    tensor o[1] = {nullptr};
    atg_ssd_state_update(o, &state, &xt, &dtt, &A, &Bt, &Ct, &D, &zt, &bias, 1);
    char* e = ssd_torch_get_and_reset_last_err();
    if (e) { std::printf("atg_ssd_state_update failed: %s\n", e); std::free(e); ++failures; return; }
    y = *o[0];
    delete o[0];
  }
  check("step y (t = 2)", y, ry.select(1, 2), true);
  check("step state", state, rfin, true);
}

void run_error_case() {
  std::printf("== error reporting\n");
  Tensor x = torch::zeros({1, 8, 2, 8}), dt = torch::zeros({1, 8, 2}), A = torch::zeros({2}), B = torch::zeros({1, 8, 1, 16});
  tensor o[2] = {nullptr, nullptr};
  atg_ssd_scan(o, &x, &dt, &A, &B, &B, nullptr, nullptr, nullptr, nullptr, 8, 0, 0);   // CPU tensors: refused
  char* e = ssd_torch_get_and_reset_last_err();
  expect("CPU tensor refused with a message", e != nullptr && o[0] == nullptr);
  if (e) { std::printf("   message: %.80s\n", e); std::free(e); }
  expect("error slot cleared", ssd_torch_get_and_reset_last_err() == nullptr);
}
}  // namespace

int main() {
  if (!torch::cuda::is_available()) { std::printf("no CUDA device\n"); return 2; }
  run_case("scan fwd+bwd, bf16, tensor-core family", torch::kBFloat16, 2, 256, 4, 32, 64, 1, 128, 2);
  run_case("scan fwd+bwd, fp32, exact family", torch::kFloat, 2, 96, 4, 16, 16, 2, 32, 1);
  run_step_case();
  run_error_case();
  std::printf(failures ? "FAILED (%d)\n" : "ALL OK\n", failures);
  return failures ? 1 : 0;
}
