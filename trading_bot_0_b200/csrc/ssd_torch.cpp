// libtorch side of the SSD operator: an autograd node over the C ABI of libssd_b200, plus C entry points in the
// calling convention of the libtch shim that tch-rs binds (`tensor` = torch::Tensor*, results returned as freshly
// allocated torch::Tensor* in out__[], C++ exceptions turned into a thread-local message:
// vendor/torch-sys-0.25.0/libtch/torch_api.h:9-23; generated wrappers such as atg_softplus,
// vendor/torch-sys-0.25.0/libtch/torch_api_generated.cpp:15775-15780).
//
// With the node, `ssd_scan(..)` takes part in `loss.backward()` and in a captured training graph like any built-in
// operator: the reference runs its forward + backward + optimizer step inside one CUDA graph on a side stream
// (trading_bots/src/torch/train/update.rs:206-328, 359-443), and extends the shim by hand for that
// (at_cuda_graph_*, vendor/torch-sys-0.25.0/libtch/torch_api.cpp:378-546).  Everything here allocates through the
// caching allocator only (legal during capture) and launches on the current stream.
//
// The file builds in two ways:
//   * stand-alone (this repository): libssd_b200_torch.so, which also registers the operators as
//     torch.ops.ssd_b200.{scan, state_update} so that Python tests drive the same node;
//   * inside the shim: compile it beside torch_api.cpp with -DSSD_TORCH_IN_LIBTCH; the error slot is then the shim's
//     own `torch_last_err`, read by get_and_reset_last_err (trading_bots/src/torch/cuda/graph.rs:107-118).
#include <ATen/ATen.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/csrc/autograd/custom_function.h>
#include <torch/library.h>

#include <cstring>
#include <optional>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../include/ssd_b200.h"

namespace {

using at::Tensor;
using torch::autograd::AutogradContext;
using torch::autograd::variable_list;
using OptTensor = std::optional<Tensor>;

int32_t storage_type(const Tensor& t) {
  if (t.scalar_type() == at::kBFloat16) return SSD_BF16;
  TORCH_CHECK(t.scalar_type() == at::kFloat, "ssd: sequence tensors must be bfloat16 or float32, got ", t.scalar_type());
  return SSD_F32;
}
const Tensor* opt(const OptTensor& t) { return (t.has_value() && t->defined()) ? &*t : nullptr; }
Tensor or_undefined(const OptTensor& t) { return opt(t) ? *t : Tensor(); }
const void* ptr(const Tensor* t) { return t ? t->data_ptr() : nullptr; }
const float* fptr(const Tensor* t) { return t ? t->data_ptr<float>() : nullptr; }

using Shape = std::vector<int64_t>;
void check_seq(const char* name, const Tensor& t, const Shape& shape, const Tensor& like) {
  TORCH_CHECK(t.defined() && t.sizes() == at::IntArrayRef(shape), "ssd: ", name, " must have shape ", at::IntArrayRef(shape),
              ", got ", t.sizes());
  TORCH_CHECK(t.scalar_type() == like.scalar_type() && t.device() == like.device(), "ssd: ", name,
              " must have x's dtype and device");
  TORCH_CHECK(t.stride(-1) == 1 && (t.dim() < 4 || t.stride(2) == t.size(3)), "ssd: ", name, ": the inner dims must be dense");
}
void check_f32(const char* name, const Tensor* t, const Shape& shape, const Tensor& like) {
  if (!t) return;
  TORCH_CHECK(t->sizes() == at::IntArrayRef(shape) && t->scalar_type() == at::kFloat && t->device() == like.device() &&
                  t->is_contiguous(),
              "ssd: ", name, " must be a contiguous float32 tensor of shape ", at::IntArrayRef(shape), " on ", like.device());
}
void check_rc(int32_t rc) { TORCH_CHECK(rc == SSD_OK, "ssd_b200 error ", rc, ": ", ssd_last_error()); }

// Geometry from the tensors, as a tch caller fills it from size() / stride().
SsdDims make_dims(const Tensor& x, const Tensor& dt, const Tensor& Bm, const Tensor& Cm, const Tensor* z, const Tensor& y,
                  int64_t chunk, bool dt_softplus, int64_t algo) {
  TORCH_CHECK(x.dim() == 4, "ssd: x must be [batch, seqlen, nheads, headdim], got ", x.dim(), " dims: ", x.sizes());
  TORCH_CHECK(Bm.dim() == 4, "ssd: B must be [batch, seqlen, ngroups, dstate], got ", Bm.dim(), " dims: ", Bm.sizes());
  TORCH_CHECK(x.is_cuda(), "ssd: x must be a CUDA tensor (there is no CPU path)");
  const int64_t Bn = x.size(0), L = x.size(1), H = x.size(2), P = x.size(3), G = Bm.size(2), N = Bm.size(3);
  check_seq("x", x, {Bn, L, H, P}, x);
  check_seq("dt", dt, {Bn, L, H}, x);
  check_seq("B", Bm, {Bn, L, G, N}, x);
  check_seq("C", Cm, {Bn, L, G, N}, x);
  check_seq("y/dy", y, {Bn, L, H, P}, x);
  TORCH_CHECK(G > 0 && H % G == 0, "ssd: nheads (", H, ") must be a multiple of ngroups (", G, ")");
  TORCH_CHECK(chunk >= 1 && chunk <= 256, "ssd: chunk must be in [1, 256], got ", chunk);
  SsdDims d;
  std::memset(&d, 0, sizeof d);
  d.batch = (int32_t)Bn; d.seqlen = (int32_t)L; d.nheads = (int32_t)H; d.headdim = (int32_t)P;
  d.dstate = (int32_t)N; d.ngroups = (int32_t)G; d.chunk = (int32_t)chunk;
  d.dtype = storage_type(x); d.algo = (int32_t)algo; d.device = x.get_device();
  d.has_z = z ? 1 : 0; d.dt_softplus = dt_softplus ? 1 : 0;
  d.x_stride_b = x.stride(0); d.x_stride_l = x.stride(1);
  d.dt_stride_b = dt.stride(0); d.dt_stride_l = dt.stride(1);
  d.b_stride_b = Bm.stride(0); d.b_stride_l = Bm.stride(1);
  d.c_stride_b = Cm.stride(0); d.c_stride_l = Cm.stride(1);
  if (z) {
    check_seq("z", *z, {Bn, L, H, P}, x);
    d.z_stride_b = z->stride(0); d.z_stride_l = z->stride(1);
  }
  d.y_stride_b = y.stride(0); d.y_stride_l = y.stride(1);
  return d;
}

Tensor workspace_for(const SsdDims& d, const Tensor& like, int32_t pass) {
  const size_t n = ssd_workspace_bytes(&d, pass);
  TORCH_CHECK(n > 0, "ssd_b200: ", ssd_last_error());
  return at::empty({(int64_t)n}, like.options().dtype(at::kByte));
}

// y, final_state = SSD(x, dt, A, B, C, D, z, init_state); saves the inputs and the forward workspace (chunk cumsums,
// chunk-entry states) so that the backward call skips recomputing them.
struct SsdScanNode : public torch::autograd::Function<SsdScanNode> {
  static variable_list forward(AutogradContext* ctx, const Tensor& x, const Tensor& dt, const Tensor& A, const Tensor& Bm,
                               const Tensor& Cm, const OptTensor& D, const OptTensor& z, const OptTensor& init_state,
                               const OptTensor& dt_bias, int64_t chunk, bool dt_softplus, int64_t algo) {
    const Tensor *pD = opt(D), *pz = opt(z), *pinit = opt(init_state), *pbias = opt(dt_bias);
    Tensor y = at::empty(x.sizes(), x.options(), at::MemoryFormat::Contiguous);
    SsdDims d = make_dims(x, dt, Bm, Cm, pz, y, chunk, dt_softplus, algo);
    const int64_t Bn = d.batch, H = d.nheads, P = d.headdim, N = d.dstate;
    check_f32("A", &A, {H}, x);
    check_f32("D", pD, {H}, x);
    check_f32("dt_bias", pbias, {H}, x);
    check_f32("init_state", pinit, {Bn, H, P, N}, x);
    bool needs_grad = false;
    for (const Tensor* t : {&x, &dt, &A, &Bm, &Cm, pD, pz, pinit, pbias}) needs_grad |= (t && t->requires_grad());
    Tensor fin = at::empty({Bn, H, P, N}, x.options().dtype(at::kFloat));
    Tensor ws = workspace_for(d, x, needs_grad ? SSD_PASS_BWD : SSD_PASS_FWD);
    SsdFwdPtrs p;
    std::memset(&p, 0, sizeof p);
    p.x = x.data_ptr(); p.dt = dt.data_ptr(); p.A = A.data_ptr<float>(); p.Bm = Bm.data_ptr(); p.Cm = Cm.data_ptr();
    p.D = fptr(pD); p.z = ptr(pz); p.init_state = fptr(pinit); p.y = y.data_ptr(); p.final_state = fin.data_ptr<float>();
    p.dt_bias = fptr(pbias);
    {
      c10::cuda::CUDAGuard guard(x.device());
      check_rc(ssd_forward(&d, &p, ws.data_ptr(), (size_t)ws.numel(), c10::cuda::getCurrentCUDAStream().stream()));
    }
    if (needs_grad) {
      ctx->save_for_backward({x, dt, A, Bm, Cm, or_undefined(D), or_undefined(z), or_undefined(init_state),
                              or_undefined(dt_bias), ws});
      ctx->saved_data["chunk"] = chunk;
      ctx->saved_data["dt_softplus"] = dt_softplus;
      ctx->saved_data["algo"] = algo;
    }
    return {y, fin};
  }

  static variable_list backward(AutogradContext* ctx, variable_list grads) {
    const variable_list s = ctx->get_saved_variables();
    const Tensor &x = s[0], &dt = s[1], &A = s[2], &Bm = s[3], &Cm = s[4], &ws = s[9];
    const Tensor *pD = s[5].defined() ? &s[5] : nullptr, *pz = s[6].defined() ? &s[6] : nullptr,
                 *pinit = s[7].defined() ? &s[7] : nullptr, *pbias = s[8].defined() ? &s[8] : nullptr;
    Tensor dy = grads[0].defined() ? grads[0] : at::zeros(x.sizes(), x.options());
    if (dy.scalar_type() != x.scalar_type()) dy = dy.to(x.scalar_type());
    if (dy.stride(-1) != 1 || dy.stride(2) != dy.size(3)) dy = dy.contiguous();
    Tensor dfin = grads[1].defined() ? grads[1].to(at::kFloat).contiguous() : Tensor();
    SsdDims d = make_dims(x, dt, Bm, Cm, pz, dy, ctx->saved_data["chunk"].toInt(), ctx->saved_data["dt_softplus"].toBool(),
                          ctx->saved_data["algo"].toInt());
    const int64_t Bn = d.batch, L = d.seqlen, H = d.nheads, P = d.headdim, N = d.dstate, G = d.ngroups;
    const auto f32 = x.options().dtype(at::kFloat);
    Tensor dx = at::empty({Bn, L, H, P}, x.options()), ddt = at::empty({Bn, L, H}, f32), dA = at::empty({H}, f32),
           dB = at::empty({Bn, L, G, N}, x.options()), dC = at::empty({Bn, L, G, N}, x.options());
    Tensor dD = pD ? at::empty({H}, f32) : Tensor(), dz = pz ? at::empty({Bn, L, H, P}, x.options()) : Tensor(),
           dinit = pinit ? at::empty({Bn, H, P, N}, f32) : Tensor(), dbias = pbias ? at::empty({H}, f32) : Tensor();
    SsdBwdPtrs p;
    std::memset(&p, 0, sizeof p);
    p.x = x.data_ptr(); p.dt = dt.data_ptr(); p.A = A.data_ptr<float>(); p.Bm = Bm.data_ptr(); p.Cm = Cm.data_ptr();
    p.D = fptr(pD); p.z = ptr(pz); p.init_state = fptr(pinit);
    p.dy = dy.data_ptr(); p.dfinal_state = dfin.defined() ? dfin.data_ptr<float>() : nullptr;
    p.dx = dx.data_ptr(); p.ddt = ddt.data_ptr<float>(); p.dA = dA.data_ptr<float>(); p.dB = dB.data_ptr(); p.dC = dC.data_ptr();
    p.dD = pD ? dD.data_ptr<float>() : nullptr; p.dz = pz ? dz.data_ptr() : nullptr;
    p.dinit_state = pinit ? dinit.data_ptr<float>() : nullptr;
    p.fwd_saved = 1;
    p.dt_bias = fptr(pbias); p.ddt_bias = pbias ? dbias.data_ptr<float>() : nullptr;
    {
      c10::cuda::CUDAGuard guard(x.device());
      check_rc(ssd_backward(&d, &p, ws.data_ptr(), (size_t)ws.numel(), c10::cuda::getCurrentCUDAStream().stream()));
    }
    return {dx, ddt.to(dt.scalar_type()), dA, dB, dC, dD, dz, dinit, dbias, Tensor(), Tensor(), Tensor()};
  }
};

std::tuple<Tensor, Tensor> ssd_scan_op(const Tensor& x, const Tensor& dt, const Tensor& A, const Tensor& Bm, const Tensor& Cm,
                                       const OptTensor& D, const OptTensor& z, const OptTensor& init_state,
                                       const OptTensor& dt_bias, int64_t chunk, bool dt_softplus, int64_t algo) {
  variable_list r = SsdScanNode::apply(x, dt, A, Bm, Cm, D, z, init_state, dt_bias, chunk, dt_softplus, algo);
  return {r[0], r[1]};
}

// One timestep over all streams, in place on `state` (no gradient: the rollout runs without autograd, as the
// reference's does, trading_bots/src/torch/train/rollout.rs:209-235).
Tensor ssd_state_update_op(Tensor state, const Tensor& x, const Tensor& dt, const Tensor& A, const Tensor& Bm,
                           const Tensor& Cm, const OptTensor& D, const OptTensor& z, const OptTensor& dt_bias,
                           bool dt_softplus) {
  TORCH_CHECK(state.is_cuda() && state.dim() == 4 && state.scalar_type() == at::kFloat && state.is_contiguous(),
              "ssd: state must be a contiguous float32 CUDA tensor [streams, nheads, headdim, dstate]");
  const int64_t S = state.size(0), H = state.size(1), P = state.size(2), N = state.size(3);
  TORCH_CHECK(Bm.dim() == 3 && Bm.size(0) == S && Bm.size(2) == N, "ssd: B must be [streams, ngroups, dstate]");
  const int64_t G = Bm.size(1);
  TORCH_CHECK(G > 0 && H % G == 0, "ssd: nheads must be a multiple of ngroups");
  const Tensor *pD = opt(D), *pz = opt(z), *pbias = opt(dt_bias);
  auto seq = [&](const char* name, const Tensor& t, const Shape& shape) {
    TORCH_CHECK(t.sizes() == at::IntArrayRef(shape) && t.scalar_type() == x.scalar_type() && t.device() == state.device(),
                "ssd: ", name, " must have shape ", at::IntArrayRef(shape), ", x's dtype and the state's device");
    TORCH_CHECK(t.stride(-1) == 1 && (t.dim() < 3 || t.stride(1) == t.size(2)), "ssd: ", name, ": the inner dims must be dense");
  };
  seq("x", x, {S, H, P}); seq("dt", dt, {S, H}); seq("B", Bm, {S, G, N}); seq("C", Cm, {S, G, N});
  if (pz) seq("z", *pz, {S, H, P});
  check_f32("A", &A, {H}, state);
  check_f32("D", pD, {H}, state);
  check_f32("dt_bias", pbias, {H}, state);
  Tensor y = at::empty({S, H, P}, x.options());
  SsdStepDims d;
  std::memset(&d, 0, sizeof d);
  d.streams = (int32_t)S; d.nheads = (int32_t)H; d.headdim = (int32_t)P; d.dstate = (int32_t)N; d.ngroups = (int32_t)G;
  d.dtype = storage_type(x); d.device = state.get_device(); d.dt_softplus = dt_softplus ? 1 : 0;
  d.x_stride_s = x.stride(0); d.dt_stride_s = dt.stride(0); d.b_stride_s = Bm.stride(0); d.c_stride_s = Cm.stride(0);
  d.z_stride_s = pz ? pz->stride(0) : 0; d.y_stride_s = y.stride(0);
  SsdStepPtrs p;
  std::memset(&p, 0, sizeof p);
  p.state = state.data_ptr<float>(); p.x = x.data_ptr(); p.dt = dt.data_ptr(); p.A = A.data_ptr<float>();
  p.Bm = Bm.data_ptr(); p.Cm = Cm.data_ptr(); p.D = fptr(pD); p.z = ptr(pz); p.y = y.data_ptr(); p.dt_bias = fptr(pbias);
  c10::cuda::CUDAGuard guard(state.device());
  check_rc(ssd_state_update(&d, &p, c10::cuda::getCurrentCUDAStream().stream()));
  return y;
}

OptTensor from_c(const Tensor* t) { return (t && t->defined()) ? OptTensor(*t) : OptTensor(); }

}  // namespace

#ifndef SSD_TORCH_IN_LIBTCH
TORCH_LIBRARY(ssd_b200, m) {
  m.def("scan(Tensor x, Tensor dt, Tensor A, Tensor B, Tensor C, Tensor? D, Tensor? z, Tensor? init_state, Tensor? dt_bias, "
        "int chunk, bool dt_softplus, int algo) -> (Tensor, Tensor)", &ssd_scan_op);
  m.def("state_update(Tensor(a!) state, Tensor x, Tensor dt, Tensor A, Tensor B, Tensor C, Tensor? D, Tensor? z, "
        "Tensor? dt_bias, bool dt_softplus) -> Tensor", &ssd_state_update_op);
}
static thread_local char* torch_last_err = nullptr;
#else
extern thread_local char* torch_last_err;
#endif

#define SSD_PROTECT(x)                         \
  try {                                        \
    x                                          \
  } catch (const std::exception& e) {          \
    torch_last_err = strdup(e.what());         \
  }

extern "C" {
typedef at::Tensor* tensor;

// out__[0] = y, out__[1] = final_state.  d, z, init_state, dt_bias may be NULL.  algo: SsdAlgo.
__attribute__((visibility("default"))) void atg_ssd_scan(tensor* out__, tensor x, tensor dt, tensor a, tensor b, tensor c,
                                                         tensor d, tensor z, tensor init_state, tensor dt_bias, int64_t chunk,
                                                         int dt_softplus, int algo) {
  SSD_PROTECT(
    auto r = ssd_scan_op(*x, *dt, *a, *b, *c, from_c(d), from_c(z), from_c(init_state), from_c(dt_bias), chunk,
                         dt_softplus != 0, algo);
    out__[0] = new at::Tensor(std::get<0>(r));
    out__[1] = new at::Tensor(std::get<1>(r));
  )
}

// out__[0] = y; `state` is updated in place.
__attribute__((visibility("default"))) void atg_ssd_state_update(tensor* out__, tensor state, tensor x, tensor dt, tensor a,
                                                                 tensor b, tensor c, tensor d, tensor z, tensor dt_bias,
                                                                 int dt_softplus) {
  SSD_PROTECT(
    out__[0] = new at::Tensor(ssd_state_update_op(*state, *x, *dt, *a, *b, *c, from_c(d), from_c(z), from_c(dt_bias),
                                                  dt_softplus != 0));
  )
}

#ifndef SSD_TORCH_IN_LIBTCH
// Stand-alone build only: the shim has its own get_and_reset_last_err.  The caller frees the string.
__attribute__((visibility("default"))) char* ssd_torch_get_and_reset_last_err() {
  char* e = torch_last_err;
  torch_last_err = nullptr;
  return e;
}
#endif
}
