// extern "C" entry points: argument validation, workspace layout, kernel-family dispatch.
#include <atomic>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include "common.cuh"
#include "ssd_internal.h"

namespace ssd {

static thread_local char g_err[512] = {0};

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}
void clear_error() { g_err[0] = 0; }

// ---- launch counter and per-kernel event profile -------------------------------------------
static std::atomic<long long> g_launches{0};
constexpr int kMaxProf = 256;
struct Profile {
  bool on = false;
  int n = 0;
  cudaEvent_t ev[kMaxProf + 1];
  const char* name[kMaxProf];
};
static thread_local Profile g_prof;

void after_launch(const char* what, cudaStream_t s) {
  g_launches.fetch_add(1, std::memory_order_relaxed);
  Profile& p = g_prof;
  if (p.on && p.n < kMaxProf) {
    if (cudaEventCreate(&p.ev[p.n + 1]) == cudaSuccess) {
      cudaEventRecord(p.ev[p.n + 1], s);
      p.name[p.n] = what;
      ++p.n;
    }
  }
}

static size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

// Returns 0 or a negative status (error string set).
static int make_geo(const SsdDims* d, Geo* g) {
  if (!d) { set_error("dims is NULL"); return SSD_ERR_NULL_POINTER; }
  if (d->batch <= 0 || d->seqlen <= 0 || d->nheads <= 0 || d->headdim <= 0 || d->dstate <= 0 || d->ngroups <= 0 ||
      d->chunk <= 0) {
    set_error("all of batch/seqlen/nheads/headdim/dstate/ngroups/chunk must be positive (got %d %d %d %d %d %d %d)",
              d->batch, d->seqlen, d->nheads, d->headdim, d->dstate, d->ngroups, d->chunk);
    return SSD_ERR_BAD_SHAPE;
  }
  if (d->nheads % d->ngroups) {
    set_error("nheads (%d) must be a multiple of ngroups (%d)", d->nheads, d->ngroups);
    return SSD_ERR_BAD_SHAPE;
  }
  if (d->chunk > 256) { set_error("chunk (%d) must be <= 256", d->chunk); return SSD_ERR_UNSUPPORTED; }
  if (d->dtype != SSD_F32 && d->dtype != SSD_BF16) { set_error("unknown dtype %d", d->dtype); return SSD_ERR_UNSUPPORTED; }
  if (d->algo < SSD_ALGO_AUTO || d->algo > SSD_ALGO_TENSOR_ONETILE) { set_error("unknown algo %d", d->algo); return SSD_ERR_UNSUPPORTED; }
  g->B = d->batch; g->L = d->seqlen; g->H = d->nheads; g->P = d->headdim; g->N = d->dstate; g->G = d->ngroups;
  g->Q = d->chunk; g->nc = (d->seqlen + d->chunk - 1) / d->chunk; g->hpg = d->nheads / d->ngroups;
  g->dt_softplus = d->dt_softplus != 0;
  g->onetile = d->algo == SSD_ALGO_TENSOR_ONETILE;
  if (g->B > 65535) { set_error("batch (%d) must be <= 65535 (grid limit)", g->B); return SSD_ERR_UNSUPPORTED; }
  const long long HP = (long long)g->H * g->P, GN = (long long)g->G * g->N;
  auto pick = [](long long v, long long dflt) { return v ? v : dflt; };
  g->xsl = pick(d->x_stride_l, HP);     g->xsb = pick(d->x_stride_b, HP * g->L);
  g->dtsl = pick(d->dt_stride_l, g->H); g->dtsb = pick(d->dt_stride_b, (long long)g->H * g->L);
  g->bsl = pick(d->b_stride_l, GN);     g->bsb = pick(d->b_stride_b, GN * g->L);
  g->csl = pick(d->c_stride_l, GN);     g->csb = pick(d->c_stride_b, GN * g->L);
  g->zsl = pick(d->z_stride_l, HP);     g->zsb = pick(d->z_stride_b, HP * g->L);
  g->ysl = pick(d->y_stride_l, HP);     g->ysb = pick(d->y_stride_b, HP * g->L);
  if (g->xsl < HP || g->zsl < HP || g->ysl < HP || g->dtsl < g->H || g->bsl < GN || g->csl < GN) {
    set_error("sequence strides must be at least the dense row size");
    return SSD_ERR_BAD_SHAPE;
  }
  if (d->device >= 0) {
    int cur = -1;
    if (cudaGetDevice(&cur) != cudaSuccess || cur != d->device) {
      set_error("current CUDA device is %d but dims.device is %d (the library never switches devices)", cur, d->device);
      return SSD_ERR_CUDA;
    }
  }
  // The chunk length only schedules the evaluation; the operator's result does not depend on it.
  // The tensor-core family works on 128-long chunks, so a requested chunk that is a larger
  // multiple of 128 is evaluated as consecutive 128-long chunks when that family will run.
  if (d->algo != SSD_ALGO_FP32_CORES && d->chunk > 128 && d->chunk % 128 == 0) {
    Geo t = *g;
    t.Q = 128;
    t.nc = (t.L + 127) / 128;
    if (tensor_supported(t, d->dtype, nullptr)) *g = t;
  }
  return SSD_OK;
}

static void make_layout(const Geo& g, bool has_z, bool tcfam, WsLayout* w) {
  const size_t f = sizeof(float);
  const size_t nq = (size_t)g.B * g.H * g.nc * g.Q * f;
  const size_t nst = (size_t)g.B * g.nc * g.H * g.P * g.N * f;
  const size_t nfin = (size_t)g.B * g.H * g.P * g.N * f;
  const size_t ncb = (size_t)g.B * g.nc * g.G * g.Q * g.Q * f;
  const size_t nbh = (size_t)g.B * g.nc * g.H * f;
  size_t o = 0;
  auto take = [&](size_t bytes) { size_t r = o; o += align256(bytes); return r; };
  w->status = take(256);
  w->cs = take(nq); w->dtf = take(nq); w->states = take(nst); w->fin = take(nfin);
  w->cb = take(tcfam ? 0 : ncb);   // C B^T stays on chip in the tensor-core family
  w->tab = take(tcfam ? (size_t)g.B * g.nc * g.H * SSD_TAB_FLOATS * f : 0);
  w->prev_bf = take(tcfam ? nst / 2 : 0);
  w->hmax = take(tcfam ? (size_t)(g.H + 1) * f : 0);   // per head: tag of the last cumsum launch that saw a strong decay; [H]: current tag
  w->total_fwd = o;
  w->dstates = take(nst);
  w->ds_bf = take(tcfam ? nst / 2 : 0);
  w->wsum = take(tcfam ? 0 : ncb);
  w->dyp = take(has_z ? (size_t)g.B * g.L * g.H * g.P * f : 0);
  w->dcsp = take(nq); w->ddtd = take(nq); w->ddot = take(nq);
  w->sdot = take(nbh * (tcfam ? 64 : 1));   // tensor family: up to 64 warp-partial sums per entry
  w->dapart = take(nbh); w->ddpart = take(nbh);
  w->dini = take(nfin);
  w->total_bwd = o;
}

static bool family_is_tensor(const Geo& g, const SsdDims* d) {
  return d->algo != SSD_ALGO_FP32_CORES && tensor_supported(g, d->dtype, nullptr);
}

// The CUDA-core kernels put (chunk, head) on one grid axis.
static int check_core_grid(const Geo& g) {
  if ((long long)g.nc * g.H > 65535) {
    set_error("CUDA-core family: nchunks*nheads (%lld) must be <= 65535 (grid limit)", (long long)g.nc * g.H);
    return SSD_ERR_UNSUPPORTED;
  }
  return 0;
}

// Kernel-family choice: 1 = tensor cores, 0 = CUDA cores, <0 = error.
static int pick_family(const Geo& g, const SsdDims* d) {
  if (d->algo == SSD_ALGO_FP32_CORES) return check_core_grid(g);
  const char* why = "";
  if (tensor_supported(g, d->dtype, &why)) return 1;
  if (d->algo != SSD_ALGO_AUTO) { set_error("algo=TENSOR not possible for these dims: %s", why); return SSD_ERR_UNSUPPORTED; }
  return check_core_grid(g);
}

// The tensor-core kernels move whole 16-byte vectors through pointers that no tensor map checks (z, y, dx, dz, dB, dC).
static int check_align16(const char* name, const void* p) {
  if (p && ((uintptr_t)p & 15)) {
    set_error("%s must be 16-byte aligned for the tensor-core kernels (got %p)", name, p);
    return SSD_ERR_BAD_ALIGNMENT;
  }
  return SSD_OK;
}

static int check_ws(const void* ws, size_t have, size_t need) {
  if (!ws) { set_error("workspace is NULL"); return SSD_ERR_NULL_POINTER; }
  if (((uintptr_t)ws) & 255) { set_error("workspace must be 256-byte aligned"); return SSD_ERR_BAD_ALIGNMENT; }
  if (have < need) { set_error("workspace too small: have %zu bytes, need %zu", have, need); return SSD_ERR_WORKSPACE_TOO_SMALL; }
  return SSD_OK;
}

int status_code_to_rc(int32_t code, const char* where) {
  if (code == 0) return SSD_OK;
  set_error("%s: a bounded wait inside a pipelined kernel ran out (wait-site code %d); the results of that call are invalid, "
            "the context is still usable", where, (int)code);
  return SSD_ERR_TIMEOUT;
}
int read_status_sync(const void* word, void* cuda_stream, int32_t* code_out, const char* where) {
  int32_t code = 0;
  cudaStream_t s = (cudaStream_t)cuda_stream;
  cudaError_t e = cudaMemcpyAsync(&code, word, sizeof(code), cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  if (e != cudaSuccess) {
    set_error("%s: reading the status word failed: %s (not usable while the stream is being captured)", where, cudaGetErrorString(e));
    return SSD_ERR_CUDA;
  }
  if (code_out) *code_out = code;
  return status_code_to_rc(code, where);
}

}  // namespace ssd

using namespace ssd;

extern "C" {

const char* ssd_last_error(void) { return g_err; }
int32_t ssd_version(void) { return 2; }
int32_t ssd_compiled_arch(void) { return 100; }
int64_t ssd_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int32_t ssd_profile_begin(void* cuda_stream) {
  clear_error();
  Profile& p = g_prof;
  if (p.on) { set_error("a profile is already open on this thread"); return SSD_ERR_UNSUPPORTED; }
  if (cudaEventCreate(&p.ev[0]) != cudaSuccess) { set_error("cudaEventCreate failed"); return SSD_ERR_CUDA; }
  cudaEventRecord(p.ev[0], (cudaStream_t)cuda_stream);
  p.n = 0;
  p.on = true;
  return SSD_OK;
}

int32_t ssd_profile_end(char* names, size_t names_bytes, float* ms, int32_t max_entries) {
  clear_error();
  Profile& p = g_prof;
  if (!p.on) { set_error("no profile is open on this thread"); return SSD_ERR_UNSUPPORTED; }
  p.on = false;
  int rc = SSD_OK;
  if (p.n > 0 && cudaEventSynchronize(p.ev[p.n]) != cudaSuccess) { set_error("cudaEventSynchronize failed"); rc = SSD_ERR_CUDA; }
  size_t off = 0;
  int out = 0;
  for (int i = 0; i < p.n; ++i) {
    float t = 0.f;
    if (rc == SSD_OK) cudaEventElapsedTime(&t, p.ev[i], p.ev[i + 1]);
    if (i < max_entries && ms && names) {
      const size_t len = strlen(p.name[i]);
      if (off + len + 2 <= names_bytes) {
        memcpy(names + off, p.name[i], len);
        off += len;
        names[off++] = '\n';
        names[off] = 0;
        ms[out++] = t;
      }
    }
  }
  for (int i = 0; i <= p.n; ++i) cudaEventDestroy(p.ev[i]);
  p.n = 0;
  return rc == SSD_OK ? out : rc;
}

size_t ssd_workspace_bytes(const SsdDims* dims, int32_t pass) {
  clear_error();
  Geo g;
  SsdDims d2;
  if (dims) { d2 = *dims; d2.device = -1; }
  if (make_geo(dims ? &d2 : nullptr, &g)) return 0;
  WsLayout w;
  make_layout(g, dims->has_z != 0, family_is_tensor(g, dims), &w);
  return pass == SSD_PASS_BWD ? w.total_bwd : w.total_fwd;
}

int32_t ssd_forward_staged(const SsdDims* dims, const SsdFwdPtrs* p, void* workspace, size_t workspace_bytes,
                           void* cuda_stream, int32_t stages) {
  clear_error();
  Geo g;
  int rc = make_geo(dims, &g);
  if (rc) return rc;
  if (!p) { set_error("ptrs is NULL"); return SSD_ERR_NULL_POINTER; }
  if (!p->x || !p->dt || !p->A || !p->Bm || !p->Cm) { set_error("x, dt, A, B, C must be non-NULL"); return SSD_ERR_NULL_POINTER; }
  if ((stages & SSD_STAGE_FINISH) && !p->y) { set_error("y must be non-NULL"); return SSD_ERR_NULL_POINTER; }
  if ((p->z != nullptr) != (dims->has_z != 0)) { set_error("dims.has_z (%d) does not match the z pointer", dims->has_z); return SSD_ERR_BAD_SHAPE; }
  if (stages == 0 || (stages & ~(SSD_STAGE_LOCAL | SSD_STAGE_TOTAL | SSD_STAGE_FINISH | SSD_STAGE_LOCAL_STATES | SSD_STAGE_LOCAL_REST))) { set_error("bad stage mask %d", stages); return SSD_ERR_BAD_SHAPE; }
  WsLayout w;
  make_layout(g, dims->has_z != 0, family_is_tensor(g, dims), &w);
  rc = check_ws(workspace, workspace_bytes, w.total_fwd);
  if (rc) return rc;
  cudaStream_t s = (cudaStream_t)cuda_stream;
  SsdFwdPtrs q = *p;
  q.final_state = nullptr;  // kernels always leave the final state in the workspace; copied out below
  const int fam = pick_family(g, dims);
  if (fam < 0) return fam;
  if (fam == 1) {
    const void* ptrs[] = {p->x, p->Bm, p->Cm, p->z, p->y};
    const char* names[] = {"x", "B", "C", "z", "y"};
    for (int i = 0; i < 5; ++i)
      if ((rc = check_align16(names[i], ptrs[i]))) return rc;
  }
  rc = run_forward(g, dims->dtype, fam == 1, q, (char*)workspace, w, s, stages);
  if (rc) return rc;
  if (p->final_state && (stages & (SSD_STAGE_TOTAL | SSD_STAGE_FINISH))) {
    cudaError_t e = cudaMemcpyAsync(p->final_state, (char*)workspace + w.fin,
                                    (size_t)g.B * g.H * g.P * g.N * sizeof(float), cudaMemcpyDeviceToDevice, s);
    if (e != cudaSuccess) { set_error("final_state copy: %s", cudaGetErrorString(e)); return SSD_ERR_CUDA; }
  }
  return SSD_OK;
}

int32_t ssd_forward(const SsdDims* dims, const SsdFwdPtrs* p, void* workspace, size_t workspace_bytes,
                    void* cuda_stream) {
  return ssd_forward_staged(dims, p, workspace, workspace_bytes, cuda_stream, SSD_STAGE_ALL);
}

int32_t ssd_backward_staged(const SsdDims* dims, const SsdBwdPtrs* p, void* workspace, size_t workspace_bytes,
                            void* cuda_stream, int32_t stages) {
  clear_error();
  Geo g;
  int rc = make_geo(dims, &g);
  if (rc) return rc;
  if (!p) { set_error("ptrs is NULL"); return SSD_ERR_NULL_POINTER; }
  if (!p->x || !p->dt || !p->A || !p->Bm || !p->Cm || !p->dy) { set_error("x, dt, A, B, C, dy must be non-NULL"); return SSD_ERR_NULL_POINTER; }
  if (stages & SSD_STAGE_FINISH) {
    if (!p->dx || !p->ddt || !p->dA || !p->dB || !p->dC) { set_error("dx, ddt, dA, dB, dC must be non-NULL"); return SSD_ERR_NULL_POINTER; }
    if (p->D && !p->dD) { set_error("dD must be non-NULL when D is given"); return SSD_ERR_NULL_POINTER; }
    if (p->dt_bias && !p->ddt_bias) { set_error("ddt_bias must be non-NULL when dt_bias is given"); return SSD_ERR_NULL_POINTER; }
  }
  if ((p->z != nullptr) != (dims->has_z != 0)) { set_error("dims.has_z (%d) does not match the z pointer", dims->has_z); return SSD_ERR_BAD_SHAPE; }
  if (p->z && !p->dz) { set_error("dz must be non-NULL when z is given"); return SSD_ERR_NULL_POINTER; }
  if (stages == 0 || (stages & ~(SSD_STAGE_LOCAL | SSD_STAGE_TOTAL | SSD_STAGE_FINISH | SSD_STAGE_LOCAL_STATES | SSD_STAGE_LOCAL_REST))) { set_error("bad stage mask %d", stages); return SSD_ERR_BAD_SHAPE; }
  WsLayout w;
  make_layout(g, dims->has_z != 0, family_is_tensor(g, dims), &w);
  rc = check_ws(workspace, workspace_bytes, w.total_bwd);
  if (rc) return rc;
  const int fam = pick_family(g, dims);
  if (fam < 0) return fam;
  if (fam == 1) {
    const void* ptrs[] = {p->x, p->Bm, p->Cm, p->z, p->dy, p->dx, p->dz, p->dB, p->dC};
    const char* names[] = {"x", "B", "C", "z", "dy", "dx", "dz", "dB", "dC"};
    for (int i = 0; i < 9; ++i)
      if ((rc = check_align16(names[i], ptrs[i]))) return rc;
  }
  return run_backward(g, dims->dtype, fam == 1, *p, (char*)workspace, w, (cudaStream_t)cuda_stream, stages);
}

int32_t ssd_backward(const SsdDims* dims, const SsdBwdPtrs* p, void* workspace, size_t workspace_bytes,
                     void* cuda_stream) {
  return ssd_backward_staged(dims, p, workspace, workspace_bytes, cuda_stream, SSD_STAGE_ALL);
}

int32_t ssd_state_update(const SsdStepDims* d, const SsdStepPtrs* p, void* cuda_stream) {
  clear_error();
  if (!d || !p) { set_error("dims/ptrs is NULL"); return SSD_ERR_NULL_POINTER; }
  if (d->streams <= 0 || d->nheads <= 0 || d->headdim <= 0 || d->dstate <= 0 || d->ngroups <= 0) {
    set_error("streams/nheads/headdim/dstate/ngroups must be positive"); return SSD_ERR_BAD_SHAPE;
  }
  if (d->nheads % d->ngroups) { set_error("nheads (%d) must be a multiple of ngroups (%d)", d->nheads, d->ngroups); return SSD_ERR_BAD_SHAPE; }
  if (d->dtype != SSD_F32 && d->dtype != SSD_BF16) { set_error("unknown dtype %d", d->dtype); return SSD_ERR_UNSUPPORTED; }
  if (!p->state || !p->x || !p->dt || !p->A || !p->Bm || !p->Cm || !p->y) { set_error("state, x, dt, A, B, C, y must be non-NULL"); return SSD_ERR_NULL_POINTER; }
  if ((long long)d->streams * d->nheads > 2147483647LL) { set_error("streams*nheads exceeds the grid limit"); return SSD_ERR_UNSUPPORTED; }
  SsdStepDims e = *d;
  const long long HP = (long long)d->nheads * d->headdim, GN = (long long)d->ngroups * d->dstate;
  if (!e.x_stride_s) e.x_stride_s = HP;
  if (!e.z_stride_s) e.z_stride_s = HP;
  if (!e.y_stride_s) e.y_stride_s = HP;
  if (!e.dt_stride_s) e.dt_stride_s = d->nheads;
  if (!e.b_stride_s) e.b_stride_s = GN;
  if (!e.c_stride_s) e.c_stride_s = GN;
  const int N = d->dstate;
  const bool vec = (N == 16 || N == 32 || N == 64 || N == 128 || N == 256);
  if (vec) {
    const size_t es = d->dtype == SSD_BF16 ? 2 : 4;
    if (((uintptr_t)p->state & 15) || ((uintptr_t)p->Bm % (4 * es)) || ((uintptr_t)p->Cm % (4 * es)) ||
        (e.b_stride_s % 4) || (e.c_stride_s % 4)) {
      set_error("state must be 16-byte aligned and B/C rows aligned to 4 elements"); return SSD_ERR_BAD_ALIGNMENT;
    }
  }
  if (d->device >= 0) {
    int cur = -1;
    if (cudaGetDevice(&cur) != cudaSuccess || cur != d->device) {
      set_error("current CUDA device is %d but dims.device is %d", cur, d->device); return SSD_ERR_CUDA;
    }
  }
  return decode_step(e, *p, (cudaStream_t)cuda_stream);
}

// ---- status word ----------------------------------------------------------------------------------

int32_t ssd_workspace_status(const void* workspace, void* cuda_stream, int32_t* code_out) {
  clear_error();
  if (!workspace) { set_error("workspace is NULL"); return SSD_ERR_NULL_POINTER; }
  return read_status_sync(workspace, cuda_stream, code_out, "ssd_workspace_status");
}

int32_t ssd_workspace_status_async(const void* workspace, int32_t* code_dst, void* cuda_stream) {
  clear_error();
  if (!workspace || !code_dst) { set_error("workspace/code_dst is NULL"); return SSD_ERR_NULL_POINTER; }
  cudaError_t e = cudaMemcpyAsync(code_dst, workspace, sizeof(int32_t), cudaMemcpyDefault, (cudaStream_t)cuda_stream);
  if (e != cudaSuccess) { set_error("ssd_workspace_status_async: %s", cudaGetErrorString(e)); return SSD_ERR_CUDA; }
  return SSD_OK;
}

int32_t ssd_status_check(int32_t code) {
  clear_error();
  return status_code_to_rc(code, "ssd_status_check");
}

int32_t ssd_selftest_bounded_wait(int32_t* device_status, int64_t max_cycles, void* cuda_stream) {
  clear_error();
  if (!device_status) { set_error("device_status is NULL"); return SSD_ERR_NULL_POINTER; }
  if (max_cycles <= 0 || max_cycles > 2000000000LL) { set_error("max_cycles must be in (0, 2e9]"); return SSD_ERR_BAD_SHAPE; }
  return tensor_selftest_wait((int*)device_status, (long long)max_cycles, (cudaStream_t)cuda_stream);
}

int32_t ssd_state_reset_rows(float* state, int64_t row_elems, const int64_t* stream_idx, int64_t count,
                             int64_t streams, void* cuda_stream) {
  clear_error();
  if (!state || (!stream_idx && count > 0)) { set_error("state/stream_idx is NULL"); return SSD_ERR_NULL_POINTER; }
  if (row_elems <= 0 || count < 0 || streams <= 0) { set_error("row_elems/streams must be positive, count >= 0"); return SSD_ERR_BAD_SHAPE; }
  if (((uintptr_t)state & 15) || (row_elems % 4)) { set_error("state must be 16-byte aligned with row_elems %% 4 == 0"); return SSD_ERR_BAD_ALIGNMENT; }
  return reset_rows(state, row_elems, (const long long*)stream_idx, count, streams, (cudaStream_t)cuda_stream);
}

int32_t ssd_sp_total_logdecay(const SsdDims* dims, const void* workspace, size_t workspace_bytes, float* out,
                              void* cuda_stream) {
  clear_error();
  Geo g;
  int rc = make_geo(dims, &g);
  if (rc) return rc;
  if (!out) { set_error("out is NULL"); return SSD_ERR_NULL_POINTER; }
  WsLayout w;
  make_layout(g, dims->has_z != 0, family_is_tensor(g, dims), &w);
  rc = check_ws(workspace, workspace_bytes, w.total_fwd);
  if (rc) return rc;
  return sp_total_logdecay(g, (const float*)((const char*)workspace + w.cs), out, (cudaStream_t)cuda_stream);
}

int32_t ssd_sp_prefix_state(const float* gathered_states, const float* gathered_logdecay, int32_t world, int32_t rank,
                            int32_t direction, int64_t batch_heads, int64_t state_elems, const float* boundary,
                            float* state_in, void* cuda_stream) {
  clear_error();
  if (!gathered_states || !gathered_logdecay || !state_in) { set_error("NULL pointer"); return SSD_ERR_NULL_POINTER; }
  if (world <= 0 || rank < 0 || rank >= world) { set_error("bad world/rank %d/%d", world, rank); return SSD_ERR_BAD_SHAPE; }
  if (direction != 1 && direction != -1) { set_error("direction must be +1 or -1"); return SSD_ERR_BAD_SHAPE; }
  if (batch_heads <= 0 || batch_heads > 65535 || state_elems <= 0) { set_error("bad batch_heads/state_elems"); return SSD_ERR_BAD_SHAPE; }
  return sp_prefix_state(gathered_states, gathered_logdecay, world, rank, direction, batch_heads, state_elems, boundary,
                         state_in, (cudaStream_t)cuda_stream);
}

}  // extern "C"
