// Sequence-parallel boundary hand-off through the C ABI: the cross-rank exclusive prefix scan of the
// (total log-decay, slice-total state) records, over NCCL.
//
// A rank that owns a contiguous slice of the sequence runs the local stages with a zero boundary
// state, then calls ssd_sp_exchange_fwd: the slice's total log-decay is read from the chunk cumsums
// in the workspace, the (state, log-decay) records of the ranks before this one arrive in a LOCAL buffer
// (one NCCL group of point-to-point transfers: a rank sends its record to the ranks after it), and
// k_sp_prefix folds them into the state entering the slice.  ssd_sp_exchange_bwd is the mirror image for the state gradient.
// Only NCCL reads a peer's memory; every kernel of this library reads the local copy.
//
// NCCL is bound at run time (dlopen of libnccl.so.2, the copy already loaded by the host program if
// there is one), so the library has no link-time dependency on it and single-GPU users never load it.
#include <dlfcn.h>
#include <nccl.h>
#include <sched.h>
#include <stdio.h>
#include <string.h>
#include <time.h>

#include <mutex>

#include "common.cuh"
#include "ssd_internal.h"

namespace ssd {
namespace {

struct NcclApi {
  ncclResult_t (*GetUniqueId)(ncclUniqueId*);
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int);
  ncclResult_t (*CommDestroy)(ncclComm_t);
  ncclResult_t (*CommAbort)(ncclComm_t);
  ncclResult_t (*CommCount)(const ncclComm_t, int*);
  ncclResult_t (*CommUserRank)(const ncclComm_t, int*);
  ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*);
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t);
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t);
  ncclResult_t (*Send)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t);
  ncclResult_t (*Recv)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t);
  ncclResult_t (*GroupStart)();
  ncclResult_t (*GroupEnd)();
  const char* (*GetErrorString)(ncclResult_t);
  bool ok = false;
};

NcclApi g_nccl;
std::once_flag g_nccl_once;
char g_nccl_why[256] = "";

const NcclApi* nccl() {
  std::call_once(g_nccl_once, [] {
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) { snprintf(g_nccl_why, sizeof(g_nccl_why), "dlopen(libnccl.so.2) failed: %s", dlerror()); return; }
    bool all = true;
    auto sym = [&](const char* name) { void* p = dlsym(h, name); if (!p) { all = false; snprintf(g_nccl_why, sizeof(g_nccl_why), "libnccl lacks %s", name); } return p; };
    g_nccl.GetUniqueId = (decltype(g_nccl.GetUniqueId))sym("ncclGetUniqueId");
    g_nccl.CommInitRank = (decltype(g_nccl.CommInitRank))sym("ncclCommInitRank");
    g_nccl.CommDestroy = (decltype(g_nccl.CommDestroy))sym("ncclCommDestroy");
    g_nccl.CommAbort = (decltype(g_nccl.CommAbort))sym("ncclCommAbort");
    g_nccl.CommCount = (decltype(g_nccl.CommCount))sym("ncclCommCount");
    g_nccl.CommUserRank = (decltype(g_nccl.CommUserRank))sym("ncclCommUserRank");
    g_nccl.CommGetAsyncError = (decltype(g_nccl.CommGetAsyncError))sym("ncclCommGetAsyncError");
    g_nccl.AllGather = (decltype(g_nccl.AllGather))sym("ncclAllGather");
    g_nccl.AllReduce = (decltype(g_nccl.AllReduce))sym("ncclAllReduce");
    g_nccl.Send = (decltype(g_nccl.Send))sym("ncclSend");
    g_nccl.Recv = (decltype(g_nccl.Recv))sym("ncclRecv");
    g_nccl.GroupStart = (decltype(g_nccl.GroupStart))sym("ncclGroupStart");
    g_nccl.GroupEnd = (decltype(g_nccl.GroupEnd))sym("ncclGroupEnd");
    g_nccl.GetErrorString = (decltype(g_nccl.GetErrorString))sym("ncclGetErrorString");
    g_nccl.ok = all;
  });
  if (!g_nccl.ok) { set_error("NCCL is not available: %s", g_nccl_why); return nullptr; }
  return &g_nccl;
}

#define SSD_NCCL_CHECK(api, call, what)                                                       \
  do {                                                                                        \
    ncclResult_t r__ = (call);                                                                \
    if (r__ != ncclSuccess && r__ != ncclInProgress) {                                        \
      set_error("%s: NCCL error %d: %s", what, (int)r__, (api)->GetErrorString(r__));          \
      return SSD_ERR_CUDA;                                                                    \
    }                                                                                         \
  } while (0)

size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

// Segments of the caller's exchange buffer.
struct ExchLayout {
  size_t gs, gl, ll, sig_all, sig_loc, total;
};
constexpr int kSigInts = 8;
ExchLayout exch_layout(long long bh, long long pn, int world) {
  ExchLayout e;
  size_t o = 0;
  auto take = [&](size_t bytes) { size_t r = o; o += align256(bytes); return r; };
  e.gs = take((size_t)world * bh * pn * sizeof(float));
  e.gl = take((size_t)world * bh * sizeof(float));
  e.ll = take((size_t)bh * sizeof(float));
  e.sig_all = take((size_t)world * kSigInts * sizeof(int32_t));
  e.sig_loc = take(kSigInts * sizeof(int32_t));
  e.total = o;
  return e;
}

double now_ms() {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return ts.tv_sec * 1e3 + ts.tv_nsec * 1e-6;
}

}  // namespace
}  // namespace ssd

using namespace ssd;

// Owning handle, a new/free pair like the reference's at_cuda_graph_new / at_cuda_graph_free
// (vendor/torch-sys-0.25.0/libtch/torch_api.cpp:378-401).
struct SsdSpComm {
  ncclComm_t comm;
  int world, rank;
  bool owned;
  int32_t* host_sig;   // pinned staging for the checked mode's signature read-back (made once, with the handle)
};

static SsdSpComm* make_handle(ncclComm_t comm, int world, int rank, bool owned) {
  int32_t* hs = nullptr;
  if (cudaHostAlloc((void**)&hs, 64 * 8 * sizeof(int32_t), cudaHostAllocDefault) != cudaSuccess) hs = nullptr;
  return new SsdSpComm{comm, world, rank, owned, hs};
}

namespace {

// Wait on the host until everything enqueued on `s` so far has completed, at most `timeout_ms`.
int wait_with_timeout(const NcclApi* api, SsdSpComm* c, cudaStream_t s, int timeout_ms, const char* what) {
  cudaEvent_t ev;
  if (cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) != cudaSuccess) { set_error("%s: cudaEventCreate failed", what); return SSD_ERR_CUDA; }
  cudaEventRecord(ev, s);
  const double t0 = now_ms();
  int rc = SSD_OK;
  for (;;) {
    const cudaError_t e = cudaEventQuery(ev);
    if (e == cudaSuccess) break;
    if (e != cudaErrorNotReady) { set_error("%s: %s", what, cudaGetErrorString(e)); rc = SSD_ERR_CUDA; break; }
    ncclResult_t ar = ncclSuccess;
    if (api->CommGetAsyncError(c->comm, &ar) == ncclSuccess && ar != ncclSuccess && ar != ncclInProgress) {
      set_error("%s: NCCL reported an asynchronous error %d: %s", what, (int)ar, api->GetErrorString(ar));
      rc = SSD_ERR_CUDA;
      break;
    }
    if (now_ms() - t0 > timeout_ms) {
      set_error("%s: the exchange did not complete within %d ms (a rank that never joined, or a stalled link); "
                "the communicator should be aborted with ssd_sp_comm_abort", what, timeout_ms);
      rc = SSD_ERR_TIMEOUT;
      break;
    }
    sched_yield();
  }
  cudaEventDestroy(ev);
  return rc;
}

int exchange(const SsdDims* dims, const void* workspace, size_t workspace_bytes, SsdSpComm* c, int direction,
             const float* local_total, const float* boundary, float* state_in, void* exch, size_t exch_bytes,
             void* cuda_stream, int timeout_ms, const char* who) {
  clear_error();
  const NcclApi* api = nccl();
  if (!api) return SSD_ERR_UNSUPPORTED;
  if (!c || !c->comm) { set_error("%s: comm is NULL", who); return SSD_ERR_NULL_POINTER; }
  if (!dims || !workspace || !local_total || !state_in || !exch) { set_error("%s: NULL pointer", who); return SSD_ERR_NULL_POINTER; }
  if (timeout_ms < 0) { set_error("%s: timeout_ms must be >= 0", who); return SSD_ERR_BAD_SHAPE; }
  const size_t need_ws = ssd_workspace_bytes(dims, SSD_PASS_FWD);
  if (need_ws == 0) return SSD_ERR_BAD_SHAPE;
  if (workspace_bytes < need_ws) { set_error("%s: workspace too small: have %zu bytes, need %zu", who, workspace_bytes, need_ws); return SSD_ERR_WORKSPACE_TOO_SMALL; }
  const long long bh = (long long)dims->batch * dims->nheads, pn = (long long)dims->headdim * dims->dstate;
  const ExchLayout e = exch_layout(bh, pn, c->world);
  if (((uintptr_t)exch) & 255) { set_error("%s: the exchange buffer must be 256-byte aligned", who); return SSD_ERR_BAD_ALIGNMENT; }
  if (exch_bytes < e.total) { set_error("%s: exchange buffer too small: have %zu bytes, need %zu", who, exch_bytes, e.total); return SSD_ERR_WORKSPACE_TOO_SMALL; }
  cudaStream_t s = (cudaStream_t)cuda_stream;
  char* eb = (char*)exch;
  float* gs = (float*)(eb + e.gs);
  float* gl = (float*)(eb + e.gl);
  float* ll = (float*)(eb + e.ll);

  if (timeout_ms > 0) {
    // Checked mode: a fixed-size signature goes round first, so that ranks that disagree about the problem are told
    // so (SSD_ERR_BAD_SHAPE) instead of entering a payload collective with different counts.
    int32_t sig[kSigInts] = {0x53534431, c->world, dims->batch, dims->nheads, dims->headdim, dims->dstate, direction, 0};
    int32_t* all = c->host_sig;
    if (c->world > 64 || !all) { set_error("%s: checked mode supports up to 64 ranks and needs its pinned staging", who); return SSD_ERR_UNSUPPORTED; }
    cudaError_t ce = cudaMemcpyAsync(eb + e.sig_loc, sig, sizeof(sig), cudaMemcpyHostToDevice, s);
    if (ce != cudaSuccess) { set_error("%s: %s", who, cudaGetErrorString(ce)); return SSD_ERR_CUDA; }
    SSD_NCCL_CHECK(api, api->AllGather(eb + e.sig_loc, eb + e.sig_all, kSigInts, ncclInt32, c->comm, s), who);
    ce = cudaMemcpyAsync(all, eb + e.sig_all, (size_t)c->world * sizeof(sig), cudaMemcpyDeviceToHost, s);
    if (ce != cudaSuccess) { set_error("%s: %s", who, cudaGetErrorString(ce)); return SSD_ERR_CUDA; }
    int rc = wait_with_timeout(api, c, s, timeout_ms, who);
    if (rc) return rc;
    for (int q = 0; q < c->world; ++q)
      if (memcmp(all + q * kSigInts, sig, sizeof(sig)) != 0) {
        const int32_t* o = all + q * kSigInts;
        set_error("%s: rank %d disagrees about the problem: it has world %d batch %d nheads %d headdim %d dstate %d direction %d, "
                  "this rank has %d %d %d %d %d %d", who, q, o[1], o[2], o[3], o[4], o[5], o[6], sig[1], sig[2], sig[3], sig[4], sig[5], sig[6]);
        return SSD_ERR_BAD_SHAPE;
      }
  }

  int rc = ssd_sp_total_logdecay(dims, workspace, workspace_bytes, ll, cuda_stream);
  if (rc) return rc;
  // A rank needs the records of the ranks before it (after it, for the gradient) and nobody else's: one grouped set of
  // point-to-point transfers, every pair at once through the switch, instead of an all-gather that walks all ranks' records
  // through every rank (exposed exchange time of a 16384-token-per-rank step at 4 ranks: 0.142 -> 0.120 ms; most of what
  // remains is the fixed cost of three collective launches per step, not wire time).
  SSD_NCCL_CHECK(api, api->GroupStart(), who);
  for (int q = 0; q < c->world; ++q) {
    if (q == c->rank) continue;
    const bool send_to = direction > 0 ? q > c->rank : q < c->rank;
    if (send_to) {
      SSD_NCCL_CHECK(api, api->Send(local_total, (size_t)(bh * pn), ncclFloat32, q, c->comm, s), who);
      SSD_NCCL_CHECK(api, api->Send(ll, (size_t)bh, ncclFloat32, q, c->comm, s), who);
    } else {
      SSD_NCCL_CHECK(api, api->Recv(gs + (size_t)q * bh * pn, (size_t)(bh * pn), ncclFloat32, q, c->comm, s), who);
      SSD_NCCL_CHECK(api, api->Recv(gl + (size_t)q * bh, (size_t)bh, ncclFloat32, q, c->comm, s), who);
    }
  }
  SSD_NCCL_CHECK(api, api->GroupEnd(), who);
  rc = ssd_sp_prefix_state(gs, gl, c->world, c->rank, direction, bh, pn, boundary, state_in, cuda_stream);
  if (rc) return rc;
  if (timeout_ms > 0) return wait_with_timeout(api, c, s, timeout_ms, who);
  return SSD_OK;
}

}  // namespace

extern "C" {

int32_t ssd_sp_unique_id(void* id128) {
  clear_error();
  const NcclApi* api = nccl();
  if (!api) return SSD_ERR_UNSUPPORTED;
  if (!id128) { set_error("id128 is NULL"); return SSD_ERR_NULL_POINTER; }
  static_assert(sizeof(ncclUniqueId) == SSD_SP_UNIQUE_ID_BYTES, "unique id size");
  ncclUniqueId id;
  SSD_NCCL_CHECK(api, api->GetUniqueId(&id), "ssd_sp_unique_id");
  memcpy(id128, &id, sizeof(id));
  return SSD_OK;
}

SsdSpComm* ssd_sp_comm_new(const void* id128, int32_t world, int32_t rank) {
  clear_error();
  const NcclApi* api = nccl();
  if (!api) return nullptr;
  if (!id128) { set_error("id128 is NULL"); return nullptr; }
  if (world <= 0 || rank < 0 || rank >= world) { set_error("bad world/rank %d/%d", world, rank); return nullptr; }
  ncclUniqueId id;
  memcpy(&id, id128, sizeof(id));
  ncclComm_t comm = nullptr;
  const ncclResult_t r = api->CommInitRank(&comm, world, id, rank);
  if (r != ncclSuccess) { set_error("ncclCommInitRank failed: %s", api->GetErrorString(r)); return nullptr; }
  return make_handle(comm, world, rank, true);
}

SsdSpComm* ssd_sp_comm_wrap(void* nccl_comm) {
  clear_error();
  const NcclApi* api = nccl();
  if (!api) return nullptr;
  if (!nccl_comm) { set_error("nccl_comm is NULL"); return nullptr; }
  int world = 0, rank = -1;
  if (api->CommCount((ncclComm_t)nccl_comm, &world) != ncclSuccess || api->CommUserRank((ncclComm_t)nccl_comm, &rank) != ncclSuccess) {
    set_error("ssd_sp_comm_wrap: the handle is not a usable ncclComm_t");
    return nullptr;
  }
  return make_handle((ncclComm_t)nccl_comm, world, rank, false);
}

int32_t ssd_sp_comm_world(const SsdSpComm* c) { return c ? c->world : -1; }
int32_t ssd_sp_comm_rank(const SsdSpComm* c) { return c ? c->rank : -1; }

void ssd_sp_comm_free(SsdSpComm* c) {
  if (!c) return;
  if (c->owned && c->comm && g_nccl.ok) g_nccl.CommDestroy(c->comm);
  if (c->host_sig) cudaFreeHost(c->host_sig);
  delete c;
}

int32_t ssd_sp_comm_abort(SsdSpComm* c) {
  clear_error();
  if (!c || !c->comm) { set_error("comm is NULL"); return SSD_ERR_NULL_POINTER; }
  const NcclApi* api = nccl();
  if (!api) return SSD_ERR_UNSUPPORTED;
  const ncclResult_t r = api->CommAbort(c->comm);
  c->comm = nullptr;
  if (r != ncclSuccess) { set_error("ncclCommAbort: %s", api->GetErrorString(r)); return SSD_ERR_CUDA; }
  return SSD_OK;
}

size_t ssd_sp_exchange_bytes(const SsdDims* dims, int32_t world) {
  clear_error();
  if (!dims || world <= 0) { set_error("dims is NULL or world <= 0"); return 0; }
  if (dims->batch <= 0 || dims->nheads <= 0 || dims->headdim <= 0 || dims->dstate <= 0) { set_error("batch/nheads/headdim/dstate must be positive"); return 0; }
  return exch_layout((long long)dims->batch * dims->nheads, (long long)dims->headdim * dims->dstate, world).total;
}

int32_t ssd_sp_exchange_fwd(const SsdDims* dims, const void* workspace, size_t workspace_bytes, SsdSpComm* comm,
                            const float* local_final_state, const float* init_state, float* state_in, void* exchange_buf,
                            size_t exchange_bytes, void* cuda_stream, int32_t timeout_ms) {
  return exchange(dims, workspace, workspace_bytes, comm, +1, local_final_state, init_state, state_in, exchange_buf,
                  exchange_bytes, cuda_stream, timeout_ms, "ssd_sp_exchange_fwd");
}

int32_t ssd_sp_exchange_bwd(const SsdDims* dims, const void* workspace, size_t workspace_bytes, SsdSpComm* comm,
                            const float* local_dinit_state, const float* dfinal_state, float* dstate_out, void* exchange_buf,
                            size_t exchange_bytes, void* cuda_stream, int32_t timeout_ms) {
  return exchange(dims, workspace, workspace_bytes, comm, -1, local_dinit_state, dfinal_state, dstate_out, exchange_buf,
                  exchange_bytes, cuda_stream, timeout_ms, "ssd_sp_exchange_bwd");
}

int32_t ssd_sp_allreduce_params(SsdSpComm* c, float* dA, float* dD, int32_t nheads, void* cuda_stream, int32_t timeout_ms) {
  clear_error();
  const NcclApi* api = nccl();
  if (!api) return SSD_ERR_UNSUPPORTED;
  if (!c || !c->comm || !dA) { set_error("comm/dA is NULL"); return SSD_ERR_NULL_POINTER; }
  if (nheads <= 0 || timeout_ms < 0) { set_error("nheads must be positive, timeout_ms >= 0"); return SSD_ERR_BAD_SHAPE; }
  cudaStream_t s = (cudaStream_t)cuda_stream;
  SSD_NCCL_CHECK(api, api->GroupStart(), "ssd_sp_allreduce_params");
  SSD_NCCL_CHECK(api, api->AllReduce(dA, dA, (size_t)nheads, ncclFloat32, ncclSum, c->comm, s), "ssd_sp_allreduce_params");
  if (dD) SSD_NCCL_CHECK(api, api->AllReduce(dD, dD, (size_t)nheads, ncclFloat32, ncclSum, c->comm, s), "ssd_sp_allreduce_params");
  SSD_NCCL_CHECK(api, api->GroupEnd(), "ssd_sp_allreduce_params");
  if (timeout_ms > 0) return wait_with_timeout(api, c, s, timeout_ms, "ssd_sp_allreduce_params");
  return SSD_OK;
}

}  // extern "C"
