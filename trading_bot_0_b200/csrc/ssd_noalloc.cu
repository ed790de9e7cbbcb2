// Forward pass for callers that have no way to allocate device memory.
//
// ssd_forward needs a scratch buffer (chunk cumsums, per-chunk states, the final state).  Most
// callers take it from their tensor allocator.  Some cannot: a rollout or paper-trading loop
// that runs after its memory pool has been frozen, a host that holds only raw device pointers
// handed over an FFI and no allocator handle, or a process whose remaining device memory is
// spoken for.  For them this file keeps the scratch in a fixed array that is part of the
// loaded library image on every GPU that loads it, and lends it to ssd_forward.
#include <mutex>

#include "common.cuh"
#include "ssd_internal.h"

namespace {

// The whole budget of the no-allocation entry point.  Lives in every context that loads the
// library, from load to exit, whether or not the entry point is ever called.
constexpr size_t kScratchBytes = SSD_NOALLOC_MAX_BYTES;
static __device__ __align__(256) unsigned char g_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
void* g_ptr[kMaxDevices] = {nullptr};   // device address of g_scratch, per device ordinal

}  // namespace

// Device address of g_scratch on the current device.  Once per device, with that device current: in host code the
// array's name is only a stand-in for the symbol, so ask the runtime where the array lives on this device.
static int scratch_address(const char* who, void** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    ssd::set_error("%s: no usable current CUDA device (ordinal %d)", who, dev);
    return SSD_ERR_CUDA;
  }
  std::lock_guard<std::mutex> lock(g_mu);
  if (!g_ptr[dev]) {
    void* q = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&q, g_scratch);
    if (e != cudaSuccess || !q) {
      ssd::set_error("%s: cudaGetSymbolAddress failed on device %d: %s", who, dev, cudaGetErrorString(e));
      return SSD_ERR_CUDA;
    }
    g_ptr[dev] = q;
  }
  *out = g_ptr[dev];
  return SSD_OK;
}

extern "C" int32_t ssd_forward_noalloc(const SsdDims* dims, const SsdFwdPtrs* p, void* cuda_stream) {
  ssd::clear_error();
  if (!dims || !p) { ssd::set_error("dims/ptrs is NULL"); return SSD_ERR_NULL_POINTER; }
  const size_t need = ssd_workspace_bytes(dims, SSD_PASS_FWD);
  if (need == 0) return SSD_ERR_BAD_SHAPE;   // message already set by ssd_workspace_bytes
  if (need > kScratchBytes) {
    ssd::set_error("ssd_forward_noalloc: these dims need %zu bytes of scratch but the built-in buffer holds %zu "
                   "(SSD_NOALLOC_MAX_BYTES); use ssd_forward with a caller-owned workspace", need, kScratchBytes);
    return SSD_ERR_WORKSPACE_TOO_SMALL;
  }
  void* scratch = nullptr;
  const int rc = scratch_address("ssd_forward_noalloc", &scratch);
  if (rc) return rc;
  return ssd_forward(dims, p, scratch, kScratchBytes, cuda_stream);
}

// The status word of the built-in scratch (its first four bytes, like any workspace): the only way a caller of
// ssd_forward_noalloc can learn that a bounded wait ran out, because the array is private to the library.
extern "C" int32_t ssd_noalloc_status(void* cuda_stream, int32_t* code_out) {
  ssd::clear_error();
  void* scratch = nullptr;
  const int rc = scratch_address("ssd_noalloc_status", &scratch);
  if (rc) return rc;
  return ssd::read_status_sync(scratch, cuda_stream, code_out, "ssd_noalloc_status");
}

extern "C" size_t ssd_noalloc_max_bytes(void) { return kScratchBytes; }
