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

namespace {

// The whole budget of the no-allocation entry point.  Lives in every context that loads the
// library, from load to exit, whether or not the entry point is ever called.
constexpr size_t kScratchBytes = SSD_NOALLOC_MAX_BYTES;
static __device__ __align__(256) unsigned char g_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
void* g_ptr[kMaxDevices] = {nullptr};   // device address of g_scratch, per device ordinal

}  // namespace

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
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    ssd::set_error("ssd_forward_noalloc: no usable current CUDA device (ordinal %d)", dev);
    return SSD_ERR_CUDA;
  }
  void* scratch = nullptr;
  {
    // Once per device, with that device current: in host code the array's name is only a
    // stand-in for the symbol, so ask the runtime where the array lives on this device.
    std::lock_guard<std::mutex> lock(g_mu);
    if (!g_ptr[dev]) {
      void* q = nullptr;
      const cudaError_t e = cudaGetSymbolAddress(&q, g_scratch);
      if (e != cudaSuccess || !q) {
        ssd::set_error("ssd_forward_noalloc: cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(e));
        return SSD_ERR_CUDA;
      }
      g_ptr[dev] = q;
    }
    scratch = g_ptr[dev];
  }
  return ssd_forward(dims, p, scratch, kScratchBytes, cuda_stream);
}

extern "C" size_t ssd_noalloc_max_bytes(void) { return kScratchBytes; }
