// Shared device/host helpers for the SSD kernels (sm_100a only).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/ssd_b200.h"

// floats per (batch, chunk, head) decay table written by the cumsum kernel for the tensor-core
// family: [cs*log2e | dt | column factors | per-step decays], 128 each
#define SSD_TAB_FLOATS 512

namespace ssd {

// Internal, fully-resolved geometry handed to every kernel by value.
struct Geo {
  int B, L, H, P, N, G, Q, nc, hpg;  // hpg = heads per group
  long long xsb, xsl, dtsb, dtsl, bsb, bsl, csb, csl, zsb, zsl, ysb, ysl;
  int dt_softplus;                     // step size = softplus(dt + dt_bias) instead of dt + dt_bias
  int onetile;                         // tensor family: the one-tile-per-CTA kernels for every shape (SSD_ALGO_TENSOR_ONETILE)
};

// The step-size pre-activation of a Mamba-2 layer, fused where dt is first read.  Above 20 softplus is the
// identity in fp32 (same cut-off as torch.nn.functional.softplus).
__device__ __forceinline__ float dt_activation(float raw, float bias, int softplus) {
  const float v = raw + bias;
  return (softplus && v <= 20.f) ? log1pf(expf(v)) : v;
}

// |sum of dt*A over a chunk| up to which exp(+-sum) stays well inside the range of bf16 / fp32 with room for the data:
// heads within it may carry their decay on the operands of the dB/dC product.  The cumsum kernel marks the heads beyond it
// without any zeroing pass: every launch has a tag of its own, writes it to word [H] of the `hmax` segment and to word [h]
// for every head h whose chunk total exceeds the range; a head is "within range" iff word [h] differs from word [H].  A
// stale or accidental match can only mark a head that did not need it (it then takes the general path): never the reverse.
constexpr float SSD_SEP_LOG_RANGE = 64.f;

// Workspace segments (offsets in bytes from the workspace base; 0-size segments unused).
struct WsLayout {
  size_t status;                                     // 256-byte status block (int32 code first)
  size_t cs, dtf, states, fin, cb;                   // forward
  size_t tab, prev_bf, hmax;                         // forward, tensor-core family only (else empty)
  size_t ds_bf;                                      // backward, tensor-core family only
  size_t dstates, wsum, dyp, dcsp, ddtd, ddot, sdot, dapart, ddpart, dini;  // backward extras (wsum: CUDA-core family only)
  size_t total_fwd, total_bwd;
};

// 16-byte asynchronous copies global -> shared, tracked per thread in groups (commit, then wait until at most N groups
// are outstanding).  With `valid` false nothing is read and the 16 bytes are written as zeros.
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc, bool valid) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(gsrc), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return __ldg(p); }
template <> __device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p) {
  return __bfloat162float(*p);
}
template <typename T> __device__ __forceinline__ void stf(T* p, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16* p, float v) {
  *p = __float2bfloat16_rn(v);
}

__device__ __forceinline__ float sigmoidf_(float z) { return 1.f / (1.f + __expf(-z)); }

// Thread-local error string shared by every translation unit of the library.
void set_error(const char* fmt, ...);
void clear_error();

// Bookkeeping after every kernel launch: counts it and, while a profile is open on this thread,
// records an event behind it on the launch stream.
void after_launch(const char* what, cudaStream_t s);

// Uses the cudaStream_t named `s` in the enclosing scope.
#define SSD_CUDA_CHECK_LAUNCH(what)                                              \
  do {                                                                           \
    cudaError_t e__ = cudaGetLastError();                                        \
    if (e__ != cudaSuccess) {                                                    \
      ::ssd::set_error("%s: launch failed: %s", what, cudaGetErrorString(e__));  \
      return SSD_ERR_CUDA;                                                       \
    }                                                                            \
    ::ssd::after_launch(what, s);                                                \
  } while (0)

static inline int cdiv(int a, int b) { return (a + b - 1) / b; }

}  // namespace ssd
