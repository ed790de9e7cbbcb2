// Streamed-rollout kernels: the single-timestep state update (in place on the caller's fp32
// state), per-stream state reset, and the small sequence-parallel prefix kernels.
//
// state_update is a pure HBM stream: every state element is read once and written once per
// step (2*H*P*N*4 bytes per stream) and the per-step vectors are tiny beside it.  Each thread
// moves 128-bit pieces of a state row; a row's dot product with C is finished with shuffles
// inside the lanes that share the row.
#include "common.cuh"
#include "ssd_internal.h"

namespace ssd {
namespace {

constexpr int DEC_THREADS = 128;

template <typename T> struct Vec4Load;
template <> struct Vec4Load<float> {
  static __device__ __forceinline__ float4 ld(const float* p) { return __ldg(reinterpret_cast<const float4*>(p)); }
};
template <> struct Vec4Load<__nv_bfloat16> {
  static __device__ __forceinline__ float4 ld(const __nv_bfloat16* p) {
    const uint2 r = __ldg(reinterpret_cast<const uint2*>(p));
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&r.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&r.y);
    const float2 fa = __bfloat1622float2(a), fb = __bfloat1622float2(b);
    return make_float4(fa.x, fa.y, fb.x, fb.y);
  }
};

__device__ __forceinline__ float ldf_shared(const float* p) { return *p; }
__device__ __forceinline__ float ldf_shared(const __nv_bfloat16* p) { return __bfloat162float(*p); }

// One block per (stream, head).  N is a power of two in [16, 256].
//   LPR = lanes that share a state row, V = float4 pieces per lane per row, RPW = rows per warp.
template <typename T, int N>
__global__ void __launch_bounds__(DEC_THREADS, 8) k_state_update(SsdStepDims d, SsdStepPtrs p) {
  constexpr int LPR = (N / 4 < 32) ? N / 4 : 32;
  constexpr int V = N / (4 * LPR);
  constexpr int RPW = 32 / LPR;
  constexpr int RPB = RPW * (DEC_THREADS / 32);  // rows per block pass
  constexpr int UNROLL = 4;
  const int sh = blockIdx.x;
  const int s = sh / d.nheads, h = sh - s * d.nheads;
  const int grp = h / (d.nheads / d.ngroups);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int lir = lane % LPR, riw = lane / LPR;
  const int P = d.headdim;

  // The state rows of the first pass are requested before anything else: the step's small vectors (dt, A, B, C, x) sit
  // behind a dependent exp, and a warp that waited for them first would request its state a memory round trip later.
  float* st = p.state + (size_t)sh * P * N;
  float4 sv[UNROLL][V];
  auto load_state = [&](int p0) {
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int pr = p0 + riw + u * RPB;
      if (pr < P) {
#pragma unroll
        for (int v = 0; v < V; ++v)
          sv[u][v] = *reinterpret_cast<const float4*>(st + (size_t)pr * N + 4 * (lir + v * LPR));
      }
    }
  };
  load_state(warp * RPW);

  const T* xs = (const T*)p.x + s * d.x_stride_s + (long long)h * P;
  const float dtv = dt_activation(ldf((const T*)p.dt + s * d.dt_stride_s + h), p.dt_bias ? __ldg(p.dt_bias + h) : 0.f, d.dt_softplus);
  const float a = expf(dtv * __ldg(p.A + h));
  const float Dh = p.D ? __ldg(p.D + h) : 0.f;
  const T* Bp = (const T*)p.Bm + s * d.b_stride_s + (long long)grp * N;
  const T* Cp = (const T*)p.Cm + s * d.c_stride_s + (long long)grp * N;
  float4 Bv[V], Cv[V];
#pragma unroll
  for (int v = 0; v < V; ++v) {
    const int n = 4 * (lir + v * LPR);
    Bv[v] = Vec4Load<T>::ld(Bp + n);
    Cv[v] = Vec4Load<T>::ld(Cp + n);
  }
  const T* zs = p.z ? (const T*)p.z + s * d.z_stride_s + (long long)h * P : nullptr;
  T* ys = (T*)p.y + s * d.y_stride_s + (long long)h * P;

  for (int p0 = warp * RPW; p0 < P; p0 += RPB * UNROLL) {  // warp-uniform trip count
    const int pbase = p0 + riw;
    if (p0 != warp * RPW) load_state(p0);
    float xv[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int pr = pbase + u * RPB;
      if (pr < P) xv[u] = ldf(xs + pr);
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int pr = pbase + u * RPB;
      float acc = 0.f;
      if (pr < P) {
        const float dx = dtv * xv[u];
#pragma unroll
        for (int v = 0; v < V; ++v) {
          float4 t = sv[u][v];
          t.x = fmaf(a, t.x, dx * Bv[v].x);
          t.y = fmaf(a, t.y, dx * Bv[v].y);
          t.z = fmaf(a, t.z, dx * Bv[v].z);
          t.w = fmaf(a, t.w, dx * Bv[v].w);
          *reinterpret_cast<float4*>(st + (size_t)pr * N + 4 * (lir + v * LPR)) = t;
          acc = fmaf(t.x, Cv[v].x, acc);
          acc = fmaf(t.y, Cv[v].y, acc);
          acc = fmaf(t.z, Cv[v].z, acc);
          acc = fmaf(t.w, Cv[v].w, acc);
        }
      }
#pragma unroll
      for (int o = LPR / 2; o; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (pr < P && lir == 0) {
        float yv = acc + Dh * xv[u];
        if (zs) {
          const float zv = ldf(zs + pr);
          yv *= zv * sigmoidf_(zv);
        }
        stf(ys + pr, yv);
      }
    }
  }
}

// The same update with the state staged through shared memory: a persistent block walks (stream, head) items and keeps
// the next DEC_STAGES - 1 items' state (and their x, B, C vectors) on the way with 16-byte cp.async copies, so the bytes in
// flight per SM are set by the ring (8 blocks x 2 items x 8 KB at headdim 32, dstate 64), not by the registers a thread can
// hold.  Measured at 8192 streams x 8 heads: 2 stages (12 blocks per SM) 0.213 ms, 3 stages (8 blocks) 0.175 ms, 4 stages
// (6 blocks) 0.193 ms, 6 stages (4 blocks) 0.223 ms; the register kernel 0.205 ms.  The step size of the next item is fetched one item ahead.  Layout of a ring slot: the item's state as it lies in
// global memory, then x, B, C.  R = state rows per thread (headdim = R * rows per block pass).
constexpr int DEC_STAGES = 3;

template <typename T, int N, int R>
__global__ void __launch_bounds__(DEC_THREADS) k_state_update_ring(SsdStepDims d, SsdStepPtrs p, long long items) {
  constexpr int LPR = (N / 4 < 32) ? N / 4 : 32;
  constexpr int V = N / (4 * LPR);
  constexpr int RPW = 32 / LPR;
  constexpr int RPB = RPW * (DEC_THREADS / 32);
  constexpr int P = R * RPB;
  constexpr int ES = (int)sizeof(T);
  constexpr int ST_B = P * N * 4, X_B = P * ES, BC_B = N * ES;
  constexpr int STAGE = ST_B + X_B + 2 * BC_B;
  constexpr int NXP = X_B / 16, NBP = BC_B / 16;   // 16-byte pieces of x and of B (C); the host checked the divisibility
  extern __shared__ __align__(16) unsigned char dec_ring[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int lir = lane % LPR, riw = lane / LPR;
  const int H = d.nheads, hpg = d.nheads / d.ngroups;
  const int row0 = warp * RPW + riw;

  auto issue = [&](long long it, int stage) {
    if (it < items) {
      const long long s = it / H;
      const int h = (int)(it - s * H);
      unsigned char* sm = dec_ring + stage * STAGE;
      const float* gst = p.state + it * (long long)(P * N);
#pragma unroll
      for (int u = 0; u < R; ++u)
#pragma unroll
        for (int v = 0; v < V; ++v) {
          const int off = (row0 + u * RPB) * N + 4 * (lir + v * LPR);
          cp_async16(sm + off * 4, gst + off, true);
        }
      const int t = threadIdx.x;
      if (t < NXP) cp_async16(sm + ST_B + t * 16, (const char*)((const T*)p.x + s * d.x_stride_s + (long long)h * P) + t * 16, true);
      else if (t < NXP + NBP)
        cp_async16(sm + ST_B + X_B + (t - NXP) * 16, (const char*)((const T*)p.Bm + s * d.b_stride_s + (long long)(h / hpg) * N) + (t - NXP) * 16, true);
      else if (t < NXP + 2 * NBP)
        cp_async16(sm + ST_B + X_B + BC_B + (t - NXP - NBP) * 16,
                   (const char*)((const T*)p.Cm + s * d.c_stride_s + (long long)(h / hpg) * N) + (t - NXP - NBP) * 16, true);
    }
    cp_async_commit();   // a group per slot even when it is empty: the wait counts groups
  };
  auto load_dt = [&](long long it) -> float {
    if (it >= items) return 0.f;
    const long long s = it / H;
    return ldf((const T*)p.dt + s * d.dt_stride_s + (it - s * H));
  };

  const long long first = blockIdx.x, stride = gridDim.x;
#pragma unroll
  for (int k = 0; k < DEC_STAGES - 1; ++k) issue(first + k * stride, k);
  float dt_next = load_dt(first);
  int stage = 0;
  for (long long it = first; it < items; it += stride) {
    cp_async_wait<DEC_STAGES - 2>();
    __syncthreads();     // every thread's pieces of this item have landed; every thread is done with the previous slot
    issue(it + (DEC_STAGES - 1) * stride, stage == 0 ? DEC_STAGES - 1 : stage - 1);
    const float dt_raw = dt_next;
    dt_next = load_dt(it + stride);
    const long long s = it / H;
    const int h = (int)(it - s * H);
    const unsigned char* sm = dec_ring + stage * STAGE;
    stage = stage + 1 == DEC_STAGES ? 0 : stage + 1;
    const float dtv = dt_activation(dt_raw, p.dt_bias ? __ldg(p.dt_bias + h) : 0.f, d.dt_softplus);
    const float a = expf(dtv * __ldg(p.A + h));
    const float Dh = p.D ? __ldg(p.D + h) : 0.f;
    const T* sx = reinterpret_cast<const T*>(sm + ST_B);
    const T* sB = reinterpret_cast<const T*>(sm + ST_B + X_B);
    const T* sC = reinterpret_cast<const T*>(sm + ST_B + X_B + BC_B);
    float Bv[V][4], Cv[V][4];
#pragma unroll
    for (int v = 0; v < V; ++v)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        Bv[v][j] = ldf_shared(sB + 4 * (lir + v * LPR) + j);
        Cv[v][j] = ldf_shared(sC + 4 * (lir + v * LPR) + j);
      }
    float* gst = p.state + it * (long long)(P * N);
    const T* zs = p.z ? (const T*)p.z + s * d.z_stride_s + (long long)h * P : nullptr;
    T* ys = (T*)p.y + s * d.y_stride_s + (long long)h * P;
#pragma unroll
    for (int u = 0; u < R; ++u) {
      const int pr = row0 + u * RPB;
      const float xv = ldf_shared(sx + pr), dx = dtv * xv;
      float acc = 0.f;
#pragma unroll
      for (int v = 0; v < V; ++v) {
        const int off = pr * N + 4 * (lir + v * LPR);
        float4 t = *reinterpret_cast<const float4*>(sm + off * 4);
        t.x = fmaf(a, t.x, dx * Bv[v][0]);
        t.y = fmaf(a, t.y, dx * Bv[v][1]);
        t.z = fmaf(a, t.z, dx * Bv[v][2]);
        t.w = fmaf(a, t.w, dx * Bv[v][3]);
        *reinterpret_cast<float4*>(gst + off) = t;
        acc = fmaf(t.x, Cv[v][0], acc);
        acc = fmaf(t.y, Cv[v][1], acc);
        acc = fmaf(t.z, Cv[v][2], acc);
        acc = fmaf(t.w, Cv[v][3], acc);
      }
#pragma unroll
      for (int o = LPR / 2; o; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (lir == 0) {
        float yv = acc + Dh * xv;
        if (zs) {
          const float zv = ldf(zs + pr);
          yv *= zv * sigmoidf_(zv);
        }
        stf(ys + pr, yv);
      }
    }
  }
  cp_async_wait<0>();
}

// Any other dstate: one warp per state row, lanes stride over n.
template <typename T>
__global__ void __launch_bounds__(DEC_THREADS) k_state_update_generic(SsdStepDims d, SsdStepPtrs p) {
  const int sh = blockIdx.x;
  const int s = sh / d.nheads, h = sh - s * d.nheads;
  const int grp = h / (d.nheads / d.ngroups);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int P = d.headdim, N = d.dstate;
  const T* xs = (const T*)p.x + s * d.x_stride_s + (long long)h * P;
  const float dtv = dt_activation(ldf((const T*)p.dt + s * d.dt_stride_s + h), p.dt_bias ? __ldg(p.dt_bias + h) : 0.f, d.dt_softplus);
  const float a = expf(dtv * __ldg(p.A + h));
  const float Dh = p.D ? __ldg(p.D + h) : 0.f;
  const T* Bp = (const T*)p.Bm + s * d.b_stride_s + (long long)grp * N;
  const T* Cp = (const T*)p.Cm + s * d.c_stride_s + (long long)grp * N;
  float* st = p.state + (size_t)sh * P * N;
  for (int pr = warp; pr < P; pr += DEC_THREADS / 32) {
    const float xv = ldf(xs + pr), dx = dtv * xv;
    float acc = 0.f;
    for (int n = lane; n < N; n += 32) {
      float t = fmaf(a, st[(size_t)pr * N + n], dx * ldf(Bp + n));
      st[(size_t)pr * N + n] = t;
      acc = fmaf(t, ldf(Cp + n), acc);
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) {
      float yv = acc + Dh * xv;
      if (p.z) {
        const float zv = ldf((const T*)p.z + s * d.z_stride_s + (long long)h * P + pr);
        yv *= zv * sigmoidf_(zv);
      }
      stf((T*)p.y + s * d.y_stride_s + (long long)h * P + pr, yv);
    }
  }
}

__global__ void k_reset_rows(float* state, long long row_elems, const long long* idx, long long count,
                             long long streams) {
  const long long r = blockIdx.y;
  if (r >= count) return;
  const long long s = idx[r];
  if (s < 0 || s >= streams) return;
  float4* row = reinterpret_cast<float4*>(state + s * row_elems);
  const long long n4 = row_elems / 4;
  for (long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x; e < n4; e += (long long)gridDim.x * blockDim.x)
    row[e] = make_float4(0.f, 0.f, 0.f, 0.f);
  if (blockIdx.x == 0)
    for (long long e = n4 * 4 + threadIdx.x; e < row_elems; e += blockDim.x) state[s * row_elems + e] = 0.f;
}

__global__ void k_total_logdecay(Geo g, const float* __restrict__ cs, float* __restrict__ out) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;  // b*H + h
  if (i >= g.B * g.H) return;
  float v = 0.f;
  for (int c = 0; c < g.nc; ++c) v += cs[((size_t)i * g.nc + c) * g.Q + g.Q - 1];
  out[i] = v;
}

// Exclusive prefix over ranks by Horner's rule:
//   direction +1: acc = init; for q = 0..rank-1:        acc = exp(ld_q)*acc + st_q
//   direction -1: acc = init; for q = world-1..rank+1:  acc = exp(ld_q)*acc + st_q
__global__ void k_sp_prefix(const float* __restrict__ gs, const float* __restrict__ gl, int world, int rank,
                            int direction, long long bh, long long elems, const float* __restrict__ init,
                            float* __restrict__ out) {
  const long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const long long r = blockIdx.y;  // b*H + h
  if (e >= elems) return;
  float acc = init ? init[r * elems + e] : 0.f;
  if (direction > 0) {
    for (int q = 0; q < rank; ++q) acc = expf(gl[q * bh + r]) * acc + gs[((size_t)q * bh + r) * elems + e];
  } else {
    for (int q = world - 1; q > rank; --q) acc = expf(gl[q * bh + r]) * acc + gs[((size_t)q * bh + r) * elems + e];
  }
  out[r * elems + e] = acc;
}

}  // namespace

// The ring kernel covers the shapes whose item (headdim x dstate fp32) is 8 KB at 4 or 8 rows per thread, with x / B / C
// rows that are whole, 16-byte aligned pieces; everything else takes the register kernels.
template <typename T, int N, int R>
static bool launch_ring(const SsdStepDims& d, const SsdStepPtrs& p, cudaStream_t s) {
  constexpr int LPR = (N / 4 < 32) ? N / 4 : 32, RPB = (32 / LPR) * (DEC_THREADS / 32), P = R * RPB, ES = (int)sizeof(T);
  constexpr int STAGE = P * N * 4 + P * ES + 2 * N * ES;
  if (d.headdim != P || (P * ES) % 16 || (N * ES) % 16) return false;
  auto al = [&](const void* q, long long stride) { return ((uintptr_t)q % 16) == 0 && (stride * ES) % 16 == 0; };
  if (!al(p.x, d.x_stride_s) || !al(p.Bm, d.b_stride_s) || !al(p.Cm, d.c_stride_s) || ((uintptr_t)p.state % 16)) return false;
  const long long items = (long long)d.streams * d.nheads;
  constexpr int smem = DEC_STAGES * STAGE;
  auto k = k_state_update_ring<T, N, R>;
  cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);   // per device, so at every launch
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int per_sm = (227 * 1024) / (smem + 1024) < 16 ? (227 * 1024) / (smem + 1024) : 16;
  long long grid = (long long)sms * (per_sm > 0 ? per_sm : 1);
  if (grid > items) grid = items;
  k<<<(unsigned)grid, DEC_THREADS, smem, s>>>(d, p, items);
  return true;
}

template <typename T>
static int decode_t(const SsdStepDims& d, const SsdStepPtrs& p, cudaStream_t s) {
  const unsigned blocks = (unsigned)((long long)d.streams * d.nheads);
  if (d.dstate == 64 && d.headdim == 32 && launch_ring<T, 64, 4>(d, p, s)) {
    SSD_CUDA_CHECK_LAUNCH("state_update");
    return SSD_OK;
  }
  switch (d.dstate) {
    case 16: k_state_update<T, 16><<<blocks, DEC_THREADS, 0, s>>>(d, p); break;
    case 32: k_state_update<T, 32><<<blocks, DEC_THREADS, 0, s>>>(d, p); break;
    case 64: k_state_update<T, 64><<<blocks, DEC_THREADS, 0, s>>>(d, p); break;
    case 128: k_state_update<T, 128><<<blocks, DEC_THREADS, 0, s>>>(d, p); break;
    case 256: k_state_update<T, 256><<<blocks, DEC_THREADS, 0, s>>>(d, p); break;
    default: k_state_update_generic<T><<<blocks, DEC_THREADS, 0, s>>>(d, p); break;
  }
  SSD_CUDA_CHECK_LAUNCH("state_update");
  return SSD_OK;
}

int decode_step(const SsdStepDims& d, const SsdStepPtrs& p, cudaStream_t s) {
  return d.dtype == SSD_BF16 ? decode_t<__nv_bfloat16>(d, p, s) : decode_t<float>(d, p, s);
}

int reset_rows(float* state, long long row_elems, const long long* idx, long long count, long long streams,
               cudaStream_t s) {
  if (count == 0) return SSD_OK;
  const long long n4 = row_elems / 4;
  const unsigned gx = (unsigned)((n4 + 255) / 256 > 0 ? ((n4 + 255) / 256 < 64 ? (n4 + 255) / 256 : 64) : 1);
  for (long long off = 0; off < count; off += 65535) {
    const long long c = (count - off < 65535) ? count - off : 65535;
    k_reset_rows<<<dim3(gx, (unsigned)c), 256, 0, s>>>(state, row_elems, idx + off, c, streams);
  }
  SSD_CUDA_CHECK_LAUNCH("state_reset_rows");
  return SSD_OK;
}

int sp_total_logdecay(const Geo& g, const float* cs, float* out, cudaStream_t s) {
  k_total_logdecay<<<cdiv(g.B * g.H, 128), 128, 0, s>>>(g, cs, out);
  SSD_CUDA_CHECK_LAUNCH("sp_total_logdecay");
  return SSD_OK;
}

int sp_prefix_state(const float* gs, const float* gl, int world, int rank, int direction, long long bh,
                    long long elems, const float* init, float* out, cudaStream_t s) {
  k_sp_prefix<<<dim3((unsigned)((elems + 255) / 256), (unsigned)bh), 256, 0, s>>>(gs, gl, world, rank, direction, bh,
                                                                                 elems, init, out);
  SSD_CUDA_CHECK_LAUNCH("sp_prefix_state");
  return SSD_OK;
}

}  // namespace ssd
