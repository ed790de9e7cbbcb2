// The two bandwidth-bound operators either side of the scan in a Mamba-2 layer:
//   before:  out = act(causal depthwise conv1d(in) + bias) over the (x | B | C) channels, act = silu or identity
//   after :  out = in * rsqrt(mean(in^2) + eps) * weight   (RMS norm of the gated scan output, weight optional)
// each with its backward.  Every tensor is read once and written once (the conv backward re-reads a
// (width-1)-row halo per 32-token tile); arithmetic is fp32, storage bf16 or fp32, 16-byte accesses.
// Reductions over tokens (dweight, dbias) are two-stage with a fixed summation order.
//
// The step-size activation softplus(dt + dt_bias) and the gate y*silu(z) need no kernel here: they are
// evaluated inside the scan's own kernels.
#include "common.cuh"
#include "ssd_internal.h"

namespace ssd {
namespace {

template <typename T> __device__ __forceinline__ void load8(const T* p, float (&v)[8]);
template <> __device__ __forceinline__ void load8<float>(const float* p, float (&v)[8]) {
  const float4 a = __ldg(reinterpret_cast<const float4*>(p)), b = __ldg(reinterpret_cast<const float4*>(p) + 1);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <> __device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 r = __ldg(reinterpret_cast<const uint4*>(p));
  const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
    v[2 * i] = f.x; v[2 * i + 1] = f.y;
  }
}
template <typename T> __device__ __forceinline__ void store8(T* p, const float (&v)[8]);
template <> __device__ __forceinline__ void store8<float>(float* p, const float (&v)[8]) {
  reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
  reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
}
template <> __device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    w[i] = *reinterpret_cast<const uint32_t*>(&h);
  }
  *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
}

// NC storage elements as loaded (kept raw so that several rows can be in flight in few registers)
template <typename T, int NC> struct RawN;
template <> struct RawN<__nv_bfloat16, 8> { uint4 v; };
template <> struct RawN<__nv_bfloat16, 4> { uint2 v; };
template <> struct RawN<float, 8> { float4 a, b; };
template <> struct RawN<float, 4> { float4 a; };
__device__ __forceinline__ void load_raw(const __nv_bfloat16* p, RawN<__nv_bfloat16, 8>& r) { r.v = __ldg(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ void load_raw(const __nv_bfloat16* p, RawN<__nv_bfloat16, 4>& r) { r.v = __ldg(reinterpret_cast<const uint2*>(p)); }
__device__ __forceinline__ void load_raw(const float* p, RawN<float, 8>& r) {
  r.a = __ldg(reinterpret_cast<const float4*>(p)); r.b = __ldg(reinterpret_cast<const float4*>(p) + 1);
}
__device__ __forceinline__ void load_raw(const float* p, RawN<float, 4>& r) { r.a = __ldg(reinterpret_cast<const float4*>(p)); }
template <> struct RawN<float, 2> { float2 a; };
__device__ __forceinline__ void store_n(float* p, const float (&v)[2]) { *reinterpret_cast<float2*>(p) = make_float2(v[0], v[1]); }
__device__ __forceinline__ float2 bf2_(uint32_t w) { return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w)); }
__device__ __forceinline__ void unpack_raw(const RawN<__nv_bfloat16, 8>& r, float (&v)[8]) {
  const float2 a = bf2_(r.v.x), b = bf2_(r.v.y), c = bf2_(r.v.z), d = bf2_(r.v.w);
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
}
__device__ __forceinline__ void unpack_raw(const RawN<__nv_bfloat16, 4>& r, float (&v)[4]) {
  const float2 a = bf2_(r.v.x), b = bf2_(r.v.y);
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}
__device__ __forceinline__ void unpack_raw(const RawN<float, 8>& r, float (&v)[8]) {
  v[0] = r.a.x; v[1] = r.a.y; v[2] = r.a.z; v[3] = r.a.w; v[4] = r.b.x; v[5] = r.b.y; v[6] = r.b.z; v[7] = r.b.w;
}
__device__ __forceinline__ void unpack_raw(const RawN<float, 4>& r, float (&v)[4]) { v[0] = r.a.x; v[1] = r.a.y; v[2] = r.a.z; v[3] = r.a.w; }
__device__ __forceinline__ uint32_t bfpack_(float lo, float hi) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ void store_n(__nv_bfloat16* p, const float (&v)[8]) {
  *reinterpret_cast<uint4*>(p) = make_uint4(bfpack_(v[0], v[1]), bfpack_(v[2], v[3]), bfpack_(v[4], v[5]), bfpack_(v[6], v[7]));
}
__device__ __forceinline__ void store_n(__nv_bfloat16* p, const float (&v)[4]) {
  *reinterpret_cast<uint2*>(p) = make_uint2(bfpack_(v[0], v[1]), bfpack_(v[2], v[3]));
}
__device__ __forceinline__ void store_n(float* p, const float (&v)[8]) {
  reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
  reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void store_n(float* p, const float (&v)[4]) { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }

// sigmoid for the silu: one tanh.approx (relative error 2^-11, below bf16 resolution) for bf16 storage, exp + fast
// division for fp32 storage
template <typename T> __device__ __forceinline__ float sig_(float a);
template <> __device__ __forceinline__ float sig_<__nv_bfloat16>(float a) {
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * a));
  return fmaf(0.5f, t, 0.5f);
}
template <> __device__ __forceinline__ float sig_<float>(float a) { return __fdividef(1.f, 1.f + __expf(-a)); }

// Packed pairs of fp32 (one 64-bit register): sm_100 executes fma / add on both halves in one instruction, with the same
// rounding as the scalar forms.
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pack2(float lo, float hi) {
  f32x2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(f32x2 v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
  f32x2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) {
  f32x2 d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
// NC storage elements -> NC/2 packed pairs
__device__ __forceinline__ void unpack_pairs(const RawN<__nv_bfloat16, 8>& r, f32x2 (&v)[4]) {
  const uint32_t w[4] = {r.v.x, r.v.y, r.v.z, r.v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) v[i] = pack2(__uint_as_float(w[i] << 16), __uint_as_float(w[i] & 0xffff0000u));
}
__device__ __forceinline__ void unpack_pairs(const RawN<__nv_bfloat16, 4>& r, f32x2 (&v)[2]) {
  v[0] = pack2(__uint_as_float(r.v.x << 16), __uint_as_float(r.v.x & 0xffff0000u));
  v[1] = pack2(__uint_as_float(r.v.y << 16), __uint_as_float(r.v.y & 0xffff0000u));
}
__device__ __forceinline__ void unpack_pairs(const RawN<float, 4>& r, f32x2 (&v)[2]) { v[0] = pack2(r.a.x, r.a.y); v[1] = pack2(r.a.z, r.a.w); }
__device__ __forceinline__ void unpack_pairs(const RawN<float, 2>& r, f32x2 (&v)[1]) { v[0] = pack2(r.a.x, r.a.y); }

constexpr int CONV_THREADS = 128;
constexpr int CONV_TL = 32;         // tokens per tile
constexpr int CONV_ROWS = 2048;     // backward: thread rows (each walks several tiles and leaves one partial sum)

// ---------------------------------------------------------------------------------------------
// conv forward.  Work item = (batch, tile of 32 tokens, vector of NC channels), channel vectors fastest so that a
// warp reads contiguous pieces of a token row; the item's thread walks the tile keeping the last K-1 input rows
// in registers, eight rows requested at a time.
template <typename T, int K, int NC>
__global__ void __launch_bounds__(CONV_THREADS) k_conv_fwd(SsdConvDims d, const T* __restrict__ in,
                                                           const float* __restrict__ weight, const float* __restrict__ bias,
                                                           T* __restrict__ out) {
  const int CV = d.channels / NC, ntile = (d.seqlen + CONV_TL - 1) / CONV_TL;
  const long long item = (long long)blockIdx.x * CONV_THREADS + threadIdx.x;
  if (item >= (long long)d.batch * ntile * CV) return;
  const int cv = (int)(item % CV);
  const long long bt = item / CV;
  const int b = (int)(bt / ntile), t0 = (int)(bt % ntile) * CONV_TL, t1 = min(t0 + CONV_TL, d.seqlen);
  const int c0 = cv * NC;
  float w[NC][K], bs[NC];
#pragma unroll
  for (int j = 0; j < NC; ++j) {
#pragma unroll
    for (int k = 0; k < K; ++k) w[j][k] = __ldg(weight + (size_t)(c0 + j) * K + k);
    bs[j] = bias ? __ldg(bias + c0 + j) : 0.f;
  }
  const T* ip = in + (long long)b * d.in_stride_b + c0;
  T* op = out + (long long)b * d.out_stride_b + c0;
  float win[K][NC];   // win[k] = input row t - (K-1) + k
#pragma unroll
  for (int k = 0; k < K - 1; ++k) {
    const int t = t0 - (K - 1) + k;
    if (t >= 0) { RawN<T, NC> r0; load_raw(ip + (long long)t * d.in_stride_l, r0); unpack_raw(r0, win[k]); }
    else {
#pragma unroll
      for (int j = 0; j < NC; ++j) win[k][j] = 0.f;
    }
  }
  constexpr int CH = 8;   // rows requested together: enough bytes in flight per thread to cover the memory latency
  for (int tc = t0; tc < t1; tc += CH) {
    RawN<T, NC> raw[CH];
#pragma unroll
    for (int i = 0; i < CH; ++i)
      if (tc + i < t1) load_raw(ip + (long long)(tc + i) * d.in_stride_l, raw[i]);
#pragma unroll
    for (int i = 0; i < CH; ++i) {
      if (tc + i < t1) {
        unpack_raw(raw[i], win[K - 1]);
        float o[NC];
#pragma unroll
        for (int j = 0; j < NC; ++j) {
          float a = bs[j];
#pragma unroll
          for (int k = 0; k < K; ++k) a = fmaf(w[j][k], win[k][j], a);
          o[j] = d.activation ? a * sig_<T>(a) : a;
        }
        store_n(op + (long long)(tc + i) * d.out_stride_l, o);
#pragma unroll
        for (int k = 0; k < K - 1; ++k)
#pragma unroll
          for (int j = 0; j < NC; ++j) win[k][j] = win[k + 1][j];
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// conv forward, shared-memory staged (the default where the channel count fills 16-byte vectors of a 256-byte
// channel block).  A persistent CTA walks tiles of 64 tokens x 256 bytes of channels; every thread requests
// 16-byte pieces of the tiles two and three ahead with cp.async (rows before the sequence start and channels past the
// end are zero-filled by the copy itself), so the bytes in flight per SM are set by the ring, not by registers.
// Thread = (16-byte channel vector, 4 consecutive tokens): K-1+4 row reads from shared memory, 4 row stores.
constexpr int CONVS_THREADS = 256;
constexpr int CONVS_TT = 64;        // tokens per tile
constexpr int CONVS_ROWB = 256;     // bytes of channels per tile row
constexpr int CONVS_STAGES = 3;
constexpr int CONVS_CTAS_PER_SM = 4;

template <typename T, int NC> __device__ __forceinline__ void lds_raw(const void* p, RawN<T, NC>& r) {
  r = *reinterpret_cast<const RawN<T, NC>*>(p);
}

// Walk of a CTA over (batch, token tile) pairs with a fixed stride, in 32-bit arithmetic without divisions in the loop.
struct PairWalk {
  int b, tt, db, dtt, ntt;
  __device__ __forceinline__ PairWalk(int first, int stride, int ntt_) : ntt(ntt_) {
    b = first / ntt_; tt = first - b * ntt_;
    db = stride / ntt_; dtt = stride - db * ntt_;
  }
  __device__ __forceinline__ void next() {
    b += db; tt += dtt;
    if (tt >= ntt) { tt -= ntt; ++b; }
  }
};

template <typename T, int K>
__global__ void __launch_bounds__(CONVS_THREADS, CONVS_CTAS_PER_SM)
k_conv_fwd_sm(SsdConvDims d, const T* __restrict__ in, const float* __restrict__ weight, const float* __restrict__ bias,
              T* __restrict__ out, int ntt) {
  constexpr int NC = 16 / (int)sizeof(T);            // channels per 16-byte copy piece
  constexpr int NP = 8 / (int)sizeof(T);             // channels per thread in the arithmetic (8 bytes: half the weights in
                                                     // registers of a 16-byte mapping, so a fourth block fits an SM)
  constexpr int CB = CONVS_ROWB / (int)sizeof(T);    // channels per tile
  constexpr int ROWS = CONVS_TT + K - 1;
  constexpr int STAGE_BYTES = ROWS * CONVS_ROWB;
  extern __shared__ __align__(128) unsigned char conv_smem[];
  const int tid = threadIdx.x, cv = tid & 15, seg = tid >> 4;      // copy role: 16-byte piece cv of rows seg, seg + 16, ...
  const int hv = tid & 31, rs = tid >> 5;                           // arithmetic role: 8-byte piece hv, tokens 8 rs .. 8 rs + 7
  // grid = (pair walkers, channel blocks): the CTAs of one x walk the same token rows side by side, one channel block
  // each, so whole rows (whole DRAM pages) are read and written at about the same time
  const int c0 = blockIdx.y * CB + cv * NC;
  const bool cok = c0 < d.channels;
  const T* ibase = in + (cok ? c0 : 0);
  const int npairs = d.batch * ntt;

  auto request = [&](const PairWalk& pw, int stage) {
    if (pw.b < d.batch) {
      const int t0 = pw.tt * CONVS_TT;
      const T* src = ibase + (long long)pw.b * d.in_stride_b + (long long)(t0 - (K - 1) + seg) * d.in_stride_l;
      unsigned char* sp = conv_smem + stage * STAGE_BYTES + cv * 16 + seg * CONVS_ROWB;
      int t = t0 - (K - 1) + seg;
#pragma unroll
      for (int j = 0; j < (ROWS + 15) / 16; ++j) {
        if (seg + 16 * j < ROWS) {
          const bool ok = cok && t >= 0 && t < d.seqlen;
          cp_async16(sp, ok ? (const void*)src : (const void*)in, ok);
        }
        sp += 16 * CONVS_ROWB; src += 16 * d.in_stride_l; t += 16;
      }
    }
    cp_async_commit();   // a group per tile slot even when it is empty: the wait below counts groups
  };

  PairWalk ahead((int)blockIdx.x, (int)gridDim.x, ntt), cur = ahead;
#pragma unroll
  for (int i = 0; i < CONVS_STAGES - 1; ++i) { request(ahead, i); ahead.next(); }
  const int c1 = blockIdx.y * CB + hv * NP;
  const bool live = c1 < d.channels;
  f32x2 w[NP / 2][K], bs[NP / 2];     // channel pairs (2j, 2j+1)
#pragma unroll
  for (int j = 0; j < NP / 2; ++j) {
#pragma unroll
    for (int k = 0; k < K; ++k)
      w[j][k] = live ? pack2(__ldg(weight + (size_t)(c1 + 2 * j) * K + k), __ldg(weight + (size_t)(c1 + 2 * j + 1) * K + k)) : 0ull;
    bs[j] = (live && bias) ? pack2(__ldg(bias + c1 + 2 * j), __ldg(bias + c1 + 2 * j + 1)) : 0ull;
  }
  int stage = 0;
  for (int pair = blockIdx.x; pair < npairs; pair += gridDim.x) {
    cp_async_wait<CONVS_STAGES - 2>();
    __syncthreads();           // this tile has landed for every thread; every thread is done with the previous one
    request(ahead, stage == 0 ? CONVS_STAGES - 1 : stage - 1);
    ahead.next();
    constexpr int TPT = CONVS_TT / (CONVS_THREADS / 32);   // tokens per thread
    const int t0 = cur.tt * CONVS_TT + rs * TPT;
    const unsigned char* sp = conv_smem + stage * STAGE_BYTES + hv * 8 + rs * TPT * CONVS_ROWB;
    T* op = out + (long long)cur.b * d.out_stride_b + (long long)t0 * d.out_stride_l + c1;
    cur.next();
    stage = stage + 1 == CONVS_STAGES ? 0 : stage + 1;
    if (!live) continue;
    f32x2 win[K][NP / 2];
#pragma unroll
    for (int k = 0; k < K - 1; ++k) { RawN<T, NP> r0; lds_raw<T, NP>(sp + k * CONVS_ROWB, r0); unpack_pairs(r0, win[k]); }
#pragma unroll
    for (int i = 0; i < TPT; ++i) {
      RawN<T, NP> r0;
      lds_raw<T, NP>(sp + (K - 1 + i) * CONVS_ROWB, r0);
      unpack_pairs(r0, win[K - 1]);
      float o[NP];
#pragma unroll
      for (int j = 0; j < NP / 2; ++j) {
        f32x2 a2 = bs[j];
#pragma unroll
        for (int k = 0; k < K; ++k) a2 = fma2(w[j][k], win[k][j], a2);
        float a, b;
        unpack2(a2, a, b);
        o[2 * j] = d.activation ? a * sig_<T>(a) : a;
        o[2 * j + 1] = d.activation ? b * sig_<T>(b) : b;
      }
      if (t0 + i < d.seqlen) store_n(op, o);
      op += d.out_stride_l;
#pragma unroll
      for (int k = 0; k < K - 1; ++k)
#pragma unroll
        for (int j = 0; j < NP / 2; ++j) win[k][j] = win[k + 1][j];
    }
  }
  cp_async_wait<0>();
}

// ---------------------------------------------------------------------------------------------
// conv backward.  Streaming forward in time over a tile: at step s the pre-activation of row s is recomputed from
// the input window, dpre[s] = dout[s] * act'(pre[s]) enters a second window, and
//   din[s-K+1] = sum_j w[K-1-j] * dpre[s-K+1+j]          (complete once dpre[s] is known)
//   dweight[k] += dpre[s] * in[s-K+1+k],  dbias += dpre[s]   (rows s of this tile only).
// dout arrives as up to three channel segments (the scan's dx, dB, dC tensors).  Thread = (row r, channel vector);
// row r walks the (batch, tile) pairs r, r+rows, ... and leaves one partial sum; k_conv_reduce adds the rows in order.
struct ConvSegs {
  const void* ptr[3];
  int c_begin[3];           // first channel of the segment; segment i covers [c_begin[i], c_begin[i+1])
  long long stride_b[3], stride_l[3];
  int n;
};

constexpr int CONV_TLB = 128;       // backward: tokens per tile (2 (K-1) halo rows per tile are recomputed: 5 % at K = 4)
constexpr int CONV_BWD_CH = 4;      // rows of the input and of the gradient requested together (two such register sets;
                                    // 8 rows per set spill at 168 registers and measured 40 % slower)
constexpr int CONV_BWD_MINB = 3;

template <typename T, int NC> __device__ __forceinline__ void zero_raw(RawN<T, NC>& r) {
  r = RawN<T, NC>{};
}

template <typename T, int K, int NC>
__global__ void __launch_bounds__(CONV_THREADS, CONV_BWD_MINB) k_conv_bwd(SsdConvDims d, int rows, const T* __restrict__ in,
                                                           const float* __restrict__ weight, const float* __restrict__ bias,
                                                           ConvSegs segs, T* __restrict__ din, long long din_stride_b,
                                                           long long din_stride_l, float* __restrict__ partial) {
  constexpr int CH = CONV_BWD_CH;
  const int CV = d.channels / NC;
  const long long item = (long long)blockIdx.x * CONV_THREADS + threadIdx.x;
  if (item >= (long long)rows * CV) return;
  const int cv = (int)(item % CV), row = (int)(item / CV);
  const int c0 = cv * NC;
  float w[NC][K], bs[NC], dw[NC][K], db[NC];
#pragma unroll
  for (int j = 0; j < NC; ++j) {
#pragma unroll
    for (int k = 0; k < K; ++k) { w[j][k] = __ldg(weight + (size_t)(c0 + j) * K + k); dw[j][k] = 0.f; }
    bs[j] = bias ? __ldg(bias + c0 + j) : 0.f;
    db[j] = 0.f;
  }
  int si = 0;
  for (int i = 1; i < segs.n; ++i) if (c0 >= segs.c_begin[i]) si = i;
  const T* dop = (const T*)segs.ptr[si] + (c0 - segs.c_begin[si]);
  const long long dosb = segs.stride_b[si], dosl = segs.stride_l[si];

  const int ntile = (d.seqlen + CONV_TLB - 1) / CONV_TLB;
  for (int pair = row; pair < d.batch * ntile; pair += rows) {
    const int b = pair / ntile, t0 = (pair - b * ntile) * CONV_TLB, t1 = min(t0 + CONV_TLB, d.seqlen);
    const T* ip = in + (long long)b * d.in_stride_b + c0;
    const T* gp = dop + (long long)b * dosb;
    T* dp = din + (long long)b * din_stride_b + c0;
    float win[K][NC], dpw[K][NC];   // win[k] = in[s-K+1+k], dpw[k] = dpre[s-K+1+k]
#pragma unroll
    for (int k = 0; k < K; ++k)
#pragma unroll
      for (int j = 0; j < NC; ++j) { win[k][j] = 0.f; dpw[k][j] = 0.f; }
    // rows s_begin .. s_end-1: K-1 rows of input before the tile, the tile, K-1 rows after it (their dpre completes the
    // tile's last din rows).  Rows outside the sequence or past s_end are zeros; a zero gradient row contributes nothing,
    // so the row loop needs no early exit and the compiler keeps both windows in renamed registers.
    const int s_begin = t0 - (K - 1), s_end = min(t1 + K - 1, d.seqlen + K - 1);
    auto load_chunk = [&](int sc, RawN<T, NC> (&rin)[CH], RawN<T, NC> (&rgo)[CH]) {
#pragma unroll
      for (int i = 0; i < CH; ++i) {
        const int s = sc + i;
        if (s >= 0 && s < d.seqlen && s < s_end) load_raw(ip + (long long)s * d.in_stride_l, rin[i]); else zero_raw(rin[i]);
        if (s >= t0 && s < d.seqlen && s < s_end) load_raw(gp + (long long)s * dosl, rgo[i]); else zero_raw(rgo[i]);
      }
    };
    auto compute_chunk = [&](int sc, const RawN<T, NC> (&rin)[CH], const RawN<T, NC> (&rgo)[CH]) {
#pragma unroll
      for (int i = 0; i < CH; ++i) {
        const int s = sc + i;
#pragma unroll
        for (int k = 0; k < K - 1; ++k)
#pragma unroll
          for (int j = 0; j < NC; ++j) { win[k][j] = win[k + 1][j]; dpw[k][j] = dpw[k + 1][j]; }
        unpack_raw(rin[i], win[K - 1]);
        float go[NC];
        unpack_raw(rgo[i], go);
        const bool own = s < t1;    // each row's weight / bias gradient is counted by exactly one tile (warp-uniform)
#pragma unroll
        for (int j = 0; j < NC; ++j) {
          float a = bs[j];
#pragma unroll
          for (int k = 0; k < K; ++k) a = fmaf(w[j][k], win[k][j], a);
          float g = go[j];
          if (d.activation) {
            const float sg = sig_<T>(a);
            g *= sg * (1.f + a * (1.f - sg));
          }
          dpw[K - 1][j] = g;
          if (own) {
            db[j] += g;
#pragma unroll
            for (int k = 0; k < K; ++k) dw[j][k] = fmaf(g, win[k][j], dw[j][k]);
          }
        }
        const int t = s - (K - 1);
        if (t >= t0 && t < t1) {
          float o[NC];
#pragma unroll
          for (int j = 0; j < NC; ++j) {
            float a = 0.f;
#pragma unroll
            for (int q = 0; q < K; ++q) a = fmaf(w[j][K - 1 - q], dpw[q][j], a);
            o[j] = a;
          }
          store_n(dp + (long long)t * din_stride_l, o);
        }
      }
    };
    // two register sets: the next chunk's rows are requested before the current chunk is worked on
    RawN<T, NC> rinA[CH], rgoA[CH], rinB[CH], rgoB[CH];
    load_chunk(s_begin, rinA, rgoA);
    for (int sc = s_begin; sc < s_end; sc += 2 * CH) {
      load_chunk(sc + CH, rinB, rgoB);
      compute_chunk(sc, rinA, rgoA);
      load_chunk(sc + 2 * CH, rinA, rgoA);
      if (sc + CH < s_end) compute_chunk(sc + CH, rinB, rgoB);
    }
  }
  float* pp = partial + ((size_t)row * d.channels + c0) * (K + 1);
#pragma unroll
  for (int j = 0; j < NC; ++j) {
#pragma unroll
    for (int k = 0; k < K; ++k) pp[j * (K + 1) + k] = dw[j][k];
    pp[j * (K + 1) + K] = db[j];
  }
}

// ---------------------------------------------------------------------------------------------
// conv backward, shared-memory staged.  Grid = (tile walkers, channel blocks of 256 bytes); a CTA walks (batch, 32-token
// tile) pairs of its channel block with the next tile's input rows and gradient rows arriving by cp.async while the
// current tile is worked on in two phases:
//   1. thread = (8 bytes of channels, 5 consecutive rows): recompute the pre-activation from a sliding input window,
//      dpre = dout * act'(pre) into a shared fp32 tile, and the weight / bias gradient of the rows this tile owns;
//   2. thread = (8 bytes of channels, 4 consecutive tokens): din from a sliding window over the dpre tile.
// The tile carries K-1 halo rows on either side (zero-filled outside the sequence), so no row is recomputed in
// registers and nothing is re-read from global memory but the halo.  A CTA leaves one partial weight-gradient row.
constexpr int CONVB_STAGES = 2;
constexpr int CONVB_CTAS_PER_SM = 3;
// 32-token tiles: 55 KB of shared memory and 80 registers per thread let three blocks (24 warps) share an SM, which an
// issue-bound kernel needs more than it needs long tiles (64-token tiles, two blocks of 126 registers: 0.424 ms; this:
// 0.357 ms; four blocks at 64 registers spill: 0.51 ms)
constexpr int CONVB_TT = 32;

template <typename T, int K>
__global__ void __launch_bounds__(CONVS_THREADS, CONVB_CTAS_PER_SM)
k_conv_bwd_sm(SsdConvDims d, const T* __restrict__ in, const float* __restrict__ weight, const float* __restrict__ bias,
              ConvSegs segs, T* __restrict__ din, long long din_stride_b, long long din_stride_l,
              float* __restrict__ partial, int ntt) {
  constexpr int NC = 16 / (int)sizeof(T);            // channels per 16-byte copy piece
  constexpr int NP = 8 / (int)sizeof(T);             // channels per thread in the arithmetic phases
  constexpr int CB = CONVS_ROWB / (int)sizeof(T);    // channels per tile
  constexpr int IN_ROWS = CONVB_TT + 2 * (K - 1), GO_ROWS = CONVB_TT + K - 1;
  constexpr int STAGE_BYTES = (IN_ROWS + GO_ROWS) * CONVS_ROWB;
  constexpr int DPRE_ROWB = CB * 4;
  constexpr int R1 = (GO_ROWS + 7) / 8;              // rows per thread in phase 1
  extern __shared__ __align__(128) unsigned char conv_smem[];
  unsigned char* dpre = conv_smem + CONVB_STAGES * STAGE_BYTES;
  const int tid = threadIdx.x, cv = tid & 15, seg = tid >> 4, hv = tid & 31, rs = tid >> 5;
  const int cb = blockIdx.y;

  // copy role: the 16-byte piece `cv` of rows seg, seg+16, ...
  const int cc = cb * CB + cv * NC;
  const bool cok = cc < d.channels;
  int si = 0;
  for (int i = 1; i < segs.n; ++i) if (cc >= segs.c_begin[i]) si = i;
  const T* gseg = (const T*)segs.ptr[si] + (cok ? cc - segs.c_begin[si] : 0);
  const long long gsb = segs.stride_b[si], gsl = segs.stride_l[si];
  const int npairs = d.batch * ntt;
  const T* ibase = in + (cok ? cc : 0);
  auto request = [&](const PairWalk& pw, int stage) {
    if (pw.b < d.batch) {
      const int t0 = pw.tt * CONVB_TT;
      unsigned char* sp = conv_smem + stage * STAGE_BYTES + cv * 16 + seg * CONVS_ROWB;
      {
        const T* src = ibase + (long long)pw.b * d.in_stride_b + (long long)(t0 - (K - 1) + seg) * d.in_stride_l;
        int t = t0 - (K - 1) + seg;
#pragma unroll
        for (int j = 0; j < (IN_ROWS + 15) / 16; ++j) {
          if (seg + 16 * j < IN_ROWS) {
            const bool ok = cok && t >= 0 && t < d.seqlen;
            cp_async16(sp + j * 16 * CONVS_ROWB, ok ? (const void*)src : (const void*)in, ok);
          }
          src += 16 * d.in_stride_l; t += 16;
        }
      }
      sp += IN_ROWS * CONVS_ROWB;
      {
        const T* src = gseg + (long long)pw.b * gsb + (long long)(t0 + seg) * gsl;
        int t = t0 + seg;
#pragma unroll
        for (int j = 0; j < (GO_ROWS + 15) / 16; ++j) {
          if (seg + 16 * j < GO_ROWS) {
            const bool ok = cok && t < d.seqlen;
            cp_async16(sp + j * 16 * CONVS_ROWB, ok ? (const void*)src : (const void*)in, ok);
          }
          src += 16 * gsl; t += 16;
        }
      }
    }
    cp_async_commit();
  };

  // arithmetic role: NP channels starting at c0, held as NP/2 packed pairs
  constexpr int NH = NP / 2;
  const int c0 = cb * CB + hv * NP;
  const bool live = c0 < d.channels;
  f32x2 w[NH][K], bs[NH], dw[NH][K], db[NH];
#pragma unroll
  for (int j = 0; j < NH; ++j) {
#pragma unroll
    for (int k = 0; k < K; ++k) {
      w[j][k] = live ? pack2(__ldg(weight + (size_t)(c0 + 2 * j) * K + k), __ldg(weight + (size_t)(c0 + 2 * j + 1) * K + k)) : 0ull;
      dw[j][k] = 0ull;
    }
    bs[j] = (live && bias) ? pack2(__ldg(bias + c0 + 2 * j), __ldg(bias + c0 + 2 * j + 1)) : 0ull;
    db[j] = 0ull;
  }

  PairWalk ahead((int)blockIdx.x, (int)gridDim.x, ntt), cur = ahead;
  request(ahead, 0);
  ahead.next();
  int stage = 0;
  for (int pair = blockIdx.x; pair < npairs; pair += gridDim.x) {
    cp_async_wait<0>();
    __syncthreads();     // the tile has landed; phase 2 of the previous tile is over (dpre and the other stage are free)
    request(ahead, stage ^ 1);
    ahead.next();
    const int b = cur.b, t0 = cur.tt * CONVB_TT;
    cur.next();
    const unsigned char* sin = conv_smem + stage * STAGE_BYTES + hv * 8;
    const unsigned char* sgo = sin + IN_ROWS * CONVS_ROWB;
    stage ^= 1;
    // ---- phase 1: rows r0 .. r0+R1-1 of the gradient tile (row r <-> token t0 + r; input rows r .. r+K-1) ----
    {
      const int r0 = rs * R1;
      f32x2 win[K][NH];
#pragma unroll
      for (int k = 0; k < K - 1; ++k) {
        RawN<T, NP> raw;
        if (r0 + k < IN_ROWS) lds_raw<T, NP>(sin + (r0 + k) * CONVS_ROWB, raw); else zero_raw(raw);
        unpack_pairs(raw, win[k]);
      }
#pragma unroll
      for (int i = 0; i < R1; ++i) {
        const int r = r0 + i;
        if (r < GO_ROWS) {
          RawN<T, NP> raw, rg;
          lds_raw<T, NP>(sin + (r + K - 1) * CONVS_ROWB, raw);
          unpack_pairs(raw, win[K - 1]);
          lds_raw<T, NP>(sgo + r * CONVS_ROWB, rg);
          f32x2 go[NH], dp[NH];
          unpack_pairs(rg, go);
          const bool own = r < CONVB_TT;    // each row's weight / bias gradient is counted by exactly one tile
#pragma unroll
          for (int j = 0; j < NH; ++j) {
            f32x2 a2 = bs[j];
#pragma unroll
            for (int k = 0; k < K; ++k) a2 = fma2(w[j][k], win[k][j], a2);
            f32x2 g = go[j];
            if (d.activation) {
              float a0, a1;
              unpack2(a2, a0, a1);
              const float s0 = sig_<T>(a0), s1 = sig_<T>(a1);
              // silu'(a) = s (1 + a (1 - s))
              g = fma2(g, pack2(fmaf(s0, fmaf(-a0, s0, a0), s0), fmaf(s1, fmaf(-a1, s1, a1), s1)), 0ull);
            }
            dp[j] = g;
            if (own) {
              db[j] = add2(db[j], g);
#pragma unroll
              for (int k = 0; k < K; ++k) dw[j][k] = fma2(g, win[k][j], dw[j][k]);
            }
          }
          f32x2* dst = reinterpret_cast<f32x2*>(dpre + r * DPRE_ROWB) + hv * NH;
          if constexpr (NH == 2) *reinterpret_cast<ulonglong2*>(dst) = make_ulonglong2(dp[0], dp[1]);
          else dst[0] = dp[0];
#pragma unroll
          for (int k = 0; k < K - 1; ++k)
#pragma unroll
            for (int j = 0; j < NH; ++j) win[k][j] = win[k + 1][j];
        }
      }
    }
    __syncthreads();
    // ---- phase 2: din[t0 + i] = sum_q w[K-1-q] * dpre[i + q], tokens i0 .. i0+7 ----
    if (live) {
      const int i0 = rs * (CONVB_TT / 8);
      const f32x2* dpp = reinterpret_cast<const f32x2*>(dpre) + hv * NH;
      auto load_row = [&](int row, f32x2 (&v)[NH]) {
        const f32x2* q = dpp + (size_t)row * (DPRE_ROWB / 8);
        if constexpr (NH == 2) { const ulonglong2 t = *reinterpret_cast<const ulonglong2*>(q); v[0] = t.x; v[1] = t.y; }
        else v[0] = q[0];
      };
      T* dp = din + (long long)b * din_stride_b + (long long)(t0 + i0) * din_stride_l + c0;
      f32x2 dwin[K][NH];
#pragma unroll
      for (int q = 0; q < K - 1; ++q) load_row(i0 + q, dwin[q]);
#pragma unroll
      for (int i = 0; i < CONVB_TT / 8; ++i) {
        load_row(i0 + i + K - 1, dwin[K - 1]);
        float o[NP];
#pragma unroll
        for (int j = 0; j < NH; ++j) {
          f32x2 a2 = 0ull;
#pragma unroll
          for (int q = 0; q < K; ++q) a2 = fma2(w[j][K - 1 - q], dwin[q][j], a2);
          unpack2(a2, o[2 * j], o[2 * j + 1]);
        }
        if (t0 + i0 + i < d.seqlen) store_n(dp, o);
        dp += din_stride_l;
#pragma unroll
        for (int q = 0; q < K - 1; ++q)
#pragma unroll
          for (int j = 0; j < NH; ++j) dwin[q][j] = dwin[q + 1][j];
      }
    }
  }
  cp_async_wait<0>();
  __syncthreads();
  // the eight row groups add their weight / bias gradients in order, through the (now idle) stage memory
  float* red = reinterpret_cast<float*>(conv_smem);
  constexpr int PER = NP * (K + 1);
#pragma unroll
  for (int j = 0; j < NH; ++j) {
    float* rp = red + (rs * 32 + hv) * PER + 2 * j * (K + 1);
#pragma unroll
    for (int k = 0; k < K; ++k) unpack2(dw[j][k], rp[k], rp[K + 1 + k]);
    unpack2(db[j], rp[K], rp[2 * K + 1]);
  }
  __syncthreads();
  for (int e = tid; e < 32 * PER; e += CONVS_THREADS) {
    const int v = e / PER, rem = e - v * PER;
    const int c = cb * CB + v * NP + rem / (K + 1);
    if (c < d.channels) {
      float a = 0.f;
#pragma unroll
      for (int g = 0; g < 8; ++g) a += red[(g * 32 + v) * PER + rem];
      partial[((size_t)blockIdx.x * d.channels + c) * (K + 1) + rem % (K + 1)] = a;
    }
  }
}

// dweight[c,k] / dbias[c] = sum over blocks of the partials, in block order
__global__ void k_conv_reduce(int nblk, int channels, int K, const float* __restrict__ partial, float* __restrict__ dweight,
                              float* __restrict__ dbias) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= channels * (K + 1)) return;
  float a = 0.f;
  for (int r = 0; r < nblk; ++r) a += partial[(size_t)r * channels * (K + 1) + i];
  const int c = i / (K + 1), k = i - c * (K + 1);
  if (k < K) dweight[(size_t)c * K + k] = a;
  else if (dbias) dbias[c] = a;
}

// ---------------------------------------------------------------------------------------------
// RMS norm.  One warp per row; a lane owns the 8-element vectors v, v+32, ... of the row.
constexpr int NORM_THREADS = 128, NORM_MAXV = 8;   // rows of up to 2048 elements stay in registers (NV = vectors per lane)

template <typename T, int NV>
__global__ void __launch_bounds__(NORM_THREADS) k_rmsnorm_fwd(SsdNormDims d, const T* __restrict__ in,
                                                              const float* __restrict__ weight, T* __restrict__ out,
                                                              float* __restrict__ rstd) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * (NORM_THREADS / 32) + (threadIdx.x >> 5);
  if (row >= d.rows) return;
  const int nv = d.width / 8;
  const T* ip = in + row * d.in_stride_row;
  T* op = out + row * d.out_stride_row;
  float v[NV][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int vi = lane + 32 * i;
    if (vi < nv) {
      load8<T>(ip + vi * 8, v[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss = fmaf(v[i][j], v[i][j], ss);
    }
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  const float r = rsqrtf(ss / (float)d.width + d.eps);
  if (lane == 0 && rstd) rstd[row] = r;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int vi = lane + 32 * i;
    if (vi < nv) {
      float o[8], wv[8];
      if (weight) load8<float>(weight + vi * 8, wv);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = v[i][j] * r * (weight ? wv[j] : 1.f);
      store8<T>(op + vi * 8, o);
    }
  }
}

// backward: n = in * rstd, dn = dout * weight, din = rstd * (dn - n * mean(dn * n)), dweight += dout * n.
// Warps walk rows with a grid stride, RU rows requested together (narrow rows would otherwise leave one 1 KB request
// per warp in flight); a block leaves one dweight partial row.
template <typename T, int NV>
__global__ void __launch_bounds__(NORM_THREADS) k_rmsnorm_bwd(SsdNormDims d, const T* __restrict__ in,
                                                              const float* __restrict__ weight, const float* __restrict__ rstd,
                                                              const T* __restrict__ dout, long long dout_stride_row,
                                                              T* __restrict__ din, long long din_stride_row,
                                                              float* __restrict__ partial) {
  constexpr int RU = NV == 1 ? 4 : (NV == 2 ? 2 : 1);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nv = d.width / 8;
  float wv[NV][8], dwv[NV][8];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int vi = lane + 32 * i;
#pragma unroll
    for (int j = 0; j < 8; ++j) { wv[i][j] = 1.f; dwv[i][j] = 0.f; }
    if (weight && vi < nv) load8<float>(weight + vi * 8, wv[i]);
  }
  const long long wstride = (long long)gridDim.x * (NORM_THREADS / 32);
  for (long long row0 = (long long)blockIdx.x * (NORM_THREADS / 32) + warp; row0 < d.rows; row0 += wstride * RU) {
    RawN<T, 8> rx[RU][NV], rg[RU][NV];
    float rs_[RU];
#pragma unroll
    for (int u = 0; u < RU; ++u) {
      const long long row = row0 + u * wstride;
      const bool rok = row < d.rows;
      rs_[u] = rok ? __ldg(rstd + row) : 0.f;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int vi = lane + 32 * i;
        if (rok && vi < nv) {
          load_raw(in + row * d.in_stride_row + vi * 8, rx[u][i]);
          load_raw(dout + row * dout_stride_row + vi * 8, rg[u][i]);
        } else {
          rx[u][i] = RawN<T, 8>{};
          rg[u][i] = RawN<T, 8>{};
        }
      }
    }
#pragma unroll
    for (int u = 0; u < RU; ++u) {
      const long long row = row0 + u * wstride;
      if (row >= d.rows) break;      // warp-uniform
      const float r = rs_[u];
      float n[NV][8], dn[NV][8];
      float dot = 0.f;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        float x[8], g[8];
        unpack_raw(rx[u][i], x);
        unpack_raw(rg[u][i], g);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          n[i][j] = x[j] * r;
          dn[i][j] = g[j] * wv[i][j];
          dwv[i][j] = fmaf(g[j], n[i][j], dwv[i][j]);
          dot = fmaf(dn[i][j], n[i][j], dot);
        }
      }
#pragma unroll
      for (int o = 16; o; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
      const float m = dot / (float)d.width;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int vi = lane + 32 * i;
        if (vi < nv) {
          float o[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = r * (dn[i][j] - n[i][j] * m);
          store8<T>(din + row * din_stride_row + vi * 8, o);
        }
      }
    }
  }
  if (!partial) return;
  // the four warps of the block add their weight-gradient rows in warp order, through shared memory
  __shared__ float sred[NORM_THREADS / 32][32 * 8 + 1];
  for (int i = 0; i < NV; ++i) {   // block-uniform trip count
    if (i * 32 >= nv) break;
    const int vi = lane + 32 * i;
#pragma unroll
    for (int j = 0; j < 8; ++j) sred[warp][lane * 8 + j] = dwv[i][j];
    __syncthreads();
    if (warp == 0 && vi < nv) {
      float* pp = partial + (size_t)blockIdx.x * d.width + vi * 8;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float a = 0.f;
        for (int ww = 0; ww < NORM_THREADS / 32; ++ww) a += sred[ww][lane * 8 + j];
        pp[j] = a;
      }
    }
    __syncthreads();
  }
}

// RMS norm backward, rows staged through shared memory: every WARP walks pairs of rows with a cp.async ring of its own
// (three stages of {two rows of in, two rows of dout}), so nothing but the warp's own copies has to be waited for and the
// bytes in flight are set by the ring and the number of resident warps (6 KB per warp at 256 bf16 features, eight blocks
// per SM) instead of by registers.  Same arithmetic and the same per-block dweight partial as k_rmsnorm_bwd.
constexpr int NORMR_ROWS = 2, NORMR_STAGES = 3;

template <typename T, int NV>
__global__ void __launch_bounds__(NORM_THREADS, 8) k_rmsnorm_bwd_ring(SsdNormDims d, const T* __restrict__ in,
                                                                      const float* __restrict__ weight, const float* __restrict__ rstd,
                                                                      const T* __restrict__ dout, long long dout_stride_row,
                                                                      T* __restrict__ din, long long din_stride_row,
                                                                      float* __restrict__ partial) {
  constexpr int ES = (int)sizeof(T), RW = NORMR_ROWS, S = NORMR_STAGES;
  extern __shared__ __align__(16) unsigned char norm_ring[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nv = d.width / 8;
  const int row_bytes = d.width * ES, ppr = row_bytes / 16;      // 16-byte pieces per row
  const int stage_bytes = 2 * RW * row_bytes;
  unsigned char* wring = norm_ring + warp * (S * stage_bytes);
  float wv[NV][8], dwv[NV][8];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int vi = lane + 32 * i;
#pragma unroll
    for (int j = 0; j < 8; ++j) { wv[i][j] = 1.f; dwv[i][j] = 0.f; }
    if (weight && vi < nv) load8<float>(weight + vi * 8, wv[i]);
  }
  const long long nitems = (d.rows + RW - 1) / RW;
  const long long first = (long long)blockIdx.x * (NORM_THREADS / 32) + warp, stride = (long long)gridDim.x * (NORM_THREADS / 32);
  auto issue = [&](long long it, int stage) {
    if (it < nitems) {
      unsigned char* sm = wring + stage * stage_bytes;
#pragma unroll
      for (int u = 0; u < RW; ++u) {
        const long long row = it * RW + u;
        const bool ok = row < d.rows;
        const char* gi = (const char*)(in + (ok ? row : 0) * d.in_stride_row);
        const char* go = (const char*)(dout + (ok ? row : 0) * dout_stride_row);
        for (int c = lane; c < ppr; c += 32) {
          cp_async16(sm + u * row_bytes + c * 16, gi + c * 16, ok);
          cp_async16(sm + (RW + u) * row_bytes + c * 16, go + c * 16, ok);
        }
      }
    }
    cp_async_commit();
  };
  auto load_rstd = [&](long long it, float (&r)[RW]) {
#pragma unroll
    for (int u = 0; u < RW; ++u) {
      const long long row = it * RW + u;
      r[u] = (it < nitems && row < d.rows) ? __ldg(rstd + row) : 0.f;
    }
  };
#pragma unroll
  for (int k = 0; k < S - 1; ++k) issue(first + k * stride, k);
  float rs_next[RW];
  load_rstd(first, rs_next);
  int stage = 0;
  for (long long it = first; it < nitems; it += stride) {
    cp_async_wait<S - 2>();
    __syncwarp();          // the warp's own copies of this item have landed; its lanes are done with the previous slot
    issue(it + (S - 1) * stride, stage == 0 ? S - 1 : stage - 1);
    float rs_[RW];
#pragma unroll
    for (int u = 0; u < RW; ++u) rs_[u] = rs_next[u];
    load_rstd(it + stride, rs_next);
    const unsigned char* sm = wring + stage * stage_bytes;
    stage = stage + 1 == S ? 0 : stage + 1;
#pragma unroll
    for (int u = 0; u < RW; ++u) {
      const long long row = it * RW + u;
      if (row >= d.rows) break;      // warp-uniform
      const float r = rs_[u];
      float n[NV][8], dn[NV][8];
      float dot = 0.f;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int vi = lane + 32 * i;
        if (vi < nv) {
          float x[8], g[8];
          RawN<T, 8> rx, rg;
          lds_raw<T, 8>(sm + u * row_bytes + vi * 8 * ES, rx);
          lds_raw<T, 8>(sm + (RW + u) * row_bytes + vi * 8 * ES, rg);
          unpack_raw(rx, x);
          unpack_raw(rg, g);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            n[i][j] = x[j] * r;
            dn[i][j] = g[j] * wv[i][j];
            dwv[i][j] = fmaf(g[j], n[i][j], dwv[i][j]);
            dot = fmaf(dn[i][j], n[i][j], dot);
          }
        }
      }
#pragma unroll
      for (int o = 16; o; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
      const float m = dot / (float)d.width;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int vi = lane + 32 * i;
        if (vi < nv) {
          float o[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = r * (dn[i][j] - n[i][j] * m);
          store8<T>(din + row * din_stride_row + vi * 8, o);
        }
      }
    }
  }
  cp_async_wait<0>();
  if (!partial) return;
  // the four warps of the block add their weight-gradient rows in warp order, through shared memory
  __shared__ float sred[NORM_THREADS / 32][32 * 8 + 1];
  for (int i = 0; i < NV; ++i) {   // block-uniform trip count
    if (i * 32 >= nv) break;
    const int vi = lane + 32 * i;
#pragma unroll
    for (int j = 0; j < 8; ++j) sred[warp][lane * 8 + j] = dwv[i][j];
    __syncthreads();
    if (warp == 0 && vi < nv) {
      float* pp = partial + (size_t)blockIdx.x * d.width + vi * 8;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float a = 0.f;
        for (int ww = 0; ww < NORM_THREADS / 32; ++ww) a += sred[ww][lane * 8 + j];
        pp[j] = a;
      }
    }
    __syncthreads();
  }
}

// dweight[i] = sum over blocks of the partials: eight row groups per column add their rows in order, then the groups
// are added in order (the same sum for the same grid, whatever the timing)
__global__ void k_norm_reduce(int nblk, int width, const float* __restrict__ partial, float* __restrict__ dweight) {
  __shared__ float red[8][32];
  const int i = blockIdx.x * 32 + threadIdx.x, g = threadIdx.y;
  float a = 0.f;
  if (i < width)
    for (int r = g; r < nblk; r += 8) a += partial[(size_t)r * width + i];
  red[g][threadIdx.x] = a;
  __syncthreads();
  if (g == 0 && i < width) {
    float t = 0.f;
#pragma unroll
    for (int q = 0; q < 8; ++q) t += red[q][threadIdx.x];
    dweight[i] = t;
  }
}

int conv_rows(const SsdConvDims* d) {   // thread rows of the backward kernel = partial sums to add
  const int ntile = (d->seqlen + CONV_TLB - 1) / CONV_TLB;
  const long long pairs = (long long)d->batch * ntile;
  return (int)(pairs < CONV_ROWS ? pairs : CONV_ROWS);
}
int norm_blocks(const SsdNormDims* d) {
  const long long need = (d->rows + NORM_THREADS / 32 - 1) / (NORM_THREADS / 32);
  return (int)(need < 1184 ? need : 1184);
}

int check_conv(const SsdConvDims* d) {
  if (!d) { set_error("dims is NULL"); return SSD_ERR_NULL_POINTER; }
  if (d->batch <= 0 || d->seqlen <= 0 || d->channels <= 0) { set_error("conv1d: batch, seqlen and channels must be positive"); return SSD_ERR_BAD_SHAPE; }
  if (d->width < 2 || d->width > 4) { set_error("conv1d: width %d not supported (2..4)", d->width); return SSD_ERR_UNSUPPORTED; }
  if (d->channels % 8) { set_error("conv1d: channels (%d) must be a multiple of 8", d->channels); return SSD_ERR_UNSUPPORTED; }
  if (d->dtype != SSD_F32 && d->dtype != SSD_BF16) { set_error("conv1d: unknown dtype %d", d->dtype); return SSD_ERR_UNSUPPORTED; }
  const int es = d->dtype == SSD_BF16 ? 2 : 4;
  const long long strides[4] = {d->in_stride_b, d->in_stride_l, d->out_stride_b, d->out_stride_l};
  for (long long st : strides)
    if (st < 0 || (st * es) % 16) { set_error("conv1d: strides must be non-negative multiples of 16 bytes"); return SSD_ERR_BAD_ALIGNMENT; }
  if (d->in_stride_l < d->channels || d->out_stride_l < d->channels) { set_error("conv1d: row strides smaller than the channel count"); return SSD_ERR_BAD_SHAPE; }
  return SSD_OK;
}
bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

}  // namespace
}  // namespace ssd

using namespace ssd;

extern "C" {

size_t ssd_conv1d_workspace_bytes(const SsdConvDims* dims) {
  clear_error();
  if (check_conv(dims)) return 0;
  return (size_t)conv_rows(dims) * dims->channels * (dims->width + 1) * sizeof(float);
}

int32_t ssd_conv1d_forward(const SsdConvDims* dims, const void* in, const float* weight, const float* bias, void* out,
                           void* cuda_stream) {
  clear_error();
  int rc = check_conv(dims);
  if (rc) return rc;
  if (!in || !weight || !out) { set_error("conv1d: in / weight / out is NULL"); return SSD_ERR_NULL_POINTER; }
  if (!aligned16(in) || !aligned16(out)) { set_error("conv1d: in and out must be 16-byte aligned"); return SSD_ERR_BAD_ALIGNMENT; }
  cudaStream_t s = (cudaStream_t)cuda_stream;
  const int esz = dims->dtype == SSD_BF16 ? 2 : 4;
  if ((long long)dims->channels * esz >= CONVS_ROWB / 2) {
    // shared-memory staged kernel: tiles of 64 tokens x 256 bytes of channels, persistent CTAs
    const int ntt = (dims->seqlen + CONVS_TT - 1) / CONVS_TT;
    const int ncb = (dims->channels * esz + CONVS_ROWB - 1) / CONVS_ROWB;
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const long long pairs = (long long)dims->batch * ntt;
    if (pairs > 0x7fffffffLL) { set_error("conv1d: batch x token tiles exceeds 2^31"); return SSD_ERR_UNSUPPORTED; }
    long long gx = ((long long)sms * CONVS_CTAS_PER_SM) / ncb;
    if (gx < 1) gx = 1;
    if (gx > pairs) gx = pairs;
    if (ncb > 65535) { set_error("conv1d: too many channels"); return SSD_ERR_UNSUPPORTED; }
    const dim3 grid((unsigned)gx, (unsigned)ncb);
#define CONV_FWD_SM(T, K) do { \
      constexpr int smem = (CONVS_TT + K - 1) * CONVS_ROWB * CONVS_STAGES; \
      cudaFuncSetAttribute(k_conv_fwd_sm<T, K>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); \
      k_conv_fwd_sm<T, K><<<grid, CONVS_THREADS, smem, s>>>(*dims, (const T*)in, weight, bias, (T*)out, ntt); } while (0)
    if (dims->dtype == SSD_BF16) {
      if (dims->width == 4) CONV_FWD_SM(__nv_bfloat16, 4); else if (dims->width == 3) CONV_FWD_SM(__nv_bfloat16, 3); else CONV_FWD_SM(__nv_bfloat16, 2);
    } else {
      if (dims->width == 4) CONV_FWD_SM(float, 4); else if (dims->width == 3) CONV_FWD_SM(float, 3); else CONV_FWD_SM(float, 2);
    }
#undef CONV_FWD_SM
    SSD_CUDA_CHECK_LAUNCH("conv1d_fwd");
    return SSD_OK;
  }
  constexpr int NCF = 8;   // channels per thread, forward
  const long long items = (long long)dims->batch * ((dims->seqlen + CONV_TL - 1) / CONV_TL) * (dims->channels / NCF);
  const unsigned grid = (unsigned)((items + CONV_THREADS - 1) / CONV_THREADS);
#define CONV_FWD(T, K) k_conv_fwd<T, K, NCF><<<grid, CONV_THREADS, 0, s>>>(*dims, (const T*)in, weight, bias, (T*)out)
  if (dims->dtype == SSD_BF16) {
    if (dims->width == 4) CONV_FWD(__nv_bfloat16, 4); else if (dims->width == 3) CONV_FWD(__nv_bfloat16, 3); else CONV_FWD(__nv_bfloat16, 2);
  } else {
    if (dims->width == 4) CONV_FWD(float, 4); else if (dims->width == 3) CONV_FWD(float, 3); else CONV_FWD(float, 2);
  }
#undef CONV_FWD
  SSD_CUDA_CHECK_LAUNCH("conv1d_fwd");
  return SSD_OK;
}

int32_t ssd_conv1d_backward(const SsdConvDims* dims, const void* in, const float* weight, const float* bias,
                            const SsdConvGrad* dout, int32_t ndout, void* din, int64_t din_stride_b, int64_t din_stride_l,
                            float* dweight, float* dbias, void* workspace, size_t workspace_bytes, void* cuda_stream) {
  clear_error();
  int rc = check_conv(dims);
  if (rc) return rc;
  if (!in || !weight || !dout || !din || !dweight || !workspace) { set_error("conv1d backward: a required pointer is NULL"); return SSD_ERR_NULL_POINTER; }
  if (ndout < 1 || ndout > 3) { set_error("conv1d backward: 1 to 3 gradient segments, got %d", ndout); return SSD_ERR_BAD_SHAPE; }
  const int es = dims->dtype == SSD_BF16 ? 2 : 4;
  ConvSegs segs;
  segs.n = ndout;
  int c = 0;
  for (int i = 0; i < 3; ++i) {
    if (i < ndout) {
      if (!dout[i].ptr || !aligned16(dout[i].ptr)) { set_error("conv1d backward: gradient segment %d is NULL or not 16-byte aligned", i); return SSD_ERR_BAD_ALIGNMENT; }
      if (dout[i].channels <= 0 || dout[i].channels % 8 || dout[i].stride_l < dout[i].channels ||
          (dout[i].stride_b * es) % 16 || (dout[i].stride_l * es) % 16) {
        set_error("conv1d backward: gradient segment %d: channels must be a positive multiple of 8, strides multiples of 16 bytes", i);
        return SSD_ERR_BAD_SHAPE;
      }
      segs.ptr[i] = dout[i].ptr; segs.c_begin[i] = c; segs.stride_b[i] = dout[i].stride_b; segs.stride_l[i] = dout[i].stride_l;
      c += dout[i].channels;
    } else {
      segs.ptr[i] = nullptr; segs.c_begin[i] = 0x7fffffff; segs.stride_b[i] = 0; segs.stride_l[i] = 0;
    }
  }
  if (c != dims->channels) { set_error("conv1d backward: gradient segments cover %d channels, expected %d", c, dims->channels); return SSD_ERR_BAD_SHAPE; }
  if (!aligned16(in) || !aligned16(din) || din_stride_l < dims->channels || (din_stride_b * es) % 16 || (din_stride_l * es) % 16) {
    set_error("conv1d backward: in / din must be 16-byte aligned with strides that are multiples of 16 bytes");
    return SSD_ERR_BAD_ALIGNMENT;
  }
  const int nblk = conv_rows(dims);
  const size_t need = (size_t)nblk * dims->channels * (dims->width + 1) * sizeof(float);
  if (workspace_bytes < need) { set_error("conv1d backward: workspace too small: %zu < %zu", workspace_bytes, need); return SSD_ERR_WORKSPACE_TOO_SMALL; }
  cudaStream_t s = (cudaStream_t)cuda_stream;
  float* partial = (float*)workspace;
  if ((long long)dims->channels * es >= CONVS_ROWB / 2) {
    const int ntt = (dims->seqlen + CONVB_TT - 1) / CONVB_TT;
    const int ncb = (dims->channels * es + CONVS_ROWB - 1) / CONVS_ROWB;
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    long long nx = ((long long)sms * CONVB_CTAS_PER_SM + ncb - 1) / ncb;
    const long long pairs = (long long)dims->batch * ntt;
    if (pairs > 0x7fffffffLL || ncb > 65535) { set_error("conv1d backward: batch x token tiles exceeds 2^31"); return SSD_ERR_UNSUPPORTED; }
    if (nx > pairs) nx = pairs;
    if (nx > nblk) nx = nblk;     // the workspace holds nblk partial rows
    const dim3 grid((unsigned)nx, (unsigned)ncb);
#define CONV_BWD_SM(T, K) do { \
      constexpr int smem = CONVB_STAGES * (2 * CONVB_TT + 3 * (K - 1)) * CONVS_ROWB + (CONVB_TT + K - 1) * (CONVS_ROWB / (int)sizeof(T)) * 4; \
      cudaFuncSetAttribute(k_conv_bwd_sm<T, K>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); \
      k_conv_bwd_sm<T, K><<<grid, CONVS_THREADS, smem, s>>>(*dims, (const T*)in, weight, bias, segs, (T*)din, din_stride_b, din_stride_l, partial, ntt); } while (0)
    if (dims->dtype == SSD_BF16) {
      if (dims->width == 4) CONV_BWD_SM(__nv_bfloat16, 4); else if (dims->width == 3) CONV_BWD_SM(__nv_bfloat16, 3); else CONV_BWD_SM(__nv_bfloat16, 2);
    } else {
      if (dims->width == 4) CONV_BWD_SM(float, 4); else if (dims->width == 3) CONV_BWD_SM(float, 3); else CONV_BWD_SM(float, 2);
    }
#undef CONV_BWD_SM
    SSD_CUDA_CHECK_LAUNCH("conv1d_bwd");
    const int n = dims->channels * (dims->width + 1);
    k_conv_reduce<<<(n + 255) / 256, 256, 0, s>>>((int)nx, dims->channels, dims->width, partial, dweight, dbias);
    SSD_CUDA_CHECK_LAUNCH("conv1d_reduce");
    return SSD_OK;
  }
  constexpr int NCB = 4;   // channels per thread, backward (half the registers of 8: twice the resident warps)
  const unsigned grid = (unsigned)(((long long)nblk * (dims->channels / NCB) + CONV_THREADS - 1) / CONV_THREADS);
#define CONV_BWD(T, K) k_conv_bwd<T, K, NCB><<<grid, CONV_THREADS, 0, s>>>(*dims, nblk, (const T*)in, weight, bias, segs, (T*)din, din_stride_b, din_stride_l, partial)
  if (dims->dtype == SSD_BF16) {
    if (dims->width == 4) CONV_BWD(__nv_bfloat16, 4); else if (dims->width == 3) CONV_BWD(__nv_bfloat16, 3); else CONV_BWD(__nv_bfloat16, 2);
  } else {
    if (dims->width == 4) CONV_BWD(float, 4); else if (dims->width == 3) CONV_BWD(float, 3); else CONV_BWD(float, 2);
  }
#undef CONV_BWD
  SSD_CUDA_CHECK_LAUNCH("conv1d_bwd");
  const int n = dims->channels * (dims->width + 1);
  k_conv_reduce<<<(n + 255) / 256, 256, 0, s>>>(nblk, dims->channels, dims->width, partial, dweight, dbias);
  SSD_CUDA_CHECK_LAUNCH("conv1d_reduce");
  return SSD_OK;
}

static int check_norm(const SsdNormDims* d) {
  if (!d) { set_error("dims is NULL"); return SSD_ERR_NULL_POINTER; }
  if (d->rows <= 0 || d->width <= 0) { set_error("rmsnorm: rows and width must be positive"); return SSD_ERR_BAD_SHAPE; }
  if (d->width % 8 || d->width > NORM_MAXV * 256) { set_error("rmsnorm: width (%d) must be a multiple of 8, at most %d", d->width, NORM_MAXV * 256); return SSD_ERR_UNSUPPORTED; }
  if (d->dtype != SSD_F32 && d->dtype != SSD_BF16) { set_error("rmsnorm: unknown dtype %d", d->dtype); return SSD_ERR_UNSUPPORTED; }
  const int es = d->dtype == SSD_BF16 ? 2 : 4;
  if (d->in_stride_row < d->width || d->out_stride_row < d->width || (d->in_stride_row * es) % 16 || (d->out_stride_row * es) % 16) {
    set_error("rmsnorm: row strides must cover the width and be multiples of 16 bytes");
    return SSD_ERR_BAD_ALIGNMENT;
  }
  return SSD_OK;
}

size_t ssd_rmsnorm_workspace_bytes(const SsdNormDims* dims) {
  clear_error();
  if (check_norm(dims)) return 0;
  return (size_t)norm_blocks(dims) * dims->width * sizeof(float);
}

int32_t ssd_rmsnorm_forward(const SsdNormDims* dims, const void* in, const float* weight, void* out, float* rstd,
                            void* cuda_stream) {
  clear_error();
  int rc = check_norm(dims);
  if (rc) return rc;
  if (!in || !out) { set_error("rmsnorm: in / out is NULL"); return SSD_ERR_NULL_POINTER; }
  if (!aligned16(in) || !aligned16(out) || (weight && !aligned16(weight))) { set_error("rmsnorm: pointers must be 16-byte aligned"); return SSD_ERR_BAD_ALIGNMENT; }
  cudaStream_t s = (cudaStream_t)cuda_stream;
  const long long nb = (dims->rows + NORM_THREADS / 32 - 1) / (NORM_THREADS / 32);
  const int nvl = (dims->width / 8 + 31) / 32;   // vectors per lane
#define NORM_FWD(T, NV) k_rmsnorm_fwd<T, NV><<<(unsigned)nb, NORM_THREADS, 0, s>>>(*dims, (const T*)in, weight, (T*)out, rstd)
#define NORM_FWD_T(T) do { if (nvl <= 1) NORM_FWD(T, 1); else if (nvl <= 2) NORM_FWD(T, 2); else if (nvl <= 4) NORM_FWD(T, 4); else NORM_FWD(T, 8); } while (0)
  if (dims->dtype == SSD_BF16) NORM_FWD_T(__nv_bfloat16); else NORM_FWD_T(float);
#undef NORM_FWD_T
#undef NORM_FWD
  SSD_CUDA_CHECK_LAUNCH("rmsnorm_fwd");
  return SSD_OK;
}

int32_t ssd_rmsnorm_backward(const SsdNormDims* dims, const void* in, const float* weight, const float* rstd,
                             const void* dout, int64_t dout_stride_row, void* din, int64_t din_stride_row, float* dweight,
                             void* workspace, size_t workspace_bytes, void* cuda_stream) {
  clear_error();
  int rc = check_norm(dims);
  if (rc) return rc;
  if (!in || !rstd || !dout || !din) { set_error("rmsnorm backward: a required pointer is NULL"); return SSD_ERR_NULL_POINTER; }
  if ((weight != nullptr) != (dweight != nullptr)) { set_error("rmsnorm backward: dweight must be given iff weight is"); return SSD_ERR_NULL_POINTER; }
  const int es = dims->dtype == SSD_BF16 ? 2 : 4;
  if (!aligned16(in) || !aligned16(dout) || !aligned16(din) || dout_stride_row < dims->width || din_stride_row < dims->width ||
      (dout_stride_row * es) % 16 || (din_stride_row * es) % 16) {
    set_error("rmsnorm backward: pointers must be 16-byte aligned, strides multiples of 16 bytes");
    return SSD_ERR_BAD_ALIGNMENT;
  }
  const int nblk = norm_blocks(dims);
  float* partial = nullptr;
  if (dweight) {
    const size_t need = (size_t)nblk * dims->width * sizeof(float);
    if (!workspace || workspace_bytes < need) { set_error("rmsnorm backward: workspace too small: %zu < %zu", workspace_bytes, need); return SSD_ERR_WORKSPACE_TOO_SMALL; }
    partial = (float*)workspace;
  }
  cudaStream_t s = (cudaStream_t)cuda_stream;
  const int nvl = (dims->width / 8 + 31) / 32;
#define NORM_BWD(T, NV) k_rmsnorm_bwd<T, NV><<<nblk, NORM_THREADS, 0, s>>>(*dims, (const T*)in, weight, rstd, (const T*)dout, dout_stride_row, (T*)din, din_stride_row, partial)
#define NORM_BWD_T(T) do { if (nvl <= 1) NORM_BWD(T, 1); else if (nvl <= 2) NORM_BWD(T, 2); else if (nvl <= 4) NORM_BWD(T, 4); else NORM_BWD(T, 8); } while (0)
  const int row_bytes = dims->width * es;
  const int ring_smem = (NORM_THREADS / 32) * NORMR_STAGES * 2 * NORMR_ROWS * row_bytes;
  const bool ring = nvl <= 1 && (row_bytes % 16) == 0 && ring_smem <= 96 * 1024 && (dims->in_stride_row * es) % 16 == 0;
  if (ring) {
#define NORM_BWD_RING(T, NV) do { \
      cudaFuncSetAttribute(k_rmsnorm_bwd_ring<T, NV>, cudaFuncAttributeMaxDynamicSharedMemorySize, ring_smem); \
      k_rmsnorm_bwd_ring<T, NV><<<nblk, NORM_THREADS, ring_smem, s>>>(*dims, (const T*)in, weight, rstd, (const T*)dout, dout_stride_row, (T*)din, din_stride_row, partial); } while (0)
    if (dims->dtype == SSD_BF16) NORM_BWD_RING(__nv_bfloat16, 1); else NORM_BWD_RING(float, 1);
#undef NORM_BWD_RING
  } else if (dims->dtype == SSD_BF16) NORM_BWD_T(__nv_bfloat16); else NORM_BWD_T(float);
#undef NORM_BWD_T
#undef NORM_BWD
  SSD_CUDA_CHECK_LAUNCH("rmsnorm_bwd");
  if (dweight) {
    k_norm_reduce<<<(dims->width + 31) / 32, dim3(32, 8), 0, s>>>(nblk, dims->width, partial, dweight);
    SSD_CUDA_CHECK_LAUNCH("rmsnorm_reduce");
  }
  return SSD_OK;
}

}  // extern "C"
