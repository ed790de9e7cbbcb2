// bf16 tensor-core kernels (tcgen05.mma, accumulators in TMEM, operands fed by TMA) for the
// intra-chunk contractions of the SSD forward and backward, chunk length 128.
//
//   k_state_tc : per (batch, chunk, group)   states[(h,p), n] = sum_l w[h,l] x[l,(h,p)] B[l,n]
//                A = x tile, scaled in place in shared memory, read MN-major; B = B tile read
//                MN-major; one 128 x N accumulator per 128 (h,p) rows.
//   k_scan_tc  : per (batch, chunk, group)   G = C B^T once (128x128 in TMEM), then per head
//                M_h = tril(G o exp(cs_i-cs_j) o dt_j) -> bf16 -> shared memory,
//                Y = M_h X_h  (+)  exp(cs_i) * (C S_prev^T);  three epilogues (forward, backward
//                recompute, dx).
//   k_dbc_tc   : per (batch, chunk, group)   W_h = dY_h X_h^T, masked/decayed like M_h, then
//                dC += W'_h B, dB += W'_h^T C accumulated over heads in TMEM, plus state terms.
//
// Everything a CTA reads arrives asynchronously: sequence tiles and the bf16 copies of the
// chunk-entry states by TMA, the per-head decay tables (written by the cumsum kernel) by 1-D
// bulk copies; the next head block's inputs are in flight while the current one is computed.
// Shared-memory tiles and descriptor conventions are described in umma.cuh.  Each CTA has 512
// threads: thread t owns accumulator row (t % 128) and part (t / 128) of the columns.
#include <stdlib.h>
#include <string.h>

#include <mutex>

#include "common.cuh"
#include "ssd_internal.h"
#include "umma.cuh"

namespace ssd {
namespace {

using namespace umma;
typedef __nv_bfloat16 bf16;

constexpr int QT = 128;               // chunk length of the tensor-core path
constexpr int TC_THREADS = 512;       // 16 warps: 4 per TMEM lane quarter
constexpr int PARTS = TC_THREADS / 128;
constexpr int BOX_BYTES = 128 * 128;  // sequence TMA box: 128 rows x 64 bf16
constexpr int SBOX_BYTES = 64 * 128;  // state TMA box: 64 (h,p) rows x 64 bf16
constexpr int TAB = SSD_TAB_FLOATS;   // floats per (batch, chunk, head) decay table
constexpr int TAB_BYTES = TAB * 4;
constexpr int T_CS = 0, T_DT = 128, T_CF = 256, T_DS = 384;   // table sections, 128 floats each

// Bounded waits: after the first one gives up every later wait is skipped, so a broken
// pipeline drains in bounded time instead of hanging; the status word tells the host.
struct Waiter {
  int* status;
  bool dead;
  __device__ __forceinline__ void wait(uint64_t* bar, uint32_t parity, int code) {
    if (dead) return;
    if (!mbar_wait(bar, parity)) {
      dead = true;
      atomicExch(status, code);
    }
  }
};

// Self-test of the bounded wait: one warp waits on an mbarrier that nothing ever arrives on.  The wait gives up after
// `max_cycles`, the kernel records the code like every pipeline kernel does and returns normally.
__global__ void k_selftest_wait(int* status, long long max_cycles) {
  __shared__ __align__(8) uint64_t bar;
  if (threadIdx.x == 0) { mbar_init(&bar, 1); mbar_fence_init(); }
  __syncthreads();
  if (!mbar_wait(&bar, 0, max_cycles) && threadIdx.x == 0) atomicExch(status, 99);
}

// ---------------------------------------------------------------------------------------------
// Decayed lower-triangular tile.  Source: a 128x128 fp32 accumulator in TMEM (C B^T or dY X^T).
// Result: out[i,j] = src[i,j] * exp(cs_i - cs_j) * dt_j for j <= i, written as bf16 into a plain
// 128x128 tile.  The tile is cut into 32x32 blocks; the four warps that share a TMEM lane quarter
// (= a block row) each take an 8-column slice of every block at or below the diagonal, so the work
// of a block row is spread over its four warps and every dependent chain is 8 long:
//   * blocks above the diagonal are never touched (zero_upper_blocks fills them once);
//   * blocks below use exp(cs_i - cs_j) dt_j = exp(cs_i - cs_r) * [exp(cs_r - cs_j) dt_j] with r the
//     last column of the block: one ex2 per block, the bracket is the per-column table T_CF, and
//     both exponents are <= 0 so nothing can overflow;
//   * in the diagonal block a slice starts from L[i, je] (je = its last column; exp(cs_i - cs_je) for
//     rows at or below je, 0 above) and walks left with the per-step decays,
//     L[i,j] = L[i,j+1] * decay_{j+1}, restarting at 1 on the diagonal.
// tab = this head's table: T_CS cs*log2(e), T_DT dt, T_CF column factors, T_DS[j] = exp(dt_{j+1} A).
__device__ __forceinline__ void decay_mask_tile(uint32_t tm_src, const float* __restrict__ tab, int row, int part,
                                                int warp, uint32_t mtile) {
  const int rb = warp & 3;                 // block row of this warp (warp-uniform)
  const uint32_t ts = smem_u32(tab);       // the table sits in shared memory: read it through the shared-memory pipe
  const float csi = lds_f32(ts + 4 * (T_CS + row));
  uint32_t raw[4][8];
#pragma unroll
  for (int cb = 0; cb < 4; ++cb)
    if (cb <= rb) tmem_ld8_issue(tmem_addr(tm_src, rb * 32, cb * 32 + part * 8), raw[cb]);
  tmem_ld_wait();
#pragma unroll
  for (int cb = 0; cb < 4; ++cb) {
    if (cb > rb) continue;
    const int c0 = cb * 32 + part * 8;
    float v[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] = __uint_as_float(raw[cb][k]);
    if (cb < rb) {
      const float rf = ex2(csi - lds_f32(ts + 4 * (T_CS + cb * 32 + 31)));
      const float4 f0 = lds_v4f32(ts + 4 * (T_CF + c0)), f1 = lds_v4f32(ts + 4 * (T_CF + c0 + 4));
      v[0] *= rf * f0.x; v[1] *= rf * f0.y; v[2] *= rf * f0.z; v[3] *= rf * f0.w;
      v[4] *= rf * f1.x; v[5] *= rf * f1.y; v[6] *= rf * f1.z; v[7] *= rf * f1.w;
    } else {
      const int je = c0 + 7;
      const float4 d0 = lds_v4f32(ts + 4 * (T_DS + c0)), d1 = lds_v4f32(ts + 4 * (T_DS + c0 + 4));
      const float4 t0 = lds_v4f32(ts + 4 * (T_DT + c0)), t1 = lds_v4f32(ts + 4 * (T_DT + c0 + 4));
      const float ds[8] = {d0.x, d0.y, d0.z, d0.w, d1.x, d1.y, d1.z, d1.w};   // ds[k] = decay of step c0+k+1
      const float dt[8] = {t0.x, t0.y, t0.z, t0.w, t1.x, t1.y, t1.z, t1.w};
      float run = (row >= je) ? ex2(csi - lds_f32(ts + 4 * (T_CS + je))) : 0.f;
      v[7] *= run * dt[7];
#pragma unroll
      for (int k = 6; k >= 0; --k) {
        run = (c0 + k == row) ? 1.f : run * ds[k];
        v[k] *= run * dt[k];
      }
    }
    st_shared_v4(mtile + plain_off(128, row, c0), pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]),
                 pack_bf16(v[6], v[7]));
  }
}
// Lower-triangular mask only: source = a 128x128 fp32 accumulator in TMEM that already carries the decay (separable heads,
// see k_dbc_ws), result = src[i,j] for j <= i as bf16 in a plain 128x128 tile.  Thread mapping of decay_mask_tile; blocks
// above the diagonal are never written (they are zero in every ring tile for the whole kernel).
__device__ __forceinline__ void mask_tril_tile(uint32_t tm_src, int row, int part, int warp, uint32_t mtile) {
  const int rb = warp & 3;
  uint32_t raw[4][8];
#pragma unroll
  for (int cb = 0; cb < 4; ++cb)
    if (cb <= rb) tmem_ld8_issue(tmem_addr(tm_src, rb * 32, cb * 32 + part * 8), raw[cb]);
  tmem_ld_wait();
#pragma unroll
  for (int cb = 0; cb < 4; ++cb) {
    if (cb > rb) continue;
    const int c0 = cb * 32 + part * 8;
    float v[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] = (cb < rb || c0 + k <= row) ? __uint_as_float(raw[cb][k]) : 0.f;
    st_shared_v4(mtile + plain_off(128, row, c0), pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]),
                 pack_bf16(v[6], v[7]));
  }
}
// zero the 32x32 blocks above the diagonal of a plain 128x128 tile (same thread mapping)
__device__ __forceinline__ void zero_upper_blocks(int row, int part, int warp, uint32_t mtile) {
#pragma unroll
  for (int cb = 1; cb < 4; ++cb)
    if (cb > (warp & 3)) st_shared_v4(mtile + plain_off(128, row, cb * 32 + part * 8), 0u, 0u, 0u, 0u);
}

// Whole-row variant for the persistent kernels.  A group of four warps (one per TMEM lane quarter)
// owns one head at a time and different groups work on different heads, so the latency of one group's
// TMEM loads, table loads and stores hides behind another group's arithmetic.  Thread = accumulator
// row; it walks the 32x32 blocks of its block row left to right (blocks below the diagonal first, the
// diagonal block last) with the next block's TMEM load in flight while the current one is scaled,
// converted and stored.  Same factorisation as decay_mask_tile.
__device__ __forceinline__ void tmem_ld16_issue(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait_2x16(uint32_t (&r)[16], uint32_t (&q)[16]) {
  // the registers are operands so that no use of them can be scheduled above the wait
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]),
                 "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]), "+r"(q[0]),
                 "+r"(q[1]), "+r"(q[2]), "+r"(q[3]), "+r"(q[4]), "+r"(q[5]), "+r"(q[6]), "+r"(q[7]), "+r"(q[8]),
                 "+r"(q[9]), "+r"(q[10]), "+r"(q[11]), "+r"(q[12]), "+r"(q[13]), "+r"(q[14]), "+r"(q[15])
               :: "memory");
}
// 16 columns of a block below the diagonal: out[k] = raw[k] * rf * cf[k]; `cf` = shared-memory address of the column factors
__device__ __forceinline__ void decay_off_half(const uint32_t (&raw)[16], float rf, uint32_t cf, uint32_t dst) {
#pragma unroll
  for (int j8 = 0; j8 < 16; j8 += 8) {
    const float4 f0 = lds_v4f32(cf + 4 * j8), f1 = lds_v4f32(cf + 4 * (j8 + 4));
    const float v0 = __uint_as_float(raw[j8]) * f0.x * rf, v1 = __uint_as_float(raw[j8 + 1]) * f0.y * rf;
    const float v2 = __uint_as_float(raw[j8 + 2]) * f0.z * rf, v3 = __uint_as_float(raw[j8 + 3]) * f0.w * rf;
    const float v4 = __uint_as_float(raw[j8 + 4]) * f1.x * rf, v5 = __uint_as_float(raw[j8 + 5]) * f1.y * rf;
    const float v6 = __uint_as_float(raw[j8 + 6]) * f1.z * rf, v7 = __uint_as_float(raw[j8 + 7]) * f1.w * rf;
    st_shared_v4(dst + (j8 >> 3) * 2048, pack_bf16(v0, v1), pack_bf16(v2, v3), pack_bf16(v4, v5), pack_bf16(v6, v7));
  }
}
// 16 columns (starting at column c0) of the diagonal block: two independent 8-column walks; `ts` = shared-memory address
// of the head's table
__device__ __forceinline__ void decay_diag_half(const uint32_t (&raw)[16], uint32_t ts, int c0, int row, float csi, uint32_t dst) {
#pragma unroll
  for (int s = 0; s < 2; ++s) {
    const int cs0 = c0 + 8 * s, je = cs0 + 7;
    const float4 d0 = lds_v4f32(ts + 4 * (T_DS + cs0)), d1 = lds_v4f32(ts + 4 * (T_DS + cs0 + 4));
    const float4 t0 = lds_v4f32(ts + 4 * (T_DT + cs0)), t1 = lds_v4f32(ts + 4 * (T_DT + cs0 + 4));
    const float ds[8] = {d0.x, d0.y, d0.z, d0.w, d1.x, d1.y, d1.z, d1.w};   // ds[k] = decay of step cs0+k+1
    const float dt[8] = {t0.x, t0.y, t0.z, t0.w, t1.x, t1.y, t1.z, t1.w};
    float v[8];
    float run = (row >= je) ? ex2(csi - lds_f32(ts + 4 * (T_CS + je))) : 0.f;
    v[7] = __uint_as_float(raw[8 * s + 7]) * (run * dt[7]);
#pragma unroll
    for (int k = 6; k >= 0; --k) {
      run = (cs0 + k == row) ? 1.f : run * ds[k];
      v[k] = __uint_as_float(raw[8 * s + k]) * (run * dt[k]);
    }
    st_shared_v4(dst + s * 2048, pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
  }
}
// rb: block row of the warp (warp-uniform); tm_row: TMEM address of (first lane of this warp's quarter, first
// source column); mrow: shared-memory address of this row's first 16 bytes in the plain 128x128 bf16 tile.
// One compact loop body for every block row (the code has to stay resident in the instruction cache while
// several groups run through it at different places); the two 16-column halves of the next block are
// requested as soon as the registers of the current ones are free.  The table (in shared memory) is read through the
// shared-memory pipe.
template <int NCH>
__device__ __forceinline__ void decay_row(int rb, int ch, uint32_t tm_row, const float* __restrict__ tab, int row, uint32_t mrow) {
  const uint32_t ts = smem_u32(tab);
  const float csi = lds_f32(ts + 4 * (T_CS + row));
  if (NCH == 1) {
    uint32_t a[16], b[16];
    tmem_ld16_issue(tm_row, a);
    tmem_ld16_issue(tm_row + 16, b);
#pragma unroll 1
    for (int cb = 0; cb < rb; ++cb) {
      const float rf = ex2(csi - lds_f32(ts + 4 * (T_CS + cb * 32 + 31)));
      const uint32_t cf = ts + 4 * (T_CF + cb * 32);
      const uint32_t dst = mrow + cb * 4 * 2048;
      tmem_ld_wait_2x16(a, b);
      decay_off_half(a, rf, cf, dst);
      tmem_ld16_issue(tm_row + (cb + 1) * 32, a);
      decay_off_half(b, rf, cf + 64, dst + 2 * 2048);
      tmem_ld16_issue(tm_row + (cb + 1) * 32 + 16, b);
    }
    tmem_ld_wait_2x16(a, b);
    decay_diag_half(a, ts, rb * 32, row, csi, mrow + rb * 4 * 2048);
    decay_diag_half(b, ts, rb * 32 + 16, row, csi, mrow + rb * 4 * 2048 + 2 * 2048);
  } else {
    // two threads per row: this one owns columns [16 ch, 16 ch + 16) of every block; two register sets so that
    // the load of the next block flies while the current one is worked on
    uint32_t a[16], b[16];
    const uint32_t tmc = tm_row + ch * 16;
    const uint32_t mr = mrow + ch * 2 * 2048;
    tmem_ld16_issue(tmc, a);
    int cb = 0;
#pragma unroll 1
    for (; cb + 1 < rb; cb += 2) {
      tmem_ld16_issue(tmc + (cb + 1) * 32, b);
      tmem_ld_wait_2x16(a, b);
      decay_off_half(a, ex2(csi - lds_f32(ts + 4 * (T_CS + cb * 32 + 31))), ts + 4 * (T_CF + cb * 32 + ch * 16), mr + cb * 4 * 2048);
      tmem_ld16_issue(tmc + (cb + 2) * 32, a);
      decay_off_half(b, ex2(csi - lds_f32(ts + 4 * (T_CS + cb * 32 + 63))), ts + 4 * (T_CF + cb * 32 + 32 + ch * 16), mr + (cb + 1) * 4 * 2048);
    }
    if (cb < rb) {   // one more block below the diagonal, then the diagonal block
      tmem_ld16_issue(tmc + (cb + 1) * 32, b);
      tmem_ld_wait_2x16(a, b);
      decay_off_half(a, ex2(csi - lds_f32(ts + 4 * (T_CS + cb * 32 + 31))), ts + 4 * (T_CF + cb * 32 + ch * 16), mr + cb * 4 * 2048);
      decay_diag_half(b, ts, rb * 32 + ch * 16, row, csi, mr + rb * 4 * 2048);
    } else {
      tmem_ld_wait_2x16(a, b);
      decay_diag_half(a, ts, rb * 32 + ch * 16, row, csi, mr + rb * 4 * 2048);
    }
  }
}

// Variant used by the one-tile-per-CTA kernels (all 16 warps meet at a CTA barrier per head anyway):
// one whole 32x32 block per thread-and-head, thread = (row, part = block column).
__device__ __forceinline__ void decay_mask_block(uint32_t tm_src, const float* __restrict__ tab, int row, int part,
                                                 int warp, uint32_t mtile) {
  const int rb = warp & 3, cb = part;   // both warp-uniform
  if (cb > rb) return;
  const int c0 = cb * 32;
  const uint32_t ts = smem_u32(tab);    // the table sits in shared memory: read it through the shared-memory pipe
  float v[32];
  tmem_ld32(tmem_addr(tm_src, rb * 32, c0), v);
  if (cb == rb) {
    float run = 0.f;
#pragma unroll
    for (int k4 = 28; k4 >= 0; k4 -= 4) {
      const float4 d = lds_v4f32(ts + 4 * (T_DS + c0 + k4)), t = lds_v4f32(ts + 4 * (T_DT + c0 + k4));   // T_DS[j] = decay of step j+1
      const float ds[4] = {d.x, d.y, d.z, d.w}, dt[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
      for (int q = 3; q >= 0; --q) {
        const int j = c0 + k4 + q;
        run = (j == row) ? 1.f : run * ds[q];
        v[k4 + q] = v[k4 + q] * run * dt[q];
      }
    }
  } else {
    const float rf = ex2(lds_f32(ts + 4 * (T_CS + row)) - lds_f32(ts + 4 * (T_CS + c0 + 31)));
#pragma unroll
    for (int k4 = 0; k4 < 32; k4 += 4) {
      const float4 f = lds_v4f32(ts + 4 * (T_CF + c0 + k4));
      v[k4] *= rf * f.x; v[k4 + 1] *= rf * f.y; v[k4 + 2] *= rf * f.z; v[k4 + 3] *= rf * f.w;
    }
  }
#pragma unroll
  for (int j8 = 0; j8 < 32; j8 += 8)
    st_shared_v4(mtile + plain_off(128, row, c0 + j8), pack_bf16(v[j8], v[j8 + 1]), pack_bf16(v[j8 + 2], v[j8 + 3]),
                 pack_bf16(v[j8 + 4], v[j8 + 5]), pack_bf16(v[j8 + 6], v[j8 + 7]));
}
// Accumulating variant for the one-tile dB / dC kernel: dC = sum_h W'_h B and dB = sum_h W'_h^T C are linear in W'_h, so
// the decayed, masked tiles of all heads of a group are added up in registers (fp32; thread = row x one 32-column block)
// and only their SUM goes to shared memory, once per tile.
__device__ __forceinline__ void decay_acc_block(uint32_t tm_src, const float* __restrict__ tab, int row, int part, int warp,
                                                float (&acc)[32]) {
  const int rb = warp & 3, cb = part;   // both warp-uniform
  if (cb > rb) return;
  const int c0 = cb * 32;
  const uint32_t ts = smem_u32(tab);
  float v[32];
  tmem_ld32(tmem_addr(tm_src, rb * 32, c0), v);
  if (cb == rb) {
    float run = 0.f;
#pragma unroll
    for (int k4 = 28; k4 >= 0; k4 -= 4) {
      const float4 d = lds_v4f32(ts + 4 * (T_DS + c0 + k4)), t = lds_v4f32(ts + 4 * (T_DT + c0 + k4));
      const float ds[4] = {d.x, d.y, d.z, d.w}, dt[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
      for (int q = 3; q >= 0; --q) {
        const int j = c0 + k4 + q;
        run = (j == row) ? 1.f : run * ds[q];
        acc[k4 + q] = fmaf(v[k4 + q], run * dt[q], acc[k4 + q]);
      }
    }
  } else {
    const float rf = ex2(lds_f32(ts + 4 * (T_CS + row)) - lds_f32(ts + 4 * (T_CS + c0 + 31)));
#pragma unroll
    for (int k4 = 0; k4 < 32; k4 += 4) {
      const float4 f = lds_v4f32(ts + 4 * (T_CF + c0 + k4));
      acc[k4] = fmaf(v[k4], rf * f.x, acc[k4]); acc[k4 + 1] = fmaf(v[k4 + 1], rf * f.y, acc[k4 + 1]);
      acc[k4 + 2] = fmaf(v[k4 + 2], rf * f.z, acc[k4 + 2]); acc[k4 + 3] = fmaf(v[k4 + 3], rf * f.w, acc[k4 + 3]);
    }
  }
}
__device__ __forceinline__ void store_acc_block(const float (&acc)[32], int row, int part, int warp, uint32_t mtile) {
  if (part > (warp & 3)) return;
#pragma unroll
  for (int j8 = 0; j8 < 32; j8 += 8)
    st_shared_v4(mtile + plain_off(128, row, part * 32 + j8), pack_bf16(acc[j8], acc[j8 + 1]), pack_bf16(acc[j8 + 2], acc[j8 + 3]),
                 pack_bf16(acc[j8 + 4], acc[j8 + 5]), pack_bf16(acc[j8 + 6], acc[j8 + 7]));
}
__device__ __forceinline__ void zero_upper_block(int row, int part, int warp, uint32_t mtile) {
  if (part <= (warp & 3)) return;
#pragma unroll
  for (int j8 = 0; j8 < 32; j8 += 8) st_shared_v4(mtile + plain_off(128, row, part * 32 + j8), 0u, 0u, 0u, 0u);
}

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const float2 a = unpack_bf16(v.x), b = unpack_bf16(v.y), c = unpack_bf16(v.z), d = unpack_bf16(v.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ uint4 pack8(const float (&o)[8]) {
  return make_uint4(pack_bf16(o[0], o[1]), pack_bf16(o[2], o[3]), pack_bf16(o[4], o[5]), pack_bf16(o[6], o[7]));
}

// Eight bf16 values (one 16-byte piece) times one fp32 factor, in packed bf16 arithmetic: the factor is split into a high
// and a low bf16 part, out = v * f_hi + v * f_lo with one fused multiply-add, so the factor itself is carried to ~16 bits and
// the result differs from an fp32 multiply followed by one rounding only by the rounding of the first product.  Two
// instructions per pair of values instead of unpack, two multiplies and a (quarter-rate) convert.
__device__ __forceinline__ uint4 scale8_bf16(const uint4& v, float f) {
  const __nv_bfloat16 fh = __float2bfloat16_rn(f);
  const __nv_bfloat16 fl = __float2bfloat16_rn(f - __bfloat162float(fh));
  const __nv_bfloat162 h2 = __halves2bfloat162(fh, fh), l2 = __halves2bfloat162(fl, fl);
  uint4 o;
  const __nv_bfloat162* in = reinterpret_cast<const __nv_bfloat162*>(&v);
  __nv_bfloat162* out = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
  for (int k = 0; k < 4; ++k) out[k] = __hfma2(in[k], l2, __hmul2(in[k], h2));
  return o;
}

// ---------------------------------------------------------------------------------------------
// chunk states (MODE 0: x, B, w = exp(cs_end-cs_l)*dt_l) and their backward twin (MODE 1: dy, C,
// w = exp(cs_l)).  grid = (nc, G, B).
template <int P, int N, int MODE>
__global__ void __launch_bounds__(TC_THREADS, 2) k_state_tc(Geo g, const __grid_constant__ CUtensorMap tmX,
                                                             const __grid_constant__ CUtensorMap tmB,
                                                             const float* __restrict__ tab, float* __restrict__ out,
                                                             int* __restrict__ status) {
  constexpr int NB = N / 64;       // 64-column boxes of the B/C tile
  constexpr int HT = 128 / P;      // heads per 128-row accumulator
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);   // 1 KB aligned, still known to be shared memory
  uint8_t* sB = smem;                          // NB boxes
  uint8_t* sX = smem + NB * BOX_BYTES;         // 2 boxes: the x tile, scaled in place (high bf16 part)
  uint8_t* sL = sX + 2 * BOX_BYTES;            // 2 boxes: low bf16 part of the scaled tile
  float* sTab = (float*)(sL + 2 * BOX_BYTES);  // [HT][TAB]
  float* sW = sTab + HT * TAB;                 // [HT][128]
  __shared__ __align__(8) uint64_t bar_b, bar_x, bar_mma;
  __shared__ uint32_t tmem_slot;
  __shared__ int s_abort;

  const int tid = threadIdx.x, warp = tid >> 5;
  if (tid == 0) s_abort = *(volatile int*)status;   // an earlier CTA gave up: drain the grid quickly
  __syncthreads();
  if (s_abort) return;
  const int c = blockIdx.x, grp = blockIdx.y, b = blockIdx.z;
  const int row = tid & 127, part = tid >> 7;
  if (tid == 0) {
    mbar_init(&bar_b, 1); mbar_init(&bar_x, 1); mbar_init(&bar_mma, 1);
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(&tmem_slot, N < 32 ? 32 : N);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = tmem_slot;
  Waiter w{status, false};

  const int MT = g.hpg * P / 128;             // accumulator tiles in this group
  const int col_base = grp * g.hpg * P;       // first (h,p) column of the group in x
  auto load_tile = [&](int mt) {              // thread 0 only
    mbar_expect_tx(&bar_x, 2 * BOX_BYTES + HT * TAB_BYTES);
    tma_load_3d(sX, &tmX, col_base + mt * 128, c * QT, b, &bar_x);
    tma_load_3d(sX + BOX_BYTES, &tmX, col_base + mt * 128 + 64, c * QT, b, &bar_x);
    bulk_load(sTab, tab + ((size_t)(b * g.nc + c) * g.H + grp * g.hpg + mt * HT) * TAB, HT * TAB_BYTES, &bar_x);
  };
  if (tid == 0) {
    mbar_expect_tx(&bar_b, NB * BOX_BYTES);
    for (int kb = 0; kb < NB; ++kb) tma_load_3d(sB + kb * BOX_BYTES, &tmB, grp * N + kb * 64, c * QT, b, &bar_b);
    load_tile(0);
    for (int mt = 1; mt < MT; ++mt) {   // later tiles: start them towards L2 now
      tma_prefetch_3d(&tmX, col_base + mt * 128, c * QT, b);
      tma_prefetch_3d(&tmX, col_base + mt * 128 + 64, c * QT, b);
      bulk_prefetch(tab + ((size_t)(b * g.nc + c) * g.H + grp * g.hpg + mt * HT) * TAB, HT * TAB_BYTES);
    }
  }
  uint32_t xphase = 0, mphase = 0;
  const uint32_t idesc = make_idesc(128, N, 1, 1);
  const uint64_t dX0 = desc_sw128_mn(smem_u32(sX), 0, 0, BOX_BYTES), dL0 = desc_sw128_mn(smem_u32(sL), 0, 0, BOX_BYTES),
                 dB0 = desc_sw128_mn(smem_u32(sB), 0, 0, BOX_BYTES);
  for (int mt = 0; mt < MT; ++mt) {
    const int h0 = grp * g.hpg + mt * HT;
    w.wait(&bar_x, xphase, 11);
    xphase ^= 1;
    for (int i = tid; i < HT * 128; i += TC_THREADS) {
      const float* t = sTab + (i >> 7) * TAB;
      const int l = i & 127;
      sW[i] = (MODE == 0) ? ex2(t[T_CS + 127] - t[T_CS + l]) * t[T_DT + l] : ex2(t[T_CS + l]);
    }
    __syncthreads();
    // scale the tile: 2 boxes x 128 rows x 8 chunks of 16 bytes.  The product w*x is split into a
    // high and a low bf16 part (two MMAs) so the chunk states keep ~16 mantissa bits: they feed
    // every later stage, and the per-chunk term of dA is a strongly cancelling sum over them.
#pragma unroll
    for (int r = 0; r < 2048 / TC_THREADS; ++r) {
      const int idx = tid + r * TC_THREADS;
      const int box = idx >> 10, l = (idx >> 3) & 127, pc = idx & 7;
      const int lc = (pc ^ l) & 7;
      const int hl = (box * 64 + lc * 8) / P;
      const float wv = sW[hl * 128 + l];
      const uint32_t off = box * BOX_BYTES + l * 128 + pc * 16;
      const uint32_t a = smem_u32(sX) + off;
      float f[8];
      unpack8(ld_shared_v4(a), f);
      uint32_t hi[4], lo[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float f0 = f[2 * k] * wv, f1 = f[2 * k + 1] * wv;
        hi[k] = pack_bf16(f0, f1);
        const float2 hf = unpack_bf16(hi[k]);
        lo[k] = pack_bf16(f0 - hf.x, f1 - hf.y);
      }
      st_shared_v4(a, hi[0], hi[1], hi[2], hi[3]);
      st_shared_v4(smem_u32(sL) + off, lo[0], lo[1], lo[2], lo[3]);
    }
    fence_async_smem();
    if (mt == 0) w.wait(&bar_b, 0, 12);
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)
        mma_bf16(tm, desc_adv(dX0, ks * 2048), desc_adv(dB0, ks * 2048), idesc, ks > 0);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)
        mma_bf16(tm, desc_adv(dL0, ks * 2048), desc_adv(dB0, ks * 2048), idesc, true);
      mma_commit(&bar_mma);
    }
    w.wait(&bar_mma, mphase, 13);
    mphase ^= 1;
    tc_fence_after();
    if (tid == 0 && mt + 1 < MT) load_tile(mt + 1);   // the tile buffers and the table are free again
    // epilogue: row = (head, p) of this tile, N / PARTS columns per thread
    float* o = out + (((size_t)(b * g.nc + c) * g.H + h0) * P + row) * N + part * (N / PARTS);
#pragma unroll
    for (int q = 0; q < N / PARTS / 16; ++q) {
      float v[16];
      tmem_ld16(tmem_addr(tm, (warp & 3) * 32, part * (N / PARTS) + q * 16), v);
#pragma unroll
      for (int j = 0; j < 16; j += 8)
        st_global_32B(o + q * 16 + j, make_uint4(__float_as_uint(v[j]), __float_as_uint(v[j + 1]), __float_as_uint(v[j + 2]), __float_as_uint(v[j + 3])),
                      make_uint4(__float_as_uint(v[j + 4]), __float_as_uint(v[j + 5]), __float_as_uint(v[j + 6]), __float_as_uint(v[j + 7])));
    }
    tc_fence_before();
    __syncthreads();
  }
  if (warp == 1) tmem_dealloc(tm, N < 32 ? 32 : N);
}

// ---------------------------------------------------------------------------------------------
// Persistent version of k_state_tc for dstate 64: one CTA per SM walks over (batch, chunk, group) items and their
// 128-row accumulator tiles.  Roles:
//   warp 17 (one lane)  producer: a four-deep ring of x tiles + the two table sections this kernel reads (TMA), so that
//                       about 100 KB of loads are in flight per SM all the time, and a two-deep ring of B (or C) tiles;
//   warps 0-15          scale the tile in place (high bf16 part) and write the low part to a second buffer, one 64-token
//                       half at a time, then store the PREVIOUS tile's accumulator;
//   warp 16 (one lane)  issues the MMAs of a half as soon as that half is scaled, into one of two TMEM accumulators.
// Every hand-over is a bounded mbarrier wait; a barrier is only ever waited on by a role that cannot fall two phases
// behind it (each completion needs that role's own next step).
template <int P, int N_>
struct PsCfg {
  static constexpr int N = N_, HT = 128 / P, NX = (N_ == 64) ? 4 : 3, NBX = N_ / 64;   // NBX: 64-column boxes of a B/C tile
  static constexpr int X_BYTES = 2 * BOX_BYTES;
  static constexpr int TBH = 256;                 // floats of a head's table that this kernel reads: the T_CS and T_DT sections
  static constexpr int TB_BYTES = HT * TBH * 4;
  static constexpr int W_MMA = 16, W_PROD = 17, THREADS = 18 * 32;
  static constexpr int B_BYTES = NBX * BOX_BYTES;
  static constexpr size_t SMEM = 1024 + NX * X_BYTES + X_BYTES + 2 * B_BYTES + NX * TB_BYTES;
  static_assert(T_CS == 0 && T_DT == 128, "the two sections must be the first 1 KB of a table");
};

template <int P, int N_, int MODE>
__global__ void __launch_bounds__(PsCfg<P, N_>::THREADS, 1) k_state_ps(Geo g, const __grid_constant__ CUtensorMap tmX,
                                                                   const __grid_constant__ CUtensorMap tmB,
                                                                   const float* __restrict__ tab, float* __restrict__ out,
                                                                   int* __restrict__ status) {
  using Cfg = PsCfg<P, N_>;
  constexpr int N = Cfg::N, HT = Cfg::HT, NX = Cfg::NX;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);   // 1 KB aligned, still known to be shared memory
  uint8_t* sX = smem;                                  // NX x {two 64-column boxes}: the tile, scaled in place (high part)
  uint8_t* sL = sX + NX * Cfg::X_BYTES;                // low bf16 part of the tile being multiplied
  uint8_t* sB = sL + Cfg::X_BYTES;                     // 2 x B (or C) tile of an item
  uint8_t* sTabs = sB + 2 * Cfg::B_BYTES;              // NX x the table sections of a tile's heads
  __shared__ __align__(8) uint64_t x_full[NX], x_free[NX], b_full[2], b_free[2], half_ready[2], h0_done, mma_done[2], acc_empty[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int s_abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) s_abort = *(volatile int*)status;
  __syncthreads();
  if (s_abort) return;
  if (tid == 0) {
    for (int i = 0; i < NX; ++i) { mbar_init(&x_full[i], 1); mbar_init(&x_free[i], 1); }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&b_full[i], 1); mbar_init(&b_free[i], 1); mbar_init(&half_ready[i], 16);
      mbar_init(&mma_done[i], 1); mbar_init(&acc_empty[i], 16);
    }
    mbar_init(&h0_done, 1);
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(&tmem_slot, 2 * N);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = tmem_slot;
  Waiter w{status, false};

  const int MT = g.hpg * P / 128;
  const int nitems = g.B * g.G * g.nc;
  const int my_items = (nitems - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
  const int total = my_items * MT;
  auto coords = [&](int n, int& b, int& grp, int& c) {   // this CTA's n-th item
    const int u = blockIdx.x + n * gridDim.x;
    c = u % g.nc;
    const int r = u / g.nc;
    grp = r % g.G;
    b = r / g.G;
  };

  if (warp == Cfg::W_PROD) {
    if (lane == 0) {
      int n = 0, mt = 0, b = 0, grp = 0, c = 0;
      for (int k = 0; k < total; ++k) {
        if (mt == 0) coords(n, b, grp, c);
        const int slot = k % NX;
        if (k >= NX) w.wait(&x_free[slot], ((k / NX) - 1) & 1, 14);
        const int col = grp * g.hpg * P + mt * 128;
        mbar_expect_tx(&x_full[slot], Cfg::X_BYTES + Cfg::TB_BYTES);
        tma_load_3d(sX + slot * Cfg::X_BYTES, &tmX, col, c * QT, b, &x_full[slot]);
        tma_load_3d(sX + slot * Cfg::X_BYTES + BOX_BYTES, &tmX, col + 64, c * QT, b, &x_full[slot]);
        const float* t0 = tab + ((size_t)(b * g.nc + c) * g.H + grp * g.hpg + mt * HT) * TAB;
        for (int hl = 0; hl < HT; ++hl)
          bulk_load(sTabs + slot * Cfg::TB_BYTES + hl * Cfg::TBH * 4, t0 + (size_t)hl * TAB, Cfg::TBH * 4, &x_full[slot]);
        if (mt == 0) {   // the item's B (or C) tile, after its first x tile so that this wait does not hold the x loads back
          if (n >= 2) w.wait(&b_free[n & 1], ((n >> 1) - 1) & 1, 15);
          mbar_expect_tx(&b_full[n & 1], Cfg::B_BYTES);
          for (int kb = 0; kb < Cfg::NBX; ++kb)
            tma_load_3d(sB + (n & 1) * Cfg::B_BYTES + kb * BOX_BYTES, &tmB, grp * N + kb * 64, c * QT, b, &b_full[n & 1]);
        }
        if (++mt == MT) { mt = 0; ++n; }
      }
    }
    __syncwarp();
  } else if (warp == Cfg::W_MMA) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc(128, N, 1, 1);
      const uint64_t dL0 = desc_sw128_mn(smem_u32(sL), 0, 0, BOX_BYTES);
      int n = 0, mt = 0;
      for (int k = 0; k < total; ++k) {
        const int slot = k % NX;
        const uint64_t dX0 = desc_sw128_mn(smem_u32(sX + slot * Cfg::X_BYTES), 0, 0, BOX_BYTES),
                       dB0 = desc_sw128_mn(smem_u32(sB + (n & 1) * Cfg::B_BYTES), 0, 0, BOX_BYTES);
        const uint32_t acc = tm + (k & 1) * N;
        if (mt == 0) w.wait(&b_full[n & 1], (n >> 1) & 1, 12);
        if (k >= 2) w.wait(&acc_empty[k & 1], ((k >> 1) - 1) & 1, 16);
        w.wait(&half_ready[0], k & 1, 17);
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) mma_bf16(acc, desc_adv(dX0, ks * 2048), desc_adv(dB0, ks * 2048), idesc, ks > 0);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) mma_bf16(acc, desc_adv(dL0, ks * 2048), desc_adv(dB0, ks * 2048), idesc, true);
        mma_commit(&h0_done);
        w.wait(&half_ready[1], k & 1, 18);
        tc_fence_after();
#pragma unroll
        for (int ks = 4; ks < 8; ++ks) mma_bf16(acc, desc_adv(dX0, ks * 2048), desc_adv(dB0, ks * 2048), idesc, true);
#pragma unroll
        for (int ks = 4; ks < 8; ++ks) mma_bf16(acc, desc_adv(dL0, ks * 2048), desc_adv(dB0, ks * 2048), idesc, true);
        mma_commit(&mma_done[k & 1]);
        mma_commit(&x_free[slot]);
        if (mt == MT - 1) mma_commit(&b_free[n & 1]);
        if (++mt == MT) { mt = 0; ++n; }
      }
    }
    __syncwarp();
  } else {
    const uint32_t ls = smem_u32(sL);
    auto scale_half = [&](int h, uint32_t xs, const float* tb) {   // rows 64 h .. 64 h + 63 of both boxes
      const int l = (tid >> 3) + 64 * h, pc = tid & 7;
      const int lc = (pc ^ l) & 7;
#pragma unroll
      for (int box = 0; box < 2; ++box) {
        const uint32_t t = smem_u32(tb) + ((box * 64 + lc * 8) / P) * Cfg::TBH * 4;   // shared-pipe reads of the table
        const float csl = lds_f32(t + 4 * (T_CS + l));
        const float wv = (MODE == 0) ? ex2(lds_f32(t + 4 * (T_CS + 127)) - csl) * lds_f32(t + 4 * (T_DT + l)) : ex2(csl);
        const uint32_t off = box * BOX_BYTES + l * 128 + pc * 16;
        float f[8];
        unpack8(ld_shared_v4(xs + off), f);
        uint32_t hi[4], lo[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float f0 = f[2 * q] * wv, f1 = f[2 * q + 1] * wv;
          hi[q] = pack_bf16(f0, f1);
          const float2 hf = unpack_bf16(hi[q]);
          lo[q] = pack_bf16(f0 - hf.x, f1 - hf.y);
        }
        st_shared_v4(xs + off, hi[0], hi[1], hi[2], hi[3]);
        st_shared_v4(ls + off, lo[0], lo[1], lo[2], lo[3]);
      }
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&half_ready[h]);
    };
    auto epilogue = [&](int k, int b, int grp, int c, int mt) {   // accumulator of tile k -> global
      const int h0 = grp * g.hpg + mt * HT;
      const int row = tid & 127, part = tid >> 7;
      float* o = out + (((size_t)(b * g.nc + c) * g.H + h0) * P + row) * N + part * (N / PARTS);
#pragma unroll
      for (int q = 0; q < N / PARTS / 16; ++q) {
        float v[16];
        tmem_ld16(tmem_addr(tm + (k & 1) * N, (warp & 3) * 32, part * (N / PARTS) + q * 16), v);
        if (q == N / PARTS / 16 - 1) {   // the accumulator is in registers: hand it back before the stores
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&acc_empty[k & 1]);
        }
#pragma unroll
        for (int j = 0; j < 16; j += 8)
          st_global_32B(o + q * 16 + j, make_uint4(__float_as_uint(v[j]), __float_as_uint(v[j + 1]), __float_as_uint(v[j + 2]), __float_as_uint(v[j + 3])),
                        make_uint4(__float_as_uint(v[j + 4]), __float_as_uint(v[j + 5]), __float_as_uint(v[j + 6]), __float_as_uint(v[j + 7])));
      }
    };
    int n = 0, mt = 0, b = 0, grp = 0, c = 0;           // tile k
    int pb = 0, pgrp = 0, pc_ = 0, pmt = 0;             // tile k - 1
    for (int k = 0; k < total; ++k) {
      if (mt == 0) coords(n, b, grp, c);
      const int slot = k % NX;
      const uint32_t xs = smem_u32(sX + slot * Cfg::X_BYTES);
      const float* tb = (const float*)(sTabs + slot * Cfg::TB_BYTES);
      w.wait(&x_full[slot], (k / NX) & 1, 11);
      if (k > 0) w.wait(&h0_done, (k - 1) & 1, 19);          // first half of the low-part buffer is free
      scale_half(0, xs, tb);
      if (k > 0) {                                           // tile k-1 is complete: second half free, accumulator ready
        w.wait(&mma_done[(k - 1) & 1], ((k - 1) >> 1) & 1, 13);
        tc_fence_after();
      }
      scale_half(1, xs, tb);
      if (k > 0) epilogue(k - 1, pb, pgrp, pc_, pmt);
      pb = b; pgrp = grp; pc_ = c; pmt = mt;
      if (++mt == MT) { mt = 0; ++n; }
    }
    w.wait(&mma_done[(total - 1) & 1], ((total - 1) >> 1) & 1, 13);
    tc_fence_after();
    epilogue(total - 1, pb, pgrp, pc_, pmt);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tm, 2 * N);
}

// ---------------------------------------------------------------------------------------------
// Chunk states AND the scan over chunks in one persistent kernel (dstate 64): k_state_ps with the work ordered so that
// one CTA walks the chunks of a (batch, group, 128-row tile) unit in scan order and keeps the running state of its
// 128 x 64 tile in registers (16 floats per thread).  The fp32 per-chunk states then never travel to memory and back
// between two kernels: the epilogue of chunk c writes the state ENTERING the chunk (fp32 for the backward pass, bf16 for
// the tensor-core scan kernels), then folds the chunk's own contribution in:  run = exp(sum of dt*A over c) * run + local_c.
//   MODE 0  forward:  units scan c = 0 .. nc-1 from `init` (or zero); `last` receives the final state.
//   MODE 1  backward: c = nc-1 .. 0 from `init` = the gradient w.r.t. the final state (or zero); the value written for
//           chunk c is the gradient w.r.t. the state LEAVING it (bf16 only: nothing reads an fp32 copy), and the epilogue
//           also emits per-warp partial sums of <dS_end_c, S_end_c> (the per-chunk term of the dt*A gradient, S_end_c read
//           from the forward pass's bf16 copy of the chunk-entry states, the fp32 final state for the last chunk), `nw` =
//           4 * P / 32 partials per (batch, chunk, head) in `sdot`;
//           `last` receives the gradient w.r.t. the initial state.
// Pipeline and barriers as in k_state_ps; the B (or C) tile now changes with every tile, so it has a ring of its own.
template <int P, int MODE>
struct PfCfg {
  // the backward kernel gives one slot of the x ring to the S_end tile (128 rows x 64: one 16 KB bf16 box, or for the last
  // chunk the fp32 final state as two swizzled 16 KB boxes)
  static constexpr int N = 64, HT = 128 / P, NX = MODE == 1 ? 3 : 4, NB = 3;
  static constexpr int X_BYTES = 2 * BOX_BYTES;
  static constexpr int TBH = 256;
  static constexpr int TB_BYTES = HT * TBH * 4;
  static constexpr int SE_BYTES = MODE == 1 ? 2 * BOX_BYTES : 0;
  static constexpr int W_MMA = 16, W_PROD = 17, W_PROD2 = 18, THREADS = (MODE == 1 ? 19 : 18) * 32;
  static constexpr int SDOT_NW = 4 * (P / 32);
  static constexpr size_t SMEM = 1024 + NX * X_BYTES + X_BYTES + NB * BOX_BYTES + SE_BYTES + NX * TB_BYTES;
};

struct StateScanArgs {
  const float* tab;
  float* st;            // [B,nc,H,P,N] fp32 out, optional
  void* st_bf;          // [B,nc,H,P,N] bf16 out
  const float* init;    // [B,H,P,N] fp32, optional
  float* last;          // [B,H,P,N] fp32 out, optional
  const void* fwd_prev_bf;  // MODE 1: bf16 copy of the forward pass's chunk-entry states (read through a tensor map)
  const float* fwd_fin;   // MODE 1: forward final state
  float* sdot;            // MODE 1: [B,nc,H,SDOT_NW]
};

template <int P, int MODE>
__global__ void __launch_bounds__(PfCfg<P, MODE>::THREADS, 1) k_state_scan_ps(Geo g, const __grid_constant__ CUtensorMap tmX,
                                                                              const __grid_constant__ CUtensorMap tmB,
                                                                              const __grid_constant__ CUtensorMap tmS,
                                                                              const __grid_constant__ CUtensorMap tmF,
                                                                              StateScanArgs a, int* __restrict__ status) {
  using Cfg = PfCfg<P, MODE>;
  constexpr int N = Cfg::N, HT = Cfg::HT, NX = Cfg::NX, NB = Cfg::NB;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);   // 1 KB aligned, still known to be shared memory
  uint8_t* sX = smem;                                  // NX x {two 64-column boxes}: the tile, scaled in place (high part)
  uint8_t* sL = sX + NX * Cfg::X_BYTES;                // low bf16 part of the tile being multiplied
  uint8_t* sB = sL + Cfg::X_BYTES;                     // NB x B (or C) tile
  uint8_t* sSE = sB + NB * BOX_BYTES;                  // MODE 1: S_end of the tile whose epilogue comes next (128B swizzle)
  uint8_t* sTabs = sSE + Cfg::SE_BYTES;                // NX x the table sections of a tile's heads
  __shared__ __align__(8) uint64_t x_full[NX], x_free[NX], b_full[NB], b_free[NB], half_ready[2], h0_done, mma_done[2], acc_empty[2],
      se_full, se_free;
  __shared__ uint32_t tmem_slot;
  __shared__ int s_abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) s_abort = *(volatile int*)status;
  __syncthreads();
  if (s_abort) return;
  if (tid == 0) {
    for (int i = 0; i < NX; ++i) { mbar_init(&x_full[i], 1); mbar_init(&x_free[i], 1); }
    for (int i = 0; i < NB; ++i) { mbar_init(&b_full[i], 1); mbar_init(&b_free[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&half_ready[i], 16); mbar_init(&mma_done[i], 1); mbar_init(&acc_empty[i], 16); }
    mbar_init(&h0_done, 1);
    mbar_init(&se_full, 1); mbar_init(&se_free, 16);
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(&tmem_slot, 128);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = tmem_slot;
  Waiter w{status, false};
  const bool want_sdot = MODE == 1 && a.sdot != nullptr;

  const int MT = g.hpg * P / 128;
  const int nunits = g.B * g.G * MT;
  const int my_units = (nunits - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
  const int total = my_units * g.nc;
  auto coords = [&](int n, int& b, int& grp, int& mt) {   // this CTA's n-th unit; neighbouring units share a B/C tile
    const int u = blockIdx.x + n * gridDim.x;
    mt = u % MT;
    const int r = u / MT;
    grp = r % g.G;
    b = r / g.G;
  };
  auto chunk_of = [&](int s) { return MODE == 0 ? s : g.nc - 1 - s; };

  if (warp == Cfg::W_PROD) {
    if (lane == 0) {
      int n = 0, sidx = 0, b = 0, grp = 0, mt = 0;
      for (int k = 0; k < total; ++k) {
        if (sidx == 0) coords(n, b, grp, mt);
        const int c = chunk_of(sidx);
        const int slot = k % NX, bs = k % NB;
        if (k >= NX) w.wait(&x_free[slot], ((k / NX) - 1) & 1, 14);
        const int col = grp * g.hpg * P + mt * 128;
        mbar_expect_tx(&x_full[slot], Cfg::X_BYTES + Cfg::TB_BYTES);
        tma_load_3d(sX + slot * Cfg::X_BYTES, &tmX, col, c * QT, b, &x_full[slot]);
        tma_load_3d(sX + slot * Cfg::X_BYTES + BOX_BYTES, &tmX, col + 64, c * QT, b, &x_full[slot]);
        const float* t0 = a.tab + ((size_t)(b * g.nc + c) * g.H + grp * g.hpg + mt * HT) * TAB;
        for (int hl = 0; hl < HT; ++hl)
          bulk_load(sTabs + slot * Cfg::TB_BYTES + hl * Cfg::TBH * 4, t0 + (size_t)hl * TAB, Cfg::TBH * 4, &x_full[slot]);
        if (k >= NB) w.wait(&b_free[bs], ((k / NB) - 1) & 1, 15);
        mbar_expect_tx(&b_full[bs], BOX_BYTES);
        tma_load_3d(sB + bs * BOX_BYTES, &tmB, grp * N, c * QT, b, &b_full[bs]);
        if (++sidx == g.nc) { sidx = 0; ++n; }
      }
    }
    __syncwarp();
  } else if (MODE == 1 && warp == Cfg::W_PROD2) {
    // second producer lane: the forward state leaving chunk c (= entering chunk c+1, or the final state), one tile ahead of
    // the epilogue that multiplies it with the running gradient
    if (lane == 0 && want_sdot) {
      int n = 0, sidx = 0, b = 0, grp = 0, mt = 0;
      for (int k = 0; k < total; ++k) {
        if (sidx == 0) coords(n, b, grp, mt);
        const int c = chunk_of(sidx);
        const int h0 = grp * g.hpg + mt * HT;
        if (k >= 1) w.wait(&se_free, (k - 1) & 1, 20);
        if (c + 1 >= g.nc) {   // the forward's final state: fp32, two boxes of 32 columns
          const int row0 = (b * g.H + h0) * P;
          mbar_expect_tx(&se_full, 2 * BOX_BYTES);
          tma_load_3d(sSE, &tmF, 0, row0, 0, &se_full);
          tma_load_3d(sSE + BOX_BYTES, &tmF, 32, row0, 0, &se_full);
        } else {               // the bf16 copy of the state entering chunk c + 1: one box of 64 columns
          mbar_expect_tx(&se_full, BOX_BYTES);
          tma_load_3d(sSE, &tmS, 0, ((b * g.nc + c + 1) * g.H + h0) * P, 0, &se_full);
        }
        if (++sidx == g.nc) { sidx = 0; ++n; }
      }
    }
    __syncwarp();
  } else if (warp == Cfg::W_MMA) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc(128, N, 1, 1);
      const uint64_t dL0 = desc_sw128_mn(smem_u32(sL), 0, 0, BOX_BYTES);
      for (int k = 0; k < total; ++k) {
        const int slot = k % NX, bs = k % NB;
        const uint64_t dX0 = desc_sw128_mn(smem_u32(sX + slot * Cfg::X_BYTES), 0, 0, BOX_BYTES),
                       dB0 = desc_sw128_mn(smem_u32(sB + bs * BOX_BYTES), 0, 0, BOX_BYTES);
        const uint32_t acc = tm + (k & 1) * 64;
        w.wait(&b_full[bs], (k / NB) & 1, 12);
        if (k >= 2) w.wait(&acc_empty[k & 1], ((k >> 1) - 1) & 1, 16);
        w.wait(&half_ready[0], k & 1, 17);
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) mma_bf16(acc, desc_adv(dX0, ks * 2048), desc_adv(dB0, ks * 2048), idesc, ks > 0);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) mma_bf16(acc, desc_adv(dL0, ks * 2048), desc_adv(dB0, ks * 2048), idesc, true);
        mma_commit(&h0_done);
        w.wait(&half_ready[1], k & 1, 18);
        tc_fence_after();
#pragma unroll
        for (int ks = 4; ks < 8; ++ks) mma_bf16(acc, desc_adv(dX0, ks * 2048), desc_adv(dB0, ks * 2048), idesc, true);
#pragma unroll
        for (int ks = 4; ks < 8; ++ks) mma_bf16(acc, desc_adv(dL0, ks * 2048), desc_adv(dB0, ks * 2048), idesc, true);
        mma_commit(&mma_done[k & 1]);
        mma_commit(&x_free[slot]);
        mma_commit(&b_free[bs]);
      }
    }
    __syncwarp();
  } else {
    const uint32_t ls = smem_u32(sL);
    const int row = tid & 127, part = tid >> 7;
    auto scale_half = [&](int h, uint32_t xs, const float* tb) {   // rows 64 h .. 64 h + 63 of both boxes
      const int l = (tid >> 3) + 64 * h, pc = tid & 7;
      const int lc = (pc ^ l) & 7;
#pragma unroll
      for (int box = 0; box < 2; ++box) {
        const uint32_t t = smem_u32(tb) + ((box * 64 + lc * 8) / P) * Cfg::TBH * 4;   // shared-pipe reads of the table
        const float csl = lds_f32(t + 4 * (T_CS + l));
        const float wv = (MODE == 0) ? ex2(lds_f32(t + 4 * (T_CS + 127)) - csl) * lds_f32(t + 4 * (T_DT + l)) : ex2(csl);
        const uint32_t off = box * BOX_BYTES + l * 128 + pc * 16;
        float f[8];
        unpack8(ld_shared_v4(xs + off), f);
        uint32_t hi[4], lo[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float f0 = f[2 * q] * wv, f1 = f[2 * q + 1] * wv;
          hi[q] = pack_bf16(f0, f1);
          const float2 hf = unpack_bf16(hi[q]);
          lo[q] = pack_bf16(f0 - hf.x, f1 - hf.y);
        }
        st_shared_v4(xs + off, hi[0], hi[1], hi[2], hi[3]);
        st_shared_v4(ls + off, lo[0], lo[1], lo[2], lo[3]);
      }
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&half_ready[h]);
    };
    float run[16];          // running state of this thread's (row, 16 columns)
    struct Tile { int b, grp, mt, s; };
    auto elem = [&](const Tile& t) {   // offset of this thread's 16 columns inside a [.., H, P, N] state
      return ((size_t)(t.grp * g.hpg + t.mt * HT) * P + row) * N + part * 16;
    };
    auto epilogue = [&](int k, const Tile& t, float dec) {
      const int c = chunk_of(t.s);
      const size_t e = elem(t), bstate = (size_t)t.b * g.H * P * N;
      if (t.s == 0) {
        if (a.init) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float4 v4 = *reinterpret_cast<const float4*>(a.init + bstate + e + 4 * j);
            run[4 * j] = v4.x; run[4 * j + 1] = v4.y; run[4 * j + 2] = v4.z; run[4 * j + 3] = v4.w;
          }
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) run[j] = 0.f;
        }
      }
      float v[16];
      tmem_ld16(tmem_addr(tm + (k & 1) * 64, (warp & 3) * 32, part * 16), v);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[k & 1]);
      const size_t o = (size_t)(t.b * g.nc + c) * g.H * P * N + e;
      if (a.st) {
#pragma unroll
        for (int j = 0; j < 16; j += 8)
          st_global_32B(a.st + o + j, make_uint4(__float_as_uint(run[j]), __float_as_uint(run[j + 1]), __float_as_uint(run[j + 2]), __float_as_uint(run[j + 3])),
                        make_uint4(__float_as_uint(run[j + 4]), __float_as_uint(run[j + 5]), __float_as_uint(run[j + 6]), __float_as_uint(run[j + 7])));
      }
      st_global_32B((bf16*)a.st_bf + o,
                    make_uint4(pack_bf16(run[0], run[1]), pack_bf16(run[2], run[3]), pack_bf16(run[4], run[5]), pack_bf16(run[6], run[7])),
                    make_uint4(pack_bf16(run[8], run[9]), pack_bf16(run[10], run[11]), pack_bf16(run[12], run[13]), pack_bf16(run[14], run[15])));
      if (want_sdot) {
        w.wait(&se_full, k & 1, 21);
        float d = 0.f;
        if (c + 1 >= g.nc) {   // block-uniform: the final state, fp32
          const uint32_t sb = smem_u32(sSE) + (part >> 1) * BOX_BYTES;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint4 u = ld_shared_v4(sb + sw128_off(row, (part & 1) * 4 + j));
            d += run[4 * j] * __uint_as_float(u.x) + run[4 * j + 1] * __uint_as_float(u.y) + run[4 * j + 2] * __uint_as_float(u.z) +
                 run[4 * j + 3] * __uint_as_float(u.w);
          }
        } else {               // the bf16 copy: this thread's 16 columns are two 16-byte pieces of its row
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const uint4 u = ld_shared_v4(smem_u32(sSE) + sw128_off(row, part * 2 + j));
            const uint32_t q[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
              d += run[8 * j + 2 * i] * __uint_as_float(q[i] << 16) + run[8 * j + 2 * i + 1] * __uint_as_float(q[i] & 0xffff0000u);
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&se_free);
#pragma unroll
        for (int off = 16; off; off >>= 1) d += __shfl_xor_sync(0xffffffffu, d, off);
        if (lane == 0) {
          const int q = warp & 3;                                  // 32-row quarter of the tile
          const int h = t.grp * g.hpg + t.mt * HT + (q * 32) / P;
          const int slot = part * (P / 32) + q % (P / 32);
          a.sdot[((size_t)(t.b * g.nc + c) * g.H + h) * Cfg::SDOT_NW + slot] = d;
        }
      }
#pragma unroll
      for (int j = 0; j < 16; ++j) run[j] = fmaf(dec, run[j], v[j]);
      if (t.s == g.nc - 1 && a.last) {
#pragma unroll
        for (int j = 0; j < 16; j += 8)
          st_global_32B(a.last + bstate + e + j, make_uint4(__float_as_uint(run[j]), __float_as_uint(run[j + 1]), __float_as_uint(run[j + 2]), __float_as_uint(run[j + 3])),
                        make_uint4(__float_as_uint(run[j + 4]), __float_as_uint(run[j + 5]), __float_as_uint(run[j + 6]), __float_as_uint(run[j + 7])));
      }
    };
    Tile cur{0, 0, 0, 0}, prev{0, 0, 0, 0};
    int n = 0;
    float dec_prev = 0.f;
    for (int k = 0; k < total; ++k) {
      if (cur.s == 0) coords(n, cur.b, cur.grp, cur.mt);
      const int slot = k % NX;
      const uint32_t xs = smem_u32(sX + slot * Cfg::X_BYTES);
      const float* tb = (const float*)(sTabs + slot * Cfg::TB_BYTES);
      w.wait(&x_full[slot], (k / NX) & 1, 11);
      const float dec = ex2(lds_f32(smem_u32(tb) + 4 * ((row / P) * Cfg::TBH + T_CS + 127)));   // decay over the whole chunk, for this tile's epilogue
      if (k > 0) w.wait(&h0_done, (k - 1) & 1, 19);            // first half of the low-part buffer is free
      scale_half(0, xs, tb);
      if (k > 0) {                                             // tile k-1 is complete: second half free, accumulator ready
        w.wait(&mma_done[(k - 1) & 1], ((k - 1) >> 1) & 1, 13);
        tc_fence_after();
      }
      scale_half(1, xs, tb);
      if (k > 0) epilogue(k - 1, prev, dec_prev);
      prev = cur;
      dec_prev = dec;
      if (++cur.s == g.nc) { cur.s = 0; ++n; }
    }
    w.wait(&mma_done[(total - 1) & 1], ((total - 1) >> 1) & 1, 13);
    tc_fence_after();
    epilogue(total - 1, prev, dec_prev);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tm, 128);
}

// ---------------------------------------------------------------------------------------------
// chunk_scan family.  grid = (nc, G, B).  G = C B^T (128x128, TMEM) once per CTA, then per head
// the masked, decayed matrix M_h[i,j] = G[i,j] exp(cs_i-cs_j) dt_j (j <= i) goes to shared
// memory as bf16 and feeds
//   MODE 0 (forward)            Y  = M_h X_h   (+) exp(cs_i) C S_prev^T      -> y (+ D x, gate)
//   MODE 1 (backward, recompute) the same Y, epilogue instead forms dz / pre-gate dy and the
//                                row sums  dcsp[i] = sum_p dy*Y,  ddot[i] = sum_p dy*x
//   MODE 2 (backward, dx)        U' = M_h^T dY_h (+) dt_j exp(cs_end-cs_j) B dS_end^T
//                                dx = D dy + U',  ddtd[j] = sum_p x*U' / dt_j
// The state block (tmS) is the bf16 copy of S_prev (modes 0,1) or dS_end (mode 2).
// IBUF = 2: the inputs of head block k+1 load while block k computes; IBUF = 1: they are
// requested as soon as block k's epilogue has copied what it needs into registers.
// Two CTAs per SM at dstate 64 (a CTA is a chain of phases that meet at CTA-wide barriers, and a second resident CTA
// fills the gaps), one at dstate 128.  These are the kernels of the one-tile arm (SSD_ALGO_TENSOR_ONETILE); the default
// path runs k_scan_ws at both state widths.
template <int P, int N, int IBUF, int MODE>
__global__ void __launch_bounds__(TC_THREADS, (N <= 64) ? 2 : 1)
k_scan_tc(Geo g, const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmDY,
          const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmC,
          const __grid_constant__ CUtensorMap tmS, const float* __restrict__ tab, const float* __restrict__ D,
          const bf16* __restrict__ z, bf16* __restrict__ y, bf16* __restrict__ dypb, bf16* __restrict__ dz,
          bf16* __restrict__ dx, float* __restrict__ rs0, float* __restrict__ rs1, int* __restrict__ status) {
  constexpr int NB = N / 64;
  constexpr int HB = 64 / P;                   // heads per 64-column box
  constexpr int NBOX = (MODE == 0) ? 1 : 2;    // sequence boxes per head block: x (and dy)
  constexpr int IN_BYTES = NBOX * BOX_BYTES + NB * SBOX_BYTES + HB * TAB_BYTES;
  constexpr uint32_t TM_COLS = 256;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);   // 1 KB aligned, still known to be shared memory
  uint8_t* sKeep = smem;                       // NB boxes kept for the whole CTA: C (modes 0,1) or B (mode 2)
  uint8_t* sBM = sKeep + NB * BOX_BYTES;       // the other tile (NB boxes), later the 32 KB M_h tile
  uint8_t* sIn = sBM + 2 * BOX_BYTES;          // IBUF x {x [, dy], state boxes, tables}
  float* sRed = (float*)(sIn + IBUF * IN_BYTES);  // [2][PARTS][128] partial row sums (modes 1, 2)
  __shared__ __align__(8) uint64_t bar_cb, bar_in[2], bar_mma;
  __shared__ uint32_t tmem_slot;
  __shared__ int s_abort;

  const int tid = threadIdx.x, warp = tid >> 5;
  if (tid == 0) s_abort = *(volatile int*)status;   // an earlier CTA gave up: drain the grid quickly
  __syncthreads();
  if (s_abort) return;
  const int c = blockIdx.x, grp = blockIdx.y, b = blockIdx.z;
  const int row = tid & 127, part = tid >> 7;
  if (tid == 0) {
    mbar_init(&bar_cb, 1); mbar_init(&bar_in[0], 1); mbar_init(&bar_in[1], 1); mbar_init(&bar_mma, 1);
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(&tmem_slot, TM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = tmem_slot;
  const uint32_t tmG = tm, tmYd = tm + 128, tmYo = tm + 192;
  Waiter w{status, false};

  const int nblk = g.hpg / HB;
  const int col_base = grp * g.hpg * P;
  auto load_block = [&](int blk, int ib) {    // thread 0 only
    uint8_t* dst = sIn + ib * IN_BYTES;
    const int h0 = grp * g.hpg + blk * HB;
    mbar_expect_tx(&bar_in[ib], IN_BYTES);
    tma_load_3d(dst, &tmX, col_base + blk * 64, c * QT, b, &bar_in[ib]);
    if (NBOX == 2) tma_load_3d(dst + BOX_BYTES, &tmDY, col_base + blk * 64, c * QT, b, &bar_in[ib]);
    for (int kb = 0; kb < NB; ++kb)
      tma_load_3d(dst + NBOX * BOX_BYTES + kb * SBOX_BYTES, &tmS, kb * 64, h0 * P, b * g.nc + c, &bar_in[ib]);
    bulk_load(dst + NBOX * BOX_BYTES + NB * SBOX_BYTES, tab + ((size_t)(b * g.nc + c) * g.H + h0) * TAB, HB * TAB_BYTES,
              &bar_in[ib]);
  };
  if (tid == 0) {
    mbar_expect_tx(&bar_cb, 2 * NB * BOX_BYTES);
    for (int kb = 0; kb < NB; ++kb) {
      tma_load_3d(sKeep + kb * BOX_BYTES, (MODE == 2) ? &tmB : &tmC, grp * N + kb * 64, c * QT, b, &bar_cb);
      tma_load_3d(sBM + kb * BOX_BYTES, (MODE == 2) ? &tmC : &tmB, grp * N + kb * 64, c * QT, b, &bar_cb);
    }
    load_block(0, 0);
    if (IBUF == 2 && nblk > 1) load_block(1, 1);
    for (int blk = IBUF; blk < nblk; ++blk) {   // later blocks: start them towards L2 now
      const int h0 = grp * g.hpg + blk * HB;
      tma_prefetch_3d(&tmX, col_base + blk * 64, c * QT, b);
      if (NBOX == 2) tma_prefetch_3d(&tmDY, col_base + blk * 64, c * QT, b);
      for (int kb = 0; kb < NB; ++kb) tma_prefetch_3d(&tmS, kb * 64, h0 * P, b * g.nc + c);
      bulk_prefetch(tab + ((size_t)(b * g.nc + c) * g.H + h0) * TAB, HB * TAB_BYTES);
    }
  }
  uint32_t inphase[2] = {0, 0}, mphase = 0;
  w.wait(&bar_cb, 0, 21);
  if (tid == 0) {
    tc_fence_after();
    const uint32_t idG = make_idesc(128, 128, 0, 0);
    const uint64_t dc = desc_sw128_k(smem_u32((MODE == 2) ? sBM : sKeep), 0), db = desc_sw128_k(smem_u32((MODE == 2) ? sKeep : sBM), 0);
#pragma unroll
    for (int kb = 0; kb < NB; ++kb)
#pragma unroll
      for (int ks = 0; ks < 4; ++ks)
        mma_bf16(tmG, desc_adv(dc, kb * BOX_BYTES + ks * 32), desc_adv(db, kb * BOX_BYTES + ks * 32), idG, (kb | ks) > 0);
    mma_commit(&bar_mma);
  }
  w.wait(&bar_mma, mphase, 22);
  mphase ^= 1;
  tc_fence_after();
  zero_upper_block(row, part, warp, smem_u32(sBM));   // the B/C tile is dead; M_h never writes these blocks

  const uint32_t idY = make_idesc(128, P, (MODE == 2) ? 1 : 0, 1), idO = make_idesc(128, 64, 0, 0);
  // descriptors of the tiles that never move (only thread 0 uses them)
  const uint64_t dM0 = (MODE == 2) ? desc_plain_mn(smem_u32(sBM), 128, 0, 0) : desc_plain_k(smem_u32(sBM), 128, 0);
  constexpr uint32_t M_STEP = (MODE == 2) ? 256 : 4096;   // bytes per K step of 16 in the M_h tile
  const uint64_t dK0 = desc_sw128_k(smem_u32(sKeep), 0);
  const int t_row = c * QT + row;
  const int hl_e = (part * 16) / P;            // head (inside the block) of this thread's epilogue columns
  for (int blk = 0; blk < nblk; ++blk) {
    const int ib = (IBUF == 2) ? (blk & 1) : 0;
    uint8_t* xt = sIn + ib * IN_BYTES;                    // x box
    uint8_t* dyt = xt + (NBOX - 1) * BOX_BYTES;           // dy box (modes 1, 2)
    uint8_t* st = xt + NBOX * BOX_BYTES;                  // state boxes
    const float* tb = (const float*)(st + NB * SBOX_BYTES);   // [HB][TAB]
    const int h0 = grp * g.hpg + blk * HB;
    const int h_e = h0 + hl_e;
    const float Dh = D ? __ldg(D + h_e) : 0.f;            // requested now, used in the epilogue
    w.wait(&bar_in[ib], inphase[ib], 23);
    inphase[ib] ^= 1;
    for (int hl = 0; hl < HB; ++hl) {
      decay_mask_block(tmG, tb + hl * TAB, row, part, warp, smem_u32(sBM));
      fence_async_smem();
      tc_fence_before();
      __syncthreads();
      if (tid == 0) {
        tc_fence_after();
        const uint64_t dO0 = desc_sw128_mn(smem_u32((MODE == 2) ? dyt : xt), 0, hl * P * 2, 16);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          mma_bf16(tmYd + hl * P, desc_adv(dM0, ks * M_STEP), desc_adv(dO0, ks * 2048), idY, ks > 0);
        if (hl == 0) {
          const uint64_t dS0 = desc_sw128_k(smem_u32(st), 0);
#pragma unroll
          for (int kb = 0; kb < NB; ++kb)
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)
              mma_bf16(tmYo, desc_adv(dK0, kb * BOX_BYTES + ks * 32), desc_adv(dS0, kb * SBOX_BYTES + ks * 32), idO,
                       (kb | ks) > 0);
        }
        mma_commit(&bar_mma);
      }
      w.wait(&bar_mma, mphase, 24);
      mphase ^= 1;
      tc_fence_after();
    }
    // ---- epilogue for the HB heads of this block: this thread has 64/PARTS = 16 of the 64 columns.
    // Copy what is needed from the input buffers into registers first, so the buffers can be refilled.
    uint4 xv[2], dv[2];
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      xv[q] = ld_shared_v4(smem_u32(xt) + sw128_off(row, part * 2 + q));
      dv[q] = (MODE != 0) ? ld_shared_v4(smem_u32(dyt) + sw128_off(row, part * 2 + q)) : make_uint4(0u, 0u, 0u, 0u);
    }
    const float cs_r = tb[hl_e * TAB + T_CS + row], dt_r = tb[hl_e * TAB + T_DT + row];
    // off-diagonal scale: exp(cs_i) for Y, dt_j exp(cs_end - cs_j) for U'
    const float osc = (MODE == 2) ? dt_r * ex2(tb[hl_e * TAB + T_CS + 127] - cs_r) : ex2(cs_r);
    if (IBUF == 1) {
      __syncthreads();
      if (tid == 0 && blk + 1 < nblk) load_block(blk + 1, 0);
    }
    float s0 = 0.f, s1 = 0.f;
    {
      float yd[16], yo[16];
      tmem_ld16(tmem_addr(tmYd, (warp & 3) * 32, part * 16), yd);
      tmem_ld16(tmem_addr(tmYo, (warp & 3) * 32, part * 16), yo);
      const long long colo = (long long)h0 * P + part * 16;
      const bf16* zp = z ? z + b * g.zsb + (long long)t_row * g.zsl + colo : nullptr;
      const size_t dense = ((size_t)b * g.L + t_row) * g.H * P + colo;
      uint4 ov[2];
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        const int k8 = q * 8;
        float xs[8], acc[8], zs[8], dys[8], o[8];
        unpack8(xv[q], xs);
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[k] = yd[k8 + k] + osc * yo[k8 + k];
        if (z) unpack8(*reinterpret_cast<const uint4*>(zp + k8), zs);
        if (MODE != 0) unpack8(dv[q], dys);
        if (MODE == 0) {
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            o[k] = acc[k] + Dh * xs[k];
            if (z) o[k] *= zs[k] * sigmoidf_(zs[k]);
          }
          ov[q] = pack8(o);
        } else if (MODE == 1) {
          float dp[8];
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            float dyv = dys[k];
            if (z) {
              const float sg = 1.f / (1.f + __expf(-zs[k]));
              o[k] = dyv * (acc[k] + Dh * xs[k]) * sg * (1.f + zs[k] * (1.f - sg));   // dz
              dyv *= zs[k] * sg;
            }
            dp[k] = dyv;
            s0 = fmaf(dyv, acc[k], s0);
            s1 = fmaf(dyv, xs[k], s1);
          }
          if (z) {
            *reinterpret_cast<uint4*>(dz + dense + k8) = pack8(o);
            *reinterpret_cast<uint4*>(dypb + dense + k8) = pack8(dp);
          }
        } else {
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            o[k] = acc[k] + Dh * dys[k];
            s0 = fmaf(xs[k], acc[k], s0);
          }
          ov[q] = pack8(o);
        }
      }
      if (MODE == 0) st_global_32B(y + b * g.ysb + (long long)t_row * g.ysl + colo, ov[0], ov[1]);
      if (MODE == 2) st_global_32B(dx + dense, ov[0], ov[1]);
      if (MODE != 0) {   // row sums: P/16 threads share a (head, row); combine through shared memory
        sRed[part * 128 + row] = s0;
        if (MODE == 1) sRed[(PARTS + part) * 128 + row] = s1;
      }
    }
    tc_fence_before();
    __syncthreads();
    if (MODE != 0 && (part % (P / 16)) == 0) {
      float t0 = 0.f, t1 = 0.f;
#pragma unroll
      for (int k = 0; k < P / 16; ++k) {
        t0 += sRed[(part + k) * 128 + row];
        if (MODE == 1) t1 += sRed[(PARTS + part + k) * 128 + row];
      }
      const size_t co = ((size_t)(b * g.H + h_e) * g.nc + c) * QT + row;
      if (MODE == 1) {
        rs0[co] = t0;   // dcsp
        rs1[co] = t1;   // ddot
      } else {
        rs0[co] = dt_r > 0.f ? t0 / dt_r : 0.f;   // ddtd
      }
    }
    if (IBUF == 2 && tid == 0 && blk + 2 < nblk) load_block(blk + 2, ib);
  }
  if (warp == 1) tmem_dealloc(tm, TM_COLS);
}

// ---------------------------------------------------------------------------------------------
// Backward chunk_scan, ungated case, one tile per CTA (dstate 128): the recompute pass (MODE 1) and the dx pass (MODE 2) of
// k_scan_tc share G and every M_h, so this kernel forms G once and does both from one decay pass per head:
//   Y  = M_h X_h    (+) exp(cs_i) C S_prev^T                   -> dcsp[i] = sum_p dy*Y, ddot[i] = sum_p dy*x
//   U' = M_h^T dY_h (+) dt_j exp(cs_end-cs_j) B dS_end^T       -> dx = D dy + U', ddtd[j] = sum_p x*U' / dt_j
// grid = (nc, G, B), 512 threads, one CTA per SM.  TMEM: G (128) + {Y, Y_off, U, U_off} (4 x 64) of 512 columns.
template <int P, int N>
__global__ void __launch_bounds__(TC_THREADS, 1)
k_bwd_tc(Geo g, const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmDY,
         const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmC,
         const __grid_constant__ CUtensorMap tmS, const __grid_constant__ CUtensorMap tmDS, const float* __restrict__ tab,
         const float* __restrict__ D, bf16* __restrict__ dx, float* __restrict__ dcsp, float* __restrict__ ddot,
         float* __restrict__ ddtd, int* __restrict__ status) {
  constexpr int NB = N / 64;
  constexpr int HB = 64 / P;                   // heads per 64-column box
  // x box, dy box and tables of a head block: two sets (the next block's is requested a whole block ahead); the S_prev and
  // dS_end boxes: one set, refilled as soon as the block's products have completed
  constexpr int XSET = 2 * BOX_BYTES + HB * TAB_BYTES;
  constexpr int ST_BYTES = 2 * NB * SBOX_BYTES;
  constexpr uint32_t TM_COLS = 512;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);   // 1 KB aligned, still known to be shared memory
  uint8_t* sC = smem;                          // NB boxes, kept for the whole CTA (state term of Y)
  uint8_t* sB = sC + NB * BOX_BYTES;           // NB boxes, kept for the whole CTA (state term of U')
  uint8_t* sM = sB + NB * BOX_BYTES;           // the 32 KB M_h tile
  uint8_t* sXset = sM + 2 * BOX_BYTES;         // 2 x {x, dy, tables}
  uint8_t* stS = sXset + 2 * XSET;             // S_prev boxes
  uint8_t* stDS = stS + NB * SBOX_BYTES;       // dS_end boxes
  float* sRed = (float*)(stDS + NB * SBOX_BYTES);      // [3][PARTS][128] partial row sums
  __shared__ __align__(8) uint64_t bar_cb, bar_x[2], bar_st, bar_mma, bar_g;
  __shared__ uint32_t tmem_slot;
  __shared__ int s_abort;

  const int tid = threadIdx.x, warp = tid >> 5;
  if (tid == 0) s_abort = *(volatile int*)status;   // an earlier CTA gave up: drain the grid quickly
  __syncthreads();
  if (s_abort) return;
  const int c = blockIdx.x, grp = blockIdx.y, b = blockIdx.z;
  const int row = tid & 127, part = tid >> 7;
  if (tid == 0) {
    mbar_init(&bar_cb, 1); mbar_init(&bar_x[0], 1); mbar_init(&bar_x[1], 1); mbar_init(&bar_st, 1);
    mbar_init(&bar_mma, 4); mbar_init(&bar_g, 1);
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(&tmem_slot, TM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = tmem_slot;
  const uint32_t tmG = tm, tmYd = tm + 128, tmYo = tm + 192, tmUd = tm + 256, tmUo = tm + 320;
  Waiter w{status, false};

  const int nblk = g.hpg / HB;
  const int col_base = grp * g.hpg * P;
  uint8_t* xt = sXset;
  uint8_t* dyt = xt + BOX_BYTES;
  const float* tb = (const float*)(dyt + BOX_BYTES);   // [HB][TAB]
  auto load_xset = [&](int blk) {     // thread 0 only
    const int h0 = grp * g.hpg + blk * HB;
    uint8_t* set = sXset + (blk & 1) * XSET;
    uint64_t* bar = &bar_x[blk & 1];
    mbar_expect_tx(bar, XSET);
    tma_load_3d(set, &tmX, col_base + blk * 64, c * QT, b, bar);
    tma_load_3d(set + BOX_BYTES, &tmDY, col_base + blk * 64, c * QT, b, bar);
    bulk_load(set + 2 * BOX_BYTES, tab + ((size_t)(b * g.nc + c) * g.H + h0) * TAB, HB * TAB_BYTES, bar);
  };
  auto load_states = [&](int blk) {   // thread 0 only
    const int h0 = grp * g.hpg + blk * HB;
    mbar_expect_tx(&bar_st, ST_BYTES);
    for (int kb = 0; kb < NB; ++kb) {
      tma_load_3d(stS + kb * SBOX_BYTES, &tmS, kb * 64, h0 * P, b * g.nc + c, &bar_st);
      tma_load_3d(stDS + kb * SBOX_BYTES, &tmDS, kb * 64, h0 * P, b * g.nc + c, &bar_st);
    }
  };
  if (tid == 0) {
    mbar_expect_tx(&bar_cb, 2 * NB * BOX_BYTES);
    for (int kb = 0; kb < NB; ++kb) {
      tma_load_3d(sC + kb * BOX_BYTES, &tmC, grp * N + kb * 64, c * QT, b, &bar_cb);
      tma_load_3d(sB + kb * BOX_BYTES, &tmB, grp * N + kb * 64, c * QT, b, &bar_cb);
    }
    load_xset(0);
    load_states(0);
    for (int blk = 1; blk < nblk; ++blk) {   // later blocks: start them towards L2 now
      const int h0 = grp * g.hpg + blk * HB;
      tma_prefetch_3d(&tmX, col_base + blk * 64, c * QT, b);
      tma_prefetch_3d(&tmDY, col_base + blk * 64, c * QT, b);
      for (int kb = 0; kb < NB; ++kb) {
        tma_prefetch_3d(&tmS, kb * 64, h0 * P, b * g.nc + c);
        tma_prefetch_3d(&tmDS, kb * 64, h0 * P, b * g.nc + c);
      }
      bulk_prefetch(tab + ((size_t)(b * g.nc + c) * g.H + h0) * TAB, HB * TAB_BYTES);
    }
  }
  uint32_t mphase = 0;
  zero_upper_block(row, part, warp, smem_u32(sM));   // M_h never writes these blocks
  w.wait(&bar_cb, 0, 21);
  if (tid == 0) {
    tc_fence_after();
    const uint32_t idG = make_idesc(128, 128, 0, 0);
    const uint64_t dc = desc_sw128_k(smem_u32(sC), 0), db = desc_sw128_k(smem_u32(sB), 0);
#pragma unroll
    for (int kb = 0; kb < NB; ++kb)
#pragma unroll
      for (int ks = 0; ks < 4; ++ks)
        mma_bf16(tmG, desc_adv(dc, kb * BOX_BYTES + ks * 32), desc_adv(db, kb * BOX_BYTES + ks * 32), idG, (kb | ks) > 0);
    mma_commit(&bar_g);
  }
  w.wait(&bar_g, 0, 22);
  tc_fence_after();

  const uint32_t idY = make_idesc(128, P, 0, 1), idU = make_idesc(128, P, 1, 1), idO = make_idesc(128, 64, 0, 0);
  const uint64_t dMk0 = desc_plain_k(smem_u32(sM), 128, 0), dMt0 = desc_plain_mn(smem_u32(sM), 128, 0, 0);
  const uint64_t dC0 = desc_sw128_k(smem_u32(sC), 0), dB0 = desc_sw128_k(smem_u32(sB), 0);
  const int t_row = c * QT + row;
  const int hl_e = (part * 16) / P;            // head (inside the block) of this thread's epilogue columns
  for (int blk = 0; blk < nblk; ++blk) {
    const int h0 = grp * g.hpg + blk * HB;
    const int h_e = h0 + hl_e;
    const float Dh = D ? __ldg(D + h_e) : 0.f;
    xt = sXset + (blk & 1) * XSET;
    dyt = xt + BOX_BYTES;
    tb = (const float*)(dyt + BOX_BYTES);
    w.wait(&bar_x[blk & 1], (blk >> 1) & 1, 23);
    w.wait(&bar_st, blk & 1, 25);
    if (tid == 0 && blk + 1 < nblk) load_xset(blk + 1);   // the other set: its readers finished with the previous block
    for (int hl = 0; hl < HB; ++hl) {
      decay_mask_block(tmG, tb + hl * TAB, row, part, warp, smem_u32(sM));
      fence_async_smem();
      tc_fence_before();
      __syncthreads();
      // four issuing lanes (one per product: Y, U', and the two state terms), each committing its own instructions
      if ((tid & 31) == 0 && warp < 4) {
        tc_fence_after();
        if (warp == 0) {
          const uint64_t dX0 = desc_sw128_mn(smem_u32(xt), 0, hl * P * 2, 16);
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) mma_bf16(tmYd + hl * P, desc_adv(dMk0, ks * 4096), desc_adv(dX0, ks * 2048), idY, ks > 0);
        } else if (warp == 1) {
          const uint64_t dY0 = desc_sw128_mn(smem_u32(dyt), 0, hl * P * 2, 16);
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) mma_bf16(tmUd + hl * P, desc_adv(dMt0, ks * 256), desc_adv(dY0, ks * 2048), idU, ks > 0);
        } else if (hl == 0) {
          const uint64_t dA0 = (warp == 2) ? dC0 : dB0;
          const uint64_t dS0 = desc_sw128_k(smem_u32(warp == 2 ? stS : stDS), 0);
          const uint32_t tmO = (warp == 2) ? tmYo : tmUo;
#pragma unroll
          for (int kb = 0; kb < NB; ++kb)
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)
              mma_bf16(tmO, desc_adv(dA0, kb * BOX_BYTES + ks * 32), desc_adv(dS0, kb * SBOX_BYTES + ks * 32), idO, (kb | ks) > 0);
        }
        mma_commit(&bar_mma);
      }
      w.wait(&bar_mma, mphase, 24);
      mphase ^= 1;
      tc_fence_after();
    }
    // ---- epilogue for the HB heads of this block: this thread has 64/PARTS = 16 of the 64 columns.
    // Copy what is needed from the input buffers into registers first, so the buffers can be refilled.
    uint4 xv[2], dv[2];
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      xv[q] = ld_shared_v4(smem_u32(xt) + sw128_off(row, part * 2 + q));
      dv[q] = ld_shared_v4(smem_u32(dyt) + sw128_off(row, part * 2 + q));
    }
    const float cs_r = tb[hl_e * TAB + T_CS + row], dt_r = tb[hl_e * TAB + T_DT + row];
    const float osc_y = ex2(cs_r), osc_u = dt_r * ex2(tb[hl_e * TAB + T_CS + 127] - cs_r);
    __syncthreads();
    if (tid == 0 && blk + 1 < nblk) load_states(blk + 1);
    float s0 = 0.f, s1 = 0.f, s2 = 0.f;
    {
      float yd[16], yo[16];
      tmem_ld16(tmem_addr(tmYd, (warp & 3) * 32, part * 16), yd);
      tmem_ld16(tmem_addr(tmYo, (warp & 3) * 32, part * 16), yo);
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        float xs[8], dys[8];
        unpack8(xv[q], xs);
        unpack8(dv[q], dys);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float acc = yd[q * 8 + k] + osc_y * yo[q * 8 + k];
          s0 = fmaf(dys[k], acc, s0);
          s1 = fmaf(dys[k], xs[k], s1);
        }
      }
    }
    {
      float ud[16], uo[16];
      tmem_ld16(tmem_addr(tmUd, (warp & 3) * 32, part * 16), ud);
      tmem_ld16(tmem_addr(tmUo, (warp & 3) * 32, part * 16), uo);
      const size_t dense = ((size_t)b * g.L + t_row) * g.H * P + (size_t)h0 * P + part * 16;
      uint4 ov[2];
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        float xs[8], dys[8], o[8];
        unpack8(xv[q], xs);
        unpack8(dv[q], dys);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float acc = ud[q * 8 + k] + osc_u * uo[q * 8 + k];
          o[k] = acc + Dh * dys[k];
          s2 = fmaf(xs[k], acc, s2);
        }
        ov[q] = pack8(o);
      }
      st_global_32B(dx + dense, ov[0], ov[1]);
    }
    sRed[part * 128 + row] = s0;
    sRed[(PARTS + part) * 128 + row] = s1;
    sRed[(2 * PARTS + part) * 128 + row] = s2;
    tc_fence_before();
    __syncthreads();
    if ((part % (P / 16)) == 0) {
      float t0 = 0.f, t1 = 0.f, t2 = 0.f;
#pragma unroll
      for (int k = 0; k < P / 16; ++k) {
        t0 += sRed[(part + k) * 128 + row];
        t1 += sRed[(PARTS + part + k) * 128 + row];
        t2 += sRed[(2 * PARTS + part + k) * 128 + row];
      }
      const size_t co = ((size_t)(b * g.H + h_e) * g.nc + c) * QT + row;
      dcsp[co] = t0;
      ddot[co] = t1;
      ddtd[co] = dt_r > 0.f ? t2 / dt_r : 0.f;
    }
  }
  if (warp == 1) tmem_dealloc(tm, TM_COLS);
}

// ---------------------------------------------------------------------------------------------
// Backward, dB and dC.  grid = (nc, G, B).  Per head W_h = dY_h X_h^T (128x128, TMEM), masked and
// decayed like M_h into W'_h (bf16, shared memory), then accumulated over the heads of the group
//   dC[i,n] += W'_h B      (+ per head block)  (exp(cs_i) dY) S_prev
//   dB[j,n] += W'_h^T C    (+ per head block)  (exp(cs_end-cs_j) dt_j X) dS_end
template <int P, int N>
__global__ void __launch_bounds__(TC_THREADS, (N <= 64) ? 2 : 1)
k_dbc_tc(Geo g, const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmDY,
         const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmC,
         const __grid_constant__ CUtensorMap tmS, const __grid_constant__ CUtensorMap tmDS,
         const float* __restrict__ tab, bf16* __restrict__ dB, bf16* __restrict__ dC, int* __restrict__ status) {
  constexpr int NB = N / 64;
  constexpr int HB = 64 / P;
  constexpr uint32_t TM_COLS = (128 + 2 * N <= 256) ? 256 : 512;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);   // 1 KB aligned, still known to be shared memory
  uint8_t* sB = smem;                          // NB boxes
  uint8_t* sC = sB + NB * BOX_BYTES;           // NB boxes
  uint8_t* sM = sC + NB * BOX_BYTES;           // 32 KB W'_h tile, plain layout
  // x box, dy box and the tables of a head block: NBUF sets, so that at dstate 128 (one CTA per SM) the next block's set is
  // requested a whole block ahead instead of behind the current block's last product
  constexpr int NBUF = (N > 64) ? 2 : 1;
  constexpr int XSET = 2 * BOX_BYTES + HB * TAB_BYTES;
  uint8_t* sXset = sM + 2 * BOX_BYTES;
  uint8_t* sS = sM;                            // S_prev boxes (NB x 8 KB): reuse the W' tile after the head loop
  uint8_t* sDS = sM + NB * SBOX_BYTES;         // dS_end boxes
  __shared__ __align__(8) uint64_t bar_cb, bar_x[2], bar_s, bar_mma;
  __shared__ uint32_t tmem_slot;
  __shared__ int s_abort;

  const int tid = threadIdx.x, warp = tid >> 5;
  if (tid == 0) s_abort = *(volatile int*)status;
  __syncthreads();
  if (s_abort) return;
  const int c = blockIdx.x, grp = blockIdx.y, b = blockIdx.z;
  const int row = tid & 127, part = tid >> 7;
  if (tid == 0) {
    mbar_init(&bar_cb, 1); mbar_init(&bar_x[0], 1); mbar_init(&bar_x[1], 1); mbar_init(&bar_s, 1); mbar_init(&bar_mma, 1);
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(&tmem_slot, TM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = tmem_slot;
  const uint32_t tmW = tm, tmDC = tm + 128, tmDB = tm + 128 + N;
  Waiter w{status, false};

  const int nblk = g.hpg / HB;
  const int col_base = grp * g.hpg * P;
  auto load_boxes = [&](int blk) {             // thread 0 only
    uint8_t* set = sXset + (blk % NBUF) * XSET;
    uint64_t* bar = &bar_x[blk % NBUF];
    mbar_expect_tx(bar, XSET);
    tma_load_3d(set, &tmX, col_base + blk * 64, c * QT, b, bar);
    tma_load_3d(set + BOX_BYTES, &tmDY, col_base + blk * 64, c * QT, b, bar);
    bulk_load(set + 2 * BOX_BYTES, tab + ((size_t)(b * g.nc + c) * g.H + grp * g.hpg + blk * HB) * TAB, HB * TAB_BYTES, bar);
  };
  if (tid == 0) {
    mbar_expect_tx(&bar_cb, 2 * NB * BOX_BYTES);
    for (int kb = 0; kb < NB; ++kb) {
      tma_load_3d(sB + kb * BOX_BYTES, &tmB, grp * N + kb * 64, c * QT, b, &bar_cb);
      tma_load_3d(sC + kb * BOX_BYTES, &tmC, grp * N + kb * 64, c * QT, b, &bar_cb);
    }
    load_boxes(0);
    for (int blk = 0; blk < nblk; ++blk) {   // everything this CTA will load later: start it towards L2 now
      const int h0 = grp * g.hpg + blk * HB;
      if (blk > 0) {
        tma_prefetch_3d(&tmX, col_base + blk * 64, c * QT, b);
        tma_prefetch_3d(&tmDY, col_base + blk * 64, c * QT, b);
        bulk_prefetch(tab + ((size_t)(b * g.nc + c) * g.H + h0) * TAB, HB * TAB_BYTES);
      }
      for (int kb = 0; kb < NB; ++kb) {
        tma_prefetch_3d(&tmS, kb * 64, h0 * P, b * g.nc + c);
        tma_prefetch_3d(&tmDS, kb * 64, h0 * P, b * g.nc + c);
      }
    }
  }
  uint32_t sphase = 0, mphase = 0;
  const uint32_t idW = make_idesc(128, 128, 0, 0), idC = make_idesc(128, N, 0, 1), idB = make_idesc(128, N, 1, 1);
  uint8_t* sX = sXset;
  uint8_t* sDY = sX + BOX_BYTES;
  const float* sTab = (const float*)(sDY + BOX_BYTES);     // [HB][TAB]
  uint64_t dDY0 = desc_sw128_k(smem_u32(sDY), 0), dX0 = desc_sw128_k(smem_u32(sX), 0);
  const uint64_t dMk0 = desc_plain_k(smem_u32(sM), 128, 0), dMt0 = desc_plain_mn(smem_u32(sM), 128, 0, 0);
  const uint64_t dBm0 = desc_sw128_mn(smem_u32(sB), 0, 0, BOX_BYTES), dCm0 = desc_sw128_mn(smem_u32(sC), 0, 0, BOX_BYTES);
  const uint64_t dSm0 = desc_sw128_mn(smem_u32(sS), 0, 0, SBOX_BYTES), dDSm0 = desc_sw128_mn(smem_u32(sDS), 0, 0, SBOX_BYTES);
  auto issue_w = [&](int hl) {   // thread 0: W = dY_h X_h^T, K = P
#pragma unroll
    for (int ks = 0; ks < P / 16; ++ks)
      mma_bf16(tmW, desc_adv(dDY0, hl * P * 2 + ks * 32), desc_adv(dX0, hl * P * 2 + ks * 32), idW, ks > 0);
  };
  w.wait(&bar_cb, 0, 31);
  bool first = true;
  // SUMW (one CTA per SM, registers to spare): W'_h is summed over the heads in registers and multiplied once per tile
  constexpr bool SUMW = N > 64;
  float acc[32];
#pragma unroll
  for (int k = 0; k < 32; ++k) acc[k] = 0.f;
  for (int blk = 0; blk < nblk; ++blk) {
    const int h0 = grp * g.hpg + blk * HB;
    if (!SUMW) zero_upper_block(row, part, warp, smem_u32(sM));   // the state boxes of the previous head block lived here
    sX = sXset + (blk % NBUF) * XSET;
    sDY = sX + BOX_BYTES;
    sTab = (const float*)(sDY + BOX_BYTES);
    dDY0 = desc_sw128_k(smem_u32(sDY), 0);
    dX0 = desc_sw128_k(smem_u32(sX), 0);
    w.wait(&bar_x[blk % NBUF], (blk / NBUF) & 1, 32);
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
      if (NBUF == 2 && blk + 1 < nblk) load_boxes(blk + 1);   // the other set: its last readers finished a block ago
      issue_w(0);
      mma_commit(&bar_mma);
      if (SUMW) {   // nothing else lives in the W' tile until the end of the CTA: fetch this block's state boxes into it now
        mbar_expect_tx(&bar_s, 2 * NB * SBOX_BYTES);
        for (int kb = 0; kb < NB; ++kb) {
          tma_load_3d(sS + kb * SBOX_BYTES, &tmS, kb * 64, h0 * P, b * g.nc + c, &bar_s);
          tma_load_3d(sDS + kb * SBOX_BYTES, &tmDS, kb * 64, h0 * P, b * g.nc + c, &bar_s);
        }
      }
    }
    w.wait(&bar_mma, mphase, 33);
    mphase ^= 1;
    tc_fence_after();
    for (int hl = 0; hl < HB; ++hl) {
      if constexpr (SUMW) {
        decay_acc_block(tmW, sTab + hl * TAB, row, part, warp, acc);
        if (hl + 1 < HB) {
          tc_fence_before();
          __syncthreads();
          if (tid == 0) {
            tc_fence_after();
            issue_w(hl + 1);
            mma_commit(&bar_mma);
          }
          w.wait(&bar_mma, mphase, 34);
          mphase ^= 1;
          tc_fence_after();
        }
        continue;
      }
      decay_mask_block(tmW, sTab + hl * TAB, row, part, warp, smem_u32(sM));
      fence_async_smem();
      tc_fence_before();
      __syncthreads();
      if (tid == 0) {
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          mma_bf16(tmDC, desc_adv(dMk0, ks * 4096), desc_adv(dBm0, ks * 2048), idC, !first || ks > 0);
          mma_bf16(tmDB, desc_adv(dMt0, ks * 256), desc_adv(dCm0, ks * 2048), idB, !first || ks > 0);
        }
        if (hl + 1 < HB) issue_w(hl + 1);
        mma_commit(&bar_mma);
      }
      first = false;
      w.wait(&bar_mma, mphase, 34);
      mphase ^= 1;
      tc_fence_after();
    }
    // state terms of this head block: fetch the bf16 S_prev and dS_end boxes over the W' tile (its
    // last readers have completed), scale the dy box by exp(cs_i) and the x box by
    // exp(cs_end - cs_j) dt_j in place meanwhile, then one K = 64 product each
    if (!SUMW && tid == 0) {
      mbar_expect_tx(&bar_s, 2 * NB * SBOX_BYTES);
      for (int kb = 0; kb < NB; ++kb) {
        tma_load_3d(sS + kb * SBOX_BYTES, &tmS, kb * 64, h0 * P, b * g.nc + c, &bar_s);
        tma_load_3d(sDS + kb * SBOX_BYTES, &tmDS, kb * 64, h0 * P, b * g.nc + c, &bar_s);
      }
    }
#pragma unroll
    for (int r = 0; r < 2048 / TC_THREADS; ++r) {
      const int idx = tid + r * TC_THREADS;
      const int box = idx >> 10, l = (idx >> 3) & 127, pc = idx & 7;
      const float* t = sTab + ((((pc ^ l) & 7) * 8) / P) * TAB;
      const float f = box ? ex2(t[T_CS + l]) : ex2(t[T_CS + 127] - t[T_CS + l]) * t[T_DT + l];
      const uint32_t a = smem_u32((box ? sDY : sX) + l * 128 + pc * 16);
      float v[8];
      unpack8(ld_shared_v4(a), v);
#pragma unroll
      for (int k = 0; k < 8; ++k) v[k] *= f;
      const uint4 o = pack8(v);
      st_shared_v4(a, o.x, o.y, o.z, o.w);
    }
    fence_async_smem();
    w.wait(&bar_s, sphase, 36);
    sphase ^= 1;
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        mma_bf16(tmDC, desc_adv(dDY0, ks * 32), desc_adv(dSm0, ks * 2048), idC, !first || ks > 0);
        mma_bf16(tmDB, desc_adv(dX0, ks * 32), desc_adv(dDSm0, ks * 2048), idC, !first || ks > 0);
      }
      mma_commit(&bar_mma);
    }
    first = false;
    w.wait(&bar_mma, mphase, 35);
    mphase ^= 1;
    tc_fence_after();
    __syncthreads();
    if (NBUF == 1 && tid == 0 && blk + 1 < nblk) load_boxes(blk + 1);
  }
  if constexpr (SUMW) {
    // the head sum -> bf16 -> the W' tile (the state boxes that lived there have been consumed), then one product per side
    zero_upper_block(row, part, warp, smem_u32(sM));
    store_acc_block(acc, row, part, warp, smem_u32(sM));
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        mma_bf16(tmDC, desc_adv(dMk0, ks * 4096), desc_adv(dBm0, ks * 2048), idC, true);
        mma_bf16(tmDB, desc_adv(dMt0, ks * 256), desc_adv(dCm0, ks * 2048), idB, true);
      }
      mma_commit(&bar_mma);
    }
    w.wait(&bar_mma, mphase, 37);
    mphase ^= 1;
    tc_fence_after();
  }
  // epilogue: this thread writes N/PARTS columns of row `row` of dC and of dB
  {
    const size_t o = (((size_t)b * g.L + c * QT + row) * g.G + grp) * N + part * (N / PARTS);
#pragma unroll
    for (int q = 0; q < N / PARTS / 16; ++q) {
      float vc[16], vb[16];
      tmem_ld16(tmem_addr(tmDC, (warp & 3) * 32, part * (N / PARTS) + q * 16), vc);
      tmem_ld16(tmem_addr(tmDB, (warp & 3) * 32, part * (N / PARTS) + q * 16), vb);
      st_global_32B(dC + o + q * 16,
                    make_uint4(pack_bf16(vc[0], vc[1]), pack_bf16(vc[2], vc[3]), pack_bf16(vc[4], vc[5]), pack_bf16(vc[6], vc[7])),
                    make_uint4(pack_bf16(vc[8], vc[9]), pack_bf16(vc[10], vc[11]), pack_bf16(vc[12], vc[13]), pack_bf16(vc[14], vc[15])));
      st_global_32B(dB + o + q * 16,
                    make_uint4(pack_bf16(vb[0], vb[1]), pack_bf16(vb[2], vb[3]), pack_bf16(vb[4], vb[5]), pack_bf16(vb[6], vb[7])),
                    make_uint4(pack_bf16(vb[8], vb[9]), pack_bf16(vb[10], vb[11]), pack_bf16(vb[12], vb[13]), pack_bf16(vb[14], vb[15])));
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tm, TM_COLS);
}

// ---------------------------------------------------------------------------------------------
// Persistent, warp-specialised version of the chunk_scan family for dstate 64: one CTA per SM walks
// over (batch, chunk, group) tiles and keeps every stage busy at once:
//   warp 16 lane 0    TMA producer: C/B tiles (2 slots) and per-head-block inputs (2 slots)
//   warp 17 lane 0    MMA issuer:   G = C B^T of the NEXT tile early, then per head Y/U' and the state term
//   warps 0-15        decay pass:   G (TMEM) -> M_h (ring of NM shared-memory tiles)
//   warps 20-27       epilogue:     accumulators (2 TMEM slots) -> global, overlapped with the next block
// Hand-offs are mbarriers: *_full arrive by TMA bytes / tcgen05.commit / one lane per producer warp,
// *_empty by tcgen05.commit or one lane per consumer warp.  Slot use n (0,1,2,...) waits `full` with
// parity n&1 and `empty` with parity (n&1)^1 (a fresh barrier passes a wait on parity 1).
// TMEM: G x2 (256 columns) + {Y, Y_off} x2 (256 columns) = 512.  Same math and operand layouts as
// k_scan_tc; MODE as there.
// sigmoid through one tanh.approx (relative error 2^-11, below the bf16 resolution of the gated output): the exact
// form costs an exp, an IEEE division and its slow path per element, which made the gated epilogue 2.4x the ungated one
__device__ __forceinline__ float sigmoid_fast(float a) {
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * a));
  return fmaf(0.5f, t, 0.5f);
}
constexpr int WS_THREADS = 28 * 32;
constexpr int WS_SCALE_WARPS = 16, WS_EPI_WARPS = 8;

template <int P, int MODE, int N_ = 64, bool GATED_ = false>
struct WsCfg {
  static constexpr int N = N_, HB = 64 / P, NB64 = N_ / 64;
  // dstate 128: the C and B tiles are 32 KB each, so there is ONE C/B slot (and one G), and the state boxes of a head
  // block live in a buffer of their own whose MMA is issued first in the block (it does not depend on M_h)
  static constexpr bool SPLIT = N_ == 128;
  static constexpr int NCBS = SPLIT ? 1 : 2;                          // C/B slots = G buffers
  static constexpr int NBOX = (MODE == 0) ? 1 : 2;
  // gated forward: the gate's box arrives by TMA beside the x box (a thread-per-row read of it from global memory costs one
  // L1 wavefront per lane and instruction); its 2 x 16 KB take the place of the third M_h slot
  static constexpr int ZB = (GATED_ && MODE == 0) ? 1 : 0;
  // M_h ring depth = decay groups.  A wait by parity is only right for a waiter that is at most one phase behind.  Slot
  // kh % NM always belongs to decay group kh % NM.  On the issuing side, with two heads per block lane hl issues head hl of
  // every block: with two slots a slot then always meets the same lane; with three it alternates between the lanes, and
  // HEAD_ORDER (below) is what keeps the second lane from reaching a slot before the first lane's head has been written.
  static constexpr int NM = (MODE == 0 && !ZB) ? 3 : 2;
  static constexpr int CB_BYTES = 2 * NB64 * BOX_BYTES;              // keep + other tile
  static constexpr int ST_BYTES = NB64 * SBOX_BYTES;                 // state boxes of one head block
  static constexpr int ZOFF = NBOX * BOX_BYTES + (SPLIT ? 0 : ST_BYTES);       // the gate's box comes last in a slot
  static constexpr int IN_BYTES = ZOFF + ZB * BOX_BYTES;                       // x [, dy] box [+ state box] [+ z box]
  // table ring depth (one 2 KB table per head): a multiple of the number of decay groups, so that a slot is always read by
  // the same group.  With a depth of 4 and three groups the slot of head 5 had last been head 1's, read by another group:
  // the group of head 5, coming from head 2, could reach the slot's barrier before head 1's table had landed, pass the wait
  // on the parity of a phase that had not even begun, and read the slot while head 5's table was still arriving (rows 0-31
  // of that head wrong about once in 10^4 CTAs).
  static constexpr int NTH = (NM == 3) ? 6 : 4 * HB;
  static_assert(NTH % NM == 0 && NTH % HB == 0 && NTH <= 8, "a table slot must belong to one decay group and one column half");
  static constexpr int RED_BYTES = (P == 64 && MODE != 0) ? 2 * 256 * 4 : 0;
  static constexpr size_t SMEM = 1024 + NCBS * CB_BYTES + NM * 2 * BOX_BYTES + 2 * IN_BYTES + (SPLIT ? ST_BYTES : 0) +
                                 NTH * TAB_BYTES + RED_BYTES;
  static_assert(SMEM <= 232448, "shared-memory plan exceeds the 227 KB a CTA can have");
  // warp roles: NM groups of 4 * NCH decay warps, then two MMA issuer warps (one per head of a head block) on the two
  // least loaded schedulers, the producer warp and an idle warp, then 8 epilogue warps
  static constexpr int NCH = 1;                                       // threads per row of the decay pass
  static constexpr int DW = 4 * NCH * NM, W_MMA = DW, W_PROD = DW + 2, W_EPI = DW + 4;
  // active issuers: warps W_MMA .. W_MMA + NI - 1, one per head of a head block; with one (64-wide) head per block and
  // dstate 128 the second lane issues the state term (8 instructions per head beside the head's own 8)
  static constexpr int NI = (SPLIT && HB == 1) ? 2 : HB;
  static constexpr bool STATE_LANE = (SPLIT && HB == 1);             // the second lane issues the state term only
  // Head 2 kb + 1 (lane 1) takes the slot head 2 kb - 2 (lane 0) had.  Lane 1 has not waited on that use, so its wait by
  // parity could pass while the slot still shows the phase before it.  Lane 0 therefore reports "head 0 of block kb is
  // written" on hz[kb % 4] as soon as it has seen it, and lane 1 waits for block kb - 1's report first.  (Lane 0 needs no
  // such report: the slot of head 2 kb was head 2 kb - 3's, whose block both lanes have finished before either starts
  // block kb, because the accumulator set of block kb is the one block kb - 2 used.  The lanes are at most two blocks
  // apart for the same reason, so four report slots never wrap.)
  static constexpr bool HEAD_ORDER = HB == 2 && NM == 3;
  static constexpr int THREADS = (DW + 4 + WS_EPI_WARPS) * 32;
  // registers per thread after re-balancing (launch share: 80 at 768 threads, 96 at 640)
  static constexpr int R_DECAY = (THREADS == 768) ? 88 : (THREADS == 640 ? 128 : (MODE == 0 ? 80 : 72)),
                       R_SPECIAL = (THREADS > 768) ? 48 : 56,
                       R_EPI = (THREADS > 768) ? (MODE == 0 ? 64 : 72) : ((MODE == 0) ? 72 : 80);
};

struct WsBars {
  uint64_t cb_full[2], cb_empty[2], g_full[2], g_empty[2], in_full[2], in_empty[2], acc_full[2], acc_empty[2];
  uint64_t m_full[3], m_empty[3], tab_full[8], tab_empty[8], st_full, st_empty, out_ready[2], hz[4], done;
};

template <int P, int MODE, int N_ = 64, bool GATED = false>
__global__ void __launch_bounds__(WsCfg<P, MODE, N_, GATED>::THREADS, 1)
k_scan_ws(Geo g, const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmDY,
          const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmC,
          const __grid_constant__ CUtensorMap tmS, const __grid_constant__ CUtensorMap tmOut,
          const __grid_constant__ CUtensorMap tmZ, const float* __restrict__ tab, const float* __restrict__ D,
          const bf16* __restrict__ z_, bf16* __restrict__ y, bf16* __restrict__ dypb, bf16* __restrict__ dz,
          bf16* __restrict__ dx, float* __restrict__ rs0, float* __restrict__ rs1, int* __restrict__ status) {
  using Cfg = WsCfg<P, MODE, N_, GATED>;
  const bf16* __restrict__ z = GATED ? z_ : nullptr;     // the ungated instantiation carries none of the gate's registers
  constexpr bool ZSMEM = Cfg::ZB != 0;                    // forward: the gate's box is in the input slot
  // Forward and dx: the output block (128 rows x 64 columns bf16) has the shape and layout of the x (dy) box the epilogue
  // reads, so the epilogue writes it over that box and a spare lane sends it out as ONE TMA tile store.  A row-per-thread
  // global store costs one L1 wavefront per lane and instruction, and the L1 data stage is what these kernels share.
  constexpr bool TSTORE = MODE != 1;
  constexpr int N = Cfg::N, HB = Cfg::HB, NBOX = Cfg::NBOX, NM = Cfg::NM, NTH = Cfg::NTH, NB64 = Cfg::NB64, NCBS = Cfg::NCBS;
  constexpr bool SPLIT = Cfg::SPLIT;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);   // 1 KB aligned, still known to be shared memory
  uint8_t* sCB = smem;                                   // NCBS x {keep tile, other tile}
  uint8_t* sM = sCB + NCBS * Cfg::CB_BYTES;              // NM x 32 KB
  uint8_t* sIn = sM + NM * 2 * BOX_BYTES;                // 2 x {x [, dy] [, state box]}
  uint8_t* sSt = sIn + 2 * Cfg::IN_BYTES;                // dstate 128: the state boxes of one head block
  uint8_t* sTab = sSt + (SPLIT ? Cfg::ST_BYTES : 0);     // NTH x decay table of one head (they run further ahead)
  float* sRed = (float*)(sTab + NTH * TAB_BYTES);          // [2][256] (P = 64 row-sum exchange)
  __shared__ __align__(8) WsBars bars;
  __shared__ uint32_t tmem_slot;
  __shared__ int s_abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) s_abort = *(volatile int*)status;
  __syncthreads();
  if (s_abort) return;
  if (tid == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars.cb_full[i], 1); mbar_init(&bars.cb_empty[i], Cfg::NI);
      mbar_init(&bars.g_full[i], 1); mbar_init(&bars.g_empty[i], Cfg::DW);
      mbar_init(&bars.in_full[i], 1); mbar_init(&bars.in_empty[i], Cfg::NI + (TSTORE ? 1 : WS_EPI_WARPS));
      mbar_init(&bars.acc_full[i], Cfg::NI); mbar_init(&bars.acc_empty[i], WS_EPI_WARPS);
      mbar_init(&bars.out_ready[i], WS_EPI_WARPS);
    }
    for (int i = 0; i < 3; ++i) { mbar_init(&bars.m_full[i], 4 * Cfg::NCH); mbar_init(&bars.m_empty[i], 1); }
    // a head's table is read by the warps of its decay group and by the epilogue warps of its columns
    for (int i = 0; i < NTH; ++i) { mbar_init(&bars.tab_full[i], 1); mbar_init(&bars.tab_empty[i], 4 * Cfg::NCH + WS_EPI_WARPS / HB); }
    mbar_init(&bars.st_full, 1); mbar_init(&bars.st_empty, 1);
    for (int i = 0; i < 4; ++i) mbar_init(&bars.hz[i], 1);
    mbar_init(&bars.done, Cfg::NI);
    mbar_fence_init();
  }
  if (warp == Cfg::W_MMA) tmem_alloc(&tmem_slot, 512);
  // the blocks above the diagonal of every M_h ring tile are zero for the whole kernel
  if (tid < 512) {
    for (int i = 0; i < NM; ++i) zero_upper_blocks(tid & 127, tid >> 7, warp, smem_u32(sM + i * 2 * BOX_BYTES));
    fence_async_smem();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = tmem_slot;
  Waiter w{status, false};

  const int nblk = g.hpg / HB;
  const int ntiles = g.B * g.G * g.nc;
  const int my_tiles = (ntiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;   // >= 1 by launch
  auto tile_coords = [&](int t, int& b, int& grp, int& c) {
    const int u = blockIdx.x + t * gridDim.x;
    c = u % g.nc;
    const int r = u / g.nc;
    grp = r % g.G;
    b = r / g.G;
  };

  if (warp >= Cfg::DW && warp < Cfg::W_EPI) reg_dec<Cfg::R_SPECIAL>();
  if (warp == Cfg::W_PROD) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      auto load_cb = [&](int t) {
        int b, grp, c;
        tile_coords(t, b, grp, c);
        const int cs_ = t % NCBS;
        w.wait(&bars.cb_empty[cs_], ((t / NCBS) & 1) ^ 1, 41);
        uint8_t* keep = sCB + cs_ * Cfg::CB_BYTES;
        mbar_expect_tx(&bars.cb_full[cs_], Cfg::CB_BYTES);
#pragma unroll
        for (int j = 0; j < NB64; ++j) {
          tma_load_3d(keep + j * BOX_BYTES, (MODE == 2) ? &tmB : &tmC, grp * N + 64 * j, c * QT, b, &bars.cb_full[cs_]);
          tma_load_3d(keep + (NB64 + j) * BOX_BYTES, (MODE == 2) ? &tmC : &tmB, grp * N + 64 * j, c * QT, b, &bars.cb_full[cs_]);
        }
      };
      const int total_blocks = my_tiles * nblk;
      auto load_tab = [&](int kg) {        // tables of the heads of global block kg: they run two blocks ahead of the boxes
        if (kg >= total_blocks) return;
        int b, grp, c;
        tile_coords(kg / nblk, b, grp, c);
        const int h0 = grp * g.hpg + (kg % nblk) * HB;
        for (int hl = 0; hl < HB; ++hl) {
          const int kh = kg * HB + hl, ts = kh % NTH;
          w.wait(&bars.tab_empty[ts], ((kh / NTH) & 1) ^ 1, 49);
          mbar_expect_tx(&bars.tab_full[ts], TAB_BYTES);
          bulk_load(sTab + ts * TAB_BYTES, tab + ((size_t)(b * g.nc + c) * g.H + h0 + hl) * TAB, TAB_BYTES, &bars.tab_full[ts]);
        }
      };
      int kb = 0;
      load_cb(0);
      load_tab(0);
      load_tab(1);
      for (int t = 0; t < my_tiles; ++t) {
        int b, grp, c;
        tile_coords(t, b, grp, c);
        for (int blk = 0; blk < nblk; ++blk, ++kb) {
          const int ib = kb & 1;
          w.wait(&bars.in_empty[ib], ((kb >> 1) & 1) ^ 1, 42);
          uint8_t* dst = sIn + ib * Cfg::IN_BYTES;
          const int h0 = grp * g.hpg + blk * HB;
          const int col = grp * g.hpg * P + blk * 64;
          mbar_expect_tx(&bars.in_full[ib], Cfg::IN_BYTES);
          tma_load_3d(dst, &tmX, col, c * QT, b, &bars.in_full[ib]);
          if (NBOX == 2) tma_load_3d(dst + BOX_BYTES, &tmDY, col, c * QT, b, &bars.in_full[ib]);
          if (ZSMEM) tma_load_3d(dst + Cfg::ZOFF, &tmZ, col, c * QT, b, &bars.in_full[ib]);
          if constexpr (!SPLIT) tma_load_3d(dst + NBOX * BOX_BYTES, &tmS, 0, h0 * P, b * g.nc + c, &bars.in_full[ib]);
          // tables two blocks ahead, behind this block's boxes: with a ring of three blocks of tables the slot's previous
          // readers (block kb - 1) start only when the box slot of block kb - 2 comes free, and the boxes must not wait for them
          load_tab(kb + 2);
          if constexpr (!SPLIT) {
            // the next tile's C/B go out right behind this tile's first block, so the MMA warp can form
            // the next G while this tile is still being worked on
            if (blk == 0 && t + 1 < my_tiles) load_cb(t + 1);
          } else {
            w.wait(&bars.st_empty, (kb & 1) ^ 1, 57);
            mbar_expect_tx(&bars.st_full, Cfg::ST_BYTES);
#pragma unroll
            for (int j = 0; j < NB64; ++j)
              tma_load_3d(sSt + j * SBOX_BYTES, &tmS, 64 * j, h0 * P, b * g.nc + c, &bars.st_full);
          }
        }
        // one C/B slot: the next tile's C/B can only follow this tile's last block
        if (SPLIT && t + 1 < my_tiles) load_cb(t + 1);
      }
    }
  } else if (warp >= Cfg::W_MMA && warp < Cfg::W_MMA + Cfg::NI) {
    // ------------------------------------------------------------------ MMA issuers: issuer mi takes head mi of every
    // head block; issuer 0 also forms G and the state term.  A commit only tracks the MMAs of its own thread, so the
    // block-level barriers expect one arrival per issuer.
    const int mi = warp - Cfg::W_MMA;
    if (lane == 0) {
      const uint32_t idG = make_idesc(128, 128, 0, 0);
      const uint32_t idY = make_idesc(128, P, (MODE == 2) ? 1 : 0, 1), idO = make_idesc(128, 64, 0, 0);
      constexpr uint32_t M_STEP = (MODE == 2) ? 256 : 4096;
      auto issue_g = [&](int t) {
        const int s_ = t % NCBS;
        w.wait(&bars.cb_full[s_], (t / NCBS) & 1, 43); w.wait(&bars.g_empty[s_], ((t / NCBS) & 1) ^ 1, 44);
        tc_fence_after();
        const uint32_t keep = smem_u32(sCB + s_ * Cfg::CB_BYTES), other = keep + NB64 * BOX_BYTES;
#pragma unroll 1
        for (int j = 0; j < NB64; ++j) {
          const uint64_t dc = desc_sw128_k(((MODE == 2) ? other : keep) + j * BOX_BYTES, 0),
                         db = desc_sw128_k(((MODE == 2) ? keep : other) + j * BOX_BYTES, 0);
#pragma unroll 1
          for (int ks = 0; ks < 4; ++ks) mma_bf16(tm + s_ * 128, desc_adv(dc, ks * 32), desc_adv(db, ks * 32), idG, (j | ks) > 0);
        }
        mma_commit(&bars.g_full[s_]);
      };
      if (mi == 0) issue_g(0);
      int kb = 0, kh = 0;
      for (int t = 0; t < my_tiles; ++t) {
        const uint32_t keep_t = smem_u32(sCB + (t % NCBS) * Cfg::CB_BYTES);
        const uint64_t dK0 = desc_sw128_k(keep_t, 0);
        // the lane that issues the state term reads the keep tile; when that is not the lane that formed G (and waited
        // for the tile there), it has to see the tile's arrival itself: the first x box of a tile can land before its C/B
        if (mi == 1) w.wait(&bars.cb_full[t % NCBS], (t / NCBS) & 1, 64);
        for (int blk = 0; blk < nblk; ++blk, ++kb) {
          const int ib = kb & 1, ab = kb & 1;
          const uint32_t inb = smem_u32(sIn + ib * Cfg::IN_BYTES);
          const uint32_t tmYd = tm + 256 + ab * 128, tmYo = tmYd + 64;
          w.wait(&bars.in_full[ib], (kb >> 1) & 1, 45);
          w.wait(&bars.acc_empty[ab], ((kb >> 1) & 1) ^ 1, 46);
          if constexpr (SPLIT) {
            if (mi == (Cfg::STATE_LANE ? 1 : 0)) {    // the state term first: it needs the keep tile and the state boxes, not M_h
              w.wait(&bars.st_full, kb & 1, 58);
              tc_fence_after();
#pragma unroll 1
              for (int j = 0; j < NB64; ++j) {
                const uint64_t dKj = desc_sw128_k(keep_t + j * BOX_BYTES, 0), dSj = desc_sw128_k(smem_u32(sSt + j * SBOX_BYTES), 0);
#pragma unroll 1
                for (int ks = 0; ks < 4; ++ks) mma_bf16(tmYo, desc_adv(dKj, ks * 32), desc_adv(dSj, ks * 32), idO, (j | ks) > 0);
              }
              mma_commit(&bars.st_empty);
            }
          }
          for (int hl = 0; hl < HB; ++hl, ++kh) {
            const int ms = kh % NM;
            if ((Cfg::STATE_LANE ? 0 : hl) != mi) continue;
            if (Cfg::HEAD_ORDER && hl == 1 && kb >= 1) w.wait(&bars.hz[(kb - 1) & 3], ((kb - 1) >> 2) & 1, 65);
            w.wait(&bars.m_full[ms], (kh / NM) & 1, 47);
            if (Cfg::HEAD_ORDER && hl == 0) mbar_arrive(&bars.hz[kb & 3]);
            tc_fence_after();
            const uint32_t mt = smem_u32(sM + ms * 2 * BOX_BYTES);
            const uint64_t dM0 = (MODE == 2) ? desc_plain_mn(mt, 128, 0, 0) : desc_plain_k(mt, 128, 0);
            const uint64_t dO0 = desc_sw128_mn(inb + ((MODE == 2) ? BOX_BYTES : 0), 0, hl * P * 2, 16);
#pragma unroll 1
            for (int ks = 0; ks < 8; ++ks)
              mma_bf16(tmYd + hl * P, desc_adv(dM0, ks * M_STEP), desc_adv(dO0, ks * 2048), idY, ks > 0);
            if (!SPLIT && hl == 0) {
              const uint64_t dS0 = desc_sw128_k(inb + NBOX * BOX_BYTES, 0);
#pragma unroll 1
              for (int ks = 0; ks < 4; ++ks) mma_bf16(tmYo, desc_adv(dK0, ks * 32), desc_adv(dS0, ks * 32), idO, ks > 0);
            }
            mma_commit(&bars.m_empty[ms]);
          }
          mma_commit(&bars.in_empty[ib]);
          if (blk == nblk - 1) mma_commit(&bars.cb_empty[t % NCBS]);
          mma_commit(&bars.acc_full[ab]);
          if (!SPLIT && mi == 0 && blk == 0 && t + 1 < my_tiles) issue_g(t + 1);
        }
        if (SPLIT && mi == 0 && t + 1 < my_tiles) issue_g(t + 1);
      }
      mma_commit(&bars.done);
      w.wait(&bars.done, 0, 48);
    }
  } else if (TSTORE && warp == Cfg::W_PROD + 1) {
    // ------------------------------------------------------------------ store lane: output blocks leave as TMA tiles
    if (lane == 0) {
      int kb = 0;
      for (int t = 0; t < my_tiles; ++t) {
        int b, grp, c;
        tile_coords(t, b, grp, c);
        for (int blk = 0; blk < nblk; ++blk, ++kb) {
          const int ib = kb & 1;
          w.wait(&bars.out_ready[ib], (kb >> 1) & 1, 59);
          tma_store_3d(&tmOut, sIn + ib * Cfg::IN_BYTES + (NBOX - 1) * BOX_BYTES, grp * g.hpg * P + blk * 64, c * QT, b);
          bulk_commit();
          bulk_wait_read0();            // the box has been read: the slot may be refilled
          mbar_arrive(&bars.in_empty[ib]);
        }
      }
      bulk_wait0();
    }
  } else if (warp < Cfg::DW) {
    // ------------------------------------------------------------------ decay pass: group wg owns heads kh = wg (mod NM)
    reg_inc<Cfg::R_DECAY>();
    const int wg = warp / (4 * Cfg::NCH), ch = (warp >> 2) % Cfg::NCH, rb = warp & 3, row = rb * 32 + lane;
    const uint32_t mrow = smem_u32(sM + wg * 2 * BOX_BYTES) + row * 16;
    int kh = 0;
    for (int t = 0; t < my_tiles; ++t) {
      const int gs = t % NCBS;
      w.wait(&bars.g_full[gs], (t / NCBS) & 1, 51);
      tc_fence_after();
      const uint32_t tm_row = tmem_addr(tm + gs * 128, rb * 32, 0);
      for (int hh = 0; hh < nblk * HB; ++hh, ++kh) {
        if (kh % NM != wg) continue;
        const int ts = kh % NTH;
        w.wait(&bars.m_empty[wg], ((kh / NM) & 1) ^ 1, 53);
        w.wait(&bars.tab_full[ts], (kh / NTH) & 1, 52);
        decay_row<Cfg::NCH>(rb, ch, tm_row, (const float*)(sTab + ts * TAB_BYTES), row, mrow);
        fence_async_smem(); __syncwarp(); if (lane == 0) { mbar_arrive(&bars.m_full[wg]); mbar_arrive(&bars.tab_empty[ts]); }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars.g_empty[gs]);
    }
  } else if (warp >= Cfg::W_EPI) {
    // ------------------------------------------------------------------ epilogue warps
    reg_dec<Cfg::R_EPI>();
    const int ew = warp - Cfg::W_EPI;
    const int row = (ew & 3) * 32 + lane, half = ew >> 2;     // 32 of the block's 64 columns
    const int hl_e = (half * 32) / P;
    int kb = 0;
    // gated recompute (MODE 1): the gate is the one operand the epilogue reads from global memory; this thread's 64 bytes
    // of it are requested at the start of the block, before the waits (the forward gets the gate's box by TMA)
    uint4 zq[GATED ? 4 : 1] = {};
    auto load_z = [&](int t_, int blk_, auto& dst) {
      if constexpr (GATED) {
        if (t_ >= my_tiles) return;
        int b_, grp_, c_;
        tile_coords(t_, b_, grp_, c_);
        const bf16* zp_ = z + b_ * g.zsb + (long long)(c_ * QT + row) * g.zsl + (long long)(grp_ * g.hpg + blk_ * HB) * P + half * 32;
        ld_global_32B(zp_, dst[0], dst[1]);
        ld_global_32B(zp_ + 16, dst[2], dst[3]);
      }
    };
    for (int t = 0; t < my_tiles; ++t) {
      int b, grp, c;
      tile_coords(t, b, grp, c);
      const int t_row = c * QT + row;
      for (int blk = 0; blk < nblk; ++blk, ++kb) {
        if constexpr (GATED && !ZSMEM) load_z(t, blk, zq);
        const int ib = kb & 1, ab = kb & 1;
        uint8_t* xt = sIn + ib * Cfg::IN_BYTES;
        uint8_t* dyt = xt + (NBOX - 1) * BOX_BYTES;
        const int khe = kb * HB + hl_e, ts = khe % NTH;
        const float* tb = (const float*)(sTab + ts * TAB_BYTES);
        const uint32_t tmYd = tm + 256 + ab * 128, tmYo = tmYd + 64;
        const int h0 = grp * g.hpg + blk * HB, h_e = h0 + hl_e;
        const float Dh = D ? __ldg(D + h_e) : 0.f;
        w.wait(&bars.tab_full[ts], (khe / NTH) & 1, 56);
        const uint32_t tbs = smem_u32(tb);
        const float cs_r = lds_f32(tbs + 4 * (T_CS + row)), dt_r = lds_f32(tbs + 4 * (T_DT + row));
        const float osc = (MODE == 2) ? dt_r * ex2(lds_f32(tbs + 4 * (T_CS + 127)) - cs_r) : ex2(cs_r);
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars.tab_empty[ts]);
        w.wait(&bars.in_full[ib], (kb >> 1) & 1, 54);
        w.wait(&bars.acc_full[ab], (kb >> 1) & 1, 55);
        tc_fence_after();
        const long long colo = (long long)h0 * P + half * 32;
        const size_t dense = ((size_t)b * g.L + t_row) * g.H * P + colo;
        float s0 = 0.f, s1 = 0.f;
#pragma unroll
        for (int h16 = 0; h16 < 2; ++h16) {
          // pull this 16-column slice out of shared memory and TMEM; after the second slice the input
          // slot and the accumulator slot are handed back before the arithmetic and the stores
          uint4 xv[2], dv[2];
          float yd[16], yo[16];
#pragma unroll
          for (int q = 0; q < 2; ++q) {
            xv[q] = ld_shared_v4(smem_u32(xt) + sw128_off(row, half * 4 + h16 * 2 + q));
            dv[q] = (MODE != 0) ? ld_shared_v4(smem_u32(dyt) + sw128_off(row, half * 4 + h16 * 2 + q)) : make_uint4(0u, 0u, 0u, 0u);
          }
          {   // both accumulator slices in flight, one wait (the two loads used to wait for one another)
            uint32_t rd[16], ro[16];
            tmem_ld16_issue(tmem_addr(tmYd, (ew & 3) * 32, half * 32 + h16 * 16), rd);
            tmem_ld16_issue(tmem_addr(tmYo, (ew & 3) * 32, half * 32 + h16 * 16), ro);
            tmem_ld_wait_2x16(rd, ro);
#pragma unroll
            for (int k = 0; k < 16; ++k) { yd[k] = __uint_as_float(rd[k]); yo[k] = __uint_as_float(ro[k]); }
          }
          if (h16 == 1) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) { mbar_arrive(&bars.acc_empty[ab]); if (!TSTORE) mbar_arrive(&bars.in_empty[ib]); }
          }
          uint4 ov[2], dpk[2];
#pragma unroll
          for (int q = 0; q < 2; ++q) {
            float xs[8], zs[8], dys[8], o[8], acc[8];
            unpack8(xv[q], xs);
#pragma unroll
            for (int k = 0; k < 8; ++k) acc[k] = yd[q * 8 + k] + osc * yo[q * 8 + k];
            if constexpr (ZSMEM) unpack8(ld_shared_v4(smem_u32(xt + Cfg::ZOFF) + sw128_off(row, half * 4 + h16 * 2 + q)), zs);
            else if (GATED) unpack8(zq[GATED ? h16 * 2 + q : 0], zs);
            if (MODE != 0) unpack8(dv[q], dys);
            if (MODE == 0) {
#pragma unroll
              for (int k = 0; k < 8; ++k) {
                o[k] = acc[k] + Dh * xs[k];
                if (GATED) o[k] *= zs[k] * sigmoid_fast(zs[k]);
              }
              ov[q] = pack8(o);
            } else if (MODE == 1) {
              float dp[8];
#pragma unroll
              for (int k = 0; k < 8; ++k) {
                float dyv = dys[k];
                if (GATED) {
                  const float sg = sigmoid_fast(zs[k]);
                  o[k] = dyv * (acc[k] + Dh * xs[k]) * sg * (1.f + zs[k] * (1.f - sg));   // dz
                  dyv *= zs[k] * sg;
                }
                dp[k] = dyv;
                s0 = fmaf(dyv, acc[k], s0);
                s1 = fmaf(dyv, xs[k], s1);
              }
              if (GATED) { ov[q] = pack8(o); dpk[q] = pack8(dp); }
            } else {
#pragma unroll
              for (int k = 0; k < 8; ++k) {
                o[k] = acc[k] + Dh * dys[k];
                s0 = fmaf(xs[k], acc[k], s0);
              }
              ov[q] = pack8(o);
            }
          }
          if (MODE == 1 && GATED) {
            st_global_32B(dz + dense + h16 * 16, ov[0], ov[1]);
            st_global_32B(dypb + dense + h16 * 16, dpk[0], dpk[1]);
          }
          if (TSTORE) {   // over the chunks of the x (dy) box this thread has just read
#pragma unroll
            for (int q = 0; q < 2; ++q)
              st_shared_v4(smem_u32(dyt) + sw128_off(row, half * 4 + h16 * 2 + q), ov[q].x, ov[q].y, ov[q].z, ov[q].w);
          }
        }
        if (TSTORE) {
          fence_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(&bars.out_ready[ib]);
        }
        if (MODE != 0) {
          if (P == 64) {   // the two column halves of a row belong to one head: combine through shared memory
            asm volatile("bar.sync 1, 256;" ::: "memory");   // previous block's exchange fully read
            if (half == 1) { sRed[row] = s0; sRed[256 + row] = s1; }
            asm volatile("bar.sync 1, 256;" ::: "memory");
            if (half == 0) { s0 += sRed[row]; s1 += sRed[256 + row]; }
          }
          if (P == 32 || half == 0) {
            const size_t co = ((size_t)(b * g.H + h_e) * g.nc + c) * QT + row;
            if (MODE == 1) {
              rs0[co] = s0;   // dcsp
              rs1[co] = s1;   // ddot
            } else {
              rs0[co] = dt_r > 0.f ? s0 / dt_r : 0.f;   // ddtd
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == Cfg::W_MMA) tmem_dealloc(tm, 512);
}

// ---------------------------------------------------------------------------------------------
// Backward chunk_scan, ungated case, dstate 64: the recompute pass (dcsp, ddot) and the dx pass of
// k_scan_ws share G and every M_h, so this kernel does both from one decay pass per head:
//   Y  = M_h X_h    (+) exp(cs_i) C S_prev^T                   -> dcsp[i] = sum_p dy*Y, ddot[i] = sum_p dy*x
//   U' = M_h^T dY_h (+) dt_j exp(cs_end-cs_j) B dS_end^T       -> dx = D dy + U', ddtd[j] = sum_p x*U' / dt_j
// Same roles, rings and parities as k_scan_ws.  TMEM: G x2 (256) + {Y, Y_off, U, U_off} (256, one
// slot: the epilogue hands it back as soon as it has read it).  The two state boxes (S_prev, dS_end)
// have a buffer of their own that is refilled while the second head of a block is worked on.
// dstate 128 (SPLIT): one C/B slot and one G; the S_prev and dS_end boxes (32 KB per head block at this width) pass as four
// 8 KB pieces through a two-slot ring with a producer lane and an issuer lane of their own (warps 19 and 18), so the state
// products run beside the head's own products and the whole plan stays inside 227 KB.
template <int P, int N_ = 64>
struct BwCfg {
  static constexpr int N = N_, NB64 = N_ / 64, HB = 64 / P, NM = 2, NT = 4;
  static constexpr bool SPLIT = N_ == 128;
  static constexpr int NCBS = SPLIT ? 1 : 2;
  static constexpr int CB_BYTES = 2 * NB64 * BOX_BYTES;      // C tile, B tile
  static constexpr int IN_BYTES = 2 * BOX_BYTES;             // x box, dy box
  static constexpr int ST_BYTES = 2 * SBOX_BYTES;            // dstate 64: S_prev box, dS_end box; dstate 128: two ring slots
  static constexpr int TB_BYTES = HB * TAB_BYTES;
  static constexpr int RED_BYTES = (P == 64) ? 3 * 256 * 4 : 0;
  static constexpr size_t SMEM = 1024 + NCBS * CB_BYTES + NM * 2 * BOX_BYTES + 2 * IN_BYTES + ST_BYTES + NT * TB_BYTES + RED_BYTES;
  static_assert(SMEM <= 232448, "shared-memory plan exceeds the 227 KB a CTA can have");
};

struct BwBars {
  uint64_t cb_full[2], cb_empty[2], g_full[2], g_empty[2], in_full[2], in_empty[2], m_full[2], m_empty[2];
  uint64_t tab_full[4], tab_empty[4], st_full, st_empty, acc_full, acc_empty, done;
  uint64_t stp_full[2], stp_empty[2];
};

template <int P, int N_ = 64>
__global__ void __launch_bounds__(WS_THREADS, 1)
k_bwd_ws(Geo g, const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmDY,
         const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmC,
         const __grid_constant__ CUtensorMap tmS, const __grid_constant__ CUtensorMap tmDS,
         const float* __restrict__ tab, const float* __restrict__ D, bf16* __restrict__ dx, float* __restrict__ dcsp,
         float* __restrict__ ddot, float* __restrict__ ddtd, int* __restrict__ status) {
  using Cfg = BwCfg<P, N_>;
  constexpr int N = Cfg::N, HB = Cfg::HB, NM = Cfg::NM, NB64 = Cfg::NB64, NCBS = Cfg::NCBS;
  constexpr bool SPLIT = Cfg::SPLIT;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);   // 1 KB aligned, still known to be shared memory
  uint8_t* sCB = smem;                                   // NCBS x {C tile, B tile}
  uint8_t* sM = sCB + NCBS * Cfg::CB_BYTES;              // NM x 32 KB
  uint8_t* sIn = sM + NM * 2 * BOX_BYTES;                // 2 x {x box, dy box}
  uint8_t* sSt = sIn + 2 * Cfg::IN_BYTES;                // S_prev box, dS_end box
  uint8_t* sTab = sSt + Cfg::ST_BYTES;                   // NT x decay tables of a head block
  float* sRed = (float*)(sTab + Cfg::NT * Cfg::TB_BYTES);
  __shared__ __align__(8) BwBars bars;
  __shared__ uint32_t tmem_slot;
  __shared__ int s_abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) s_abort = *(volatile int*)status;
  __syncthreads();
  if (s_abort) return;
  if (tid == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars.cb_full[i], 1); mbar_init(&bars.cb_empty[i], SPLIT ? 2 : 1);
      mbar_init(&bars.stp_full[i], 1); mbar_init(&bars.stp_empty[i], 1);
      mbar_init(&bars.g_full[i], 1); mbar_init(&bars.g_empty[i], WS_SCALE_WARPS);
      mbar_init(&bars.in_full[i], 1); mbar_init(&bars.in_empty[i], 1 + WS_EPI_WARPS);
      mbar_init(&bars.m_full[i], WS_SCALE_WARPS); mbar_init(&bars.m_empty[i], 1);
    }
    for (int i = 0; i < 4; ++i) { mbar_init(&bars.tab_full[i], 1); mbar_init(&bars.tab_empty[i], WS_SCALE_WARPS + WS_EPI_WARPS); }
    mbar_init(&bars.st_full, 1); mbar_init(&bars.st_empty, 1);
    mbar_init(&bars.acc_full, SPLIT ? 2 : 1); mbar_init(&bars.acc_empty, WS_EPI_WARPS);
    mbar_init(&bars.done, 1);
    mbar_fence_init();
  }
  if (warp == 17) tmem_alloc(&tmem_slot, 512);
  if (tid < 512) {
    for (int i = 0; i < NM; ++i) zero_upper_blocks(tid & 127, tid >> 7, warp, smem_u32(sM + i * 2 * BOX_BYTES));
    fence_async_smem();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = tmem_slot;
  const uint32_t tmYd = tm + 256, tmYo = tm + 320, tmUd = tm + 384, tmUo = tm + 448;
  Waiter w{status, false};

  const int nblk = g.hpg / HB;
  const int ntiles = g.B * g.G * g.nc;
  const int my_tiles = (ntiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
  auto tile_coords = [&](int t, int& b, int& grp, int& c) {
    const int u = blockIdx.x + t * gridDim.x;
    c = u % g.nc;
    const int r = u / g.nc;
    grp = r % g.G;
    b = r / g.G;
  };

  // the single-thread roles give registers back, the epilogue (widest live set) takes them
  if (warp == 16) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      auto load_cb = [&](int t) {
        int b, grp, c;
        tile_coords(t, b, grp, c);
        const int cs_ = t % NCBS;
        w.wait(&bars.cb_empty[cs_], ((t / NCBS) & 1) ^ 1, 41);
        uint8_t* dst = sCB + cs_ * Cfg::CB_BYTES;
        mbar_expect_tx(&bars.cb_full[cs_], Cfg::CB_BYTES);
#pragma unroll
        for (int j = 0; j < NB64; ++j) {
          tma_load_3d(dst + j * BOX_BYTES, &tmC, grp * N + 64 * j, c * QT, b, &bars.cb_full[cs_]);
          tma_load_3d(dst + (NB64 + j) * BOX_BYTES, &tmB, grp * N + 64 * j, c * QT, b, &bars.cb_full[cs_]);
        }
      };
      const int total_blocks = my_tiles * nblk;
      auto load_tab = [&](int kg) {
        if (kg >= total_blocks) return;
        int b, grp, c;
        tile_coords(kg / nblk, b, grp, c);
        const int h0 = grp * g.hpg + (kg % nblk) * HB, ts = kg % Cfg::NT;
        w.wait(&bars.tab_empty[ts], ((kg / Cfg::NT) & 1) ^ 1, 49);
        mbar_expect_tx(&bars.tab_full[ts], Cfg::TB_BYTES);
        bulk_load(sTab + ts * Cfg::TB_BYTES, tab + ((size_t)(b * g.nc + c) * g.H + h0) * TAB, Cfg::TB_BYTES, &bars.tab_full[ts]);
      };
      int kb = 0;
      load_cb(0);
      load_tab(0);
      load_tab(1);
      for (int t = 0; t < my_tiles; ++t) {
        int b, grp, c;
        tile_coords(t, b, grp, c);
        for (int blk = 0; blk < nblk; ++blk, ++kb) {
          load_tab(kb + 2);
          const int ib = kb & 1;
          const int h0 = grp * g.hpg + blk * HB, col = grp * g.hpg * P + blk * 64;
          w.wait(&bars.in_empty[ib], ((kb >> 1) & 1) ^ 1, 42);
          uint8_t* dst = sIn + ib * Cfg::IN_BYTES;
          mbar_expect_tx(&bars.in_full[ib], Cfg::IN_BYTES);
          tma_load_3d(dst, &tmX, col, c * QT, b, &bars.in_full[ib]);
          tma_load_3d(dst + BOX_BYTES, &tmDY, col, c * QT, b, &bars.in_full[ib]);
          if constexpr (!SPLIT) {
            w.wait(&bars.st_empty, (kb & 1) ^ 1, 50);
            mbar_expect_tx(&bars.st_full, Cfg::ST_BYTES);
            tma_load_3d(sSt, &tmS, 0, h0 * P, b * g.nc + c, &bars.st_full);
            tma_load_3d(sSt + SBOX_BYTES, &tmDS, 0, h0 * P, b * g.nc + c, &bars.st_full);
            if (blk == 0 && t + 1 < my_tiles) load_cb(t + 1);
          }
        }
        if (SPLIT && t + 1 < my_tiles) load_cb(t + 1);   // one C/B slot: after the tile's last block
      }
    }
  } else if (SPLIT && warp == 19) {
    // ------------------------------------------------------------------ dstate 128: producer of the state pieces
    // piece p of a head block: 0,1 = the two 64-column halves of S_prev, 2,3 = those of dS_end; piece q = 4 kb + p uses
    // ring slot q & 1 for the (q >> 1)-th time
    if (lane == 0) {
      int q = 0;
      for (int t = 0; t < my_tiles; ++t) {
        int b, grp, c;
        tile_coords(t, b, grp, c);
        for (int blk = 0; blk < nblk; ++blk) {
          const int h0 = grp * g.hpg + blk * HB;
          for (int p = 0; p < 4; ++p, ++q) {
            const int slot = q & 1;
            w.wait(&bars.stp_empty[slot], ((q >> 1) & 1) ^ 1, 60);
            mbar_expect_tx(&bars.stp_full[slot], SBOX_BYTES);
            tma_load_3d(sSt + slot * SBOX_BYTES, p < 2 ? &tmS : &tmDS, 64 * (p & 1), h0 * P, b * g.nc + c, &bars.stp_full[slot]);
          }
        }
      }
    }
  } else if (SPLIT && warp == 18) {
    // ------------------------------------------------------------------ dstate 128: issuer of the state products
    if (lane == 0) {
      const uint32_t idO = make_idesc(128, 64, 0, 0);
      const uint32_t tmYo_ = tm + 320, tmUo_ = tm + 448;
      int kb = 0, q = 0;
      for (int t = 0; t < my_tiles; ++t) {
        w.wait(&bars.cb_full[0], t & 1, 61);
        const uint32_t ct = smem_u32(sCB);
        for (int blk = 0; blk < nblk; ++blk, ++kb) {
          w.wait(&bars.acc_empty, (kb & 1) ^ 1, 62);
          for (int p = 0; p < 4; ++p, ++q) {
            const int slot = q & 1;
            w.wait(&bars.stp_full[slot], (q >> 1) & 1, 63);
            tc_fence_after();
            // C boxes 0,1 then B boxes 0,1 lie one after the other in the C/B slot: piece p multiplies box p
            const uint64_t dA = desc_sw128_k(ct + p * BOX_BYTES, 0), dS = desc_sw128_k(smem_u32(sSt + slot * SBOX_BYTES), 0);
#pragma unroll 1
            for (int ks = 0; ks < 4; ++ks)
              mma_bf16(p < 2 ? tmYo_ : tmUo_, desc_adv(dA, ks * 32), desc_adv(dS, ks * 32), idO, ((p & 1) | ks) > 0);
            mma_commit(&bars.stp_empty[slot]);
          }
          if (blk == nblk - 1) mma_commit(&bars.cb_empty[0]);
          mma_commit(&bars.acc_full);
        }
      }
    }
  } else if (warp == 17) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idG = make_idesc(128, 128, 0, 0);
      const uint32_t idY = make_idesc(128, P, 0, 1), idU = make_idesc(128, P, 1, 1), idO = make_idesc(128, 64, 0, 0);
      auto issue_g = [&](int t) {
        const int s_ = t % NCBS;
        w.wait(&bars.cb_full[s_], (t / NCBS) & 1, 43);
        w.wait(&bars.g_empty[s_], ((t / NCBS) & 1) ^ 1, 44);
        tc_fence_after();
        const uint32_t ct = smem_u32(sCB + s_ * Cfg::CB_BYTES);
#pragma unroll 1
        for (int j = 0; j < NB64; ++j) {
          const uint64_t dc = desc_sw128_k(ct + j * BOX_BYTES, 0), db = desc_sw128_k(ct + (NB64 + j) * BOX_BYTES, 0);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) mma_bf16(tm + s_ * 128, desc_adv(dc, ks * 32), desc_adv(db, ks * 32), idG, (j | ks) > 0);
        }
        mma_commit(&bars.g_full[s_]);
      };
      issue_g(0);
      const uint64_t dS0 = desc_sw128_k(smem_u32(sSt), 0), dDS0 = desc_sw128_k(smem_u32(sSt + SBOX_BYTES), 0);
      int kb = 0, kh = 0;
      for (int t = 0; t < my_tiles; ++t) {
        const uint32_t ct = smem_u32(sCB + (t % NCBS) * Cfg::CB_BYTES);
        const uint64_t dC0 = desc_sw128_k(ct, 0), dB0 = desc_sw128_k(ct + BOX_BYTES, 0);
        for (int blk = 0; blk < nblk; ++blk, ++kb) {
          const int ib = kb & 1;
          const uint32_t inb = smem_u32(sIn + ib * Cfg::IN_BYTES);
          w.wait(&bars.in_full[ib], (kb >> 1) & 1, 45);
          if (!SPLIT) w.wait(&bars.st_full, kb & 1, 57);
          w.wait(&bars.acc_empty, (kb & 1) ^ 1, 46);
          for (int hl = 0; hl < HB; ++hl, ++kh) {
            const int ms = kh % NM;
            w.wait(&bars.m_full[ms], (kh / NM) & 1, 47);
            tc_fence_after();
            const uint32_t mt = smem_u32(sM + ms * 2 * BOX_BYTES);
            const uint64_t dMk = desc_plain_k(mt, 128, 0), dMt = desc_plain_mn(mt, 128, 0, 0);
            const uint64_t dX0 = desc_sw128_mn(inb, 0, hl * P * 2, 16), dY0 = desc_sw128_mn(inb + BOX_BYTES, 0, hl * P * 2, 16);
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
              mma_bf16(tmYd + hl * P, desc_adv(dMk, ks * 4096), desc_adv(dX0, ks * 2048), idY, ks > 0);
              mma_bf16(tmUd + hl * P, desc_adv(dMt, ks * 256), desc_adv(dY0, ks * 2048), idU, ks > 0);
            }
            if (!SPLIT && hl == 0) {
#pragma unroll
              for (int ks = 0; ks < 4; ++ks) {
                mma_bf16(tmYo, desc_adv(dC0, ks * 32), desc_adv(dS0, ks * 32), idO, ks > 0);
                mma_bf16(tmUo, desc_adv(dB0, ks * 32), desc_adv(dDS0, ks * 32), idO, ks > 0);
              }
              mma_commit(&bars.st_empty);
            }
            mma_commit(&bars.m_empty[ms]);
          }
          mma_commit(&bars.in_empty[ib]);
          if (blk == nblk - 1) mma_commit(&bars.cb_empty[t % NCBS]);
          mma_commit(&bars.acc_full);
          if (!SPLIT && blk == 0 && t + 1 < my_tiles) issue_g(t + 1);
        }
        if (SPLIT && t + 1 < my_tiles) issue_g(t + 1);
      }
      mma_commit(&bars.done);
      w.wait(&bars.done, 0, 48);
    }
  } else if (warp < WS_SCALE_WARPS) {
    // ------------------------------------------------------------------ decay pass warps (they hand registers to the epilogue)
    reg_dec<64>();
    const int row = tid & 127, part = tid >> 7;
    int kb = 0, kh = 0;
    for (int t = 0; t < my_tiles; ++t) {
      const int gs = t % NCBS;
      w.wait(&bars.g_full[gs], (t / NCBS) & 1, 51);
      tc_fence_after();
      for (int blk = 0; blk < nblk; ++blk, ++kb) {
        const int ts = kb % Cfg::NT;
        const float* tb = (const float*)(sTab + ts * Cfg::TB_BYTES);
        w.wait(&bars.tab_full[ts], (kb / Cfg::NT) & 1, 52);
        for (int hl = 0; hl < HB; ++hl, ++kh) {
          const int ms = kh % NM;
          w.wait(&bars.m_empty[ms], ((kh / NM) & 1) ^ 1, 53);
          decay_mask_tile(tm + gs * 128, tb + hl * TAB, row, part, warp, smem_u32(sM + ms * 2 * BOX_BYTES));
          fence_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(&bars.m_full[ms]);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars.tab_empty[ts]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars.g_empty[gs]);
    }
  } else if (warp >= 20) {
    // ------------------------------------------------------------------ epilogue warps
    reg_inc<88>();
    const int ew = warp - 20;
    const int row = (ew & 3) * 32 + lane, half = ew >> 2;     // 32 of the block's 64 columns
    const int hl_e = (half * 32) / P;
    int kb = 0;
    for (int t = 0; t < my_tiles; ++t) {
      int b, grp, c;
      tile_coords(t, b, grp, c);
      const int t_row = c * QT + row;
      for (int blk = 0; blk < nblk; ++blk, ++kb) {
        const int ib = kb & 1, ts = kb % Cfg::NT;
        const uint32_t xt = smem_u32(sIn + ib * Cfg::IN_BYTES), dyt = xt + BOX_BYTES;
        const float* tb = (const float*)(sTab + ts * Cfg::TB_BYTES) + hl_e * TAB;
        const int h0 = grp * g.hpg + blk * HB, h_e = h0 + hl_e;
        const float Dh = D ? __ldg(D + h_e) : 0.f;
        w.wait(&bars.tab_full[ts], (kb / Cfg::NT) & 1, 56);
        const uint32_t tbs = smem_u32(tb);
        const float cs_r = lds_f32(tbs + 4 * (T_CS + row)), dt_r = lds_f32(tbs + 4 * (T_DT + row));
        const float osc_y = ex2(cs_r), osc_u = dt_r * ex2(lds_f32(tbs + 4 * (T_CS + 127)) - cs_r);
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars.tab_empty[ts]);
        w.wait(&bars.in_full[ib], (kb >> 1) & 1, 54);
        w.wait(&bars.acc_full, kb & 1, 55);
        tc_fence_after();
        const size_t dense = ((size_t)b * g.L + t_row) * g.H * P + (size_t)h0 * P + half * 32;
        float s0 = 0.f, s1 = 0.f, s2 = 0.f;
#pragma unroll
        for (int ph = 0; ph < 4; ++ph) {          // ph 0,1: Y slices; ph 2,3: U' slices (16 columns each)
          const int h16 = ph & 1;
          const bool upass = ph >= 2;
          uint4 xv[2], dv[2];
          float a16[16], o16[16];
#pragma unroll
          for (int q = 0; q < 2; ++q) {
            xv[q] = ld_shared_v4(xt + sw128_off(row, half * 4 + h16 * 2 + q));
            dv[q] = ld_shared_v4(dyt + sw128_off(row, half * 4 + h16 * 2 + q));
          }
          {   // both accumulator slices in flight, one wait
            uint32_t ra[16], ro[16];
            tmem_ld16_issue(tmem_addr(upass ? tmUd : tmYd, (ew & 3) * 32, half * 32 + h16 * 16), ra);
            tmem_ld16_issue(tmem_addr(upass ? tmUo : tmYo, (ew & 3) * 32, half * 32 + h16 * 16), ro);
            tmem_ld_wait_2x16(ra, ro);
#pragma unroll
            for (int k = 0; k < 16; ++k) { a16[k] = __uint_as_float(ra[k]); o16[k] = __uint_as_float(ro[k]); }
          }
          if (ph == 3) {   // everything read: hand the accumulators and the input slot back
            tc_fence_before();
            __syncwarp();
            if (lane == 0) { mbar_arrive(&bars.acc_empty); mbar_arrive(&bars.in_empty[ib]); }
          }
          const float osc = upass ? osc_u : osc_y;
          uint4 ov[2];
#pragma unroll
          for (int q = 0; q < 2; ++q) {
            float xs[8], dys[8];
            unpack8(xv[q], xs);
            unpack8(dv[q], dys);
            if (!upass) {
#pragma unroll
              for (int k = 0; k < 8; ++k) {
                const float acc = a16[q * 8 + k] + osc * o16[q * 8 + k];
                s0 = fmaf(dys[k], acc, s0);
                s1 = fmaf(dys[k], xs[k], s1);
              }
            } else {
              float o[8];
#pragma unroll
              for (int k = 0; k < 8; ++k) {
                const float acc = a16[q * 8 + k] + osc * o16[q * 8 + k];
                o[k] = acc + Dh * dys[k];
                s2 = fmaf(xs[k], acc, s2);
              }
              ov[q] = pack8(o);
            }
          }
          if (upass) st_global_32B(dx + dense + h16 * 16, ov[0], ov[1]);
        }
        if (P == 64) {   // the two column halves of a row belong to one head: combine through shared memory
          asm volatile("bar.sync 1, 256;" ::: "memory");
          if (half == 1) { sRed[row] = s0; sRed[256 + row] = s1; sRed[512 + row] = s2; }
          asm volatile("bar.sync 1, 256;" ::: "memory");
          if (half == 0) { s0 += sRed[row]; s1 += sRed[256 + row]; s2 += sRed[512 + row]; }
        }
        if (P == 32 || half == 0) {
          const size_t co = ((size_t)(b * g.H + h_e) * g.nc + c) * QT + row;
          dcsp[co] = s0;
          ddot[co] = s1;
          ddtd[co] = dt_r > 0.f ? s2 / dt_r : 0.f;
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 17) tmem_dealloc(tm, 512);
}

// ---------------------------------------------------------------------------------------------
// Backward dB / dC, dstate 64, persistent and warp-specialised like k_scan_ws.
//
// Block path (any head).  Per head W_h = dY_h X_h^T (K = P) into one of two TMEM slots -> decay pass (32x32 blocks, the
// factorisation of decay_mask_tile) -> W'_h as bf16 in shared memory -> dC += W'_h B, dB += W'_h^T C.
// Per head block, once its raw x / dy boxes are no longer needed by a W product, the decay warps scale them in place and
// one K = 64 product each adds the state terms dC += dY' S_prev, dB += X' dS_end.  dC / dB stay in TMEM for the whole tile.
//
// Separable heads.  exp(cs_i - cs_j) dt_j = a_i b_j with a_i = exp(cs_i), b_j = exp(-cs_j) dt_j, and dC, dB are linear in
// W'_h, so for a head whose decay over a chunk stays inside the range of the storage type (|cs_end| <= SSD_SEP_LOG_RANGE for
// every chunk of the call; the cumsum kernel records the per-head maximum) the decay can ride on the OPERANDS:
//   sum_h W'_h = tril( sum_h (a_h o dY_h) (b_h o X_h)^T ),
// one accumulator for all such heads of the tile, filled by the tensor core from the boxes the decay warps scale in place
// anyway for the state terms (dy by a, x by b; the factor exp(cs_end) that the x-side state term then lacks goes onto the
// rows of the dS_end box).  Those heads need no per-head pass over a 128x128 tile at all; once per tile the accumulator is
// masked to its lower triangle and multiplied like one more W'_h.  Heads outside the range (strong decay: a_i or b_j alone
// would leave the range although every a_i b_j with j <= i is at most dt_j) keep the block path.
//
// With the per-head pass gone for most heads a tile is a short chain of scale -> multiply steps, and what bounds the kernel
// is how far the loads run ahead of it: the x/dy boxes have a ring of three, the state boxes of two, the tables of four;
// the B/C tiles (read at the END of a tile by the separable path) and the W' tile are single.

template <int P>
struct DbCfg {
  static constexpr int N = 64, HB = 64 / P, NT = 4, NIN = 3, NST = 2;
  static constexpr int CB_BYTES = 2 * BOX_BYTES;             // B tile, C tile
  static constexpr int IN_BYTES = 2 * BOX_BYTES;             // x box, dy box
  static constexpr int ST_BYTES = 2 * SBOX_BYTES;            // S_prev box, dS_end box
  static constexpr int TB_BYTES = HB * TAB_BYTES;
  static constexpr size_t SMEM = 1024 + CB_BYTES + 2 * BOX_BYTES + NIN * IN_BYTES + NST * ST_BYTES + NT * TB_BYTES;
};

struct DbBars {
  uint64_t cb_full, cb_empty, in_full[3], in_empty[3], w_full[2], w_empty[2], m_full, m_empty;
  uint64_t tab_full[4], tab_empty[4], st_full[2], st_empty[2], wraw_done[3], sc_full[3], acc_full, acc_empty, done;
  uint64_t wsep_full, wsep_empty;
};

template <int P>
__global__ void __launch_bounds__(WS_THREADS, 1)
k_dbc_ws(Geo g, const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmDY,
         const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmC,
         const __grid_constant__ CUtensorMap tmS, const __grid_constant__ CUtensorMap tmDS,
         const float* __restrict__ tab, const float* __restrict__ hmax, bf16* __restrict__ dB, bf16* __restrict__ dC,
         int* __restrict__ status) {
  using Cfg = DbCfg<P>;
  constexpr int N = Cfg::N, HB = Cfg::HB, NIN = Cfg::NIN, NST = Cfg::NST, NT = Cfg::NT;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);   // 1 KB aligned, still known to be shared memory
  uint8_t* sCB = smem;                                   // {B tile, C tile} of the current tile
  uint8_t* sM = sCB + Cfg::CB_BYTES;                     // one 32 KB W' tile
  uint8_t* sIn = sM + 2 * BOX_BYTES;                     // NIN x {x box, dy box}
  uint8_t* sSt = sIn + NIN * Cfg::IN_BYTES;              // NST x {S_prev box, dS_end box}
  uint8_t* sTab = sSt + NST * Cfg::ST_BYTES;             // NT x decay tables of a head block
  __shared__ __align__(8) DbBars bars;
  __shared__ uint32_t tmem_slot;
  __shared__ int s_abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) s_abort = *(volatile int*)status;
  __syncthreads();
  if (s_abort) return;
  if (tid == 0) {
    // two MMA issuer lanes (dC side, dB side): tcgen05.commit tracks the MMAs of its own thread only, so every barrier that
    // releases something both of them read expects one commit from each
    mbar_init(&bars.cb_full, 1); mbar_init(&bars.cb_empty, 2);
    for (int i = 0; i < NIN; ++i) {
      mbar_init(&bars.in_full[i], 1); mbar_init(&bars.in_empty[i], 2);
      mbar_init(&bars.wraw_done[i], 1); mbar_init(&bars.sc_full[i], WS_SCALE_WARPS);
    }
    for (int i = 0; i < 2; ++i) { mbar_init(&bars.w_full[i], 1); mbar_init(&bars.w_empty[i], WS_SCALE_WARPS); }
    mbar_init(&bars.m_full, WS_SCALE_WARPS); mbar_init(&bars.m_empty, 2);
    for (int i = 0; i < NT; ++i) { mbar_init(&bars.tab_full[i], 1); mbar_init(&bars.tab_empty[i], WS_SCALE_WARPS); }
    for (int i = 0; i < NST; ++i) { mbar_init(&bars.st_full[i], 1); mbar_init(&bars.st_empty[i], 2); }
    mbar_init(&bars.acc_full, 2); mbar_init(&bars.acc_empty, WS_EPI_WARPS);
    mbar_init(&bars.done, 2);
    mbar_init(&bars.wsep_full, 1); mbar_init(&bars.wsep_empty, WS_SCALE_WARPS);
    mbar_fence_init();
  }
  if (warp == 17) tmem_alloc(&tmem_slot, 512);
  if (tid < 512) {
    zero_upper_blocks(tid & 127, tid >> 7, warp, smem_u32(sM));
    fence_async_smem();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = tmem_slot;
  const uint32_t tmDC = tm + 256, tmDB = tm + 320, tmWsep = tm + 384;
  Waiter w{status, false};
  // which heads take the separable path: one bit per head, the same in every role (up to 64 heads; beyond that none)
  unsigned long long sepmask = 0ull;
  if (hmax && g.H <= 64) {
    const int* tags = reinterpret_cast<const int*>(hmax);
    const int cur = __ldg(tags + g.H);
    for (int h = 0; h < g.H; ++h)
      if (__ldg(tags + h) != cur) sepmask |= 1ull << h;
  }
  auto is_sep = [&](int h) { return ((sepmask >> h) & 1ull) != 0; };
  auto group_has_sep = [&](int grp) {
    const unsigned long long gm = (g.hpg >= 64 ? ~0ull : ((1ull << g.hpg) - 1ull)) << (grp * g.hpg);
    return (sepmask & gm) != 0ull;
  };

  const int nblk = g.hpg / HB;
  const int ntiles = g.B * g.G * g.nc;
  const int my_tiles = (ntiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
  auto tile_coords = [&](int t, int& b, int& grp, int& c) {
    const int u = blockIdx.x + t * gridDim.x;
    c = u % g.nc;
    const int r = u / g.nc;
    grp = r % g.G;
    b = r / g.G;
  };
  // use n (0, 1, 2, ...) of a ring of depth D sits in slot n % D; its `full` wait has parity (n / D) & 1, its `empty` wait the
  // opposite (a fresh barrier passes a wait on parity 1)
  auto par = [](int n, int depth) { return (uint32_t)((n / depth) & 1); };

  // registers: the single-thread roles (warps 16-19, one aligned group of four) and the epilogue hand some back, the decay
  // warps take them (80 * 512 + 64 * 128 + 48 * 256 <= the launch-time 72 * 896)
  if (warp >= 16 && warp < 20) reg_dec<64>();
  if (warp == 16) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      const int total_blocks = my_tiles * nblk;
      auto load_tab = [&](int kg) {
        if (kg >= total_blocks) return;
        int b, grp, c;
        tile_coords(kg / nblk, b, grp, c);
        const int h0 = grp * g.hpg + (kg % nblk) * HB, ts = kg % NT;
        w.wait(&bars.tab_empty[ts], par(kg, NT) ^ 1, 49);
        mbar_expect_tx(&bars.tab_full[ts], Cfg::TB_BYTES);
        bulk_load(sTab + ts * Cfg::TB_BYTES, tab + ((size_t)(b * g.nc + c) * g.H + h0) * TAB, Cfg::TB_BYTES, &bars.tab_full[ts]);
      };
      int kb = 0;
      load_tab(0);
      load_tab(1);
      for (int t = 0; t < my_tiles; ++t) {
        int b, grp, c;
        tile_coords(t, b, grp, c);
        for (int blk = 0; blk < nblk; ++blk, ++kb) {
          load_tab(kb + 2);
          const int ib = kb % NIN, sb = kb % NST;
          const int h0 = grp * g.hpg + blk * HB, col = grp * g.hpg * P + blk * 64;
          w.wait(&bars.in_empty[ib], par(kb, NIN) ^ 1, 42);
          uint8_t* dst = sIn + ib * Cfg::IN_BYTES;
          mbar_expect_tx(&bars.in_full[ib], Cfg::IN_BYTES);
          tma_load_3d(dst, &tmX, col, c * QT, b, &bars.in_full[ib]);
          tma_load_3d(dst + BOX_BYTES, &tmDY, col, c * QT, b, &bars.in_full[ib]);
          w.wait(&bars.st_empty[sb], par(kb, NST) ^ 1, 50);
          uint8_t* sd = sSt + sb * Cfg::ST_BYTES;
          mbar_expect_tx(&bars.st_full[sb], Cfg::ST_BYTES);
          tma_load_3d(sd, &tmS, 0, h0 * P, b * g.nc + c, &bars.st_full[sb]);
          tma_load_3d(sd + SBOX_BYTES, &tmDS, 0, h0 * P, b * g.nc + c, &bars.st_full[sb]);
          // this tile's B / C: single buffer, free once the previous tile's last products have completed; requested behind
          // the tile's first boxes so that this wait does not hold the box stream back
          if (blk == (nblk > 1 ? 1 : 0)) {
            w.wait(&bars.cb_empty, (t & 1) ^ 1, 41);
            mbar_expect_tx(&bars.cb_full, Cfg::CB_BYTES);
            tma_load_3d(sCB, &tmB, grp * N, c * QT, b, &bars.cb_full);
            tma_load_3d(sCB + BOX_BYTES, &tmC, grp * N, c * QT, b, &bars.cb_full);
          }
        }
      }
    }
  } else if (warp == 17 || warp == 18) {
    // ------------------------------------------------------------------ MMA issuers.  The products are split by side:
    // lane A (warp 17) issues every W product and everything that accumulates into dC, lane B (warp 18) everything into dB.
    if (lane == 0) {
      const bool side_c = warp == 17;
      const uint32_t idW = make_idesc(128, 128, 0, 0), idC = make_idesc(128, N, 0, 1), idB = make_idesc(128, N, 1, 1);
      const int total_blocks = my_tiles * nblk;
      int kw = 0;   // W products of block-path heads issued so far
      auto issue_w_block = [&](int kg) {   // the W products of global block kg's heads on the block path (lane A only)
        if (kg >= total_blocks) return;
        const int ib = kg % NIN;
        int bb, gg, cc;
        tile_coords(kg / nblk, bb, gg, cc);
        const int h0 = gg * g.hpg + (kg % nblk) * HB;
        bool any_block_path = false;
        for (int hl = 0; hl < HB; ++hl) any_block_path |= !is_sep(h0 + hl);
        if (!any_block_path) {   // nothing reads the raw boxes: release them at once, without waiting for them to land
          mbar_arrive(&bars.wraw_done[ib]);
          return;
        }
        w.wait(&bars.in_full[ib], par(kg, NIN), 45);
        tc_fence_after();
        const uint32_t inb = smem_u32(sIn + ib * Cfg::IN_BYTES);
        const uint64_t dX0 = desc_sw128_k(inb, 0), dDY0 = desc_sw128_k(inb + BOX_BYTES, 0);
        for (int hl = 0; hl < HB; ++hl) {
          if (is_sep(h0 + hl)) continue;
          const int ws = kw & 1;
          w.wait(&bars.w_empty[ws], par(kw, 2) ^ 1, 58);
          tc_fence_after();
#pragma unroll
          for (int ks = 0; ks < P / 16; ++ks)
            mma_bf16(tm + ws * 128, desc_adv(dDY0, hl * P * 2 + ks * 32), desc_adv(dX0, hl * P * 2 + ks * 32), idW, ks > 0);
          mma_commit(&bars.w_full[ws]);
          ++kw;
        }
        mma_commit(&bars.wraw_done[ib]);   // the raw boxes of this block have been read by every W product
      };
      if (side_c) issue_w_block(0);
      const uint64_t dBm0 = desc_sw128_mn(smem_u32(sCB), 0, 0, BOX_BYTES), dCm0 = desc_sw128_mn(smem_u32(sCB) + BOX_BYTES, 0, 0, BOX_BYTES);
      const uint32_t mt = smem_u32(sM);
      const uint64_t dMk = desc_plain_k(mt, 128, 0), dMt = desc_plain_mn(mt, 128, 0, 0);
      int kb = 0, kh = 0, ksep = 0;   // kh: W' tiles consumed; ksep: tiles with separable heads so far
      for (int t = 0; t < my_tiles; ++t) {
        w.wait(&bars.acc_empty, (t & 1) ^ 1, 46);
        tc_fence_after();
        int tb_, tg_, tc_;
        tile_coords(t, tb_, tg_, tc_);
        const bool anysep = group_has_sep(tg_);
        bool first = true, firstsep = true, have_cb = false;
        auto issue_m = [&]() {   // the W' tile -> dC (lane A) or dB (lane B)
          if (!have_cb) { w.wait(&bars.cb_full, t & 1, 43); have_cb = true; }
          w.wait(&bars.m_full, kh & 1, 47);
          tc_fence_after();
          if (side_c) {
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) mma_bf16(tmDC, desc_adv(dMk, ks * 4096), desc_adv(dBm0, ks * 2048), idC, !first || ks > 0);
          } else {
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) mma_bf16(tmDB, desc_adv(dMt, ks * 256), desc_adv(dCm0, ks * 2048), idB, !first || ks > 0);
          }
          first = false;
          mma_commit(&bars.m_empty);
          ++kh;
        };
        for (int blk = 0; blk < nblk; ++blk, ++kb) {
          const int ib = kb % NIN, sb = kb % NST;
          const uint32_t inb = smem_u32(sIn + ib * Cfg::IN_BYTES), stb = smem_u32(sSt + sb * Cfg::ST_BYTES);
          const int h0 = tg_ * g.hpg + blk * HB;
          for (int hl = 0; hl < HB; ++hl)
            if (!is_sep(h0 + hl)) issue_m();
          // the next block's W products go out before this block's state terms, so the decay warps
          // find their next input ready when they come back from scaling this block's boxes
          if (side_c) issue_w_block(kb + 1);
          w.wait(&bars.sc_full[ib], par(kb, NIN), 59);
          w.wait(&bars.st_full[sb], par(kb, NST), 57);
          tc_fence_after();
          if (side_c) {
            const uint64_t dDYk = desc_sw128_k(inb + BOX_BYTES, 0), dXk = desc_sw128_k(inb, 0);
            const uint64_t dSm0 = desc_sw128_mn(stb, 0, 0, SBOX_BYTES);
            // separable heads of this block: their W, decay included, adds up in one accumulator for the whole tile
            for (int hl = 0; hl < HB; ++hl) {
              if (!is_sep(h0 + hl)) continue;
              if (firstsep) w.wait(&bars.wsep_empty, (ksep & 1) ^ 1, 60);   // the decay warps have read the previous tile's sum
#pragma unroll
              for (int ks = 0; ks < P / 16; ++ks)
                mma_bf16(tmWsep, desc_adv(dDYk, hl * P * 2 + ks * 32), desc_adv(dXk, hl * P * 2 + ks * 32), idW, !firstsep || ks > 0);
              firstsep = false;
            }
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) mma_bf16(tmDC, desc_adv(dDYk, ks * 32), desc_adv(dSm0, ks * 2048), idC, !first || ks > 0);
          } else {
            const uint64_t dXk = desc_sw128_k(inb, 0);
            const uint64_t dDSm0 = desc_sw128_mn(stb + SBOX_BYTES, 0, 0, SBOX_BYTES);
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) mma_bf16(tmDB, desc_adv(dXk, ks * 32), desc_adv(dDSm0, ks * 2048), idC, !first || ks > 0);
          }
          first = false;
          mma_commit(&bars.st_empty[sb]);
          mma_commit(&bars.in_empty[ib]);
        }
        if (anysep) {
          if (side_c) mma_commit(&bars.wsep_full);
          ++ksep;
          issue_m();   // the masked sum of the separable heads, handed over by the decay warps like one more W'_h
        }
        if (!have_cb) w.wait(&bars.cb_full, t & 1, 43);   // keep the barrier's phases in step even if nothing read the tiles
        mma_commit(&bars.cb_empty);
        mma_commit(&bars.acc_full);
      }
      mma_commit(&bars.done);
      w.wait(&bars.done, 0, 48);
    }
  } else if (warp < WS_SCALE_WARPS) {
    // ------------------------------------------------------------------ decay pass warps
    reg_inc<80>();
    const int row = tid & 127, part = tid >> 7;
    int kb = 0, kh = 0, kw = 0, ksep = 0;
    for (int t = 0; t < my_tiles; ++t) {
      int tb_, tg_, tc_;
      tile_coords(t, tb_, tg_, tc_);
      const bool anysep = group_has_sep(tg_);
      for (int blk = 0; blk < nblk; ++blk, ++kb) {
        const int ts = kb % NT, ib = kb % NIN, sb = kb % NST;
        const int h0 = tg_ * g.hpg + blk * HB;
        const float* tb = (const float*)(sTab + ts * Cfg::TB_BYTES);
        const uint32_t tbs = smem_u32(sTab + ts * Cfg::TB_BYTES);
        w.wait(&bars.tab_full[ts], par(kb, NT), 52);
        for (int hl = 0; hl < HB; ++hl) {
          if (is_sep(h0 + hl)) continue;
          const int ws = kw & 1;
          w.wait(&bars.w_full[ws], par(kw, 2), 51);
          w.wait(&bars.m_empty, (kh & 1) ^ 1, 53);
          tc_fence_after();
          decay_mask_tile(tm + ws * 128, tb + hl * TAB, row, part, warp, smem_u32(sM));
          fence_async_smem();

          tc_fence_before();
          __syncwarp();
          if (lane == 0) { mbar_arrive(&bars.m_full); mbar_arrive(&bars.w_empty[ws]); }
          ++kh;
          ++kw;
        }
        // scale this block's boxes in place for the state terms (x: box 0, dy: box 1).  Block-path heads: x by
        // exp(cs_end - cs_j) dt_j.  Separable heads: x by b_j = exp(-cs_j) dt_j (the operand of their W product as well),
        // and the missing exp(cs_end) goes onto their rows of the dS_end box.
        w.wait(&bars.in_full[ib], par(kb, NIN), 54);
        w.wait(&bars.wraw_done[ib], par(kb, NIN), 55);
        uint8_t* xb = sIn + ib * Cfg::IN_BYTES;
        // four 16-byte pieces per thread (x box: two, dy box: two): all loads first, then the factors, then the arithmetic,
        // so that one warp has several independent chains in flight (four decay warps share a scheduler)
        {
          uint32_t adr[4];
          uint4 raw[4];
          float fac[4];
#pragma unroll
          for (int r = 0; r < 4; ++r) {
            const int idx = tid + r * 512;
            const int box = idx >> 10, l = (idx >> 3) & 127, pc = idx & 7;
            adr[r] = smem_u32(xb + box * BOX_BYTES + l * 128 + pc * 16);
            raw[r] = ld_shared_v4(adr[r]);
          }
#pragma unroll
          for (int r = 0; r < 4; ++r) {
            const int idx = tid + r * 512;
            const int box = idx >> 10, l = (idx >> 3) & 127, pc = idx & 7;
            const int hl = (((pc ^ l) & 7) * 8) / P;
            const uint32_t tt = tbs + hl * TAB_BYTES;
            const float csl = lds_f32(tt + 4 * (T_CS + l));
            fac[r] = box ? ex2(csl)
                         : (is_sep(h0 + hl) ? ex2(-csl) : ex2(lds_f32(tt + 4 * (T_CS + 127)) - csl)) * lds_f32(tt + 4 * (T_DT + l));
          }
#pragma unroll
          for (int r = 0; r < 4; ++r) raw[r] = scale8_bf16(raw[r], fac[r]);
#pragma unroll
          for (int r = 0; r < 4; ++r) st_shared_v4(adr[r], raw[r].x, raw[r].y, raw[r].z, raw[r].w);
        }
        if (anysep) {
          w.wait(&bars.st_full[sb], par(kb, NST), 61);
          const int r = tid >> 3;                      // row (h,p) of the 64 x 64 dS_end box, one 16-byte piece per thread
          const int hl = r / P;
          if (is_sep(h0 + hl)) {
            const float f = ex2(lds_f32(tbs + hl * TAB_BYTES + 4 * (T_CS + 127)));
            const uint32_t a = smem_u32(sSt + sb * Cfg::ST_BYTES + SBOX_BYTES + r * 128 + (tid & 7) * 16);
            const uint4 o = scale8_bf16(ld_shared_v4(a), f);
            st_shared_v4(a, o.x, o.y, o.z, o.w);
          }
        }
        fence_async_smem();
        __syncwarp();
        if (lane == 0) { mbar_arrive(&bars.sc_full[ib]); mbar_arrive(&bars.tab_empty[ts]); }
      }
      if (anysep) {   // the separable heads' sum: mask to the lower triangle, hand over like one more W'_h
        w.wait(&bars.wsep_full, ksep & 1, 62);
        ++ksep;
        w.wait(&bars.m_empty, (kh & 1) ^ 1, 53);
        tc_fence_after();
        mask_tril_tile(tmWsep, row, part, warp, smem_u32(sM));
        fence_async_smem();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) { mbar_arrive(&bars.m_full); mbar_arrive(&bars.wsep_empty); }
        ++kh;
      }
    }
  } else if (warp >= 20) {
    // ------------------------------------------------------------------ epilogue warps: dC, dB of a finished tile
    reg_dec<48>();
    const int ew = warp - 20;
    const int row = (ew & 3) * 32 + lane, half = ew >> 2;     // 32 of the 64 columns
    for (int t = 0; t < my_tiles; ++t) {
      int b, grp, c;
      tile_coords(t, b, grp, c);
      w.wait(&bars.acc_full, t & 1, 56);
      tc_fence_after();
      const size_t o = (((size_t)b * g.L + c * QT + row) * g.G + grp) * N + half * 32;
#pragma unroll
      for (int j = 0; j < 32; j += 16) {
        float vc[16], vb[16];
        tmem_ld16(tmem_addr(tmDC, (ew & 3) * 32, half * 32 + j), vc);
        tmem_ld16(tmem_addr(tmDB, (ew & 3) * 32, half * 32 + j), vb);
        if (j == 16) {   // both accumulators are in registers: hand them back before the stores
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&bars.acc_empty);
        }
        st_global_32B(dC + o + j,
                      make_uint4(pack_bf16(vc[0], vc[1]), pack_bf16(vc[2], vc[3]), pack_bf16(vc[4], vc[5]), pack_bf16(vc[6], vc[7])),
                      make_uint4(pack_bf16(vc[8], vc[9]), pack_bf16(vc[10], vc[11]), pack_bf16(vc[12], vc[13]), pack_bf16(vc[14], vc[15])));
        st_global_32B(dB + o + j,
                      make_uint4(pack_bf16(vb[0], vb[1]), pack_bf16(vb[2], vb[3]), pack_bf16(vb[4], vb[5]), pack_bf16(vb[6], vb[7])),
                      make_uint4(pack_bf16(vb[8], vb[9]), pack_bf16(vb[10], vb[11]), pack_bf16(vb[12], vb[13]), pack_bf16(vb[14], vb[15])));
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 17) tmem_dealloc(tm, 512);
}

// ---------------------------------------------------------------------------------------------
// Exclusive scan over chunks, 4 state elements per thread, decays staged in shared memory.
// Optionally also writes the bf16 copy of the chunk-entry states that the tensor kernels load.
// The reverse scan (state gradient) can also emit, per chunk, this block's warp-partial sums of
// <dS_end_c, S_end_c> (S_end_c = forward state entering chunk c+1, or the final state), which is
// the per-chunk term of the dt*A gradient: `sdot` [B, nc, H, gridDim.x * 8].
template <bool WRITE, bool BFDOT = false>
__global__ void __launch_bounds__(256, BFDOT ? 3 : 1) k_state_passing_v4(Geo g, float* __restrict__ st, const float* __restrict__ cs,
                                                          const float* __restrict__ init, float* __restrict__ last,
                                                          bf16* __restrict__ st_bf, int reverse,
                                                          const float* __restrict__ fwd_prev,
                                                          const bf16* __restrict__ fwd_prev_bf,
                                                          const float* __restrict__ fwd_fin, float* __restrict__ sdot) {
  extern __shared__ float sdec[];  // [nc]
  // fp32 chunk-entry states have no reader in this family: the reverse scans form <dS_end, S_end> from the bf16 copy (here
  // given as `fwd_prev_bf`), so a scan that writes the copy leaves the fp32 values unwritten: 2 of its 5 bytes per element
  const int h = blockIdx.y, b = blockIdx.z;
  const int PN = g.P * g.N;
  for (int c = threadIdx.x; c < g.nc; c += blockDim.x)
    sdec[c] = expf(cs[((size_t)(b * g.H + h) * g.nc + c) * g.Q + g.Q - 1]);
  __syncthreads();
  const int e = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
  const bool valid = e < PN;
  const int eo = valid ? e : 0;
  float4 run = (init && valid) ? *reinterpret_cast<const float4*>(init + ((size_t)(b * g.H + h)) * PN + eo)
                               : make_float4(0.f, 0.f, 0.f, 0.f);
  const size_t cstride = (size_t)g.H * PN;
  const size_t boff = ((size_t)b * g.nc * g.H + h) * PN + eo;
  float* base = st + boff;
  const int nw = gridDim.x * 8, wslot = blockIdx.x * 8 + (threadIdx.x >> 5);
  // chunks in flight per thread.  The scan is bound by the bytes it keeps in flight (B * H * P * N / 4 threads, each with U
  // loads per stream outstanding): the narrower bf16 loads need more steps to keep as many, within the 85 registers
  // that leave three blocks per SM (two would put the 384 blocks of a B2 H24 pass into two waves)
  // chunks in flight per thread.  The scan is bound by the bytes it keeps in flight (B * H * P * N / 4 threads): the
  // narrower bf16 loads get six steps instead of four, within the 85 registers that leave three blocks per SM (two would
  // put the 384 blocks of a B2 H24 pass into two waves)
  constexpr int U = BFDOT ? 6 : 4;
  float4 fin4 = make_float4(0.f, 0.f, 0.f, 0.f);
  if (BFDOT && sdot && valid) fin4 = *reinterpret_cast<const float4*>(fwd_fin + ((size_t)(b * g.H + h)) * PN + eo);
  for (int s0 = 0; s0 < g.nc; s0 += U) {
    float4 v[U], se[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int s = s0 + u;
      v[u] = se[u] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (s < g.nc && valid) {
        const int c = reverse ? g.nc - 1 - s : s;
        v[u] = *reinterpret_cast<const float4*>(base + (size_t)c * cstride);
        if (sdot) {
          if constexpr (BFDOT) {
            // an unconditional load (index clamped; the last chunk takes the final state read before the loop instead) and
            // nothing else: with the bf16 -> fp32 conversion here the loads of the U steps were issued one round after the
            // other instead of together (0.25 instead of 0.17 ms on 0.8 GB)
            const bool inner = c + 1 < g.nc;
            const uint2 q = *reinterpret_cast<const uint2*>(fwd_prev_bf + boff + (size_t)(inner ? c + 1 : c) * cstride);
            se[u].x = __uint_as_float(q.x);   // raw bits, converted where they are used
            se[u].y = __uint_as_float(q.y);
          } else {
            se[u] = (c + 1 < g.nc) ? *reinterpret_cast<const float4*>(fwd_prev + boff + (size_t)(c + 1) * cstride)
                                   : *reinterpret_cast<const float4*>(fwd_fin + ((size_t)(b * g.H + h)) * PN + eo);
          }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int s = s0 + u;
      if (s < g.nc) {   // block-uniform
        const int c = reverse ? g.nc - 1 - s : s;
        if (WRITE && valid) {
          // the reverse scan's fp32 values have no reader in this family (the scans take the bf16 copy, the state
          // gradient entering the slice leaves through `last`): a third of its bytes stay unwritten
          if (!st_bf) *reinterpret_cast<float4*>(base + (size_t)c * cstride) = run;
          if (st_bf)
            *reinterpret_cast<uint2*>(st_bf + boff + (size_t)c * cstride) =
                make_uint2(pack_bf16(run.x, run.y), pack_bf16(run.z, run.w));
        }
        if (sdot) {
          if constexpr (BFDOT) {
            const uint32_t q0 = __float_as_uint(se[u].x), q1 = __float_as_uint(se[u].y);
            se[u] = (c + 1 < g.nc) ? make_float4(__uint_as_float(q0 << 16), __uint_as_float(q0 & 0xffff0000u),
                                                 __uint_as_float(q1 << 16), __uint_as_float(q1 & 0xffff0000u))
                                   : fin4;
          }
          float d = run.x * se[u].x + run.y * se[u].y + run.z * se[u].z + run.w * se[u].w;
#pragma unroll
          for (int o = 16; o; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
          if ((threadIdx.x & 31) == 0) sdot[((size_t)(b * g.nc + c) * g.H + h) * nw + wslot] = d;
        }
        const float d = sdec[c];
        run.x = fmaf(d, run.x, v[u].x); run.y = fmaf(d, run.y, v[u].y);
        run.z = fmaf(d, run.z, v[u].z); run.w = fmaf(d, run.w, v[u].w);
      }
    }
  }
  if (last && valid) *reinterpret_cast<float4*>(last + ((size_t)(b * g.H + h)) * PN + eo) = run;
}

// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                             const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                             CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn get_encode() {
  static EncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeFn)p;
  });
  return fn;
}

// 3-D bf16 map, 128B swizzle: dims (fastest first) {d0, d1, d2}, strides in ELEMENTS, box {64, box1, 1}.
int make_map3(CUtensorMap* m, const void* ptr, long long d0, long long d1, long long d2, long long s1, long long s2,
              int box1, const char* what) {
  EncodeFn enc = get_encode();
  if (!enc) { set_error("cuTensorMapEncodeTiled is not available from the driver"); return SSD_ERR_CUDA; }
  cuuint64_t dims[3] = {(cuuint64_t)d0, (cuuint64_t)d1, (cuuint64_t)d2};
  cuuint64_t strides[2] = {(cuuint64_t)s1 * 2, (cuuint64_t)s2 * 2};
  cuuint32_t box[3] = {64, (cuuint32_t)box1, 1};
  cuuint32_t es[3] = {1, 1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, es,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled(%s) failed with CUresult %d", what, (int)r); return SSD_ERR_CUDA; }
  return SSD_OK;
}
// fp32 [rows, 64] state rows (dstate 64), 128B swizzle: box = 32 columns (128 bytes) x 128 rows
int make_f32_rows_map(CUtensorMap* m, const float* ptr, long long rows, const char* what) {
  EncodeFn enc = get_encode();
  if (!enc) { set_error("cuTensorMapEncodeTiled is not available from the driver"); return SSD_ERR_CUDA; }
  cuuint64_t dims[3] = {64, (cuuint64_t)rows, 1};
  cuuint64_t strides[2] = {64 * 4, (cuuint64_t)rows * 64 * 4};
  cuuint32_t box[3] = {32, 128, 1};
  cuuint32_t es[3] = {1, 1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(ptr), dims, strides, box, es,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled(%s) failed with CUresult %d", what, (int)r); return SSD_ERR_CUDA; }
  return SSD_OK;
}
// [batch, seqlen, cols] sequence tensor: box = 64 cols x 128 rows
int make_seq_map(CUtensorMap* m, const void* ptr, long long cols, long long L, long long B, long long stride_l,
                 long long stride_b, const char* what) {
  return make_map3(m, ptr, cols, L, B, stride_l, stride_b, 128, what);
}
// dense [B*nc, H*P, N] bf16 chunk states: box = 64 cols (n) x 64 rows ((h,p))
int make_state_map(CUtensorMap* m, const Geo& g, const void* ptr, const char* what) {
  return make_map3(m, ptr, g.N, (long long)g.H * g.P, (long long)g.B * g.nc, g.N, (long long)g.H * g.P * g.N, 64, what);
}

template <int P, int N>
constexpr size_t state_smem() { return 1024 + (N / 64) * BOX_BYTES + 4 * BOX_BYTES + (128 / P) * (TAB_BYTES + 512); }
template <int P, int N, int IBUF, int MODE>
constexpr size_t scan_smem() {
  return 1024 + (N / 64) * BOX_BYTES + 2 * BOX_BYTES +
         IBUF * ((MODE == 0 ? 1 : 2) * BOX_BYTES + (N / 64) * SBOX_BYTES + (64 / P) * TAB_BYTES) +
         (MODE == 0 ? 0 : 2 * PARTS * 128 * 4);
}
template <int P, int N>
constexpr size_t dbc_smem() {
  return 1024 + 2 * (N / 64) * BOX_BYTES + 2 * BOX_BYTES + (N > 64 ? 2 : 1) * (2 * BOX_BYTES + (64 / P) * TAB_BYTES);
}

int sm_count();

template <int P, int N, int MODE>
int launch_state(const Geo& g, const CUtensorMap& tx, const CUtensorMap& tb, const float* tab, float* out, int* status,
                 cudaStream_t s) {
  if (!g.onetile) {   // persistent, ring-fed version
    auto kp = k_state_ps<P, N, MODE>;
    constexpr size_t sm = PsCfg<P, N>::SMEM;
    cudaFuncSetAttribute(kp, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
    const int nitems = g.B * g.G * g.nc;
    const int grid = nitems < sm_count() ? nitems : sm_count();
    kp<<<grid, PsCfg<P, N>::THREADS, sm, s>>>(g, tx, tb, tab, out, status);
    SSD_CUDA_CHECK_LAUNCH(MODE == 0 ? "chunk_state_ps" : "dstates_local_ps");
    return SSD_OK;
  }
  auto k = k_state_tc<P, N, MODE>;
  cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)state_smem<P, N>());
  k<<<dim3(g.nc, g.G, g.B), TC_THREADS, state_smem<P, N>(), s>>>(g, tx, tb, tab, out, status);
  SSD_CUDA_CHECK_LAUNCH(MODE == 0 ? "chunk_state_tc" : "dstates_local_tc");
  return SSD_OK;
}

struct ScanArgs {
  const float *tab, *D;
  const void* z;
  void *y, *dypb, *dz, *dx;
  float *rs0, *rs1;
};
struct SeqMaps {
  CUtensorMap x, dy, b, c, s, ds;
  CUtensorMap out;     // the output of the persistent scan kernels (y, or the dense dx), written by TMA tile stores
  CUtensorMap z;       // the gate (forward of the persistent scan kernel)
};

int sm_count() {
  static int n[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return 132;
  if (!n[dev]) cudaDeviceGetAttribute(&n[dev], cudaDevAttrMultiProcessorCount, dev);
  return n[dev] > 0 ? n[dev] : 132;
}

template <int P, int MODE, int N, bool GATED = false>
int launch_scan_ws(const Geo& g, const SeqMaps& m, const CUtensorMap& ts, const ScanArgs& a, int* status, cudaStream_t s) {
  if constexpr (!GATED && MODE != 2) {
    if (a.z) return launch_scan_ws<P, MODE, N, true>(g, m, ts, a, status, s);
  }
  auto k = k_scan_ws<P, MODE, N, GATED>;
  constexpr size_t sm = WsCfg<P, MODE, N, GATED>::SMEM;
  cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
  const int ntiles = g.B * g.G * g.nc;
  const int grid = ntiles < sm_count() ? ntiles : sm_count();
  k<<<grid, WsCfg<P, MODE, N, GATED>::THREADS, sm, s>>>(g, m.x, m.dy, m.b, m.c, ts, m.out, m.z, a.tab, a.D, (const bf16*)a.z, (bf16*)a.y, (bf16*)a.dypb,
                                 (bf16*)a.dz, (bf16*)a.dx, a.rs0, a.rs1, status);
  SSD_CUDA_CHECK_LAUNCH(MODE == 0 ? "chunk_scan_ws" : (MODE == 1 ? "chunk_scan_bwd_ws" : "dx_ws"));
  return SSD_OK;
}

template <int P, int N, int MODE>
int launch_scan(const Geo& g, const SeqMaps& m, const CUtensorMap& ts, const ScanArgs& a, int* status, cudaStream_t s) {
  if (!g.onetile) return launch_scan_ws<P, MODE, N>(g, m, ts, a, status, s);
  constexpr int IBUF = (MODE == 0 && N < 128) ? 2 : 1;
  auto k = k_scan_tc<P, N, IBUF, MODE>;
  constexpr size_t sm = scan_smem<P, N, IBUF, MODE>();
  cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
  k<<<dim3(g.nc, g.G, g.B), TC_THREADS, sm, s>>>(g, m.x, m.dy, m.b, m.c, ts, a.tab, a.D, (const bf16*)a.z, (bf16*)a.y,
                                                 (bf16*)a.dypb, (bf16*)a.dz, (bf16*)a.dx, a.rs0, a.rs1, status);
  SSD_CUDA_CHECK_LAUNCH(MODE == 0 ? "chunk_scan_tc" : (MODE == 1 ? "chunk_scan_bwd_tc" : "dx_tc"));
  return SSD_OK;
}

template <int P, int N = 64>
int launch_bwd_ws(const Geo& g, const SeqMaps& m, const float* tab, const float* D, void* dx, float* dcsp, float* ddot,
                  float* ddtd, int* status, cudaStream_t s) {
  auto k = k_bwd_ws<P, N>;
  constexpr size_t sm = BwCfg<P, N>::SMEM;
  cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
  const int ntiles = g.B * g.G * g.nc;
  const int grid = ntiles < sm_count() ? ntiles : sm_count();
  k<<<grid, WS_THREADS, sm, s>>>(g, m.x, m.dy, m.b, m.c, m.s, m.ds, tab, D, (bf16*)dx, dcsp, ddot, ddtd, status);
  SSD_CUDA_CHECK_LAUNCH("scan_bwd_dx_ws");
  return SSD_OK;
}

template <int P, int N>
constexpr size_t bwd_tc_smem() {
  return 1024 + 2 * (N / 64) * BOX_BYTES + 2 * BOX_BYTES + 2 * (2 * BOX_BYTES + (64 / P) * TAB_BYTES) + 2 * (N / 64) * SBOX_BYTES +
         3 * PARTS * 128 * 4;
}
template <int P, int N>
int launch_bwd_tc(const Geo& g, const SeqMaps& m, const float* tab, const float* D, void* dx, float* dcsp, float* ddot,
                  float* ddtd, int* status, cudaStream_t s) {
  auto k = k_bwd_tc<P, N>;
  constexpr size_t sm = bwd_tc_smem<P, N>();
  cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
  k<<<dim3(g.nc, g.G, g.B), TC_THREADS, sm, s>>>(g, m.x, m.dy, m.b, m.c, m.s, m.ds, tab, D, (bf16*)dx, dcsp, ddot, ddtd, status);
  SSD_CUDA_CHECK_LAUNCH("scan_bwd_dx_tc");
  return SSD_OK;
}

template <int P>
int launch_dbc_ws(const Geo& g, const SeqMaps& m, const float* tab, const float* hmax, void* dB, void* dC, int* status, cudaStream_t s) {
  auto k = k_dbc_ws<P>;
  constexpr size_t sm = DbCfg<P>::SMEM;
  cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
  const int ntiles = g.B * g.G * g.nc;
  const int grid = ntiles < sm_count() ? ntiles : sm_count();
  k<<<grid, WS_THREADS, sm, s>>>(g, m.x, m.dy, m.b, m.c, m.s, m.ds, tab, hmax, (bf16*)dB, (bf16*)dC, status);
  SSD_CUDA_CHECK_LAUNCH("dBdC_ws");
  return SSD_OK;
}

template <int P, int N>
int launch_dbc(const Geo& g, const SeqMaps& m, const float* tab, const float* hmax, void* dB, void* dC, int* status, cudaStream_t s) {
  if (N == 64 && !g.onetile) return launch_dbc_ws<P>(g, m, tab, hmax, dB, dC, status, s);
  auto k = k_dbc_tc<P, N>;
  cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dbc_smem<P, N>());
  k<<<dim3(g.nc, g.G, g.B), TC_THREADS, dbc_smem<P, N>(), s>>>(g, m.x, m.dy, m.b, m.c, m.s, m.ds, tab, (bf16*)dB, (bf16*)dC,
                                                               status);
  SSD_CUDA_CHECK_LAUNCH("dBdC_tc");
  return SSD_OK;
}

// dy may be NULL (forward); dy strides are the y strides of the geometry unless `dy_dense`.
int make_maps(const Geo& g, const void* x, const void* dy, bool dy_dense, const void* Bm, const void* Cm,
              const void* s_bf, const void* ds_bf, SeqMaps* m) {
  const long long HP = (long long)g.H * g.P, GN = (long long)g.G * g.N;
  int rc = make_seq_map(&m->x, x, HP, g.L, g.B, g.xsl, g.xsb, "x");
  if (rc) return rc;
  if (dy) {
    rc = dy_dense ? make_seq_map(&m->dy, dy, HP, g.L, g.B, HP, HP * g.L, "dy")
                  : make_seq_map(&m->dy, dy, HP, g.L, g.B, g.ysl, g.ysb, "dy");
    if (rc) return rc;
  } else {
    m->dy = m->x;
  }
  rc = make_seq_map(&m->b, Bm, GN, g.L, g.B, g.bsl, g.bsb, "B");
  if (rc) return rc;
  rc = make_seq_map(&m->c, Cm, GN, g.L, g.B, g.csl, g.csb, "C");
  if (rc) return rc;
  if (s_bf) {
    rc = make_state_map(&m->s, g, s_bf, "states");
    if (rc) return rc;
  } else {
    m->s = m->x;
  }
  if (ds_bf) {
    rc = make_state_map(&m->ds, g, ds_bf, "dstates");
    if (rc) return rc;
  } else {
    m->ds = m->s;
  }
  return SSD_OK;
}

}  // namespace

bool tensor_supported(const Geo& g, int dtype, const char** why) {
  auto no = [&](const char* m) { if (why) *why = m; return false; };
  if (dtype != SSD_BF16) return no("tensor-core kernels need bf16 storage");
  if (g.Q != QT) return no("tensor-core kernels need chunk == 128 (or a multiple of it)");
  if (g.L % QT) return no("tensor-core kernels need seqlen % 128 == 0");
  if (!((g.P == 32 || g.P == 64) && (g.N == 64 || g.N == 128))) return no("tensor-core kernels cover headdim in {32,64}, dstate in {64,128}");
  if ((g.hpg * g.P) % 128) return no("heads_per_group * headdim must be a multiple of 128");
  if ((g.xsl % 8) || (g.xsb % 8) || (g.bsl % 8) || (g.bsb % 8) || (g.csl % 8) || (g.csb % 8) || (g.ysl % 8) || (g.ysb % 8) ||
      (g.zsl % 8) || (g.zsb % 8))
    return no("strides must be multiples of 8 elements (16 bytes) for TMA");
  return true;
}

int tensor_state_passing(const Geo& g, float* st, const float* cs, const float* init, float* last, void* st_bf,
                         int reverse, bool write, const float* fwd_prev, const void* fwd_prev_bf, const float* fwd_fin,
                         float* sdot, int* sdot_nw, cudaStream_t s) {
  const int PN = g.P * g.N;
  const dim3 grid(cdiv(PN / 4, 256), g.H, g.B);
  const size_t sm = (size_t)g.nc * sizeof(float);
  if (sdot_nw) *sdot_nw = (int)grid.x * 8;
  // the bf16 copy stands in for the fp32 chunk-entry states wherever the forward scan no longer writes those
  const bf16* prev_bf = (const bf16*)fwd_prev_bf;
  if (write && prev_bf && sdot)
    k_state_passing_v4<true, true><<<grid, 256, sm, s>>>(g, st, cs, init, last, (bf16*)st_bf, reverse, nullptr, prev_bf, fwd_fin, sdot);
  else if (write) k_state_passing_v4<true><<<grid, 256, sm, s>>>(g, st, cs, init, last, (bf16*)st_bf, reverse, fwd_prev, nullptr, fwd_fin, sdot);
  else k_state_passing_v4<false><<<grid, 256, sm, s>>>(g, st, cs, init, last, nullptr, reverse, nullptr, nullptr, nullptr, nullptr);
  SSD_CUDA_CHECK_LAUNCH(reverse ? (write ? "dstate_passing" : "dstate_total") : (write ? "state_passing" : "state_total"));
  return SSD_OK;
}

#define DISPATCH_PN(CALL)                                                 \
  if (g.P == 32 && g.N == 64) { CALL(32, 64) }                            \
  else if (g.P == 32 && g.N == 128) { CALL(32, 128) }                     \
  else if (g.P == 64 && g.N == 64) { CALL(64, 64) }                       \
  else { CALL(64, 128) }

// chunk states (mode 0: x, B) or local state gradients (mode 1: dy, C) on tensor cores
int tensor_chunk_state(const Geo& g, int mode, const void* xdy, long long sb, long long sl, const void* bc,
                       long long bsb, long long bsl, const float* tab, float* out, int* status, cudaStream_t s) {
  CUtensorMap tx, tb;
  int rc = make_seq_map(&tx, xdy, (long long)g.H * g.P, g.L, g.B, sl, sb, "x/dy");
  if (rc) return rc;
  rc = make_seq_map(&tb, bc, (long long)g.G * g.N, g.L, g.B, bsl, bsb, "B/C");
  if (rc) return rc;
#define CALL(PP, NN) return mode == 0 ? launch_state<PP, NN, 0>(g, tx, tb, tab, out, status, s) \
                                      : launch_state<PP, NN, 1>(g, tx, tb, tab, out, status, s);
  DISPATCH_PN(CALL)
#undef CALL
}

// Chunk states and the scan over chunks in one launch (see k_state_scan_ps): dstate 64, persistent family.
bool tensor_state_fused_applies(const Geo& g) { return g.N == 64 && !g.onetile; }

template <int P, int MODE>
static int launch_state_scan(const Geo& g, const CUtensorMap& tx, const CUtensorMap& tb, const CUtensorMap& ts, const CUtensorMap& tf,
                             const StateScanArgs& a, int* status, cudaStream_t s) {
  auto k = k_state_scan_ps<P, MODE>;
  constexpr size_t sm = PfCfg<P, MODE>::SMEM;
  cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
  const int nunits = g.B * g.G * (g.hpg * P / 128);
  const int grid = nunits < sm_count() ? nunits : sm_count();
  k<<<grid, PfCfg<P, MODE>::THREADS, sm, s>>>(g, tx, tb, ts, tf, a, status);
  SSD_CUDA_CHECK_LAUNCH(MODE == 0 ? "chunk_state_scan" : "dstate_scan");
  return SSD_OK;
}

int tensor_state_fused(const Geo& g, int mode, const void* xdy, long long sb, long long sl, const void* bc, long long bsb,
                       long long bsl, const float* tab, float* st, void* st_bf, const float* init, float* last,
                       const void* fwd_prev_bf, const float* fwd_fin, float* sdot, int* sdot_nw, int* status, cudaStream_t s) {
  CUtensorMap tx, tb;
  int rc = make_seq_map(&tx, xdy, (long long)g.H * g.P, g.L, g.B, sl, sb, "x/dy");
  if (rc) return rc;
  rc = make_seq_map(&tb, bc, (long long)g.G * g.N, g.L, g.B, bsl, bsb, "B/C");
  if (rc) return rc;
  StateScanArgs a{tab, st, st_bf, init, last, fwd_prev_bf, fwd_fin, sdot};
  if (sdot_nw) *sdot_nw = 4 * (g.P / 32);
  CUtensorMap ts = tx, tf = tx;   // placeholders unless the backward kernel reads the forward states
  if (mode == 1 && sdot) {
    const long long rows = (long long)g.B * g.nc * g.H * g.P;   // bf16 [rows, 64]: boxes of 128 rows x 64 columns
    rc = make_map3(&ts, fwd_prev_bf, 64, rows, 1, 64, rows * 64, 128, "forward chunk-entry states (bf16 copy)");
    if (rc) return rc;
    rc = make_f32_rows_map(&tf, fwd_fin, (long long)g.B * g.H * g.P, "forward final state");
    if (rc) return rc;
  }
  if (g.P == 32) return mode == 0 ? launch_state_scan<32, 0>(g, tx, tb, ts, tf, a, status, s) : launch_state_scan<32, 1>(g, tx, tb, ts, tf, a, status, s);
  if (g.P == 64) return mode == 0 ? launch_state_scan<64, 0>(g, tx, tb, ts, tf, a, status, s) : launch_state_scan<64, 1>(g, tx, tb, ts, tf, a, status, s);
  set_error("tensor_state_fused: unsupported headdim %d", g.P);
  return SSD_ERR_UNSUPPORTED;
}

int tensor_chunk_scan(const Geo& g, const SsdFwdPtrs& p, const float* tab, const void* prev_bf, int* status,
                      cudaStream_t s) {
  SeqMaps m;
  int rc = make_maps(g, p.x, nullptr, false, p.Bm, p.Cm, prev_bf, nullptr, &m);
  if (rc) return rc;
  rc = make_seq_map(&m.out, p.y, (long long)g.H * g.P, g.L, g.B, g.ysl, g.ysb, "y");
  if (rc) return rc;
  if (p.z) {
    rc = make_seq_map(&m.z, p.z, (long long)g.H * g.P, g.L, g.B, g.zsl, g.zsb, "z");
    if (rc) return rc;
  } else {
    m.z = m.x;
  }
  ScanArgs a{tab, p.D, p.z, p.y, nullptr, nullptr, nullptr, nullptr, nullptr};
#define CALL(PP, NN) return launch_scan<PP, NN, 0>(g, m, m.s, a, status, s);
  DISPATCH_PN(CALL)
#undef CALL
}

// backward, forward-recompute pass: dcsp, ddot, and for the gated case dz and the bf16 pre-gate dy
int tensor_scan_bwd(const Geo& g, const SsdBwdPtrs& p, const float* tab, const void* prev_bf, void* dypb, float* dcsp,
                    float* ddot, int* status, cudaStream_t s) {
  SeqMaps m;
  int rc = make_maps(g, p.x, p.dy, false, p.Bm, p.Cm, prev_bf, nullptr, &m);
  if (rc) return rc;
  m.out = m.x;
  m.z = m.x;
  ScanArgs a{tab, p.D, p.z, nullptr, dypb, p.dz, nullptr, dcsp, ddot};
#define CALL(PP, NN) return launch_scan<PP, NN, 1>(g, m, m.s, a, status, s);
  DISPATCH_PN(CALL)
#undef CALL
}

// backward, dx and ddtd; `dyp` is the pre-gate gradient (dy itself, or the dense bf16 copy)
int tensor_dx(const Geo& g, const SsdBwdPtrs& p, const void* dyp, bool dy_dense, const float* tab, const void* ds_bf,
              float* ddtd, int* status, cudaStream_t s) {
  SeqMaps m;
  int rc = make_maps(g, p.x, dyp, dy_dense, p.Bm, p.Cm, nullptr, ds_bf, &m);
  if (rc) return rc;
  {
    const long long HP = (long long)g.H * g.P;
    rc = make_seq_map(&m.out, p.dx, HP, g.L, g.B, HP, HP * g.L, "dx");
    if (rc) return rc;
    m.z = m.x;
  }
  ScanArgs a{tab, p.D, nullptr, nullptr, nullptr, nullptr, p.dx, ddtd, nullptr};
#define CALL(PP, NN) return launch_scan<PP, NN, 2>(g, m, m.ds, a, status, s);
  DISPATCH_PN(CALL)
#undef CALL
}

// ungated backward: recompute pass and dx pass in one kernel (persistent for dstate 64, one tile per CTA for dstate 128)
bool tensor_bwd_merged_applies(const Geo& g, const SsdBwdPtrs& p) { return !p.z && (g.N == 128 || !g.onetile); }
int tensor_bwd_merged(const Geo& g, const SsdBwdPtrs& p, const float* tab, const void* prev_bf, const void* ds_bf,
                      float* dcsp, float* ddot, float* ddtd, int* status, cudaStream_t s) {
  SeqMaps m;
  int rc = make_maps(g, p.x, p.dy, false, p.Bm, p.Cm, prev_bf, ds_bf, &m);
  if (rc) return rc;
  if (g.N == 128 && g.onetile) {   // one tile per CTA
    if (g.P == 32) return launch_bwd_tc<32, 128>(g, m, tab, p.D, p.dx, dcsp, ddot, ddtd, status, s);
    return launch_bwd_tc<64, 128>(g, m, tab, p.D, p.dx, dcsp, ddot, ddtd, status, s);
  }
  if (g.N == 128) {
    if (g.P == 32) return launch_bwd_ws<32, 128>(g, m, tab, p.D, p.dx, dcsp, ddot, ddtd, status, s);
    return launch_bwd_ws<64, 128>(g, m, tab, p.D, p.dx, dcsp, ddot, ddtd, status, s);
  }
  if (g.P == 32) return launch_bwd_ws<32>(g, m, tab, p.D, p.dx, dcsp, ddot, ddtd, status, s);
  return launch_bwd_ws<64>(g, m, tab, p.D, p.dx, dcsp, ddot, ddtd, status, s);
}

int tensor_dbc(const Geo& g, const SsdBwdPtrs& p, const void* dyp, bool dy_dense, const float* tab, const float* hmax,
               const void* prev_bf, const void* ds_bf, int* status, cudaStream_t s) {
  SeqMaps m;
  int rc = make_maps(g, p.x, dyp, dy_dense, p.Bm, p.Cm, prev_bf, ds_bf, &m);
  if (rc) return rc;
#define CALL(PP, NN) return launch_dbc<PP, NN>(g, m, tab, hmax, p.dB, p.dC, status, s);
  DISPATCH_PN(CALL)
#undef CALL
}

int tensor_selftest_wait(int* status, long long max_cycles, cudaStream_t s) {
  k_selftest_wait<<<1, 32, 0, s>>>(status, max_cycles);
  SSD_CUDA_CHECK_LAUNCH("selftest_wait");
  return SSD_OK;
}

}  // namespace ssd
