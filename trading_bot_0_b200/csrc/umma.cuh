// Thin inline-PTX layer over the Blackwell (sm_100a) tensor-core path: tcgen05.mma with
// accumulators in tensor memory (TMEM), shared-memory matrix descriptors, mbarriers and TMA
// (cp.async.bulk.tensor) tile loads.  No cluster multicast anywhere: every load is a plain
// per-CTA load of this GPU's own memory.
//
// Conventions used by the kernels built on top of this file
//   * cta_group::1, M = 128: accumulator row r lives in TMEM lane r; a warp w may read lanes
//     32*(w%4) .. 32*(w%4)+31 only.
//   * bf16 operands, fp32 accumulation (kind::f16).
//   * "SW128" tiles are what a TMA box with a 128-byte inner extent and 128B swizzle leaves in
//     shared memory: row pitch 128 B, the 16-byte chunk index XOR-ed with (row % 8); tile bases
//     are 1024-byte aligned.  Read as a K-major operand the rows are M/N and the 64 columns are
//     K (SBO = 1024 B between 8-row groups; a K step of 16 elements advances the start address
//     by 32 B).  Read as an MN-major operand the rows are K and the 64 columns are M/N
//     (SBO = 1024 B between 8-row K groups, LBO = distance between 64-column blocks).
//   * "plain" tiles are written by threads in the no-swizzle core-matrix layout:
//     byte offset(row, col) = (col/8)*rows*16 + row*16 + (col%8)*2.  The same bytes are a K-major
//     operand (rows = M/N, cols = K; LBO = rows*16 between K groups, SBO = 128) and the
//     transposed MN-major operand (cols = M/N, rows = K; SBO = rows*16, LBO = 128).
//   * every wait is bounded; a wait that gives up records a code in a status word and the
//     kernel runs on to its clean-up (results are then garbage, the context stays usable).
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ssd {
namespace umma {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// ---- mbarrier ------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Bounded wait on a phase parity.  Each try_wait may suspend the thread (up to the hint, in ns) until
// the phase completes, so waiting warps stay off the issue slots; the bound is in elapsed clock
// cycles, not in polls: about 2 s, because a profiler pass that instruments every instruction can
// slow a kernel a thousandfold and must not be mistaken for a broken pipeline.  Returns false when
// the bound ran out.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, long long max_cycles = 4000000000LL) {
  const uint32_t a = smem_u32(bar);
  long long t0 = 0;
  for (int i = 0;; ++i) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(a), "r"(parity), "r"(20000u) : "memory");
    if (ok) return true;
    if (i == 0) t0 = clock64();
    else if ((i & 15) == 0 && clock64() - t0 > max_cycles) return false;
  }
}

// ---- TMA -------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, int c0, int c1, int c2,
                                            uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(smem_u32(bar)) : "memory");
}
// Tile store shared -> global through the same kind of map (coordinates must not be negative; rows past the tensor's
// extent are dropped).  Stores are tracked per thread in bulk groups: commit, then wait until the group's shared-memory
// reads are done (the source may be overwritten) or until the group has completed.
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, const void* smem_src, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4}], [%1];"
               ::"l"(map), "r"(smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// 1-D bulk copy global -> shared (both 16-byte aligned, size a multiple of 16), completing on `bar`.
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
// Ask for a tile / a byte range to be brought into L2 (no shared memory, no completion to wait for):
// used to take the DRAM latency of loads that will be issued a little later off the critical path.
__device__ __forceinline__ void tma_prefetch_3d(const CUtensorMap* map, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global.tile [%0, {%1, %2, %3}];" ::"l"(map), "r"(c0), "r"(c1), "r"(c2)
               : "memory");
}
__device__ __forceinline__ void bulk_prefetch(const void* gsrc, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(gsrc), "r"(bytes) : "memory");
}
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// ---- proxies / fences --------------------------------------------------------------------------
// generic-proxy smem writes -> visible to the async proxy (tcgen05.mma operand reads)
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// ---- TMEM --------------------------------------------------------------------------------------
// One full warp allocates `ncols` (power of two >= 32) columns; the base address lands in *slot.
__device__ __forceinline__ void tmem_alloc(uint32_t* slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(ncols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(ncols) : "memory");
}
// 32 lanes x 32 consecutive fp32 columns: thread t of the warp gets lane (lane_base + t).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
// 32 lanes x 16 consecutive fp32 columns.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
// 32 lanes x 8 consecutive fp32 columns, WITHOUT the wait: issue several, then tmem_ld_wait() once.
__device__ __forceinline__ void tmem_ld8_issue(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr));
}
// 32 lanes x 32 consecutive fp32 columns, WITHOUT the wait (raw bits): lets the next block's load fly
// while the current block is being worked on.
__device__ __forceinline__ void tmem_ld32_issue(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ uint32_t tmem_addr(uint32_t base, int lane, int col) {
  return base + ((uint32_t)lane << 16) + (uint32_t)col;
}

// ---- descriptors -------------------------------------------------------------------------------
enum : uint32_t { LAYOUT_NONE = 0, LAYOUT_SW128 = 2 };

__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;  // descriptor version of sm_100
  d |= (uint64_t)(layout & 7) << 61;
  return d;
}
// SW128 tile read K-major: rows are M/N, 64 K-columns per tile; kbyte = byte offset of the K step.
__device__ __forceinline__ uint64_t desc_sw128_k(uint32_t tile, uint32_t kbyte) {
  return make_desc(tile + kbyte, 16, 1024, LAYOUT_SW128);
}
// SW128 tile(s) read MN-major: rows are K (8-row groups 1024 B apart), 64 M/N columns per tile,
// `lbo` bytes between consecutive 64-column tiles; krow = first K row, mnbyte = byte offset of
// the first M/N column inside the 128-byte row.
__device__ __forceinline__ uint64_t desc_sw128_mn(uint32_t tile, uint32_t krow, uint32_t mnbyte, uint32_t lbo) {
  return make_desc(tile + krow * 128 + mnbyte, lbo, 1024, LAYOUT_SW128);
}
// plain tile with `rows` rows read K-major (rows = M/N); k0 = first K column (multiple of 8).
__device__ __forceinline__ uint64_t desc_plain_k(uint32_t tile, uint32_t rows, uint32_t k0) {
  return make_desc(tile + (k0 >> 3) * rows * 16, rows * 16, 128, LAYOUT_NONE);
}
// the same plain tile read as its transpose, MN-major (cols = M/N); k0 = first K ROW (multiple of 8),
// mn0 = first M/N column (multiple of 8).
__device__ __forceinline__ uint64_t desc_plain_mn(uint32_t tile, uint32_t rows, uint32_t k0, uint32_t mn0) {
  return make_desc(tile + k0 * 16 + (mn0 >> 3) * rows * 16, 128, rows * 16, LAYOUT_NONE);
}
// Advance the start address of a descriptor by `bytes` (a multiple of 16).  Shared-memory addresses
// stay below 256 KB, so the 14-bit address field never carries into its neighbours.  Building a
// descriptor costs a chain of dependent integer ops in the single issuing thread; loops over K
// steps should build the first one and add to it.
__device__ __forceinline__ uint64_t desc_adv(uint64_t d, uint32_t bytes) { return d + (uint64_t)(bytes >> 4); }
// byte offset of (row, col) in a plain tile; col multiple of 8 addresses one 16-byte chunk
__device__ __forceinline__ uint32_t plain_off(uint32_t rows, uint32_t row, uint32_t col) {
  return (col >> 3) * rows * 16 + row * 16 + (col & 7) * 2;
}
// byte offset of the 16-byte chunk holding columns [8*chunk, 8*chunk+8) of `row` in a SW128 tile
__device__ __forceinline__ uint32_t sw128_off(uint32_t row, uint32_t chunk) {
  return row * 128 + (((chunk ^ row) & 7) << 4);
}

// instruction descriptor, kind::f16, bf16 x bf16 -> fp32
__device__ __forceinline__ uint32_t make_idesc(int m, int n, int a_mn_major, int b_mn_major) {
  uint32_t d = 0;
  d |= 1u << 4;   // D format fp32
  d |= 1u << 7;   // A format bf16
  d |= 1u << 10;  // B format bf16
  d |= (uint32_t)(a_mn_major & 1) << 15;
  d |= (uint32_t)(b_mn_major & 1) << 16;
  d |= (uint32_t)(n >> 3) << 17;
  d |= (uint32_t)(m >> 4) << 24;
  return d;
}

// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread.  One instruction covers K = 16.
__device__ __forceinline__ void mma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, bool accumulate) {
  const uint32_t acc = accumulate ? 1u : 0u;
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
               ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc) : "memory");
}
// All MMAs issued so far by this thread arrive on `bar` when they complete (implies
// tcgen05.fence::before_thread_sync).
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// ---- register re-balancing between warp roles ------------------------------------------------
// All four warps of an aligned group of four must execute the same one.  A role that needs few registers
// gives some back (dec) so that the arithmetic-heavy role can take more (inc) than the launch-time share.
template <int R> __device__ __forceinline__ void reg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(R)); }
template <int R> __device__ __forceinline__ void reg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(R)); }

// ---- small helpers -----------------------------------------------------------------------------
__device__ __forceinline__ float ex2(float x) {   // 2^x, flushes results below 2^-126 to zero
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float2 unpack_bf16(uint32_t u) {
  return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u));
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
// 32 contiguous bytes to global memory: one full sector per thread when `p` is 32-byte aligned, else two halves
// 32 read-only bytes per thread in one request where the address allows it (two 16-byte requests otherwise): rows read by
// one thread each cost one L1 wavefront per lane and instruction, so half the instructions is half the wavefronts.
__device__ __forceinline__ void ld_global_32B(const void* p, uint4& a, uint4& b) {
  if ((reinterpret_cast<uintptr_t>(p) & 31) == 0) {
    asm volatile("ld.global.nc.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w), "=r"(b.x), "=r"(b.y), "=r"(b.z), "=r"(b.w) : "l"(p));
  } else {
    a = __ldg(reinterpret_cast<const uint4*>(p));
    b = __ldg(reinterpret_cast<const uint4*>(p) + 1);
  }
}
__device__ __forceinline__ void st_global_32B(void* p, const uint4& a, const uint4& b) {
  if ((reinterpret_cast<uintptr_t>(p) & 31) == 0) {
    asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b.x),
                 "r"(b.y), "r"(b.z), "r"(b.w) : "memory");
  } else {
    reinterpret_cast<uint4*>(p)[0] = a;
    reinterpret_cast<uint4*>(p)[1] = b;
  }
}
// fp32 reads of shared memory through the shared-memory pipe.  A read through a plain `const float*` compiles to a generic
// load when the compiler has lost track of the address space (pointers into the dynamic shared memory handed through
// helper functions): generic loads take the long-latency path, and the decay passes are chains of dependent table reads.
__device__ __forceinline__ float lds_f32(uint32_t addr) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ float4 lds_v4f32(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint4 ld_shared_v4(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}

}  // namespace umma
}  // namespace ssd
