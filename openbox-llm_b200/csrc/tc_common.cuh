// sm_100a building blocks shared by the tcgen05 attention kernels: mbarrier and TMA wrappers
// with bounded waits, TMEM allocation, UMMA shared-memory / instruction descriptors,
// tcgen05.mma / ld / st wrappers.
#pragma once

#include <cuda.h>   // CUtensorMap (types only; the encode entry point is fetched at run time)

#include "common.cuh"

namespace nsa {
namespace tc {

constexpr int kRows = 128;     // (query, head) rows per CTA tile = UMMA M
constexpr int kKeys = 64;      // keys per tile = one 64-token selection block
constexpr long long kWaitLimitCycles = 2000000000LL;   // about one second

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

// ---- mbarrier ------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait.  When the limit runs out the kernel raises the device status word, marks the
// CTA as aborted and every later wait of the CTA returns at once, so the grid drains; other
// CTAs notice the status word the next time one of their waits is slow.
// Returns true when the phase completed, false when the wait was given up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* status,
                                          volatile int* s_abort, int code) {
  if (*s_abort) return false;
  if (mbar_try_wait(bar, parity)) return true;
  const long long start = clock64();
  uint32_t polls = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++polls & 0xffu) == 0) {
      if (*s_abort) return false;
      if (*(volatile int*)status != 0) { *s_abort = 1; return false; }
      if (clock64() - start > kWaitLimitCycles) {
        atomicOr(status, code);
        *s_abort = 1;
        return false;
      }
    }
  }
  return true;
}

// Wait of an aborted CTA for something of its own that is still in flight (a TMA load into its
// shared memory, MMAs reading it) before it gives the memory back: bounded like every other wait,
// and not cut short by the abort flag.
constexpr long long kDrainLimitCycles = 20000000LL;   // about ten milliseconds
__device__ __forceinline__ bool mbar_wait_drain(uint64_t* bar, uint32_t parity) {
  const long long start = clock64();
  while (!mbar_try_wait(bar, parity))
    if (clock64() - start > kDrainLimitCycles) return false;
  return true;
}

// ---- selection work list -----------------------------------------------------------------------
// The block-outer selection kernels take one work item per CTA: a 64-token block of one
// (batch, kv head) and a chunk of at most kSelChunkTiles of its row tiles.  A block that many
// queries list (an attention-sink block, a forced initial block) becomes several items, so no
// single CTA walks its whole query list.
constexpr int kSelChunkTiles = 128;
struct SelWorkHeader { int n_items; int pad[63]; };   // 256 bytes in front of the int4 items

// ---- TMA -------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* tm, uint64_t* bar, int c0,
                                            int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(smem_u32(dst)),
      "l"(tm), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
// Tiled store shared -> global as part of the thread's bulk async-group.  Rows of the box that
// fall outside the tensor are dropped.
__device__ __forceinline__ void tma_store_5d(const CUtensorMap* tm, const void* src, int c0, int c1,
                                             int c2, int c3, int c4) {
  asm volatile(
      "cp.async.bulk.tensor.5d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5, %6}], [%1];" ::"l"(tm),
      "r"(smem_u32(src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
      : "memory");
}
// Tiled reduction shared -> global (element-wise add in the map's data type, here fp32), part of
// the thread's bulk async-group like a store.  Rows of the box outside the tensor are dropped.
__device__ __forceinline__ void tma_reduce_add_4d(const CUtensorMap* tm, const void* src, int c0, int c1,
                                                  int c2, int c3) {
  asm volatile(
      "cp.reduce.async.bulk.tensor.4d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(tm),
      "r"(smem_u32(src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// the shared-memory source of every committed bulk store of this thread has been read
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// every committed bulk store of this thread is complete
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* tm) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tm) : "memory");
}

// ---- TMEM ------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(dst_smem)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// 32 lanes x 32 consecutive 32-bit columns; lane i of the warp reads TMEM lane base+i
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
      "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]),
      "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
      "r"(r[30]), "r"(r[31])
      : "memory");
}

// ---- UMMA descriptors ------------------------------------------------------------------------
// Shared-memory tiles are stored the way a 128B-swizzled TMA box lands: rows of 128 bytes
// (64 bf16), 8-row groups of 1024 bytes, 16-byte chunk index XOR (row & 7); a tile wider than
// 64 elements is a sequence of such "slabs".
//
// K-major operand (the contraction index runs inside a 128-byte row):
//   canonical ((8,n),2):((8,SBO),1) in 16-byte units -> LBO field 1, SBO = 1024 bytes.
// MN-major operand (the M/N index runs inside a 128-byte row, one contraction index per row):
//   canonical ((8,n),(8,k)):((1,LBO),(8,SBO)) -> LBO = byte distance between 64-element slabs,
//   SBO = 1024 bytes between 8-row groups.
__device__ __forceinline__ uint64_t desc_sw128(uint32_t saddr, uint32_t lbo_bytes,
                                               uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3fffu);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3fffu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3fffu) << 32;
  d |= 1ull << 46;   // descriptor version of sm_100
  d |= 2ull << 61;   // SWIZZLE_128B
  return d;
}
// The upper word of every descriptor used here is the same constant (SBO = 1024 bytes, version,
// 128B swizzle); the lower word is address >> 4 plus the LBO field, so stepping a descriptor by
// a byte offset that is a multiple of 16 is one 32-bit add.
constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
__device__ __forceinline__ uint32_t desc_lo_kmajor(uint32_t saddr) { return ((saddr >> 4) & 0x3fffu) | (1u << 16); }
__device__ __forceinline__ uint32_t desc_lo_mnmajor(uint32_t saddr, uint32_t slab_bytes) {
  return ((saddr >> 4) & 0x3fffu) | (((slab_bytes >> 4) & 0x3fffu) << 16);
}
__device__ __forceinline__ uint64_t desc_at(uint32_t lo, uint32_t byte_offset) {
  uint64_t d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo + (byte_offset >> 4)), "r"(kDescHi));
  return d;
}
// the same with another distance between 8-row groups (tiles whose 64-column slabs interleave)
__device__ __forceinline__ uint64_t desc_at_sbo(uint32_t lo, uint32_t byte_offset, uint32_t sbo_bytes) {
  uint64_t d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo + (byte_offset >> 4)),
      "r"((sbo_bytes >> 4) | (1u << 14) | (2u << 29)));
  return d;
}
// 5-D tiled load: coordinates innermost first
__device__ __forceinline__ void tma_load_5d(void* dst, const CUtensorMap* tm, uint64_t* bar, int c0, int c1,
                                            int c2, int c3, int c4) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6, %7}], [%2];" ::"r"(smem_u32(dst)),
      "l"(tm), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
      : "memory");
}
// L2 eviction-priority hints.  The block-outer selection kernels stream 17 GB of partial rows out
// through L2 while they gather the q (and dO) rows of one (batch, kv head), which would fit L2 by
// themselves: the partial stores are marked evict-first.  (Marking the gathers evict-last as well
// bought the two kernels 2-3 % and cost the kernels after them as much: the lines stay.)
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ uint64_t l2_policy_evict_normal() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_normal.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ void tma_load_5d_hint(void* dst, const CUtensorMap* tm, uint64_t* bar, int c0, int c1,
                                                 int c2, int c3, int c4, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1, {%3, %4, %5, %6, %7}], [%2], %8;" ::"r"(smem_u32(dst)),
      "l"(tm), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void tma_store_5d_hint(const CUtensorMap* tm, const void* src, int c0, int c1,
                                                  int c2, int c3, int c4, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.5d.global.shared::cta.bulk_group.L2::cache_hint [%0, {%2, %3, %4, %5, %6}], [%1], %7;" ::"l"(tm),
      "r"(smem_u32(src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4), "l"(policy)
      : "memory");
}
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t saddr) { return desc_sw128(saddr, 16, 1024); }
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t saddr, uint32_t slab_bytes) {
  return desc_sw128(saddr, slab_bytes, 1024);
}

// kind::f16 instruction descriptor: bf16 x bf16 -> f32, M x N tile
__host__ __device__ constexpr uint32_t idesc_bf16(int M, int N, int a_mn_major, int b_mn_major) {
  return (1u << 4)                         // D format f32
         | (1u << 7) | (1u << 10)          // A, B format bf16
         | ((uint32_t)a_mn_major << 15) | ((uint32_t)b_mn_major << 16)
         | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                       uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc,
                                       uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Loads that must be issued where they are written: ptxas otherwise sinks a prefetch down to its
// first use (a whole loop iteration later) and the warp then waits out the full memory latency.
__device__ __forceinline__ float ldg_f32_now(const float* ptr) {
  float v;
  asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(v) : "l"(ptr));
  return v;
}
__device__ __forceinline__ int ldg_s32_now(const int32_t* ptr) {
  int v;
  asm volatile("ld.global.nc.s32 %0, [%1];" : "=r"(v) : "l"(ptr));
  return v;
}

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);   // .x = lo -> low 16 bits
  return *reinterpret_cast<uint32_t*>(&h);
}

// ---- which selection-forward variant does the work ------------------------------------------
// stats[0] = number of (query tile, distinct block) pairs of the query-outer kernel.
// The query-outer kernel runs one 64-key tile per such pair; this kernel runs one row tile per
// nq (query, block) pairs, at about three times the cost of a query-outer tile.
__device__ __forceinline__ bool prefer_pairs(const unsigned long long* stats, const int32_t* offsets,
                                             int units, int n_ktiles, int nq, int force) {
  if (force) return force == 2;
  const unsigned long long union_tiles = stats[0];
  const unsigned long long pairs = (unsigned long long)__ldg(offsets + (size_t)units * (n_ktiles + 1) - 1);
  return union_tiles * (unsigned long long)nq > 3ull * pairs;
}

// byte offset of element (row, col) inside a 128B-swizzled slab sequence; col in elements
__device__ __forceinline__ uint32_t sw128_offset(int row, int col, int rows_per_slab) {
  const int slab = col >> 6, c = col & 63;
  const int chunk = (c >> 3) ^ (row & 7);
  return (uint32_t)(slab * rows_per_slab * 128 + row * 128 + chunk * 16 + (c & 7) * 2);
}

}  // namespace tc
}  // namespace nsa
