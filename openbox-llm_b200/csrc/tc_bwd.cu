// tcgen05 / TMEM backward of the three attention branches, key-tile outer.
//
// One CTA owns a tile of 64 keys of one (batch, kv head): K and V of the tile are loaded
// once (TMA), dK^T and dV^T of the tile stay in TMEM for the whole CTA and are written once,
// with no atomics.  The CTA walks the (query, head) rows that attend the tile, 128 rows at a
// time (nq queries x the G heads of the group):
//   window      queries [64 j, 64 j + 63 + W - 1]
//   compression queries t >= (64 j + 1) * Bsz - 1
//   selection   the queries that list block j, from the block -> query CSR
// Q and dO rows arrive by TMA into 128B-swizzled tiles: one box per row tile for the window and
// compression branches (consecutive queries), one box per query and 64-column slab for
// selection.  Selection CTAs take (block, chunk of row tiles) items from a device-built work list.
// Per row tile, five MMAs:
//   S    = Q K^T          (A: Q  K-major,   B: K  K-major)
//   dP   = dO V^T         (A: dO K-major,   B: V  K-major)
//   dV^T += dO^T P        (A: dO MN-major,  B: P  MN-major)      P, dS: bf16 tiles the threads
//   dK^T += Q^T dS        (A: Q  MN-major,  B: dS MN-major)      write to shared memory
//   dQ   = dS K           (A: dS K-major,   B: K  MN-major)
// with p = exp2(s*scale*log2e - lse*log2e) and dS = scale * p * (dP - delta) computed by the
// thread that owns the row (TMEM lane = row).  dQ of a row is the sum over the key tiles it
// attends.  Two ways out of the CTA:
//   slots        every (row tile, key tile) result leaves as a bf16 partial tile (TMA store) and a
//                second kernel adds the partials of each query in fp32, in a fixed order
//                (selection always; window / compression when the caller wants dq itself);
//   accumulator  window / compression inside the whole op: the fp32 tile is added to one fp32
//                accumulator [units][T][G][D] by TMA reduce-add.  Consecutive key tiles hit the same
//                consecutive query rows at nearby times, so the adds meet in L2 and no partial
//                buffer exists; the order of the adds, hence the last bits of dq, is not fixed.
#include "tc_common.cuh"
#include "tc_host.cuh"

namespace nsa {
namespace tc {

struct BwdArgs {
  const __nv_bfloat16* q;
  const __nv_bfloat16* d_o;
  const float* lse;
  const float* delta;          // sum_d dO * O per row (unscaled)
  const float* row_scale;      // gate value per row of a gated branch, or null
  const int32_t* q_of_block;
  const int32_t* offsets;      // [B*Hkv, n_ktiles + 1] global pair offsets (selection)
  __nv_bfloat16* dk;
  __nv_bfloat16* dv;
  __nv_bfloat16* dq_part;
  float* dk_acc;               // fp32 accumulators, used when the row tiles of a key tile are split
  float* dv_acc;
  const SelWorkHeader* work;   // selection: work items {bh, block, first row tile, chunks of the block}
  int* status;
  int split_chunk;             // row tiles per CTA when split
  int B, Hq, Hkv, T, Lk, G, nq;
  int kind, window, block_size;
  int n_ktiles, n_slots;
  int merged;                  // selection: one TMA box per (query, tensor) brings both 64-column slabs
  int dq_acc_mode;             // 1: dQ tiles are added to the fp32 accumulator (window / compression)
  float scale, scale_log2;
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d)
               : "memory");
}

constexpr int kRowTileBytes = kRows * 128 * 2;   // Q or dO row tile: always two 64-element slabs
constexpr int kPBytes = kRows * 128;             // P or dS: 128 rows x 64 keys bf16
constexpr int kGroupThreads = 256;               // one compute group: 2 warps per TMEM lane quadrant
constexpr int kGroupBytes = 2 * kRowTileBytes + 2 * kPBytes;   // Q, dO, P, dS of one group
constexpr int kMaxNq = 64;                       // queries per row tile (group size >= 2)

__host__ __device__ inline size_t bwd_smem_bytes(int D) {
  return (size_t)2 * kKeys * 128 * (D / 64)      // K, V
         + 2 * (size_t)kGroupBytes               // two groups
         + 256                                   // barriers
         + 2 * 2 * kMaxNq * 4                    // query positions, double buffered, per group
         + 2 * 128 * 4                           // partial-row index of each tile row, per group
         + 768;                                  // alignment slack (checked at run time)
}

__device__ __forceinline__ void group_sync(int group) {
  asm volatile("bar.sync %0, %1;" ::"r"(group + 1), "r"(kGroupThreads) : "memory");
}
// Named barrier that also tells every thread whether any of them brought a non-zero `pred`: the
// way a group of warps decides together to leave after a given-up wait.
__device__ __forceinline__ bool named_or_b(int id, int threads, int pred) {
  uint32_t out;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %3, 0;\n\t"
      "bar.red.or.pred p, %1, %2, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(out)
      : "r"(id), "r"(threads), "r"(pred)
      : "memory");
  return out != 0;
}

// Two compute groups of 256 threads share the key tile and the dK^T / dV^T accumulators and
// take alternate row tiles, so that one group's MMAs and memory waits overlap the other
// group's arithmetic.  Inside a group, the two warps of a TMEM lane quadrant split the 64 key
// columns of a row between them.  Row r of a tile is head r % G of the tile's query r / G: the
// G rows of a query arrive by one TMA box each for Q and dO (128B swizzle), whatever the query
// list looks like, and leave as bf16 dQ partials through a 128B-swizzled staging tile: a full
// tile by one asynchronous TMA store per slab, the ragged last tile as whole rows by hand.
template <int D>
__global__ void __launch_bounds__(512, 1)
tc_bwd_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
              const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
              const __grid_constant__ CUtensorMap tm_q_run, const __grid_constant__ CUtensorMap tm_do_run,
              const __grid_constant__ CUtensorMap tm_dq, const __grid_constant__ CUtensorMap tm_dqacc,
              const BwdArgs p) {
  constexpr int kSlabs = D / 64;
  constexpr int kKVBytes = kKeys * 128 * kSlabs;
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kColDV = 256, kColDK = 320;   // group g: S at 128 g, dP at 128 g + 64, dQ over both
  constexpr uint32_t kIdescS = idesc_bf16(128, kKeys, 0, 0);     // rows x keys
  constexpr uint32_t kIdescT = idesc_bf16(128, kKeys, 1, 1);     // d x keys, both MN-major
  constexpr uint32_t kIdescDQ = idesc_bf16(128, D, 0, 1);        // rows x d

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);   // pointer arithmetic keeps the shared address space
  uint8_t* sK = smem;
  uint8_t* sV = sK + kKVBytes;
  uint8_t* sGroup = sV + kKVBytes;
  uint64_t* bars = (uint64_t*)(sGroup + 2 * kGroupBytes);
  uint64_t* bar_kv = bars + 0;
  uint32_t* s_tmem = (uint32_t*)(bars + 8);
  volatile int* s_abort = (volatile int*)(s_tmem + 1);
  int* s_rowt_all = (int*)(bars + 10);               // [2 groups][2 buffers][kMaxNq]
  uint32_t* s_prow_all = (uint32_t*)(s_rowt_all + 2 * 2 * kMaxNq);   // [2][128]

  const int tid = threadIdx.x;
  const int grp = tid / kGroupThreads, lt = tid % kGroupThreads;
  const int wg = lt >> 5, lane = lt & 31;
  const int quad = wg & 3, half = wg >> 2;           // TMEM lane quadrant, key-column half
  const int row = quad * 32 + lane;                  // row of the tile this thread works on
  uint8_t* sQ = sGroup + grp * kGroupBytes;
  uint8_t* sDO = sQ + kRowTileBytes;
  uint8_t* sP = sDO + kRowTileBytes;
  uint8_t* sDS = sP + kPBytes;
  uint64_t* bar_sp = bars + 1 + 3 * grp;
  uint64_t* bar_acc = bars + 2 + 3 * grp;
  uint64_t* bar_g = bars + 3 + 3 * grp;
  uint64_t* bar_drain = bars + 7 + 2 * grp;
  int* s_rowt = s_rowt_all + grp * 2 * kMaxNq;
  uint32_t* s_prow = s_prow_all + grp * 128;

  int4 item = make_int4((int)blockIdx.y, (int)blockIdx.x, 0, 1);
  if (p.kind == 2) {                                 // selection: one work item per CTA
    if ((int)blockIdx.x >= p.work->n_items) return;
    item = reinterpret_cast<const int4*>(p.work + 1)[blockIdx.x];
  }
  const int j = item.y;                              // key tile
  const int bh = item.x;
  const int b = bh / p.Hkv, hkv = bh % p.Hkv;
  const int key0 = j * kKeys;
  const int ql = row / p.G, g = row % p.G;
  const int head = hkv * p.G + g;
  const bool row_slot_ok = ql < p.nq;

  // ---- the queries that attend this key tile ---------------------------------------------
  int t_lo = 0, n_q = 0, pair_base = 0;
  if (p.kind == 0) {
    t_lo = key0;
    n_q = min(p.T - 1, key0 + kKeys - 1 + p.window - 1) - t_lo + 1;
  } else if (p.kind == 1) {
    t_lo = key0 * p.window + p.block_size - 1;       // first query that sees summary key0 (window: the stride)
    n_q = p.T - t_lo;
  } else {
    pair_base = __ldg(p.offsets + (size_t)bh * (p.n_ktiles + 1) + j);
    n_q = __ldg(p.offsets + (size_t)bh * (p.n_ktiles + 1) + j + 1) - pair_base;
  }
  n_q = max(n_q, 0);
  const int n_rt_all = (n_q + p.nq - 1) / p.nq;
  // gridDim.z > 1: the row tiles are split in chunks and dK / dV go through fp32 atomics
  const int chunk = p.kind == 2 ? kSelChunkTiles : ((int)gridDim.z > 1 ? p.split_chunk : n_rt_all);
  const int rt_begin = p.kind == 2 ? item.z : (int)blockIdx.z * chunk;
  const int rt_end = min(n_rt_all, rt_begin + chunk);
  const bool split = p.kind == 2 ? item.w > 1 : gridDim.z > 1;

  if (rt_end <= rt_begin) {
    if (!split && n_rt_all == 0) {   // nobody attends these keys: their gradients are zero
      for (int i = tid; i < kKeys * D / 8; i += blockDim.x) {
        const int key = key0 + i / (D / 8);
        if (key < p.Lk) {
          const size_t off = ((size_t)bh * p.Lk + key) * D + (i % (D / 8)) * 8;
          *reinterpret_cast<uint4*>(p.dk + off) = make_uint4(0, 0, 0, 0);
          *reinterpret_cast<uint4*>(p.dv + off) = make_uint4(0, 0, 0, 0);
        }
      }
    }
    return;
  }

  if (tid == 0) {
    int bad = (*(volatile int*)p.status != 0) ? 1 : 0;
    if ((size_t)((uint8_t*)(s_prow_all + 2 * 128) - smem_raw) > bwd_smem_bytes(D)) {
      atomicOr(p.status, 256);   // the shared-memory window is less aligned than assumed
      bad = 1;
    }
    *s_abort = bad;
    // S / dP ready (bars 1 and 4) = the MMAs have completed and the previous tile's dQ store
    // has left the staging tile, which is the P / dS tile: two arrivals
    for (int k = 0; k <= 6; ++k) mbar_init(bars + k, (k == 1 || k == 4) ? 2 : 1);
    mbar_init(bars + 7, 1); mbar_init(bars + 9, 1);   // per group: an aborted CTA waits here for its last MMAs
    fence_barrier_init();
    prefetch_tensormap(&tm_k); prefetch_tensormap(&tm_v);
    prefetch_tensormap(&tm_q); prefetch_tensormap(&tm_do);
    prefetch_tensormap(p.dq_acc_mode ? &tm_dqacc : &tm_dq);
  }
  __syncthreads();
  if (*s_abort) return;
  // Rows past nq * G of a tile (and, for D = 64, the second slab) are never loaded: keep them 0.
  for (int i = tid; i < 2 * 2 * kRowTileBytes / 16; i += blockDim.x) {
    const int buf = i / (kRowTileBytes / 16), o16 = i % (kRowTileBytes / 16);
    uint8_t* base = sGroup + (buf >> 1) * kGroupBytes + (buf & 1) * kRowTileBytes;
    *reinterpret_cast<uint4*>(base + o16 * 16) = make_uint4(0, 0, 0, 0);
  }
  fence_proxy_async();

  if (tid < 32) {
    tmem_alloc(s_tmem, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *s_tmem;
  const uint32_t lane_base = tmem + ((uint32_t)(quad * 32) << 16);
  const uint32_t colS = grp * 128, colDP = grp * 128 + 64, colDQ = grp * 128;
  // Q / dO tiles: slab-major (8-row groups 1024 bytes apart, slabs kRows * 128 apart) or, with merged
  // boxes, the two slabs of an 8-row group side by side (groups 2048 bytes apart)
  const uint32_t q_slab = p.merged ? 1024u : (uint32_t)(kRows * 128), q_sbo = p.merged ? 2048u : 1024u;

  if (tid == 0) {
    mbar_expect_tx(bar_kv, 2 * kKVBytes);
#pragma unroll
    for (int s = 0; s < kSlabs; ++s) {
      tma_load_3d(sK + s * (kKeys * 128), &tm_k, bar_kv, s * 64, key0, bh);
      tma_load_3d(sV + s * (kKeys * 128), &tm_v, bar_kv, s * 64, key0, bh);
    }
  }
  // dK^T / dV^T start at zero so that every MMA into them accumulates
  if (grp == 0 && half == 0) {
    uint32_t z[32];
#pragma unroll
    for (int c = 0; c < 32; ++c) z[c] = 0u;
#pragma unroll
    for (int cc = 0; cc < 4; ++cc) tmem_st32(lane_base + kColDV + cc * 32, z);
    tmem_wait_st();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (tid == 0 || tid == kGroupThreads) mbar_wait(bar_kv, 0, p.status, s_abort, 32);

  // query position of this thread's row in row tile i (-1: no row)
  auto row_query = [&](int i) -> int {
    const int qi = i * p.nq + ql;
    if (!row_slot_ok || qi >= n_q) return -1;
    if (p.kind == 2) return ldg_s32_now(p.q_of_block + pair_base + qi);
    return t_lo + qi;
  };
  auto row_index = [&](int t) -> size_t { return (size_t)(b * p.Hq + head) * p.T + t; };
  // one TMA box per query and slab for Q and for dO; a missing query reads past T: zeros
  const uint32_t gather_bytes = (uint32_t)(p.nq * p.G * 128 * kSlabs * 2);
  // part (window / compression only): 0 = Q and dO, 1 = Q now (the byte count of both is
  // announced), 2 = dO, issued later because its tile served as staging meanwhile
  auto gather = [&](const int* rowt, int part = 0) {
    if (p.kind != 2) {
      // window / compression: the tile's queries are consecutive tokens, one box per slab
      if (lt == 0) {
        if (part != 2) mbar_expect_tx(bar_g, gather_bytes);
        const int tq = rowt[0] >= 0 ? rowt[0] : p.T;
#pragma unroll
        for (int s = 0; s < kSlabs; ++s) {
          if (part != 2) tma_load_3d(sQ + s * (kRows * 128), &tm_q_run, bar_g, s * 64, b * p.Hq + hkv * p.G, tq);
          if (part != 1) tma_load_3d(sDO + s * (kRows * 128), &tm_do_run, bar_g, s * 64, b * p.Hq + hkv * p.G, tq);
        }
      }
    } else {
      // selection: one box per (query, slab, tensor); the boxes are dealt out over the eight
      // warps of the group (a few lanes each) because one warp issues them one after another
      if (lt == 0) mbar_expect_tx(bar_g, gather_bytes);
      const int op = lane * 8 + wg;                       // op id -> (query, slab, Q or dO)
      if (p.merged) {
        // a box costs the TMA unit a fixed time whatever its size, and the boxes of a tile are what
        // bounds the kernel: one box per (query, tensor) brings both slabs, laid out side by side
        for (int o = op; o < p.nq * 2; o += kGroupThreads) {
          const int qq = o >> 1;
          const int tq = rowt[qq] >= 0 ? rowt[qq] : p.T;
          tma_load_5d(((o & 1) ? sDO : sQ) + qq * (p.G / 8) * 2048, (o & 1) ? &tm_do : &tm_q, bar_g, 0, 0, 0, tq,
                      (b * p.Hq + hkv * p.G) >> 3);
        }
      }
      const int n_ops = p.merged ? 0 : p.nq * kSlabs * 2;
      for (int o = op; o < n_ops; o += kGroupThreads) {
        const int qq = o / (kSlabs * 2), k = o % (kSlabs * 2);
        const int s = k >> 1;
        const int tq = rowt[qq] >= 0 ? rowt[qq] : p.T;   // a missing query reads past T: zeros
        if (k & 1)
          tma_load_3d(sDO + s * (kRows * 128) + qq * p.G * 128, &tm_do, bar_g, s * 64,
                      b * p.Hq + hkv * p.G, tq);
        else
          tma_load_3d(sQ + s * (kRows * 128) + qq * p.G * 128, &tm_q, bar_g, s * 64,
                      b * p.Hq + hkv * p.G, tq);
      }
    }
  };

  // Row metadata runs ahead of the work: the query position two tiles ahead (t_nxt) and, one
  // iteration later, its lse / delta, so that no dependent global load is waited for in line.
  int i = rt_begin + grp;
  int t_cur = i < rt_end ? row_query(i) : -1;
  int t_nxt = i + 2 < rt_end ? row_query(i + 2) : -1;
  float lse_cur = 0.f, delta_cur = 0.f, gate_cur = 1.f;
  if (t_cur >= 0) {
    lse_cur = __ldg(p.lse + row_index(t_cur));
    delta_cur = __ldg(p.delta + row_index(t_cur));
    if (p.row_scale) gate_cur = __ldg(p.row_scale + row_index(t_cur));
  }
  int buf = 0;
  bool g_pending = false;     // a gather of this group is on its way and its arrival has not been seen
  if (i < rt_end) {
    if (g == 0 && half == 0 && row_slot_ok) s_rowt[ql] = t_cur;
    group_sync(grp);
    gather(s_rowt);
    g_pending = true;
  }
  uint32_t phase = 0;
  for (; i < rt_end; i += 2, phase ^= 1, buf ^= 1) {
    const int t_nn = (i + 4 < rt_end) ? row_query(i + 4) : -1;
    float lse_nxt = 0.f, delta_nxt = 0.f, gate_nxt = 1.f;
    if (t_nxt >= 0) {
      lse_nxt = ldg_f32_now(p.lse + row_index(t_nxt));
      delta_nxt = ldg_f32_now(p.delta + row_index(t_nxt));
      if (p.row_scale) gate_nxt = ldg_f32_now(p.row_scale + row_index(t_nxt));
    }
    // query positions of this group's next tile, for the gather issued further down
    if (g == 0 && half == 0 && row_slot_ok) s_rowt[(buf ^ 1) * kMaxNq + ql] = t_nxt;
    if (mbar_wait(bar_g, phase, p.status, s_abort, 512)) g_pending = false;
    // also: the staging tile of the previous iteration has been read.  One decision for the whole
    // group: after a given-up wait it issues and writes nothing more
    if (named_or_b(grp + 1, kGroupThreads, *s_abort)) break;
    if (lt == 0) {
      tc_fence_after();
      const uint32_t qa = desc_lo_kmajor(smem_u32(sQ)), da = desc_lo_kmajor(smem_u32(sDO));
      const uint32_t ka = desc_lo_kmajor(smem_u32(sK)), va = desc_lo_kmajor(smem_u32(sV));
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        const uint32_t slab = kk >> 2, in = (kk & 3) * 32;
        mma_ss(tmem + colS, desc_at_sbo(qa, slab * q_slab + in, q_sbo),
               desc_at(ka, slab * (kKeys * 128) + in), kIdescS, kk > 0);
      }
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        const uint32_t slab = kk >> 2, in = (kk & 3) * 32;
        mma_ss(tmem + colDP, desc_at_sbo(da, slab * q_slab + in, q_sbo),
               desc_at(va, slab * (kKeys * 128) + in), kIdescS, kk > 0);
      }
      tc_commit(bar_sp);
      bulk_wait_read();
      mbar_arrive(bar_sp);
    }
    // valid key columns of this row: one range [lo, hi]
    int lo = 0, hi = -1;
    if (t_cur >= 0) {
      if (p.kind == 0) {
        lo = max(0, t_cur - p.window + 1 - key0);
        hi = min(kKeys - 1, t_cur - key0);
      } else if (p.kind == 1) {
        hi = min(kKeys - 1, cmp_visible(t_cur, p.block_size, p.window, p.Lk) - 1 - key0);
      } else {
        hi = min(kKeys - 1, min(t_cur, p.T - 1) - key0);
      }
    }
    const float lse2_cur = lse_cur * kLog2e;
    mbar_wait(bar_sp, phase, p.status, s_abort, 64);
    tc_fence_after();
    __syncwarp();
    {
      uint32_t rs[32], rp[32];
      tmem_ld32(lane_base + colS + half * 32, rs);
      tmem_ld32(lane_base + colDP + half * 32, rp);
      tmem_wait_ld();
      uint32_t pp[16], pd[16];
#pragma unroll
      for (int c2 = 0; c2 < 16; ++c2) {
        float pv[2], dv[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int c = half * 32 + c2 * 2 + e;
          const bool ok = (c >= lo) && (c <= hi);
          // gate_cur * p: the branch's dO is gate * dO, so dV takes (gate p)^T dO and
          // dS = scale * gate * p * (dO.v - dO.o)
          const float pr = ok ? gate_cur * ex2(__uint_as_float(rs[c2 * 2 + e]) * p.scale_log2 - lse2_cur) : 0.f;
          pv[e] = pr;
          dv[e] = pr * (__uint_as_float(rp[c2 * 2 + e]) - delta_cur) * p.scale;
        }
        pp[c2] = pack_bf16(pv[0], pv[1]);
        pd[c2] = pack_bf16(dv[0], dv[1]);
      }
      const uint32_t p_row = smem_u32(sP) + row * 128, ds_row = smem_u32(sDS) + row * 128;
#pragma unroll
      for (int k4 = 0; k4 < 4; ++k4) {
        const uint32_t chunk16 = (uint32_t)((half * 4 + k4) ^ (row & 7)) << 4;
        st_shared_v4(p_row + chunk16, pp[k4 * 4], pp[k4 * 4 + 1], pp[k4 * 4 + 2], pp[k4 * 4 + 3]);
        st_shared_v4(ds_row + chunk16, pd[k4 * 4], pd[k4 * 4 + 1], pd[k4 * 4 + 2], pd[k4 * 4 + 3]);
      }
    }
    fence_proxy_async();
    tc_fence_before();
    group_sync(grp);
    if (lt == 0) {
      tc_fence_after();
      const uint32_t qa = desc_lo_mnmajor(smem_u32(sQ), q_slab);
      const uint32_t da = desc_lo_mnmajor(smem_u32(sDO), q_slab);
      const uint32_t pa = desc_lo_mnmajor(smem_u32(sP), 0), dsa = desc_lo_mnmajor(smem_u32(sDS), 0);
      const uint32_t dsk = desc_lo_kmajor(smem_u32(sDS)), ka = desc_lo_mnmajor(smem_u32(sK), kKeys * 128);
#pragma unroll
      for (int kk = 0; kk < kRows / 16; ++kk)        // contraction over the 128 rows, 16 (two 8-row groups) a step
        mma_ss(tmem + kColDV, desc_at_sbo(da, kk * 2 * q_sbo, q_sbo), desc_at(pa, kk * 2048), kIdescT, 1);
#pragma unroll
      for (int kk = 0; kk < kRows / 16; ++kk)
        mma_ss(tmem + kColDK, desc_at_sbo(qa, kk * 2 * q_sbo, q_sbo), desc_at(dsa, kk * 2048), kIdescT, 1);
#pragma unroll
      for (int kk = 0; kk < kKeys / 16; ++kk)        // contraction over the 64 keys
        mma_ss(tmem + colDQ, desc_at(dsk, kk * 32), desc_at(ka, kk * 2048), kIdescDQ, kk > 0);
      tc_commit(bar_acc);
    }
    // row of the partial buffer that takes this row's dQ
    if (half == 0) {
      uint32_t prow = 0xffffffffu;
      if (t_cur >= 0) {
        if (p.kind == 2) {
          prow = (uint32_t)((size_t)(pair_base + i * p.nq + ql) * p.G + g);
        } else {
          const int slot = p.kind == 0 ? j % p.n_slots : j;
          prow = (uint32_t)((((size_t)bh * p.T + t_cur) * p.n_slots + slot) * p.G + g);
        }
      }
      s_prow[row] = prow;
    }
    mbar_wait(bar_acc, phase, p.status, s_abort, 128);
    tc_fence_after();
    if (p.dq_acc_mode) {
      // dQ: TMEM -> fp32 staging -> TMA reduce-add into the accumulator.  The fp32 tile is D / 32
      // slabs of 128 rows x 128 bytes (128B swizzle): the first two lie over the P / dS tiles, the
      // other two (D = 128) over the dO tile, whose refill therefore waits until the reduction has
      // read them; Q is refilled at once.
      constexpr bool kTwoStep = D > 64;
      if (i + 2 < rt_end) { gather(s_rowt + (buf ^ 1) * kMaxNq, kTwoStep ? 1 : 0); g_pending = true; }
      __syncwarp();
#pragma unroll
      for (int cc = 0; cc < D / 64; ++cc) {          // this thread's half of the D columns
        const int col0 = half * (D / 2) + cc * 32;
        const int slab = col0 >> 5;
        uint8_t* sbase = slab < 2 ? sP + slab * (kRows * 128) : sDO + (slab - 2) * (kRows * 128);
        uint32_t r32[32];
        tmem_ld32(lane_base + colDQ + col0, r32);
        tmem_wait_ld();
        const uint32_t rbase = smem_u32(sbase) + row * 128;
#pragma unroll
        for (int c = 0; c < 8; ++c)
          st_shared_v4(rbase + (((uint32_t)c ^ (uint32_t)(row & 7)) << 4), r32[c * 4], r32[c * 4 + 1],
                       r32[c * 4 + 2], r32[c * 4 + 3]);
      }
      fence_proxy_async();
      tc_fence_before();
      group_sync(grp);
      if (lt == 0) {
        // rows of queries past the tile's range carry zeros (p = 0 there); rows past T are dropped
        const int t_tile = t_lo + i * p.nq;
#pragma unroll
        for (int sl = 0; sl < D / 32; ++sl) {
          const uint8_t* sbase = sl < 2 ? sP + sl * (kRows * 128) : sDO + (sl - 2) * (kRows * 128);
          tma_reduce_add_4d(&tm_dqacc, sbase, sl * 32, 0, t_tile, bh);
        }
        bulk_commit();
        if (kTwoStep && i + 2 < rt_end) {
          bulk_wait_read();
          gather(s_rowt + (buf ^ 1) * kMaxNq, 2);
        }
      }
    } else {
      // the row tiles are free again: fetch this group's next tile
      if (i + 2 < rt_end) { gather(s_rowt + (buf ^ 1) * kMaxNq); g_pending = true; }
      __syncwarp();
      // dQ: TMEM -> bf16 -> staging tile (the P / dS region): one slab of 128-byte rows per 64
      // columns, 16-byte chunks XOR row, which is the layout of a 128B-swizzled TMA box
      {
#pragma unroll
        for (int cc = 0; cc < D / 64; ++cc) {          // this thread's half of the D columns
          const int col0 = half * (D / 2) + cc * 32;
          uint32_t r32[32];
          tmem_ld32(lane_base + colDQ + col0, r32);
          tmem_wait_ld();
#pragma unroll
          for (int v4 = 0; v4 < 4; ++v4) {
            const uint32_t chunk = (uint32_t)((col0 >> 3) + v4);
            st_shared_v4(smem_u32(sP) + (chunk >> 3) * (kRows * 128) + row * 128 + (((chunk & 7) ^ (row & 7)) << 4),
                         pack_bf16(__uint_as_float(r32[v4 * 8 + 0]), __uint_as_float(r32[v4 * 8 + 1])),
                         pack_bf16(__uint_as_float(r32[v4 * 8 + 2]), __uint_as_float(r32[v4 * 8 + 3])),
                         pack_bf16(__uint_as_float(r32[v4 * 8 + 4]), __uint_as_float(r32[v4 * 8 + 5])),
                         pack_bf16(__uint_as_float(r32[v4 * 8 + 6]), __uint_as_float(r32[v4 * 8 + 7])));
          }
        }
      }
      fence_proxy_async();
      tc_fence_before();
      group_sync(grp);
      if ((i + 1) * p.nq <= n_q) {
        // a full tile: its rows are consecutive in the partial buffer, one TMA store per slab
        if (lt == 0) {
          const int slot = p.kind == 2 ? 0 : (p.kind == 0 ? j % p.n_slots : j);
          const int mid = p.kind == 2 ? pair_base + i * p.nq : t_lo + i * p.nq;
          const int outer = p.kind == 2 ? 0 : bh;
#pragma unroll
          for (int sl = 0; sl < kSlabs; ++sl)
            tma_store_5d(&tm_dq, sP + sl * (kRows * 128), sl * 64, 0, slot, mid, outer);
          bulk_commit();
        }
      } else {   // the ragged last tile: 16 lanes write the 256 (D = 128) or 128 bytes of one row
        constexpr int kChunks = D / 8;
        constexpr int kRowsPerPass = kGroupThreads / kChunks;
        const int c = lt % kChunks;
#pragma unroll 4
        for (int r = lt / kChunks; r < kRows; r += kRowsPerPass) {
          const uint32_t prow = s_prow[r];
          if (prow != 0xffffffffu) {
            const uint4 v = *reinterpret_cast<const uint4*>(sP + (c >> 3) * (kRows * 128) + r * 128 +
                                                            (((c & 7) ^ (r & 7)) << 4));
            *reinterpret_cast<uint4*>(p.dq_part + (size_t)prow * D + c * 8) = v;
          }
        }
      }
    }
    t_cur = t_nxt; t_nxt = t_nn; lse_cur = lse_nxt; delta_cur = delta_nxt; gate_cur = gate_nxt;
  }

  if (lt == 0) bulk_wait_all();
  tc_fence_before();
  if (__syncthreads_or(*s_abort)) {
    // Give-up path: dK / dV are not written.  Each group's issuing thread waits (bounded) for the
    // gather still on its way into shared memory and for the MMAs it has issued; then the tensor
    // memory goes back.
    if (lt == 0) {
      if (grp == 0) mbar_wait_drain(bar_kv, 0);
      if (g_pending) mbar_wait_drain(bar_g, phase);
      tc_commit(bar_drain);
      mbar_wait_drain(bar_drain, 0);
    }
    tc_fence_before();
    __syncthreads();
    if (tid < 32) tmem_dealloc(tmem, kTmemCols);
    return;
  }
  // ---- dK^T, dV^T: lane = d, column = key; group 0 writes dV, group 1 writes dK ---------------
  tc_fence_after();
  if (half == 0) {
    const uint32_t col = grp == 0 ? kColDV : kColDK;
    const int d = row;
#pragma unroll
    for (int hc = 0; hc < 2; ++hc) {
      uint32_t r32[32];
      tmem_ld32(lane_base + col + hc * 32, r32);
      tmem_wait_ld();
      if (d < D) {
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          const int key = key0 + hc * 32 + c;
          if (key < p.Lk) {
            const size_t o = ((size_t)bh * p.Lk + key) * D + d;
            if (split) atomicAdd((grp == 0 ? p.dv_acc : p.dk_acc) + o, __uint_as_float(r32[c]));
            else (grp == 0 ? p.dv : p.dk)[o] = __float2bfloat16_rn(__uint_as_float(r32[c]));
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (tid < 32) tmem_dealloc(tmem, kTmemCols);
}

// ---- the same backward with the issuing taken out of the compute groups ---------------------------
// Two row tiles are in flight (shared memory holds no more: Q, dO, P, dS of a tile are 96 KB), one
// per slot.  Three producer warps refill a slot's Q / dO the moment its MMAs are done; one thread
// issues whichever batch of MMAs is ready next (S / dP of the tile that has landed, or dV / dK / dQ
// of the tile whose probabilities are written); each slot has a compute group of 256 threads (two
// warps per TMEM lane quadrant, half of the key columns each) that turns S / dP into P / dS and,
// while the slot's next tile is on its way, moves the tile's dQ from TMEM to the staging tile and
// stores it.  Each hand-over is an mbarrier with a bounded wait.  The tensor pipe needs about 2.9 k
// cycles per row tile (80-100 cycles per MMA instruction: their shared-memory operands, not the
// arithmetic); the aim of this arrangement is to keep it fed.
constexpr int kB2Threads = 640;   // 2 x 8 compute warps, 3 producer warps, MMA warp
constexpr int kB2Producers = 3;
constexpr int kB2Compute = 16;    // compute warps

template <int D>
__global__ void __launch_bounds__(kB2Threads, 1)
tc_bwd2_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
               const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
               const __grid_constant__ CUtensorMap tm_q_run, const __grid_constant__ CUtensorMap tm_do_run,
               const __grid_constant__ CUtensorMap tm_dq, const BwdArgs p) {
  constexpr int kSlabs = D / 64;
  constexpr int kKVBytes = kKeys * 128 * kSlabs;
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kColDV = 256, kColDK = 320;   // slot s: S at 128 s, dP at 128 s + 64, dQ over both
  constexpr uint32_t kIdescS = idesc_bf16(128, kKeys, 0, 0);
  constexpr uint32_t kIdescT = idesc_bf16(128, kKeys, 1, 1);
  constexpr uint32_t kIdescDQ = idesc_bf16(128, D, 0, 1);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* sK = smem;
  uint8_t* sV = sK + kKVBytes;
  uint8_t* sGroup = sV + kKVBytes;
  uint64_t* bars = (uint64_t*)(sGroup + 2 * kGroupBytes);
  uint64_t* bar_kv = bars + 0;
  uint64_t* g_full = bars + 1;       // [2] Q / dO of the slot have landed
  uint64_t* sp_full = bars + 3;      // [2] S / dP of the slot are in TMEM
  uint64_t* pds_full = bars + 5;     // [2] P / dS of the slot are in shared memory (128 arrivals)
  uint64_t* acc_full = bars + 7;     // [2] dV / dK / dQ MMAs of the slot are done
  uint64_t* dq_read = bars + 9;      // [2] dQ of the slot has left TMEM (256 arrivals)
  uint64_t* qdo_free = bars + 13;    // [2] the dV / dK MMAs of the slot are done: Q / dO may be refilled
  uint64_t* bar_drain = bars + 11;
  uint32_t* s_tmem = (uint32_t*)(bars + 16);
  volatile int* s_abort = (volatile int*)(s_tmem + 1);
  uint32_t* s_prow = (uint32_t*)(s_tmem + 4);        // [2][128] partial row of each tile row (ragged tile), per slot

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  int4 item = make_int4((int)blockIdx.y, (int)blockIdx.x, 0, 1);
  if (p.kind == 2) {                                 // selection: one work item per CTA
    if ((int)blockIdx.x >= p.work->n_items) return;
    item = reinterpret_cast<const int4*>(p.work + 1)[blockIdx.x];
  }
  const int j = item.y;                              // key tile
  const int bh = item.x;
  const int b = bh / p.Hkv, hkv = bh % p.Hkv;
  const int key0 = j * kKeys;

  // ---- the queries that attend this key tile ---------------------------------------------
  int t_lo = 0, n_q = 0, pair_base = 0;
  if (p.kind == 0) {
    t_lo = key0;
    n_q = min(p.T - 1, key0 + kKeys - 1 + p.window - 1) - t_lo + 1;
  } else if (p.kind == 1) {
    t_lo = key0 * p.window + p.block_size - 1;       // first query that sees summary key0 (window: the stride)
    n_q = p.T - t_lo;
  } else {
    pair_base = __ldg(p.offsets + (size_t)bh * (p.n_ktiles + 1) + j);
    n_q = __ldg(p.offsets + (size_t)bh * (p.n_ktiles + 1) + j + 1) - pair_base;
  }
  n_q = max(n_q, 0);
  const int n_rt_all = (n_q + p.nq - 1) / p.nq;
  const int chunk = p.kind == 2 ? kSelChunkTiles : ((int)gridDim.z > 1 ? p.split_chunk : n_rt_all);
  const int rt_begin = p.kind == 2 ? item.z : (int)blockIdx.z * chunk;
  const int rt_end = min(n_rt_all, rt_begin + chunk);
  const bool split = p.kind == 2 ? item.w > 1 : gridDim.z > 1;
  const int n_tiles = rt_end - rt_begin;

  if (n_tiles <= 0) {
    if (!split && n_rt_all == 0) {   // nobody attends these keys: their gradients are zero
      for (int i = tid; i < kKeys * D / 8; i += blockDim.x) {
        const int key = key0 + i / (D / 8);
        if (key < p.Lk) {
          const size_t off = ((size_t)bh * p.Lk + key) * D + (i % (D / 8)) * 8;
          *reinterpret_cast<uint4*>(p.dk + off) = make_uint4(0, 0, 0, 0);
          *reinterpret_cast<uint4*>(p.dv + off) = make_uint4(0, 0, 0, 0);
        }
      }
    }
    return;
  }

  if (tid == 0) {
    int bad = (*(volatile int*)p.status != 0) ? 1 : 0;
    if ((size_t)((uint8_t*)(s_prow + 256) - smem_raw) > bwd_smem_bytes(D)) {
      atomicOr(p.status, 256);   // the shared-memory window is less aligned than assumed
      bad = 1;
    }
    *s_abort = bad;
    mbar_init(bar_kv, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(g_full + s, 1); mbar_init(sp_full + s, 1); mbar_init(pds_full + s, 256);
      mbar_init(acc_full + s, 1); mbar_init(dq_read + s, 256); mbar_init(qdo_free + s, 1);
    }
    mbar_init(bar_drain, 1);
    fence_barrier_init();
    prefetch_tensormap(&tm_k); prefetch_tensormap(&tm_v);
    prefetch_tensormap(&tm_q); prefetch_tensormap(&tm_do); prefetch_tensormap(&tm_dq);
  }
  __syncthreads();
  if (*s_abort) return;
  // Rows past nq * G of a tile (and, for D = 64, the second slab) are never loaded: keep them 0.
  for (int i = tid; i < 2 * 2 * kRowTileBytes / 16; i += kB2Threads) {
    const int buf = i / (kRowTileBytes / 16), o16 = i % (kRowTileBytes / 16);
    uint8_t* base = sGroup + (buf >> 1) * kGroupBytes + (buf & 1) * kRowTileBytes;
    *reinterpret_cast<uint4*>(base + o16 * 16) = make_uint4(0, 0, 0, 0);
  }
  fence_proxy_async();
  if (warp == 0) {
    tmem_alloc(s_tmem, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *s_tmem;
  // dK^T / dV^T start at zero so that every MMA into them accumulates
  if (warp < 4) {
    uint32_t z[32];
#pragma unroll
    for (int c = 0; c < 32; ++c) z[c] = 0u;
    const uint32_t lb = tmem + ((uint32_t)(warp * 32) << 16);
#pragma unroll
    for (int cc = 0; cc < 4; ++cc) tmem_st32(lb + kColDV + cc * 32, z);
    tmem_wait_st();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  if (warp >= kB2Compute && warp < kB2Compute + kB2Producers) {
    // ---- producers: K / V once, then Q and dO of every tile.  A warp gets a TMA box out every
    // 60-100 cycles whatever its size, so the boxes of a tile are dealt out over three warps
    // (box o to warp o % 3) and, where the shape allows, one box brings both column slabs ---------
    const int pw = warp - kB2Compute;
    if (pw == 0 && lane == 0) {
      mbar_expect_tx(bar_kv, 2 * kKVBytes);
#pragma unroll
      for (int s = 0; s < kSlabs; ++s) {
        tma_load_3d(sK + s * (kKeys * 128), &tm_k, bar_kv, s * 64, key0, bh);
        tma_load_3d(sV + s * (kKeys * 128), &tm_v, bar_kv, s * 64, key0, bh);
      }
    }
    const uint32_t gather_bytes = (uint32_t)(p.nq * p.G * 128 * kSlabs * 2);
    const int per_q = p.merged ? 2 : kSlabs * 2;     // boxes per query: Q and dO, per slab unless merged
    const int n_ops = p.nq * per_q;                  // selection: the boxes of a tile
    constexpr int kRounds = (kMaxNq * kSlabs * 2 + 32 * kB2Producers - 1) / (32 * kB2Producers);
    auto box_of = [&](int r) -> int { return (r * 32 + lane) * kB2Producers + pw; };
    auto tq_of = [&](int k, int o) -> int {          // query position of box o of tile k (none: past T, zeros)
      const int qi = (rt_begin + k) * p.nq + o / per_q;
      return (o < n_ops && qi < n_q) ? ldg_s32_now(p.q_of_block + pair_base + qi) : p.T;
    };
    int tq[kRounds];
    if (p.kind == 2) {
#pragma unroll
      for (int r = 0; r < kRounds; ++r) tq[r] = tq_of(0, box_of(r));
    }
    const uint64_t pol_keep = l2_policy_evict_normal();   // gathered q / dO rows: read again by other blocks
    int issued = 0;                                  // tiles whose loads this warp has sent off
    for (int k = 0; k < n_tiles; ++k) {
      const int sb = k & 1;
      // the slot's Q / dO are free once the dV / dK MMAs of tile k-2 are done (dQ reads dS and K only)
      if (k >= 2) mbar_wait(qdo_free + sb, ((k >> 1) - 1) & 1, p.status, s_abort, 128);
      if (__any_sync(0xffffffffu, *s_abort)) break;           // the whole warp leaves together
      uint8_t* sQ = sGroup + sb * kGroupBytes;
      uint8_t* sDO = sQ + kRowTileBytes;
      if (pw == 0 && lane == 0) mbar_expect_tx(g_full + sb, gather_bytes);
      __syncwarp();
      if (p.kind != 2) {
        // window / compression: the tile's queries are consecutive tokens, one box per slab
        if (pw == 0 && lane == 0) {
          const int qi = (rt_begin + k) * p.nq;
          const int t0 = qi < n_q ? t_lo + qi : p.T;
#pragma unroll
          for (int s = 0; s < kSlabs; ++s) {
            tma_load_3d(sQ + s * (kRows * 128), &tm_q_run, g_full + sb, s * 64, b * p.Hq + hkv * p.G, t0);
            tma_load_3d(sDO + s * (kRows * 128), &tm_do_run, g_full + sb, s * 64, b * p.Hq + hkv * p.G, t0);
          }
        }
      } else {
#pragma unroll
        for (int r = 0; r < kRounds; ++r) {
          const int o = box_of(r);
          if (o < n_ops && p.merged) {
            tma_load_5d_hint(((o & 1) ? sDO : sQ) + (o >> 1) * (p.G / 8) * 2048, (o & 1) ? &tm_do : &tm_q, g_full + sb,
                             0, 0, 0, tq[r], (b * p.Hq + hkv * p.G) >> 3, pol_keep);
          } else if (o < n_ops) {
            const int qq = o / (kSlabs * 2), kx = o % (kSlabs * 2);
            const int s = kx >> 1;
            if (kx & 1)
              tma_load_3d(sDO + s * (kRows * 128) + qq * p.G * 128, &tm_do, g_full + sb, s * 64,
                          b * p.Hq + hkv * p.G, tq[r]);
            else
              tma_load_3d(sQ + s * (kRows * 128) + qq * p.G * 128, &tm_q, g_full + sb, s * 64,
                          b * p.Hq + hkv * p.G, tq[r]);
          }
        }
        if (k + 1 < n_tiles) {
#pragma unroll
          for (int r = 0; r < kRounds; ++r) tq[r] = tq_of(k + 1, box_of(r));
        }
      }
      issued = k + 1;
    }
    if (*s_abort && pw == 0 && lane == 0) {
      // give-up path: the loads still on their way into this CTA's shared memory land (bounded
      // wait on the last phase of each slot) before the CTA ends
      mbar_wait_drain(bar_kv, 0);
      for (int k = max(0, issued - 2); k < issued; ++k) mbar_wait_drain(g_full + (k & 1), (k >> 1) & 1);
    }
  } else if (warp == kB2Compute + kB2Producers) {
    // ---- MMA issuer: whichever batch is ready next ---------------------------------------------
    if (lane == 0) {
      mbar_wait(bar_kv, 0, p.status, s_abort, 32);
      const uint32_t ka = desc_lo_kmajor(smem_u32(sK)), va = desc_lo_kmajor(smem_u32(sV));
      const uint32_t kb = desc_lo_mnmajor(smem_u32(sK), kKeys * 128);
      const uint32_t q_slab = p.merged ? 1024u : (uint32_t)(kRows * 128), q_sbo = p.merged ? 2048u : 1024u;
      int next_a = 0, next_b = 0;                    // next tile for S / dP, next tile for dV / dK / dQ
      long long idle_since = clock64();
      uint32_t polls = 0;
      while (next_b < n_tiles) {
        bool progressed = false;
        if (next_a < n_tiles) {
          const int k = next_a, sb = k & 1, u = k >> 1;
          // Q / dO have landed; dQ of tile k-2, which lies over the slot's S / dP columns, has been read
          if (mbar_try_wait(g_full + sb, u & 1) && (k < 2 || mbar_try_wait(dq_read + sb, (u - 1) & 1))) {
            tc_fence_after();
            const uint8_t* sQ = sGroup + sb * kGroupBytes;
            const uint32_t qa = desc_lo_kmajor(smem_u32(sQ)), da = desc_lo_kmajor(smem_u32(sQ + kRowTileBytes));
            const uint32_t colS = tmem + sb * 128, colDP = colS + 64;
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
              const uint32_t slab = kk >> 2, in = (kk & 3) * 32;
              mma_ss(colS, desc_at_sbo(qa, slab * q_slab + in, q_sbo), desc_at(ka, slab * (kKeys * 128) + in),
                     kIdescS, kk > 0);
            }
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
              const uint32_t slab = kk >> 2, in = (kk & 3) * 32;
              mma_ss(colDP, desc_at_sbo(da, slab * q_slab + in, q_sbo), desc_at(va, slab * (kKeys * 128) + in),
                     kIdescS, kk > 0);
            }
            tc_commit(sp_full + sb);
            ++next_a;
            progressed = true;
          }
        }
        if (next_b < next_a) {
          const int k = next_b, sb = k & 1, u = k >> 1;
          if (mbar_try_wait(pds_full + sb, u & 1)) {
            tc_fence_after();
            const uint8_t* sQ = sGroup + sb * kGroupBytes;
            const uint8_t* sP = sQ + 2 * kRowTileBytes;
            const uint8_t* sDS = sP + kPBytes;
            const uint32_t qa = desc_lo_mnmajor(smem_u32(sQ), q_slab);
            const uint32_t da = desc_lo_mnmajor(smem_u32(sQ + kRowTileBytes), q_slab);
            const uint32_t pa = desc_lo_mnmajor(smem_u32(sP), 0), dsa = desc_lo_mnmajor(smem_u32(sDS), 0);
            const uint32_t dsk = desc_lo_kmajor(smem_u32(sDS));
#pragma unroll
            for (int kk = 0; kk < kRows / 16; ++kk)        // contraction over the 128 rows, 16 a step
              mma_ss(tmem + kColDV, desc_at_sbo(da, kk * 2 * q_sbo, q_sbo), desc_at(pa, kk * 2048), kIdescT, 1);
#pragma unroll
            for (int kk = 0; kk < kRows / 16; ++kk)
              mma_ss(tmem + kColDK, desc_at_sbo(qa, kk * 2 * q_sbo, q_sbo), desc_at(dsa, kk * 2048), kIdescT, 1);
            tc_commit(qdo_free + sb);
#pragma unroll
            for (int kk = 0; kk < kKeys / 16; ++kk)        // contraction over the 64 keys
              mma_ss(tmem + sb * 128, desc_at(dsk, kk * 32), desc_at(kb, kk * 2048), kIdescDQ, kk > 0);
            tc_commit(acc_full + sb);
            ++next_b;
            progressed = true;
          }
        }
        if (progressed) {
          idle_since = clock64();
        } else if ((++polls & 0xffu) == 0) {
          if (*s_abort) break;
          if (*(volatile int*)p.status != 0) { *s_abort = 1; break; }
          if (clock64() - idle_since > kWaitLimitCycles) { atomicOr(p.status, 2048); *s_abort = 1; break; }
        }
      }
      // the tensor pipe is idle before TMEM is read for dK / dV and given back, whatever happened
      tc_commit(bar_drain);
      if (!mbar_wait(bar_drain, 0, p.status, s_abort, 4096)) mbar_wait_drain(bar_drain, 0);
    }
  } else if (warp < kB2Compute) {
    // ---- compute group of slot sb: S, dP -> P, dS; then the tile's dQ out -----------------------------
    const int sb = warp >> 3, wg = warp & 7, lt = (warp & 7) * 32 + lane;
    const int quad = wg & 3, half = wg >> 2;           // TMEM lane quadrant, key-column half
    const int row = quad * 32 + lane;
    const int ql = row / p.G, g = row % p.G;
    const int head = hkv * p.G + g;
    const bool row_slot_ok = ql < p.nq;
    uint8_t* sP = sGroup + sb * kGroupBytes + 2 * kRowTileBytes;
    uint8_t* sDS = sP + kPBytes;
    uint32_t* s_prow_g = s_prow + sb * 128;
    const uint32_t lane_base = tmem + ((uint32_t)(quad * 32) << 16) + sb * 128;
    auto row_query = [&](int k) -> int {
      const int qi = (rt_begin + k) * p.nq + ql;
      if (!row_slot_ok || qi >= n_q) return -1;
      if (p.kind == 2) return ldg_s32_now(p.q_of_block + pair_base + qi);
      return t_lo + qi;
    };
    auto row_index = [&](int t) -> size_t { return (size_t)(b * p.Hq + head) * p.T + t; };
    int t_cur = sb < n_tiles ? row_query(sb) : -1;
    int t_nxt = sb + 2 < n_tiles ? row_query(sb + 2) : -1;
    float lse_cur = 0.f, delta_cur = 0.f, gate_cur = 1.f;
    if (t_cur >= 0) {
      lse_cur = __ldg(p.lse + row_index(t_cur));
      delta_cur = __ldg(p.delta + row_index(t_cur));
      if (p.row_scale) gate_cur = __ldg(p.row_scale + row_index(t_cur));
    }
    for (int k = sb; k < n_tiles; k += 2) {
      const int u = k >> 1, i = rt_begin + k;
      const int t_nn = (k + 4 < n_tiles) ? row_query(k + 4) : -1;
      float lse_nxt = 0.f, delta_nxt = 0.f, gate_nxt = 1.f;
      if (t_nxt >= 0) {
        lse_nxt = ldg_f32_now(p.lse + row_index(t_nxt));
        delta_nxt = ldg_f32_now(p.delta + row_index(t_nxt));
        if (p.row_scale) gate_nxt = ldg_f32_now(p.row_scale + row_index(t_nxt));
      }
      int lo = 0, hi = -1;                           // valid key columns of this row: one range [lo, hi]
      if (t_cur >= 0) {
        if (p.kind == 0) {
          lo = max(0, t_cur - p.window + 1 - key0);
          hi = min(kKeys - 1, t_cur - key0);
        } else if (p.kind == 1) {
          hi = min(kKeys - 1, cmp_visible(t_cur, p.block_size, p.window, p.Lk) - 1 - key0);
        } else {
          hi = min(kKeys - 1, min(t_cur, p.T - 1) - key0);
        }
      }
      // gate * p = 2^(s * scale * log2e - lse * log2e + log2(gate)): the branch's dO is gate * dO, so dV takes
      // (gate p)^T dO; dS = scale * gate * p * (dP - delta), the constant factors folded once per row
      const float lse2 = lse_cur * kLog2e - __log2f(gate_cur);
      const float dscale = p.scale, ddelta = delta_cur * p.scale;
      // every column of this thread's half is attended (the usual case away from the diagonal)?
      const bool all_cols = lo <= half * 32 && hi >= half * 32 + 31;
      mbar_wait(sp_full + sb, u & 1, p.status, s_abort, 64);
      // the P / dS tiles double as the dQ staging tile: this group's store of tile k-2 has read it
      if (lt == 0) bulk_wait_read();
      if (named_or_b(1 + sb, 256, *s_abort)) break;            // the whole group leaves together
      tc_fence_after();
      {
        uint32_t rs[32], rp[32];
        tmem_ld32(lane_base + half * 32, rs);
        tmem_ld32(lane_base + 64 + half * 32, rp);
        tmem_wait_ld();
        uint32_t pp[16], pd[16];
        if (__all_sync(0xffffffffu, all_cols)) {
#pragma unroll
          for (int c2 = 0; c2 < 16; ++c2) {
            const float p0 = ex2(fmaf(__uint_as_float(rs[c2 * 2]), p.scale_log2, -lse2));
            const float p1 = ex2(fmaf(__uint_as_float(rs[c2 * 2 + 1]), p.scale_log2, -lse2));
            pp[c2] = pack_bf16(p0, p1);
            pd[c2] = pack_bf16(p0 * fmaf(__uint_as_float(rp[c2 * 2]), dscale, -ddelta),
                               p1 * fmaf(__uint_as_float(rp[c2 * 2 + 1]), dscale, -ddelta));
          }
        } else {
#pragma unroll
          for (int c2 = 0; c2 < 16; ++c2) {
            float pv[2], dv[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int c = half * 32 + c2 * 2 + e;
              const bool ok = (c >= lo) && (c <= hi);
              const float pr = ok ? ex2(fmaf(__uint_as_float(rs[c2 * 2 + e]), p.scale_log2, -lse2)) : 0.f;
              pv[e] = pr;
              dv[e] = pr * fmaf(__uint_as_float(rp[c2 * 2 + e]), dscale, -ddelta);
            }
            pp[c2] = pack_bf16(pv[0], pv[1]);
            pd[c2] = pack_bf16(dv[0], dv[1]);
          }
        }
        const uint32_t p_row = smem_u32(sP) + row * 128, ds_row = smem_u32(sDS) + row * 128;
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4) {
          const uint32_t chunk16 = (uint32_t)((half * 4 + k4) ^ (row & 7)) << 4;
          st_shared_v4(p_row + chunk16, pp[k4 * 4], pp[k4 * 4 + 1], pp[k4 * 4 + 2], pp[k4 * 4 + 3]);
          st_shared_v4(ds_row + chunk16, pd[k4 * 4], pd[k4 * 4 + 1], pd[k4 * 4 + 2], pd[k4 * 4 + 3]);
        }
      }
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive(pds_full + sb);
      // ---- the tile's dQ: TMEM -> bf16 -> staging tile (the P / dS region, free once the MMAs are
      // done) -> partial buffer, while the producers fetch the slot's next tile
      mbar_wait(acc_full + sb, u & 1, p.status, s_abort, 128);
      tc_fence_after();
#pragma unroll
      for (int cc = 0; cc < D / 64; ++cc) {          // this thread's half of the D columns
        const int col0 = half * (D / 2) + cc * 32;
        uint32_t r32[32];
        tmem_ld32(lane_base + col0, r32);
        tmem_wait_ld();
        if (cc == D / 64 - 1) {            // dQ is in registers: S / dP of the slot's next tile may land
          tc_fence_before();
          mbar_arrive(dq_read + sb);
        }
#pragma unroll
        for (int v4 = 0; v4 < 4; ++v4) {
          const uint32_t chunk = (uint32_t)((col0 >> 3) + v4);
          st_shared_v4(smem_u32(sP) + (chunk >> 3) * (kRows * 128) + row * 128 + (((chunk & 7) ^ (row & 7)) << 4),
                       pack_bf16(__uint_as_float(r32[v4 * 8 + 0]), __uint_as_float(r32[v4 * 8 + 1])),
                       pack_bf16(__uint_as_float(r32[v4 * 8 + 2]), __uint_as_float(r32[v4 * 8 + 3])),
                       pack_bf16(__uint_as_float(r32[v4 * 8 + 4]), __uint_as_float(r32[v4 * 8 + 5])),
                       pack_bf16(__uint_as_float(r32[v4 * 8 + 6]), __uint_as_float(r32[v4 * 8 + 7])));
        }
      }
      const bool full_tile = (i + 1) * p.nq <= n_q;
      if (!full_tile && half == 0) {
        uint32_t prow = 0xffffffffu;
        const int qi = i * p.nq + ql;
        if (row_slot_ok && qi < n_q) {
          if (p.kind == 2) {
            prow = (uint32_t)((size_t)(pair_base + qi) * p.G + g);
          } else {
            const int slot = p.kind == 0 ? j % p.n_slots : j;
            prow = (uint32_t)((((size_t)bh * p.T + t_lo + qi) * p.n_slots + slot) * p.G + g);
          }
        }
        s_prow_g[row] = prow;
      }
      fence_proxy_async();
      if (named_or_b(1 + sb, 256, *s_abort)) break;
      if (full_tile) {
        // its rows are consecutive in the partial buffer: one TMA store per slab
        if (lt == 0) {
          const int slot = p.kind == 2 ? 0 : (p.kind == 0 ? j % p.n_slots : j);
          const int mid = p.kind == 2 ? pair_base + i * p.nq : t_lo + i * p.nq;
          const int outer = p.kind == 2 ? 0 : bh;
#pragma unroll
          for (int sl = 0; sl < kSlabs; ++sl)
            tma_store_5d_hint(&tm_dq, sP + sl * (kRows * 128), sl * 64, 0, slot, mid, outer, l2_policy_evict_first());
          bulk_commit();
        }
      } else {   // the ragged last tile: 16 lanes write the 256 (D = 128) or 128 bytes of one row
        constexpr int kChunks = D / 8;
        constexpr int kRowsPerPass = 256 / kChunks;
        const int c = lt % kChunks;
        for (int r = lt / kChunks; r < kRows; r += kRowsPerPass) {
          const uint32_t prow = s_prow_g[r];
          if (prow != 0xffffffffu) {
            const uint4 v = *reinterpret_cast<const uint4*>(sP + (c >> 3) * (kRows * 128) + r * 128 +
                                                            (((c & 7) ^ (r & 7)) << 4));
            *reinterpret_cast<uint4*>(p.dq_part + (size_t)prow * D + c * 8) = v;
          }
        }
      }
      t_cur = t_nxt; t_nxt = t_nn; lse_cur = lse_nxt; delta_cur = delta_nxt; gate_cur = gate_nxt;
    }
    if (lt == 0) bulk_wait_all();
  }

  // ---- dK^T, dV^T: lane = d, column = key; compute group 0 writes dV, group 1 writes dK ----------
  __syncthreads();           // the MMA thread has seen the tensor pipe drain (bar_drain)
  tc_fence_after();
  if (warp < kB2Compute && ((warp >> 2) & 1) == 0 && !*s_abort) {
    const int grp = warp >> 3, quad = warp & 3;
    const uint32_t col = grp == 0 ? kColDV : kColDK;
    const uint32_t lane_base = tmem + ((uint32_t)(quad * 32) << 16);
    const int d = quad * 32 + lane;
#pragma unroll
    for (int hc = 0; hc < 2; ++hc) {
      uint32_t r32[32];
      tmem_ld32(lane_base + col + hc * 32, r32);
      tmem_wait_ld();
      if (d < D) {
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          const int key = key0 + hc * 32 + c;
          if (key < p.Lk) {
            const size_t o = ((size_t)bh * p.Lk + key) * D + d;
            if (split) atomicAdd((grp == 0 ? p.dv_acc : p.dk_acc) + o, __uint_as_float(r32[c]));
            else (grp == 0 ? p.dv : p.dk)[o] = __float2bfloat16_rn(__uint_as_float(r32[c]));
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, kTmemCols);
}

// delta[b,h,t] = sum_d dO * O (fp32), one warp per row
__global__ void delta_kernel(const __nv_bfloat16* __restrict__ d_o, const __nv_bfloat16* __restrict__ o,
                             float* __restrict__ delta, size_t rows, int D) {
  const size_t row = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  float s = 0.f;
  for (int d = lane * 2; d < D; d += 64) {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(d_o + row * D + d));
    const float2 c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(o + row * D + d));
    s = fmaf(a.x, c.x, fmaf(a.y, c.y, s));
  }
  s = warp_sum(s);
  if (lane == 0) delta[row] = s;
}

// dq[b, hkv*G+g, t, :] = sum over the partial slots of query (bh, t); one thread per 8 elements
template <int D>
__global__ void dq_reduce_kernel(const __nv_bfloat16* __restrict__ part, const int32_t* __restrict__ pair_of_slot,
                                 __nv_bfloat16* __restrict__ dq, int B, int Hq, int Hkv, int T, int G,
                                 int kind, int window, int block_size, int Lk, int n_slots, int S) {
  constexpr int kVec = D / 8;
  const size_t gid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t total = (size_t)B * Hkv * T * G * kVec;
  if (gid >= total) return;
  const int v = (int)(gid % kVec);
  const int g = (int)((gid / kVec) % G);
  const int t = (int)((gid / ((size_t)kVec * G)) % T);
  const size_t bh = gid / ((size_t)kVec * G * T);
  float acc[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) acc[e] = 0.f;
  auto add = [&](size_t row_index) {
    const uint4 u = __ldg(reinterpret_cast<const uint4*>(part + (row_index * G + g) * D + v * 8));
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = __bfloat1622float2(h[e]);
      acc[2 * e] += f.x;
      acc[2 * e + 1] += f.y;
    }
  };
  if (kind == 2) {
    const int32_t* ps = pair_of_slot + (bh * T + t) * S;
    for (int s = 0; s < S; ++s) {
      const int pr = __ldg(ps + s);
      if (pr >= 0) add((size_t)pr);
    }
  } else {
    int first, last;   // key tiles this query attends
    if (kind == 0) { first = max(0, t - window + 1) >> 6; last = t >> 6; }
    else { first = 0; last = cmp_visible(t, block_size, window, Lk) - 1; last = last < 0 ? -1 : last >> 6; }
    for (int jt = first; jt <= last; ++jt) {
      const int slot = kind == 0 ? jt % n_slots : jt;
      add((bh * T + t) * n_slots + slot);
    }
  }
  const int b = (int)(bh / Hkv), hkv = (int)(bh % Hkv);
  uint4 u;
  u.x = pack_bf16(acc[0], acc[1]); u.y = pack_bf16(acc[2], acc[3]);
  u.z = pack_bf16(acc[4], acc[5]); u.w = pack_bf16(acc[6], acc[7]);
  *reinterpret_cast<uint4*>(dq + (((size_t)b * Hq + hkv * G + g) * T + t) * D + v * 8) = u;
}

// dq of the whole op in one pass: the partials of the compression, selection and window branches
// of query (bh, t) are added in fp32 and rounded once.  A branch whose buffer is null is absent.
struct Reduce3Args {
  const __nv_bfloat16* part_cmp; int slots_cmp, Lk_cmp, cmp_len, cmp_stride;
  const __nv_bfloat16* part_slc; const int32_t* pair_of_slot; int S;
  const __nv_bfloat16* part_win; int slots_win, window;
  const float* acc;            // fp32 accumulator [units][T][G][D] holding the window + compression part, or null
  __nv_bfloat16* dq;
  int B, Hq, Hkv, T, G;
};

// One thread adds up 8 columns of a query's dQ for HG heads (g, g + G / HG, ...): the heads of a
// query share the partial rows, so their index loads and address arithmetic are paid once.  The
// kernel moves 32 GB at the benchmark shape and was held back by its instruction count, not by
// memory, when every thread served a single head.
template <int D, int HG>
__global__ void dq_reduce3_kernel(const Reduce3Args a) {
  constexpr int kVec = D / 8;
  const int Gp = a.G / HG;                               // head groups per query
  const size_t gid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t total = (size_t)a.B * a.Hkv * a.T * Gp * kVec;
  if (gid >= total) return;
  const int v = (int)(gid % kVec);
  const int g = (int)((gid / kVec) % Gp);
  const int t = (int)((gid / ((size_t)kVec * Gp)) % a.T);
  const size_t bh = gid / ((size_t)kVec * Gp * a.T);
  float acc[HG][8];
#pragma unroll
  for (int h = 0; h < HG; ++h)
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[h][e] = 0.f;
  const size_t row_elems = (size_t)a.G * D;              // elements of one partial row (all heads)
  const size_t in_row = (size_t)g * D + v * 8;           // this thread's first head inside a row
  const size_t head_step = (size_t)Gp * D;               // to its next head
  // eight partial rows per trip: their loads are issued before the first is added
  constexpr int kTrip = 8;
  auto add_rows = [&](const __nv_bfloat16* part, const long long (&rows)[kTrip]) {
    uint4 u[kTrip][HG];
#pragma unroll
    for (int k = 0; k < kTrip; ++k) {
      const __nv_bfloat16* src = part + (size_t)(rows[k] >= 0 ? rows[k] : 0) * row_elems + in_row;
#pragma unroll
      for (int h = 0; h < HG; ++h)
        u[k][h] = rows[k] >= 0 ? __ldg(reinterpret_cast<const uint4*>(src + h * head_step))
                               : make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int k = 0; k < kTrip; ++k)
#pragma unroll
      for (int h = 0; h < HG; ++h) {
        const uint32_t w[4] = {u[k][h].x, u[k][h].y, u[k][h].z, u[k][h].w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {                    // bf16 -> fp32 is a shift
          acc[h][2 * e] += __uint_as_float(w[e] << 16);
          acc[h][2 * e + 1] += __uint_as_float(w[e] & 0xffff0000u);
        }
      }
  };
  const long long qrow = (long long)(bh * a.T + t);
  if (a.acc) {
#pragma unroll
    for (int h = 0; h < HG; ++h) {
      const float4* src = reinterpret_cast<const float4*>(a.acc + (size_t)qrow * row_elems + in_row + h * head_step);
      const float4 lo = __ldg(src), hi = __ldg(src + 1);
      acc[h][0] = lo.x; acc[h][1] = lo.y; acc[h][2] = lo.z; acc[h][3] = lo.w;
      acc[h][4] = hi.x; acc[h][5] = hi.y; acc[h][6] = hi.z; acc[h][7] = hi.w;
    }
  }
  if (a.part_slc) {
    const int32_t* ps = a.pair_of_slot + (size_t)qrow * a.S;
    for (int s0 = 0; s0 < a.S; s0 += kTrip) {
      long long rows[kTrip];
#pragma unroll
      for (int k = 0; k < kTrip; ++k) rows[k] = s0 + k < a.S ? (long long)__ldg(ps + s0 + k) : -1;
      add_rows(a.part_slc, rows);
    }
  }
  if (a.part_win) {
    const int first = max(0, t - a.window + 1) >> 6, last = t >> 6;
    for (int j0 = first; j0 <= last; j0 += kTrip) {
      long long rows[kTrip];
#pragma unroll
      for (int k = 0; k < kTrip; ++k) rows[k] = j0 + k <= last ? qrow * a.slots_win + (j0 + k) % a.slots_win : -1;
      add_rows(a.part_win, rows);
    }
  }
  if (a.part_cmp) {
    const int n_vis = cmp_visible(t, a.cmp_len, a.cmp_stride, a.Lk_cmp);
    const int last = n_vis > 0 ? (n_vis - 1) >> 6 : -1;
    for (int j0 = 0; j0 <= last; j0 += kTrip) {
      long long rows[kTrip];
#pragma unroll
      for (int k = 0; k < kTrip; ++k) rows[k] = j0 + k <= last ? qrow * a.slots_cmp + j0 + k : -1;
      add_rows(a.part_cmp, rows);
    }
  }
  const int b = (int)(bh / a.Hkv), hkv = (int)(bh % a.Hkv);
#pragma unroll
  for (int h = 0; h < HG; ++h) {
    uint4 u;
    u.x = pack_bf16(acc[h][0], acc[h][1]); u.y = pack_bf16(acc[h][2], acc[h][3]);
    u.z = pack_bf16(acc[h][4], acc[h][5]); u.w = pack_bf16(acc[h][6], acc[h][7]);
    *reinterpret_cast<uint4*>(a.dq + (((size_t)b * a.Hq + hkv * a.G + g + h * Gp) * a.T + t) * D + v * 8) = u;
  }
}

// Selection blocks whose row tiles were split over several work items collect dK / dV in the fp32
// accumulators: this kernel clears the accumulator rows of those blocks before the backward
// kernel (finalize = 0) and turns them into the bf16 outputs after it (finalize = 1).
__global__ void sel_split_blocks_kernel(const int32_t* __restrict__ offsets, float* __restrict__ dk_acc,
                                        float* __restrict__ dv_acc, __nv_bfloat16* __restrict__ dk,
                                        __nv_bfloat16* __restrict__ dv, int n_ktiles, int nq, int Lk, int D,
                                        int finalize) {
  const int j = blockIdx.x, bh = blockIdx.y;
  const int n_q = offsets[(size_t)bh * (n_ktiles + 1) + j + 1] - offsets[(size_t)bh * (n_ktiles + 1) + j];
  const int n_rt = (n_q + nq - 1) / nq;
  if (n_rt <= kSelChunkTiles) return;                 // one work item: written directly
  const int rows = min(kKeys, Lk - j * kKeys);
  const size_t base = ((size_t)bh * Lk + (size_t)j * kKeys) * D;
  for (int i = threadIdx.x; i < rows * D; i += blockDim.x) {
    if (finalize) {
      dk[base + i] = __float2bfloat16_rn(dk_acc[base + i]);
      dv[base + i] = __float2bfloat16_rn(dv_acc[base + i]);
    } else {
      dk_acc[base + i] = 0.f;
      dv_acc[base + i] = 0.f;
    }
  }
}

static const char* const kBwdNames[3] = {"tc_bwd_win", "tc_bwd_cmp", "tc_bwd_slc"};
static const char* const kRedNames[3] = {"dq_reduce_win", "dq_reduce_cmp", "dq_reduce_slc"};

struct BwdPlan {
  int n_ktiles, n_slots, nq, n_splits, split_chunk;
  size_t off_acc;
  size_t cap_pairs;          // selection: pairs the CSR may hold
  size_t off_delta, off_part, off_csr_ws, off_qob, off_off, off_pbh, off_pos, off_work, total;
  size_t sel_region_bytes;   // selection: bytes from off_qob to the end of the work list
};

struct SelRegion { size_t qob, pbh, off, pos, work, total; };                     // tc_fwdpair.cu
SelRegion sel_region(size_t units, int n_ktiles, size_t cap_pairs, int nq);
size_t sel_work_max_items(size_t units, int n_ktiles, size_t cap_pairs, int nq);
size_t sel_work_bytes(size_t units, int n_ktiles, size_t cap_pairs, int nq);
int sel_build_worklist(const int32_t* offsets, int n_ktiles, size_t units, size_t cap_pairs, int nq,
                       void* work, cudaStream_t st);

}  // namespace tc
int get_option_merged_boxes();   // api.cu
int get_option_bwd_kernel();
namespace tc {

static BwdPlan plan_bwd(const AttnArgs& a) {
  BwdPlan pl;
  const int G = a.Hq / a.Hkv;
  pl.nq = kRows / G;
  pl.n_ktiles = (a.Lk + kKeys - 1) / kKeys;
  const size_t units = (size_t)a.B * a.Hkv;
  size_t part_rows;
  if (a.kind == 2) {
    pl.n_slots = a.S;
    pl.cap_pairs = units * a.T * a.S;
    part_rows = pl.cap_pairs;
  } else {
    pl.n_slots = a.kind == 0 ? (a.window + kKeys - 2) / kKeys + 1 : pl.n_ktiles;
    pl.cap_pairs = 0;
    part_rows = a.dq_acc ? 0 : units * a.T * pl.n_slots;   // accumulator mode: no partial buffer
  }
  size_t off = 0;
  pl.off_delta = off; off += align_up((size_t)a.B * a.Hq * a.T * sizeof(float), 256);
  pl.off_part = off; off += align_up(part_rows * G * a.D * 2, 256);
  pl.off_csr_ws = pl.off_qob = pl.off_off = pl.off_pbh = pl.off_pos = off;
  if (a.kind == 2) {
    pl.off_csr_ws = off; off += align_up(nsa_csr_workspace_bytes(a.B, a.Hkv, pl.n_ktiles * kKeys, a.S, kKeys), 256);
    const SelRegion r = sel_region(units, pl.n_ktiles, pl.cap_pairs, pl.nq);   // same layout as the forward's
    pl.off_qob = off + r.qob; pl.off_pbh = off + r.pbh; pl.off_off = off + r.off;
    pl.off_pos = off + r.pos; pl.off_work = off + r.work;
    pl.sel_region_bytes = r.total;
    off += r.total;
  }
  // compression: a few key tiles are attended by (almost) every query; split their row tiles
  pl.n_splits = 1;
  pl.split_chunk = 0;
  pl.off_acc = off;
  if (a.kind == 1) {
    const int max_rt = (a.T + pl.nq - 1) / pl.nq;
    pl.split_chunk = 48;
    pl.n_splits = (max_rt + pl.split_chunk - 1) / pl.split_chunk;
    if (pl.n_splits > 1) off += 2 * align_up((size_t)a.B * a.Hkv * a.Lk * a.D * sizeof(float), 256);
    else pl.n_splits = 1;
  }
  // selection: blocks split over several work items use the same accumulators
  if (a.kind == 2) off += 2 * align_up((size_t)a.B * a.Hkv * a.Lk * a.D * sizeof(float), 256);
  pl.total = off;
  return pl;
}

}  // namespace tc

// defined in aux.cu: CSR with an explicit block count and the (query, slot) -> pair map
int build_csr_internal(const int32_t* block_idx, int B, int Hkv, int T, int S, int block_size,
                       int n_blk, int32_t* q_of_block, int32_t* block_offsets, int32_t* pair_bh,
                       int32_t* pair_of_slot, void* workspace, size_t workspace_bytes, cudaStream_t st);

size_t tc_attn_bwd_workspace(const AttnArgs& a) { return tc::plan_bwd(a).total; }

int tc_attn_bwd(const AttnArgs& a, void* ws, size_t ws_bytes, cudaStream_t st) {
  using namespace tc;
  const BwdPlan pl = plan_bwd(a);
  if (!ws || ws_bytes < pl.total) {
    set_error("backward workspace too small: need %zu bytes", pl.total);
    return NSA_ERR_WORKSPACE;
  }
  char* base = (char*)ws;
  const int G = a.Hq / a.Hkv;
  BwdArgs p;
  p.q = (const __nv_bfloat16*)a.q;
  p.d_o = (const __nv_bfloat16*)a.d_o;
  p.lse = a.lse;
  p.delta = a.row_dot ? a.row_dot : (float*)(base + pl.off_delta);
  p.row_scale = a.row_scale;
  p.q_of_block = (const int32_t*)(base + pl.off_qob);
  p.offsets = (const int32_t*)(base + pl.off_off);
  p.dk = (__nv_bfloat16*)a.dk_acc;     // the API passes the dk / dv outputs through these fields
  p.dv = (__nv_bfloat16*)a.dv_acc;
  p.dq_part = (__nv_bfloat16*)(base + pl.off_part);
  p.work = nullptr;
  p.status = device_status_ptr();
  if (!p.status) { set_error("device status word unavailable"); return NSA_ERR_CUDA; }
  p.B = a.B; p.Hq = a.Hq; p.Hkv = a.Hkv; p.T = a.T; p.Lk = a.Lk; p.G = G; p.nq = pl.nq;
  p.kind = a.kind; p.window = a.window; p.block_size = a.block_size;
  p.n_ktiles = pl.n_ktiles; p.n_slots = pl.n_slots;
  p.dq_acc_mode = (a.dq_acc && a.kind != 2) ? 1 : 0;
  p.merged = (a.kind == 2 && a.D == 128 && G % 8 == 0 && get_option_merged_boxes()) ? 1 : 0;
  p.scale = a.scale; p.scale_log2 = a.scale * kLog2e;
  p.split_chunk = pl.split_chunk;
  const size_t n_kv = (size_t)a.B * a.Hkv * a.Lk * a.D;
  p.dk_acc = (float*)(base + pl.off_acc);
  p.dv_acc = (float*)(base + pl.off_acc + align_up(n_kv * sizeof(float), 256));
  if (pl.n_splits > 1)
    NSA_CUDA_OK(cudaMemsetAsync(base + pl.off_acc, 0, 2 * align_up(n_kv * sizeof(float), 256), st));

  const size_t rows = (size_t)a.B * a.Hq * a.T;
  if (!a.row_dot) {
    KernelScope ks("delta_kernel", st);
    delta_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, st>>>((const __nv_bfloat16*)a.d_o,
                                                             (const __nv_bfloat16*)a.o,
                                                             (float*)(base + pl.off_delta), rows, a.D);
  }
  NSA_LAUNCH_OK("delta_kernel");
  int32_t* pair_of_slot = (int32_t*)(base + pl.off_pos);
  if (a.kind == 2) {
    if (a.sel_plan) {      // built earlier for this block list: one copy instead of the build
      NSA_CUDA_OK(cudaMemcpyAsync(base + pl.off_qob, a.sel_plan, pl.sel_region_bytes, cudaMemcpyDeviceToDevice, st));
    } else {
      int rc = build_csr_internal(a.block_idx, a.B, a.Hkv, a.T, a.S, kKeys, pl.n_ktiles,
                                  (int32_t*)(base + pl.off_qob), (int32_t*)(base + pl.off_off),
                                  (int32_t*)(base + pl.off_pbh), pair_of_slot, base + pl.off_csr_ws,
                                  pl.off_qob - pl.off_csr_ws, st);
      if (rc != NSA_OK) return rc;
      rc = sel_build_worklist(p.offsets, pl.n_ktiles, (size_t)a.B * a.Hkv, pl.cap_pairs, pl.nq, base + pl.off_work, st);
      if (rc != NSA_OK) return rc;
    }
    p.work = (const SelWorkHeader*)(base + pl.off_work);
    KernelScope ks("sel_split_blocks_kernel", st);
    sel_split_blocks_kernel<<<dim3(pl.n_ktiles, a.B * a.Hkv), 256, 0, st>>>(p.offsets, p.dk_acc, p.dv_acc, p.dk, p.dv,
                                                                        pl.n_ktiles, pl.nq, a.Lk, a.D, 0);
  }
  CUtensorMap tm_k, tm_v, tm_q, tm_do;
  int rc = make_map(&tm_k, a.k, a.D, a.Lk, a.B * a.Hkv, kKeys, 1);
  if (rc == NSA_OK) rc = make_map(&tm_v, a.v, a.D, a.Lk, a.B * a.Hkv, kKeys, 1);
  if (rc == NSA_OK) rc = p.merged ? make_map_query_both_slabs(&tm_q, a.q, a.T, a.B * a.Hq, G)
                                  : make_map_query_rows(&tm_q, a.q, a.D, a.T, a.B * a.Hq, G);
  if (rc == NSA_OK) rc = p.merged ? make_map_query_both_slabs(&tm_do, a.d_o, a.T, a.B * a.Hq, G)
                                  : make_map_query_rows(&tm_do, a.d_o, a.D, a.T, a.B * a.Hq, G);
  CUtensorMap tm_q_run, tm_do_run;
  if (rc == NSA_OK) rc = make_map_query_rows(&tm_q_run, a.q, a.D, a.T, a.B * a.Hq, G, pl.nq);
  if (rc == NSA_OK) rc = make_map_query_rows(&tm_do_run, a.d_o, a.D, a.T, a.B * a.Hq, G, pl.nq);
  CUtensorMap tm_dq, tm_dqacc;
  if (rc == NSA_OK && p.dq_acc_mode) {
    rc = make_map_dq_acc(&tm_dqacc, a.dq_acc, a.D, G, (size_t)a.T, (size_t)a.B * a.Hkv, pl.nq);
    tm_dq = tm_dqacc;        // the partial-tile map is not used in this mode
  } else if (rc == NSA_OK) {
    rc = a.kind == 2 ? make_map_partial(&tm_dq, p.dq_part, a.D, G, 1, pl.cap_pairs ? pl.cap_pairs : 1, 1, pl.nq)
                     : make_map_partial(&tm_dq, p.dq_part, a.D, G, pl.n_slots, a.T, (size_t)a.B * a.Hkv, pl.nq);
    tm_dqacc = tm_dq;        // likewise
  }
  if (rc != NSA_OK) return rc;
  const size_t smem = bwd_smem_bytes(a.D);
  dim3 grid(pl.n_ktiles, a.B * a.Hkv, pl.n_splits);
  if (a.kind == 2)
    grid = dim3((unsigned)sel_work_max_items((size_t)a.B * a.Hkv, pl.n_ktiles, pl.cap_pairs, pl.nq));
  if (get_option_bwd_kernel() == 1 && !p.dq_acc_mode) {       // compute groups relieved of the issuing
    KernelScope ks(branch_name(kBwdNames, a.kind), st);
    if (a.D == 128) {
      NSA_CUDA_OK(cudaFuncSetAttribute(tc_bwd2_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      tc_bwd2_kernel<128><<<grid, kB2Threads, smem, st>>>(tm_k, tm_v, tm_q, tm_do, tm_q_run, tm_do_run, tm_dq, p);
    } else {
      NSA_CUDA_OK(cudaFuncSetAttribute(tc_bwd2_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      tc_bwd2_kernel<64><<<grid, kB2Threads, smem, st>>>(tm_k, tm_v, tm_q, tm_do, tm_q_run, tm_do_run, tm_dq, p);
    }
  } else if (a.D == 128) {
    NSA_CUDA_OK(cudaFuncSetAttribute(tc_bwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    KernelScope ks(branch_name(kBwdNames, a.kind), st);
    tc_bwd_kernel<128><<<grid, 512, smem, st>>>(tm_k, tm_v, tm_q, tm_do, tm_q_run, tm_do_run, tm_dq, tm_dqacc, p);
  } else {
    NSA_CUDA_OK(cudaFuncSetAttribute(tc_bwd_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    KernelScope ks(branch_name(kBwdNames, a.kind), st);
    tc_bwd_kernel<64><<<grid, 512, smem, st>>>(tm_k, tm_v, tm_q, tm_do, tm_q_run, tm_do_run, tm_dq, tm_dqacc, p);
  }
  NSA_LAUNCH_OK("tc_bwd_kernel");
  if (a.kind == 2) {
    KernelScope ks("sel_split_blocks_kernel", st);
    sel_split_blocks_kernel<<<dim3(pl.n_ktiles, a.B * a.Hkv), 256, 0, st>>>(p.offsets, p.dk_acc, p.dv_acc, p.dk, p.dv,
                                                                        pl.n_ktiles, pl.nq, a.Lk, a.D, 1);
    NSA_LAUNCH_OK("sel_split_blocks_kernel");
  }
  if (pl.n_splits > 1) {
    int rc2 = cast_f32_to(p.dk_acc, p.dk, n_kv, NSA_DTYPE_BF16, st);
    if (rc2 == NSA_OK) rc2 = cast_f32_to(p.dv_acc, p.dv, n_kv, NSA_DTYPE_BF16, st);
    if (rc2 != NSA_OK) return rc2;
  }
  if (!a.dq) return NSA_OK;   // the partials stay in the workspace (or the accumulator) for tc_dq_reduce3
  const size_t nthreads = (size_t)a.B * a.Hkv * a.T * G * (a.D / 8);
  const unsigned rgrid = (unsigned)((nthreads + 255) / 256);
  {
    KernelScope ks(branch_name(kRedNames, a.kind), st);
    if (a.D == 128)
      dq_reduce_kernel<128><<<rgrid, 256, 0, st>>>(p.dq_part, pair_of_slot, (__nv_bfloat16*)a.dq, a.B, a.Hq,
                                                  a.Hkv, a.T, G, a.kind, a.window, a.block_size, a.Lk,
                                                  pl.n_slots, a.S);
    else
      dq_reduce_kernel<64><<<rgrid, 256, 0, st>>>(p.dq_part, pair_of_slot, (__nv_bfloat16*)a.dq, a.B, a.Hq,
                                                 a.Hkv, a.T, G, a.kind, a.window, a.block_size, a.Lk,
                                                 pl.n_slots, a.S);
  }
  NSA_LAUNCH_OK("dq_reduce_kernel");
  return NSA_OK;
}


// dq of the whole op from the three branch workspaces (each written by tc_attn_bwd with a null
// dq) and / or the fp32 accumulator: `base` carries B, Hq, Hkv, T, D; a null workspace means the
// branch is absent (or sits in the accumulator).
int tc_dq_reduce3(const AttnArgs& base, int Lk_cmp, int cmp_len, int cmp_stride, int S, int block_size,
                  int window, const void* ws_cmp, const void* ws_slc, const void* ws_win,
                  const float* dq_acc, void* dq, cudaStream_t st) {
  using namespace tc;
  Reduce3Args r;
  r.acc = dq_acc;
  r.part_cmp = r.part_slc = r.part_win = nullptr;
  r.pair_of_slot = nullptr;
  r.slots_cmp = r.slots_win = 1;
  r.Lk_cmp = Lk_cmp; r.cmp_len = cmp_len; r.cmp_stride = cmp_stride; r.S = S; r.window = window;
  r.dq = (__nv_bfloat16*)dq;
  r.B = base.B; r.Hq = base.Hq; r.Hkv = base.Hkv; r.T = base.T; r.G = base.Hq / base.Hkv;
  if (ws_cmp) {
    AttnArgs a = base; a.kind = 1; a.Lk = Lk_cmp; a.block_size = cmp_len; a.window = cmp_stride;
    const BwdPlan pl = plan_bwd(a);
    r.part_cmp = (const __nv_bfloat16*)((const char*)ws_cmp + pl.off_part);
    r.slots_cmp = pl.n_slots;
  }
  if (ws_slc) {
    AttnArgs a = base; a.kind = 2; a.Lk = base.T; a.S = S; a.block_size = block_size;
    const BwdPlan pl = plan_bwd(a);
    r.part_slc = (const __nv_bfloat16*)((const char*)ws_slc + pl.off_part);
    r.pair_of_slot = (const int32_t*)((const char*)ws_slc + pl.off_pos);
  }
  if (ws_win) {
    AttnArgs a = base; a.kind = 0; a.Lk = base.T; a.window = window;
    const BwdPlan pl = plan_bwd(a);
    r.part_win = (const __nv_bfloat16*)((const char*)ws_win + pl.off_part);
    r.slots_win = pl.n_slots;
  }
  const int hg = r.G % 2 == 0 ? 2 : 1;                    // heads of a query served by one thread
  const size_t nthreads = (size_t)r.B * r.Hkv * r.T * (r.G / hg) * (base.D / 8);
  if (nthreads == 0) return NSA_OK;
  const unsigned grid = (unsigned)((nthreads + 255) / 256);
  KernelScope ks("dq_reduce3", st);
  if (base.D == 128) {
    if (hg == 2) dq_reduce3_kernel<128, 2><<<grid, 256, 0, st>>>(r);
    else dq_reduce3_kernel<128, 1><<<grid, 256, 0, st>>>(r);
  } else {
    if (hg == 2) dq_reduce3_kernel<64, 2><<<grid, 256, 0, st>>>(r);
    else dq_reduce3_kernel<64, 1><<<grid, 256, 0, st>>>(r);
  }
  NSA_LAUNCH_OK("dq_reduce3_kernel");
  return NSA_OK;
}

}  // namespace nsa
