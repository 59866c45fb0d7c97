// Selected-block attention forward, key-block outer, warp-specialised.
//
// One CTA per (64-token block, chunk of its row tiles), launched by tc_sel_fwd (tc_fwdpair.cu); per row
// tile S = Q K^T, p = exp2(s - m_block), O_part = P V; O_part, m and the sum of p leave per
// (pair, head) and sel_combine_kernel merges them.  The row tiles of a CTA flow through a
// pipeline of roles:
//   3 producer warps  gather the Q rows of tile k into a 3-stage ring, three tiles ahead of the
//                     arithmetic: one TMA box per query (both 64-column slabs, where the shape
//                     allows) or per query and slab.  A warp gets a box out every 60-100 cycles,
//                     whatever its size, and at 32 boxes a tile that bounded the kernel; several
//                     warps issue side by side
//   MMA warp          one thread issues S(k) as soon as stage k has landed, then P V of tile k-1
//   2 softmax groups  128 threads each (thread = row = TMEM lane), tiles alternate between them:
//                     S from TMEM, row maximum, exponentials, P back to TMEM as packed bf16 (it is
//                     the TMEM A operand of P V, so it never touches shared memory)
//   epilogue group    128 threads: O_part from TMEM to a bf16 staging tile, one TMA store per slab
// Each hand-over is an mbarrier with a bounded wait.  TMEM: two slots of S/P (64 columns) + O (D).
#include "tc_common.cuh"
#include "tc_host.cuh"

namespace nsa {
namespace tc {

struct PairArgs {
  const int32_t* q_of_block;
  const int32_t* offsets;        // [B*Hkv, n_ktiles + 1]
  __nv_bfloat16* o_part;         // [pairs, G, D]
  float* ml;                     // [pairs, G, 2]: the row maximum m and the sum of p
  const unsigned long long* stats;
  const SelWorkHeader* work;     // n_items, then int4 items {bh, block, first row tile, chunks of the block}
  int* status;
  int force;                     // 0: device-side choice, 1: query-outer kernel, 2: this kernel
  int B, Hq, Hkv, T, G, nq, n_ktiles, nq_union;
  int merged;                    // 1: one TMA box per query brings both 64-column slabs (D = 128, G % 8 == 0)
  float scale_log2;
};

constexpr int kPairThreads = 512;            // 2 x 4 softmax warps, 4 epilogue warps, 3 producer warps, MMA warp
constexpr int kPairProducers = 3;
constexpr int kPairQStages = 3;

__host__ __device__ inline size_t pair_smem_bytes(int D) {
  const size_t q = (size_t)kRows * 128 * (D / 64);
  return (size_t)2 * kKeys * 128 * (D / 64) + kPairQStages * q + 2 * q /*staging*/ + 512 /*barriers*/ +
         128 * 4 /*partial-row index*/ + 1024 /*alignment slack*/;
}

__device__ __forceinline__ void named_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
// barrier over `threads` threads that also ORs a predicate over them: every participant gets the
// same answer, so a group never splits over a decision (a split group would hang in bar.sync)
__device__ __forceinline__ bool named_or(int id, int threads, int pred) {
  uint32_t out;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %3, 0;\n\t"
      "bar.red.or.pred p, %1, %2, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(out)
      : "r"(id), "r"(threads), "r"(pred)
      : "memory");
  return out != 0;
}
__device__ __forceinline__ void bulk_wait_read_1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }

template <int D>
__global__ void __launch_bounds__(kPairThreads, 1)
tc_fwdpair_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                   const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_o,
                   const PairArgs p) {
  constexpr int kSlabs = D / 64;
  constexpr int kKVBytes = kKeys * 128 * kSlabs;
  constexpr int kQBytes = kRows * 128 * kSlabs;
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kSlotCols = 64 + D;           // S / P then O
  constexpr uint32_t kIdescS = idesc_bf16(128, kKeys, 0, 0);
  constexpr uint32_t kIdescPV = idesc_bf16(128, D, 0, 1);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* sK = smem;
  uint8_t* sV = sK + kKVBytes;
  uint8_t* sQ = sV + kKVBytes;                      // [kPairQStages][kQBytes]
  uint8_t* sStage = sQ + kPairQStages * kQBytes;      // [2][kQBytes]
  uint64_t* bars = (uint64_t*)(sStage + 2 * kQBytes);
  uint64_t* bar_kv = bars + 0;
  uint64_t* q_full = bars + 1;      // [3]
  uint64_t* q_empty = bars + 4;     // [3]
  uint64_t* s_full = bars + 7;      // [2]
  uint64_t* p_full = bars + 9;      // [2]
  uint64_t* o_full = bars + 11;     // [2]
  uint64_t* o_empty = bars + 13;    // [2]
  uint64_t* bar_drain = bars + 15;
  uint32_t* s_tmem = (uint32_t*)(bars + 16);
  volatile int* s_abort = (volatile int*)(s_tmem + 1);
  volatile int* s_issued = (volatile int*)(s_tmem + 2);   // row tiles whose gather has been issued
  uint32_t* s_prow = (uint32_t*)(s_tmem + 4);             // [128] partial row of each tile row (ragged tile)

  if (!prefer_pairs(p.stats, p.offsets, p.B * p.Hkv, p.n_ktiles, p.nq_union, p.force)) return;
  if ((int)blockIdx.x >= p.work->n_items) return;
  const int4 item = reinterpret_cast<const int4*>(p.work + 1)[blockIdx.x];
  const int bh = item.x, j = item.y;
  const int b = bh / p.Hkv, hkv = bh % p.Hkv;
  const int key0 = j * kKeys;
  const int pair_base = __ldg(p.offsets + (size_t)bh * (p.n_ktiles + 1) + j);
  const int n_q = __ldg(p.offsets + (size_t)bh * (p.n_ktiles + 1) + j + 1) - pair_base;
  const int rt_end = min((n_q + p.nq - 1) / p.nq, item.z + kSelChunkTiles);
  const int n_tiles = rt_end - item.z;              // row tiles of this work item
  if (n_tiles <= 0) return;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    int bad = (*(volatile int*)p.status != 0) ? 1 : 0;
    if ((size_t)((uint8_t*)(s_prow + 128) - smem_raw) > pair_smem_bytes(D)) {
      atomicOr(p.status, 256);   // the shared-memory window is less aligned than assumed
      bad = 1;
    }
    *s_abort = bad;
    *s_issued = 0;
    mbar_init(bar_kv, 1);
    for (int s = 0; s < kPairQStages; ++s) { mbar_init(q_full + s, 1); mbar_init(q_empty + s, 1); }
    for (int s = 0; s < 2; ++s) {
      mbar_init(s_full + s, 1); mbar_init(p_full + s, 128);
      mbar_init(o_full + s, 1); mbar_init(o_empty + s, 128);
    }
    mbar_init(bar_drain, 1);
    fence_barrier_init();
    prefetch_tensormap(&tm_k); prefetch_tensormap(&tm_v);
    prefetch_tensormap(&tm_q); prefetch_tensormap(&tm_o);
  }
  __syncthreads();
  if (*s_abort) return;
  // rows past nq * G of a tile are never loaded: keep them zero in every stage
  for (int i = tid; i < kPairQStages * kQBytes / 16; i += kPairThreads)
    *reinterpret_cast<uint4*>(sQ + (size_t)i * 16) = make_uint4(0, 0, 0, 0);
  fence_proxy_async();
  if (warp == 0) {
    tmem_alloc(s_tmem, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *s_tmem;

  if (warp >= 12 && warp < 12 + kPairProducers) {
    // ---- producers: K / V once, then the Q rows of every tile; box o of a tile goes to warp o % 3 ----
    const int pw = warp - 12;
    if (pw == 0 && lane == 0) {
      mbar_expect_tx(bar_kv, 2 * kKVBytes);
#pragma unroll
      for (int s = 0; s < kSlabs; ++s) {
        tma_load_3d(sK + s * (kKeys * 128), &tm_k, bar_kv, s * 64, key0, bh);
        tma_load_3d(sV + s * (kKeys * 128), &tm_v, bar_kv, s * 64, key0, bh);
      }
    }
    const uint32_t gather_bytes = (uint32_t)(p.nq * p.G * 128 * kSlabs);
    // A TMA box costs its issuing warp a fixed time of the order of a hundred cycles whatever its size:
    // where the shape allows (`merged`), one box per query brings both column slabs, else one box per
    // query and slab.
    const int per_q = p.merged ? 1 : kSlabs;
    const int n_ops = p.nq * per_q;                  // at most 128: up to two per lane of the three warps
    const int o0 = lane * kPairProducers + pw, o1 = o0 + 32 * kPairProducers;   // this lane's boxes
    // query position of one of this lane's boxes in tile k (a missing query reads past T: zeros)
    auto tq_of = [&](int k, int o) -> int {
      const int qi = (item.z + k) * p.nq + o / per_q;
      return (o < n_ops && qi < n_q) ? ldg_s32_now(p.q_of_block + pair_base + qi) : p.T;
    };
    int tq0 = tq_of(0, o0), tq1 = tq_of(0, o1);
    for (int k = 0; k < n_tiles; ++k) {
      const int st = k % kPairQStages;
      mbar_wait(q_empty + st, ((k / kPairQStages) + 1) & 1, p.status, s_abort, 512);
      const int tn0 = k + 1 < n_tiles ? tq_of(k + 1, o0) : p.T;          // next tile's positions, ahead
      const int tn1 = k + 1 < n_tiles ? tq_of(k + 1, o1) : p.T;
      if (__any_sync(0xffffffffu, *s_abort)) break;          // the whole warp leaves together
      if (pw == 0 && lane == 0) { mbar_expect_tx(q_full + st, gather_bytes); *s_issued = k + 1; }
      __syncwarp();
      uint8_t* dst = sQ + st * kQBytes;
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int o = r ? o1 : o0, tq = r ? tq1 : tq0;
        if (o < n_ops) {
          if (p.merged) {
            tma_load_5d_hint(dst + o * (p.G / 8) * 2048, &tm_q, q_full + st, 0, 0, 0, tq, (b * p.Hq + hkv * p.G) >> 3,
                             l2_policy_evict_normal());
          } else {
            const int qq = o / kSlabs, sl = o % kSlabs;
            tma_load_3d(dst + sl * (kRows * 128) + qq * p.G * 128, &tm_q, q_full + st, sl * 64,
                        b * p.Hq + hkv * p.G, tq);
          }
        }
      }
      tq0 = tn0; tq1 = tn1;
    }
  } else if (warp == 12 + kPairProducers) {
    // ---- MMA issuer ------------------------------------------------------------------------
    if (lane == 0) {
      mbar_wait(bar_kv, 0, p.status, s_abort, 32);
      const uint32_t ka = desc_lo_kmajor(smem_u32(sK));
      const uint32_t va = desc_lo_mnmajor(smem_u32(sV), kKeys * 128);
      for (int k = 0; k <= n_tiles; ++k) {
        if (*s_abort) break;
        if (k < n_tiles) {
          const int st = k % kPairQStages, sb = k & 1;
          mbar_wait(q_full + st, (k / kPairQStages) & 1, p.status, s_abort, 512);
          // the S / P columns of the slot are free once P V of tile k-2 has completed
          if (k >= 2) mbar_wait(o_full + sb, ((k >> 1) - 1) & 1, p.status, s_abort, 128);
          if (*s_abort) break;
          tc_fence_after();
          const uint32_t qa = desc_lo_kmajor(smem_u32(sQ + st * kQBytes));
          const uint32_t colS = tmem + sb * kSlotCols;
          // Q tile: slab-major (8-row groups 1024 bytes apart, slabs kRows * 128 apart) or, with merged
          // boxes, the two slabs of an 8-row group side by side (groups 2048 bytes apart)
          const uint32_t q_slab = p.merged ? 1024u : (uint32_t)(kRows * 128), q_sbo = p.merged ? 2048u : 1024u;
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint32_t slab = kk >> 2, in = (kk & 3) * 32;
            mma_ss(colS, desc_at_sbo(qa, slab * q_slab + in, q_sbo), desc_at(ka, slab * (kKeys * 128) + in),
                   kIdescS, kk > 0);
          }
          tc_commit(q_empty + st);     // the stage may be refilled once S has read it
          tc_commit(s_full + sb);
        }
        if (k >= 1) {
          const int jt = k - 1, sb = jt & 1;
          mbar_wait(p_full + sb, (jt >> 1) & 1, p.status, s_abort, 64);
          // the O columns of the slot are free once the epilogue has read O of tile jt-2
          if (jt >= 2) mbar_wait(o_empty + sb, ((jt >> 1) - 1) & 1, p.status, s_abort, 1024);
          if (*s_abort) break;
          tc_fence_after();
          const uint32_t colP = tmem + sb * kSlotCols, colO = colP + 64;
#pragma unroll
          for (int kk = 0; kk < kKeys / 16; ++kk)
            mma_ts(colO, colP + kk * 8, desc_at(va, kk * 2048), kIdescPV, kk > 0);
          tc_commit(o_full + sb);
        }
      }
      // the tensor pipe is idle before TMEM is given back, whatever happened above
      tc_commit(bar_drain);
      if (!mbar_wait(bar_drain, 0, p.status, s_abort, 2048)) mbar_wait_drain(bar_drain, 0);
    }
  } else if (warp < 8) {
    // ---- softmax group `sb` ------------------------------------------------------------------
    const int sb = warp >> 2, quad = warp & 3;
    const int row = quad * 32 + lane;
    const int ql = row / p.G, g = row % p.G;
    const bool row_slot_ok = ql < p.nq;
    const uint32_t lane_base = tmem + ((uint32_t)(quad * 32) << 16) + sb * kSlotCols;
    auto row_query = [&](int k) -> int {
      const int qi = (item.z + k) * p.nq + ql;
      if (!row_slot_ok || qi >= n_q) return -1;
      return ldg_s32_now(p.q_of_block + pair_base + qi);
    };
    int t_cur = sb < n_tiles ? row_query(sb) : -1;
    for (int k = sb; k < n_tiles; k += 2) {
      if (*s_abort) break;
      const int t_nxt = k + 2 < n_tiles ? row_query(k + 2) : -1;
      const int hi = t_cur >= 0 ? min(kKeys - 1, min(t_cur, p.T - 1) - key0) : -1;
      mbar_wait(s_full + sb, (k >> 1) & 1, p.status, s_abort, 64);
      if (*s_abort) break;
      tc_fence_after();
      uint32_t r[64];
      tmem_ld32(lane_base, r);
      tmem_ld32(lane_base + 32, r + 32);
      tmem_wait_ld();
      float mx = -INFINITY;
      if (hi >= kKeys - 1) {
#pragma unroll
        for (int c = 0; c < 64; ++c) {
          const float x = __uint_as_float(r[c]) * p.scale_log2;
          r[c] = __float_as_uint(x);
          mx = fmaxf(mx, x);
        }
      } else {
#pragma unroll
        for (int c = 0; c < 64; ++c) {
          const float x = c <= hi ? __uint_as_float(r[c]) * p.scale_log2 : -INFINITY;
          r[c] = __float_as_uint(x);
          mx = fmaxf(mx, x);
        }
      }
      const float msub = (mx == -INFINITY) ? 0.f : mx;
      float lsum = 0.f;
      uint32_t pk[32];
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        const float p0 = ex2(__uint_as_float(r[2 * c]) - msub), p1 = ex2(__uint_as_float(r[2 * c + 1]) - msub);
        lsum += p0 + p1;
        pk[c] = pack_bf16(p0, p1);
      }
      tmem_st32(lane_base, pk);            // P over the first half of S: this lane's S is in registers
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(p_full + sb);
      if (t_cur >= 0) {
        const size_t prow = (size_t)(pair_base + (item.z + k) * p.nq + ql) * p.G + g;
        *reinterpret_cast<float2*>(p.ml + prow * 2) = make_float2(mx, lsum);
      }
      t_cur = t_nxt;
    }
  } else if (warp < 12) {
    // ---- epilogue group: O_part of every tile, in order ---------------------------------------
    const int quad = warp & 3, et = tid - 8 * 32;
    const int row = quad * 32 + lane;
    const int ql = row / p.G, g = row % p.G;
    for (int k = 0; k < n_tiles; ++k) {
      const int sb = k & 1;
      const int i = item.z + k;
      mbar_wait(o_full + sb, (k >> 1) & 1, p.status, s_abort, 128);
      tc_fence_after();
      // the staging tile of this slot is free once the store of tile k-2 has read it
      if (et == 0 && k >= 2) bulk_wait_read_1();
      if (named_or(1, 128, *s_abort)) break;                   // the whole group leaves together
      uint8_t* stage = sStage + sb * kQBytes;
      const uint32_t lane_base = tmem + ((uint32_t)(quad * 32) << 16) + sb * kSlotCols + 64;
#pragma unroll
      for (int cc = 0; cc < D / 32; ++cc) {
        uint32_t r32[32];
        tmem_ld32(lane_base + cc * 32, r32);
        tmem_wait_ld();
        if (cc == D / 32 - 1) {            // O of this slot is in registers: the MMA warp may overwrite it
          tc_fence_before();
          mbar_arrive(o_empty + sb);
        }
#pragma unroll
        for (int v4 = 0; v4 < 4; ++v4) {
          const uint32_t chunk = (uint32_t)(cc * 4 + v4);
          const uint32_t dst = smem_u32(stage) + (chunk >> 3) * (kRows * 128) + row * 128 +
                               (((chunk & 7) ^ (row & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst),
                       "r"(pack_bf16(__uint_as_float(r32[v4 * 8 + 0]), __uint_as_float(r32[v4 * 8 + 1]))),
                       "r"(pack_bf16(__uint_as_float(r32[v4 * 8 + 2]), __uint_as_float(r32[v4 * 8 + 3]))),
                       "r"(pack_bf16(__uint_as_float(r32[v4 * 8 + 4]), __uint_as_float(r32[v4 * 8 + 5]))),
                       "r"(pack_bf16(__uint_as_float(r32[v4 * 8 + 6]), __uint_as_float(r32[v4 * 8 + 7])))
                       : "memory");
        }
      }
      const bool full_tile = (i + 1) * p.nq <= n_q;
      if (!full_tile) {
        const int qi = i * p.nq + ql;
        s_prow[row] = (ql < p.nq && qi < n_q) ? (uint32_t)((size_t)(pair_base + qi) * p.G + g) : 0xffffffffu;
      }
      fence_proxy_async();
      named_sync(1, 128);
      if (full_tile) {
        // its pairs are consecutive rows of the partial buffer: one TMA store per slab
        if (et == 0) {
#pragma unroll
          for (int sl = 0; sl < kSlabs; ++sl)
            tma_store_5d_hint(&tm_o, stage + sl * (kRows * 128), sl * 64, 0, 0, pair_base + i * p.nq, 0,
                              l2_policy_evict_first());
          bulk_commit();
        }
      } else {   // the ragged last tile: whole rows out by hand
        constexpr int kChunks = D / 8;
        constexpr int kRowsPerPass = 128 / kChunks;
        const int c = et % kChunks;
        for (int r = et / kChunks; r < kRows; r += kRowsPerPass) {
          const uint32_t pr = s_prow[r];
          if (pr != 0xffffffffu) {
            const uint4 v = *reinterpret_cast<const uint4*>(stage + (c >> 3) * (kRows * 128) + r * 128 +
                                                            (((c & 7) ^ (r & 7)) << 4));
            *reinterpret_cast<uint4*>(p.o_part + (size_t)pr * D + c * 8) = v;
          }
        }
      }
    }
    if (et == 0) bulk_wait_all();
  }

  // ---- teardown: every gather that was issued has landed, the tensor pipe is idle -----------------
  __syncthreads();
  if (*s_abort && tid == 0) {
    const int issued = *s_issued;
    for (int k = max(0, issued - kPairQStages); k < issued; ++k) {
      // bounded: a gather that never lands was what made the CTA give up in the first place
      mbar_wait_drain(q_full + k % kPairQStages, (k / kPairQStages) & 1);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, kTmemCols);
}

}  // namespace tc

int get_option_merged_boxes();   // api.cu

// launched by tc_sel_fwd (tc_fwdpair.cu)
int tc_fwdpair_launch(const AttnArgs& a, const int32_t* q_of_block, const int32_t* offsets, void* o_part,
                       float* ml, const unsigned long long* stats, const void* work, int force, int nq,
                       int n_ktiles, int nq_union, size_t cap_pairs, unsigned grid, cudaStream_t st) {
  using namespace tc;
  const int G = a.Hq / a.Hkv;
  PairArgs p;
  p.q_of_block = q_of_block; p.offsets = offsets;
  p.o_part = (__nv_bfloat16*)o_part; p.ml = ml; p.stats = stats;
  p.work = (const SelWorkHeader*)work;
  p.status = device_status_ptr();
  if (!p.status) { set_error("device status word unavailable"); return NSA_ERR_CUDA; }
  p.force = force;
  p.B = a.B; p.Hq = a.Hq; p.Hkv = a.Hkv; p.T = a.T; p.G = G; p.nq = nq;
  p.n_ktiles = n_ktiles; p.nq_union = nq_union;
  p.scale_log2 = a.scale * kLog2e;
  p.merged = (a.D == 128 && G % 8 == 0 && get_option_merged_boxes()) ? 1 : 0;
  CUtensorMap tm_k, tm_v, tm_q, tm_o;
  int rc = make_map(&tm_k, a.k, a.D, a.T, a.B * a.Hkv, kKeys, 1);
  if (rc == NSA_OK) rc = make_map(&tm_v, a.v, a.D, a.T, a.B * a.Hkv, kKeys, 1);
  if (rc == NSA_OK) rc = p.merged ? make_map_query_both_slabs(&tm_q, a.q, a.T, a.B * a.Hq, G)
                                  : make_map_query_rows(&tm_q, a.q, a.D, a.T, a.B * a.Hq, G);
  if (rc == NSA_OK) rc = make_map_partial(&tm_o, o_part, a.D, G, 1, cap_pairs ? cap_pairs : 1, 1, nq);
  if (rc != NSA_OK) return rc;
  const size_t smem = pair_smem_bytes(a.D);
  KernelScope ks("tc_fwd_slc_pairs", st);
  if (a.D == 128) {
    NSA_CUDA_OK(cudaFuncSetAttribute(tc_fwdpair_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    tc_fwdpair_kernel<128><<<grid, kPairThreads, smem, st>>>(tm_k, tm_v, tm_q, tm_o, p);
  } else {
    NSA_CUDA_OK(cudaFuncSetAttribute(tc_fwdpair_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    tc_fwdpair_kernel<64><<<grid, kPairThreads, smem, st>>>(tm_k, tm_v, tm_q, tm_o, p);
  }
  NSA_LAUNCH_OK("tc_fwdpair_kernel");
  return NSA_OK;
}

}  // namespace nsa
