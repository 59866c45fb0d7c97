// Selected-block attention forward, key-block outer ("split-K over blocks").
//
// When neighbouring queries list unrelated blocks, a query-outer tile wastes most of every MMA
// on rows that do not attend the block.  This kernel instead gives one CTA one 64-token block:
// K and V of the block are loaded once, the (query, head) rows that list the block are
// gathered from the block -> query CSR, 128 rows at a time, and for each row tile
//   S = Q K^T ,  p = exp2(s*scale*log2e - m) with m the row's maximum over this block,
//   O_part = P V   (P: bf16 tile in shared memory, K-major A operand; V: MN-major B operand)
// are computed; O_part (bf16), m and the sum of p (fp32) are written per (pair, head).  A second
// kernel merges the partials of each query: o = sum_j 2^(m_j-M) O_j / sum_j 2^(m_j-M) l_j.
// A small statistics kernel counts the distinct blocks per query tile; the launchers of both
// forward variants read it on the device and only the cheaper variant does the work.
#include "tc_common.cuh"
#include "tc_host.cuh"

namespace nsa {
namespace tc {

struct PairArgs {
  const __nv_bfloat16* q;
  const int32_t* q_of_block;
  const int32_t* offsets;        // [B*Hkv, n_ktiles + 1]
  __nv_bfloat16* o_part;         // [pairs, G, D]
  float* ml;                     // [pairs, G, 3]: m, sum of p over columns 0..31, over 32..63
  const unsigned long long* stats;
  const SelWorkHeader* work;     // n_items, then int4 items {bh, block, first row tile, chunks of the block}
  int* status;
  int force;                     // 0: device-side choice, 1: query-outer kernel, 2: this kernel
  int B, Hq, Hkv, T, G, nq, n_ktiles, nq_union;
  float scale_log2;
};

__device__ __forceinline__ void cp_async16p(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes)
               : "memory");
}

constexpr int kPairGroupThreads = 256;

constexpr int kPairMaxNq = 64;

__host__ __device__ inline size_t pair_smem_bytes(int D) {
  return (size_t)2 * kKeys * 128 * (D / 64) +
         2 * ((size_t)kRows * 128 * (D / 64) + kRows * 128 + kRows * 256) +   // Q, P, staging
         256 + 2 * 2 * kPairMaxNq * 4 + 2 * 128 * 4 + 2 * 128 * 2 * 4 + 1024;
}

template <int D>
__global__ void __launch_bounds__(512, 1)
tc_fwdpair_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                  const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_o,
                  const PairArgs p) {
  constexpr int kSlabs = D / 64;
  constexpr int kKVBytes = kKeys * 128 * kSlabs;
  constexpr int kQBytes = kRows * 128 * kSlabs;
  constexpr int kPBytes = kRows * 128;
  constexpr int kStageBytes = kRows * 256;
  constexpr int kGroupBytes = kQBytes + kPBytes + kStageBytes;
  constexpr uint32_t kTmemCols = 256;
  constexpr uint32_t kIdescS = idesc_bf16(128, kKeys, 0, 0);
  constexpr uint32_t kIdescPV = idesc_bf16(128, D, 0, 1);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);   // pointer arithmetic keeps the shared address space
  uint8_t* sK = smem;
  uint8_t* sV = sK + kKVBytes;
  uint8_t* sGroup = sV + kKVBytes;
  uint64_t* bars = (uint64_t*)(sGroup + 2 * kGroupBytes);
  uint64_t* bar_kv = bars + 0;
  uint32_t* s_tmem = (uint32_t*)(bars + 8);
  volatile int* s_abort = (volatile int*)(s_tmem + 1);
  int* s_rowt_all = (int*)(bars + 10);                  // [2 groups][2 buffers][kPairMaxNq]
  uint32_t* s_prow_all = (uint32_t*)(s_rowt_all + 2 * 2 * kPairMaxNq);   // [2][128]
  float* s_max_all = (float*)(s_prow_all + 2 * 128);    // [2][128][2]

  const int tid = threadIdx.x;
  const int grp = tid / kPairGroupThreads, lt = tid % kPairGroupThreads;
  const int wg = lt >> 5, lane = lt & 31;
  const int quad = wg & 3, half = wg >> 2;
  const int row = quad * 32 + lane;
  uint8_t* sQ = sGroup + grp * kGroupBytes;
  uint8_t* sP = sQ + kQBytes;
  uint8_t* sStage = sP + kPBytes;
  uint64_t* bar_s = bars + 1 + 3 * grp;
  uint64_t* bar_o = bars + 2 + 3 * grp;
  uint64_t* bar_g = bars + 3 + 3 * grp;
  int* s_rowt = s_rowt_all + grp * 2 * kPairMaxNq;
  uint32_t* s_prow = s_prow_all + grp * 128;
  float* s_max = s_max_all + grp * 256;

  if (!prefer_pairs(p.stats, p.offsets, p.B * p.Hkv, p.n_ktiles, p.nq_union, p.force)) return;
  if ((int)blockIdx.x >= p.work->n_items) return;
  const int4 item = reinterpret_cast<const int4*>(p.work + 1)[blockIdx.x];
  const int bh = item.x, j = item.y;
  const int b = bh / p.Hkv, hkv = bh % p.Hkv;
  const int key0 = j * kKeys;
  const int ql = row / p.G, g = row % p.G;
  const bool row_slot_ok = ql < p.nq;

  const int pair_base = __ldg(p.offsets + (size_t)bh * (p.n_ktiles + 1) + j);
  const int n_q = __ldg(p.offsets + (size_t)bh * (p.n_ktiles + 1) + j + 1) - pair_base;
  const int n_rt = min((n_q + p.nq - 1) / p.nq, item.z + kSelChunkTiles);   // end of this item's chunk
  if (n_rt <= item.z) return;

  if (tid == 0) {
    *s_abort = (*(volatile int*)p.status != 0) ? 1 : 0;
    for (int k = 0; k <= 6; ++k) mbar_init(bars + k, 1);
    fence_barrier_init();
    prefetch_tensormap(&tm_k);
    prefetch_tensormap(&tm_v);
    prefetch_tensormap(&tm_q);
    prefetch_tensormap(&tm_o);
  }
  __syncthreads();
  if (*s_abort) return;
  // rows past nq * G of a tile are never loaded: keep them zero
  for (int i = tid; i < 2 * kQBytes / 16; i += blockDim.x) {
    uint8_t* base = sGroup + (i / (kQBytes / 16)) * kGroupBytes;
    *reinterpret_cast<uint4*>(base + (i % (kQBytes / 16)) * 16) = make_uint4(0, 0, 0, 0);
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
  const uint32_t col0 = grp * 128;        // S (64 columns) and, after S is read, O (D columns)

  if (tid == 0) {
    mbar_expect_tx(bar_kv, 2 * kKVBytes);
#pragma unroll
    for (int s = 0; s < kSlabs; ++s) {
      tma_load_3d(sK + s * (kKeys * 128), &tm_k, bar_kv, s * 64, key0, bh);
      tma_load_3d(sV + s * (kKeys * 128), &tm_v, bar_kv, s * 64, key0, bh);
    }
  }
  if (tid == 0 || tid == kPairGroupThreads) mbar_wait(bar_kv, 0, p.status, s_abort, 32);

  auto row_query = [&](int i) -> int {
    const int qi = i * p.nq + ql;
    if (!row_slot_ok || qi >= n_q) return -1;
    return ldg_s32_now(p.q_of_block + pair_base + qi);
  };

  const uint32_t gather_bytes = (uint32_t)(p.nq * p.G * 128 * kSlabs);
  auto gather = [&](const int* rowt) {      // one TMA box per query and slab; no query: zeros
    // the boxes are dealt out over the eight warps of the group (a few lanes each): one warp
    // issues its boxes one after another
    if (lt == 0) mbar_expect_tx(bar_g, gather_bytes);
    const int n_ops = p.nq * kSlabs;
    for (int o = lane * 8 + wg; o < n_ops; o += kPairGroupThreads) {
      const int qq = o / kSlabs, s = o % kSlabs;
      const int tq = rowt[qq] >= 0 ? rowt[qq] : p.T;
      tma_load_3d(sQ + s * (kRows * 128) + qq * p.G * 128, &tm_q, bar_g, s * 64,
                  b * p.Hq + hkv * p.G, tq);
    }
  };

  int i = item.z + grp;
  int t_cur = i < n_rt ? row_query(i) : -1;
  int t_nxt = i + 2 < n_rt ? row_query(i + 2) : -1;
  int buf = 0;
  if (i < n_rt) {
    if (g == 0 && half == 0 && row_slot_ok) s_rowt[ql] = t_cur;
    asm volatile("bar.sync %0, %1;" ::"r"(grp + 1), "r"(kPairGroupThreads) : "memory");
    gather(s_rowt);
  }
  uint32_t phase = 0;
  for (; i < n_rt; i += 2, phase ^= 1, buf ^= 1) {
    const int t_nn = (i + 4 < n_rt) ? row_query(i + 4) : -1;
    if (g == 0 && half == 0 && row_slot_ok) s_rowt[(buf ^ 1) * kPairMaxNq + ql] = t_nxt;
    mbar_wait(bar_g, phase, p.status, s_abort, 512);
    asm volatile("bar.sync %0, %1;" ::"r"(grp + 1), "r"(kPairGroupThreads) : "memory");
    if (lt == 0) {
      tc_fence_after();
      const uint32_t qa = desc_lo_kmajor(smem_u32(sQ)), ka = desc_lo_kmajor(smem_u32(sK));
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        const uint32_t slab = kk >> 2, in = (kk & 3) * 32;
        mma_ss(tmem + col0, desc_at(qa, slab * (kRows * 128) + in),
               desc_at(ka, slab * (kKeys * 128) + in), kIdescS, kk > 0);
      }
      tc_commit(bar_s);
    }
    const int hi = t_cur >= 0 ? min(kKeys - 1, min(t_cur, p.T - 1) - key0) : -1;
    mbar_wait(bar_s, phase, p.status, s_abort, 64);
    tc_fence_after();
    __syncwarp();
    uint32_t rs[32];
    tmem_ld32(lane_base + col0 + half * 32, rs);
    tmem_wait_ld();
    // S is done, so the Q tile is free: fetch this group's next tile
    if (i + 2 < n_rt) gather(s_rowt + (buf ^ 1) * kPairMaxNq);
    __syncwarp();
    float x[32];
    float mx = -INFINITY;
#pragma unroll
    for (int c = 0; c < 32; ++c) {
      x[c] = (half * 32 + c <= hi) ? __uint_as_float(rs[c]) * p.scale_log2 : -INFINITY;
      mx = fmaxf(mx, x[c]);
    }
    s_max[row * 2 + half] = mx;
    tc_fence_before();
    asm volatile("bar.sync %0, %1;" ::"r"(grp + 1), "r"(kPairGroupThreads) : "memory");
    const float m = fmaxf(s_max[row * 2], s_max[row * 2 + 1]);
    const float msub = (m == -INFINITY) ? 0.f : m;
    float lsum = 0.f;
    uint32_t pp[16];
#pragma unroll
    for (int c2 = 0; c2 < 16; ++c2) {
      const float p0 = ex2(x[2 * c2] - msub), p1 = ex2(x[2 * c2 + 1] - msub);
      lsum += p0 + p1;
      pp[c2] = pack_bf16(p0, p1);
    }
    const uint32_t p_row = smem_u32(sP) + row * 128;
#pragma unroll
    for (int k4 = 0; k4 < 4; ++k4) {
      const uint32_t chunk16 = (uint32_t)((half * 4 + k4) ^ (row & 7)) << 4;
      asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(p_row + chunk16), "r"(pp[k4 * 4]),
                   "r"(pp[k4 * 4 + 1]), "r"(pp[k4 * 4 + 2]), "r"(pp[k4 * 4 + 3])
                   : "memory");
    }
    fence_proxy_async();
    if (lt == 0) bulk_wait_read();   // the previous tile's store has left the staging tile
    asm volatile("bar.sync %0, %1;" ::"r"(grp + 1), "r"(kPairGroupThreads) : "memory");
    if (lt == 0) {
      tc_fence_after();
      const uint32_t pa = desc_lo_kmajor(smem_u32(sP)), va = desc_lo_mnmajor(smem_u32(sV), kKeys * 128);
#pragma unroll
      for (int kk = 0; kk < kKeys / 16; ++kk)
        mma_ss(tmem + col0, desc_at(pa, kk * 32), desc_at(va, kk * 2048), kIdescPV, kk > 0);
      tc_commit(bar_o);
    }
    const size_t prow = (size_t)(pair_base + i * p.nq + ql) * p.G + g;
    if (t_cur >= 0) {
      if (half == 0) p.ml[prow * 3] = m;
      p.ml[prow * 3 + 1 + half] = lsum;
    }
    if (half == 0) s_prow[row] = t_cur >= 0 ? (uint32_t)prow : 0xffffffffu;
    mbar_wait(bar_o, phase, p.status, s_abort, 128);
    tc_fence_after();
    __syncwarp();
    {   // O_part: TMEM -> bf16 -> staging tile: one slab of 128-byte rows per 64 columns, 16-byte
        // chunks XOR row, the layout of a 128B-swizzled TMA box
#pragma unroll
      for (int cc = 0; cc < D / 64; ++cc) {
        const int c0 = half * (D / 2) + cc * 32;
        uint32_t r32[32];
        tmem_ld32(lane_base + col0 + c0, r32);
        tmem_wait_ld();
#pragma unroll
        for (int v4 = 0; v4 < 4; ++v4) {
          const uint32_t chunk = (uint32_t)((c0 >> 3) + v4);
          const uint32_t dst = smem_u32(sStage) + (chunk >> 3) * (kRows * 128) + row * 128 +
                               (((chunk & 7) ^ (row & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst),
                       "r"(pack_bf16(__uint_as_float(r32[v4 * 8 + 0]), __uint_as_float(r32[v4 * 8 + 1]))),
                       "r"(pack_bf16(__uint_as_float(r32[v4 * 8 + 2]), __uint_as_float(r32[v4 * 8 + 3]))),
                       "r"(pack_bf16(__uint_as_float(r32[v4 * 8 + 4]), __uint_as_float(r32[v4 * 8 + 5]))),
                       "r"(pack_bf16(__uint_as_float(r32[v4 * 8 + 6]), __uint_as_float(r32[v4 * 8 + 7])))
                       : "memory");
        }
      }
    }
    fence_proxy_async();
    tc_fence_before();
    asm volatile("bar.sync %0, %1;" ::"r"(grp + 1), "r"(kPairGroupThreads) : "memory");
    if ((i + 1) * p.nq <= n_q) {
      // a full tile: its pairs are consecutive rows of the partial buffer, one TMA store per slab
      if (lt == 0) {
#pragma unroll
        for (int sl = 0; sl < kSlabs; ++sl)
          tma_store_5d(&tm_o, sStage + sl * (kRows * 128), sl * 64, 0, 0, pair_base + i * p.nq, 0);
        bulk_commit();
      }
    } else {   // the ragged last tile: whole rows out by hand
      constexpr int kChunks = D / 8;
      constexpr int kRowsPerPass = kPairGroupThreads / kChunks;
      const int c = lt % kChunks;
#pragma unroll 4
      for (int r = lt / kChunks; r < kRows; r += kRowsPerPass) {
        const uint32_t pr = s_prow[r];
        if (pr != 0xffffffffu) {
          const uint4 v = *reinterpret_cast<const uint4*>(sStage + (c >> 3) * (kRows * 128) + r * 128 +
                                                          (((c & 7) ^ (r & 7)) << 4));
          *reinterpret_cast<uint4*>(p.o_part + (size_t)pr * D + c * 8) = v;
        }
      }
    }
    tc_fence_before();
    t_cur = t_nxt; t_nxt = t_nn;
  }
  if (lt == 0) bulk_wait_all();
  tc_fence_before();
  __syncthreads();
  if (tid < 32) tmem_dealloc(tmem, kTmemCols);
}

// o[b, hkv*G+g, t, :] and lse from the per-(pair, head) partials of query (bh, t)
template <int D>
__global__ void sel_combine_kernel(const __nv_bfloat16* __restrict__ o_part, const float* __restrict__ ml,
                                   const int32_t* __restrict__ pair_of_slot,
                                   const int32_t* __restrict__ offsets,
                                   const unsigned long long* __restrict__ stats,
                                   __nv_bfloat16* __restrict__ o, float* __restrict__ lse, int B, int Hq,
                                   int Hkv, int T, int G, int S, int n_ktiles, int nq_union, int force) {
  if (!prefer_pairs(stats, offsets, B * Hkv, n_ktiles, nq_union, force)) return;
  constexpr int kVec = D / 8;
  const size_t gid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t total = (size_t)B * Hkv * T * G * kVec;
  if (gid >= total) return;
  const int v = (int)(gid % kVec);
  const int g = (int)((gid / kVec) % G);
  const int t = (int)((gid / ((size_t)kVec * G)) % T);
  const size_t bh = gid / ((size_t)kVec * G * T);
  const int32_t* ps = pair_of_slot + (bh * T + t) * S;
  // one pass with a running maximum: o = sum_j 2^(m_j - M) O_j / sum_j 2^(m_j - M) l_j
  float M = -INFINITY, L = 0.f;
  float acc[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) acc[e] = 0.f;
  // four slots per trip: all loads of a trip are issued before the first is used
  for (int s0 = 0; s0 < S; s0 += 4) {
    int pr[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) pr[j] = s0 + j < S ? __ldg(ps + s0 + j) : -1;
    float m[4], l[4];
    uint4 u[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      m[j] = -INFINITY; l[j] = 0.f; u[j] = make_uint4(0u, 0u, 0u, 0u);
      if (pr[j] >= 0) {
        const size_t prow = (size_t)pr[j] * G + g;
        m[j] = __ldg(ml + prow * 3);
        l[j] = __ldg(ml + prow * 3 + 1) + __ldg(ml + prow * 3 + 2);
        u[j] = __ldg(reinterpret_cast<const uint4*>(o_part + prow * D + v * 8));
      }
    }
    const float Mn = fmaxf(fmaxf(fmaxf(m[0], m[1]), fmaxf(m[2], m[3])), M);
    if (Mn == -INFINITY) continue;                          // nothing in this trip, nothing before
    const float a_old = ex2(M - Mn);                        // M = -inf: 0
    L *= a_old;
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] *= a_old;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float w = ex2(m[j] - Mn);                       // absent slot: 0
      L = fmaf(w, l[j], L);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u[j]);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(h[e]);
        acc[2 * e] = fmaf(w, f.x, acc[2 * e]);
        acc[2 * e + 1] = fmaf(w, f.y, acc[2 * e + 1]);
      }
    }
    M = Mn;
  }
  const float inv = L > 0.f ? 1.f / L : 0.f;
  const int b = (int)(bh / Hkv), hkv = (int)(bh % Hkv);
  const size_t orow = ((size_t)b * Hq + hkv * G + g) * T + t;
  uint4 u;
  u.x = pack_bf16(acc[0] * inv, acc[1] * inv); u.y = pack_bf16(acc[2] * inv, acc[3] * inv);
  u.z = pack_bf16(acc[4] * inv, acc[5] * inv); u.w = pack_bf16(acc[6] * inv, acc[7] * inv);
  *reinterpret_cast<uint4*>(o + orow * D + v * 8) = u;
  if (v == 0) lse[orow] = L > 0.f ? (M + log2f(L)) * kLn2 : kLseEmpty;
}

// distinct causally useful blocks per query tile of nq queries, summed into stats[0];
// one warp per query tile, its bitmap in shared memory
__global__ void sel_stats_kernel(const int32_t* __restrict__ block_idx, unsigned long long* __restrict__ stats,
                                 int T, int S, int nq, int n_qtiles, int nb, size_t n_tiles_total) {
  extern __shared__ uint32_t bm_all[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int words = (nb + 31) / 32;
  uint32_t* bm = bm_all + warp * words;
  const size_t tile = (size_t)blockIdx.x * (blockDim.x >> 5) + warp;
  if (tile >= n_tiles_total) return;
  const size_t bh = tile / n_qtiles;
  const int t0 = (int)(tile % n_qtiles) * nq;
  for (int w = lane; w < words; w += 32) bm[w] = 0u;
  __syncwarp();
  const int n_entries = (min(T, t0 + nq) - t0) * S;
  const int32_t* idx = block_idx + (bh * T + t0) * S;
  for (int e = lane; e < n_entries; e += 32) {
    const int blk = __ldg(idx + e);
    if (blk >= 0 && blk < nb && blk * kKeys <= t0 + e / S) atomicOr(&bm[blk >> 5], 1u << (blk & 31));
  }
  __syncwarp();
  int cnt = 0;
  for (int w = lane; w < words; w += 32) cnt += __popc(bm[w]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
  if (lane == 0 && cnt) atomicAdd(stats, (unsigned long long)cnt);
}

// One CTA walks the (batch, kv head, block) entries in order: each block's row tiles in chunks of
// kSelChunkTiles, one work item each (at least one, so that a block nobody lists still gets its
// zero gradients).  An exclusive scan of the chunk counts places the items, so the list is in
// (batch, kv head, block, chunk) order: CTAs that run together work on one (batch, kv head) and
// share its q rows in L2.
__global__ void sel_worklist_kernel(const int32_t* __restrict__ offsets, int n_ktiles, int units, int nq,
                                    SelWorkHeader* __restrict__ work, int max_items) {
  __shared__ int part[1024];
  __shared__ int carry;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  int4* items = reinterpret_cast<int4*>(work + 1);
  const int total = units * n_ktiles;
  for (int base0 = 0; base0 < total; base0 += 1024) {
    const int idx = base0 + threadIdx.x;
    int n_chunks = 0, bh = 0, j = 0;
    if (idx < total) {
      bh = idx / n_ktiles; j = idx % n_ktiles;
      const int n_q = offsets[(size_t)bh * (n_ktiles + 1) + j + 1] - offsets[(size_t)bh * (n_ktiles + 1) + j];
      const int n_rt = (n_q + nq - 1) / nq;
      n_chunks = max(1, (n_rt + kSelChunkTiles - 1) / kSelChunkTiles);
    }
    part[threadIdx.x] = n_chunks;
    __syncthreads();
    for (int o = 1; o < 1024; o <<= 1) {
      const int v = threadIdx.x >= o ? part[threadIdx.x - o] : 0;
      __syncthreads();
      part[threadIdx.x] += v;
      __syncthreads();
    }
    const int incl = part[threadIdx.x] + carry;
    const int first = incl - n_chunks;
    for (int c = 0; c < n_chunks && first + c < max_items; ++c)
      items[first + c] = make_int4(bh, j, c * kSelChunkTiles, n_chunks);
    __syncthreads();
    if (threadIdx.x == 1023) carry = incl;
    __syncthreads();
  }
  if (threadIdx.x == 0) work->n_items = min(carry, max_items);
}

size_t sel_work_max_items(size_t units, int n_ktiles, size_t cap_pairs, int nq) {
  // sum over blocks of max(1, ceil(ceil(n_q / nq) / chunk)) <= blocks * (1 + 1/chunk) + pairs / (chunk * nq)
  const size_t blocks = units * n_ktiles;
  return blocks + blocks / kSelChunkTiles + cap_pairs / ((size_t)kSelChunkTiles * nq) + 2;
}
size_t sel_work_bytes(size_t units, int n_ktiles, size_t cap_pairs, int nq) {
  return sizeof(SelWorkHeader) + sel_work_max_items(units, n_ktiles, cap_pairs, nq) * sizeof(int4);
}
int sel_build_worklist(const int32_t* offsets, int n_ktiles, size_t units, size_t cap_pairs, int nq,
                       void* work, cudaStream_t st) {
  NSA_CUDA_OK(cudaMemsetAsync(work, 0, sizeof(SelWorkHeader), st));
  const size_t n = units * n_ktiles;
  if (n == 0) return NSA_OK;
  KernelScope ks("sel_worklist_kernel", st);
  sel_worklist_kernel<<<1, 1024, 0, st>>>(
      offsets, n_ktiles, (int)units, nq, (SelWorkHeader*)work,
      (int)sel_work_max_items(units, n_ktiles, cap_pairs, nq));
  NSA_LAUNCH_OK("sel_worklist_kernel");
  return NSA_OK;
}

struct PairPlan {
  int n_ktiles, nq;
  size_t cap_pairs;
  size_t off_stats, off_part, off_ml, off_csr_ws, off_qob, off_off, off_pbh, off_pos, off_work, total;
};

static PairPlan plan_pairs(const AttnArgs& a) {
  PairPlan pl;
  const int G = a.Hq / a.Hkv;
  pl.nq = kRows / G;
  pl.n_ktiles = (a.T + kKeys - 1) / kKeys;
  const size_t units = (size_t)a.B * a.Hkv;
  pl.cap_pairs = units * a.T * a.S;
  size_t off = 0;
  pl.off_stats = off; off += 256;
  pl.off_part = off; off += align_up(pl.cap_pairs * G * a.D * 2, 256);
  pl.off_ml = off; off += align_up(pl.cap_pairs * G * 3 * 4, 256);
  pl.off_csr_ws = off; off += align_up(nsa_csr_workspace_bytes(a.B, a.Hkv, pl.n_ktiles * kKeys, a.S, kKeys), 256);
  pl.off_qob = off; off += align_up(pl.cap_pairs * 4, 256);
  pl.off_pbh = off; off += align_up(pl.cap_pairs * 4, 256);
  pl.off_off = off; off += align_up(units * (pl.n_ktiles + 1) * 4, 256);
  pl.off_pos = off; off += align_up(pl.cap_pairs * 4, 256);
  pl.off_work = off; off += align_up(sel_work_bytes(units, pl.n_ktiles, pl.cap_pairs, pl.nq), 256);
  pl.total = off;
  return pl;
}

}  // namespace tc

int build_csr_internal(const int32_t* block_idx, int B, int Hkv, int T, int S, int block_size,
                       int n_blk, int32_t* q_of_block, int32_t* block_offsets, int32_t* pair_bh,
                       int32_t* pair_of_slot, void* workspace, size_t workspace_bytes, cudaStream_t st);
int tc_fwd_union_launch(const AttnArgs& a, const unsigned long long* stats, const int32_t* offsets,
                        int force, cudaStream_t st);
int get_option_sel_fwd();
int get_option_pair_kernel();
int tc_fwdpair2_launch(const AttnArgs& a, const int32_t* q_of_block, const int32_t* offsets, void* o_part,
                       float* ml, const unsigned long long* stats, const void* work, int force, int nq,
                       int n_ktiles, int nq_union, size_t cap_pairs, unsigned grid, cudaStream_t st);

size_t tc_sel_fwd_workspace(const AttnArgs& a) { return tc::plan_pairs(a).total; }

// Selection forward: statistics, CSR, then both variants are launched; the device-side rule
// lets exactly one of them do the work.
int tc_sel_fwd(const AttnArgs& a, void* ws, size_t ws_bytes, cudaStream_t st) {
  using namespace tc;
  const PairPlan pl = plan_pairs(a);
  if (!ws || ws_bytes < pl.total) {
    set_error("selection forward workspace too small: need %zu bytes", pl.total);
    return NSA_ERR_WORKSPACE;
  }
  char* base = (char*)ws;
  const int G = a.Hq / a.Hkv;
  const int nq_union = kRows / group_pad(G);
  unsigned long long* stats = (unsigned long long*)(base + pl.off_stats);
  NSA_CUDA_OK(cudaMemsetAsync(stats, 0, 256, st));
  {
    const int n_qtiles = (a.T + nq_union - 1) / nq_union;
    const size_t tiles = (size_t)a.B * a.Hkv * n_qtiles;
    const int words = (pl.n_ktiles + 31) / 32;
    KernelScope ks("sel_stats_kernel", st);
    sel_stats_kernel<<<(unsigned)((tiles + 3) / 4), 128, 4 * words * sizeof(uint32_t), st>>>(
        a.block_idx, stats, a.T, a.S, nq_union, n_qtiles, pl.n_ktiles, tiles);
  }
  NSA_LAUNCH_OK("sel_stats_kernel");
  int32_t* offsets = (int32_t*)(base + pl.off_off);
  int32_t* pair_of_slot = (int32_t*)(base + pl.off_pos);
  int rc = build_csr_internal(a.block_idx, a.B, a.Hkv, a.T, a.S, kKeys, pl.n_ktiles,
                              (int32_t*)(base + pl.off_qob), offsets, (int32_t*)(base + pl.off_pbh),
                              pair_of_slot, base + pl.off_csr_ws, pl.off_qob - pl.off_csr_ws, st);
  if (rc != NSA_OK) return rc;
  rc = sel_build_worklist(offsets, pl.n_ktiles, (size_t)a.B * a.Hkv, pl.cap_pairs, pl.nq, base + pl.off_work, st);
  if (rc != NSA_OK) return rc;
  const int force = get_option_sel_fwd();
  rc = tc_fwd_union_launch(a, stats, offsets, force, st);
  if (rc != NSA_OK) return rc;

  PairArgs p;
  p.q = (const __nv_bfloat16*)a.q;
  p.q_of_block = (const int32_t*)(base + pl.off_qob);
  p.offsets = offsets;
  p.o_part = (__nv_bfloat16*)(base + pl.off_part);
  p.ml = (float*)(base + pl.off_ml);
  p.stats = stats;
  p.work = (const SelWorkHeader*)(base + pl.off_work);
  p.status = device_status_ptr();
  if (!p.status) { set_error("device status word unavailable"); return NSA_ERR_CUDA; }
  p.B = a.B; p.Hq = a.Hq; p.Hkv = a.Hkv; p.T = a.T; p.G = G; p.nq = pl.nq;
  p.n_ktiles = pl.n_ktiles; p.nq_union = nq_union; p.force = force;
  p.scale_log2 = a.scale * kLog2e;
  CUtensorMap tm_k, tm_v, tm_q;
  rc = make_map(&tm_k, a.k, a.D, a.T, a.B * a.Hkv, kKeys, 1);
  if (rc == NSA_OK) rc = make_map(&tm_v, a.v, a.D, a.T, a.B * a.Hkv, kKeys, 1);
  if (rc == NSA_OK) rc = make_map_query_rows(&tm_q, a.q, a.D, a.T, a.B * a.Hq, G);
  CUtensorMap tm_o;
  if (rc == NSA_OK) rc = make_map_partial(&tm_o, p.o_part, a.D, G, 1, pl.cap_pairs ? pl.cap_pairs : 1, 1, pl.nq);
  if (rc != NSA_OK) return rc;
  const size_t smem = pair_smem_bytes(a.D);
  const dim3 grid((unsigned)sel_work_max_items((size_t)a.B * a.Hkv, pl.n_ktiles, pl.cap_pairs, pl.nq));
  const size_t nthreads = (size_t)a.B * a.Hkv * a.T * G * (a.D / 8);
  const unsigned cgrid = (unsigned)((nthreads + 255) / 256);
  const bool v2 = get_option_pair_kernel() == 1;
  if (v2) {
    rc = tc_fwdpair2_launch(a, p.q_of_block, offsets, p.o_part, p.ml, stats, p.work, force, pl.nq, pl.n_ktiles,
                            nq_union, pl.cap_pairs, grid.x, st);
    if (rc != NSA_OK) return rc;
  }
  if (a.D == 128) {
    NSA_CUDA_OK(cudaFuncSetAttribute(tc_fwdpair_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    if (!v2) { KernelScope ks("tc_fwd_slc_pairs", st); tc_fwdpair_kernel<128><<<grid, 512, smem, st>>>(tm_k, tm_v, tm_q, tm_o, p); }
    { KernelScope ks("sel_combine_kernel", st);
      sel_combine_kernel<128><<<cgrid, 256, 0, st>>>(p.o_part, p.ml, pair_of_slot, offsets, stats,
                                                    (__nv_bfloat16*)a.o, a.lse, a.B, a.Hq, a.Hkv, a.T, G,
                                                    a.S, pl.n_ktiles, nq_union, p.force); }
  } else {
    NSA_CUDA_OK(cudaFuncSetAttribute(tc_fwdpair_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    if (!v2) { KernelScope ks("tc_fwd_slc_pairs", st); tc_fwdpair_kernel<64><<<grid, 512, smem, st>>>(tm_k, tm_v, tm_q, tm_o, p); }
    { KernelScope ks("sel_combine_kernel", st);
      sel_combine_kernel<64><<<cgrid, 256, 0, st>>>(p.o_part, p.ml, pair_of_slot, offsets, stats,
                                                   (__nv_bfloat16*)a.o, a.lse, a.B, a.Hq, a.Hkv, a.T, G,
                                                   a.S, pl.n_ktiles, nq_union, p.force); }
  }
  NSA_LAUNCH_OK("tc_fwdpair_kernel");
  return NSA_OK;
}

}  // namespace nsa
