// Block scoring + top-n on the tensor cores (replaces the dense scoring pass of
// nsa_model.py:343-355).
//
// Same row tile as the forward kernel: 128 rows = nq queries x Gp heads of one (batch, kv head).
// For every 64-summary tile: S = Q Kc^T by tcgen05.mma; the thread that owns a row turns it
// into compression-branch probabilities p = exp2(s*scale*log2e - lse*log2e) with the LSE the
// compression forward stored; the probabilities go to shared memory and are summed over the Gp
// heads of each query (ascending head order, fp32).  The 128 threads are dealt out 128 / nq per
// query; each keeps in registers the best 16 of the candidates it scanned, ordered by
// (importance descending, block index ascending), and a tournament over the lists' heads writes
// the query's top-n at the end.  Slots with no causally valid block are -1.
#include "tc_common.cuh"
#include "tc_host.cuh"

namespace nsa {
namespace tc {

struct ScoreArgs {
  const float* lse;
  int32_t* block_idx;
  float* imp_out;
  int* status;
  int B, Hq, Hkv, T, n_blk, G, Gp, nq, block_size, n_sel, n_qtiles, n_init, n_local;
  // general geometry (lanes kernel): n_blk summaries of block_size tokens every `stride`; selection
  // blocks of sel_block = r * stride tokens; overlap: block_size == 2 * stride; imp_out has imp_cols columns
  int stride, sel_block, r, overlap, imp_cols;
  float scale_log2;
};


__host__ __device__ inline size_t score_smem_bytes(int D, int nq) {
  return (size_t)(kRows * 128 + 2 * kKeys * 128) * (D / 64) + (size_t)kRows * kKeys * 4 +
         (size_t)nq * kKeys * 4 + 256 + 4 * 32 * 8 + 1024;
}

template <int D>
__global__ void __launch_bounds__(128, 2)
tc_score_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const ScoreArgs p) {
  constexpr int kSlabs = D / 64;
  constexpr int kQBytes = kRows * 128 * kSlabs, kKBytes = kKeys * 128 * kSlabs;
  constexpr uint32_t kTmemCols = 64;
  constexpr uint32_t kIdescQK = idesc_bf16(128, kKeys, 0, 0);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);   // pointer arithmetic keeps the shared address space
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + kQBytes;                        // 2 stages
  float* sP = (float*)(sK + 2 * kKBytes);            // [128][64] probabilities
  float* sImp = sP + kRows * kKeys;                  // [nq][64] group sums
  uint64_t* bars = (uint64_t*)(sImp + p.nq * kKeys);
  uint64_t* bar_q = bars + 0;
  uint64_t* bar_k = bars + 1;   // [2]
  uint64_t* bar_s = bars + 3;
  uint64_t* bar_drain = bars + 4;   // an aborted CTA waits here for its last MMAs
  uint32_t* s_tmem = (uint32_t*)(bars + 5);
  volatile int* s_abort = (volatile int*)(s_tmem + 1);

  const int tid = threadIdx.x, warp = tid >> 5;
  const int qtile = p.n_qtiles - 1 - (int)blockIdx.x;
  const int bh = blockIdx.y;
  const int b = bh / p.Hkv, hkv = bh % p.Hkv;
  const int t0 = qtile * p.nq;
  const int t_last = min(p.T - 1, t0 + p.nq - 1);
  const int g = tid / p.nq, ql = tid % p.nq;
  const int t = t0 + ql;
  const bool row_ok = (g < p.G) && (t < p.T);

  if (tid == 0) {
    *s_abort = (*(volatile int*)p.status != 0) ? 1 : 0;
    mbar_init(bar_q, 1);
    mbar_init(bar_k + 0, 1); mbar_init(bar_k + 1, 1);
    mbar_init(bar_s, 1);
    mbar_init(bar_drain, 1);
    fence_barrier_init();
    prefetch_tensormap(&tm_q); prefetch_tensormap(&tm_k);
  }
  __syncthreads();
  if (*s_abort) return;

  const int hi_last = min(p.n_blk, (t_last + 1) / p.block_size) - 1;
  int n_tiles = hi_last < 0 ? 0 : hi_last / kKeys + 1;
  // forced blocks (the first n_init, the n_local most recent including the block holding t)
  // are candidates even when incomplete: the tiles reach the block holding the last query
  const bool forcing = p.n_init > 0 || p.n_local > 0;
  if (forcing) n_tiles = max(n_tiles, (t_last / p.block_size) / kKeys + 1);

  // Running top-16 lists: the 128 threads are dealt out Lq = 128 / nq per query; each keeps, in
  // registers, the best 16 of the candidates it has scanned (64 / Lq per tile), ordered by
  // (importance descending, block index ascending).  The Lq lists of a query are merged at the
  // end by a 16-round tournament over their heads.
  constexpr int kList = 16;
  const int Lq = kRows / p.nq;
  const int my_q = tid / Lq, my_sub = tid % Lq;
  const int per_lane = kKeys / Lq;
  const int my_t = t0 + my_q;
  float lv[kList];
  int li[kList];
#pragma unroll
  for (int k = 0; k < kList; ++k) { lv[k] = -1.f; li[k] = -1; }

  uint32_t tmem = 0;
  bool aborted = false;
  int k_loaded = 0, k_seen = 0;   // thread 0: K tiles whose load was issued / whose arrival was seen
  bool q_seen = false;
  if (n_tiles > 0) {
    if (warp == 0) {
      tmem_alloc(s_tmem, kTmemCols);
      tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    tmem = *s_tmem;
    const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);
    const float lse2 = row_ok ? __ldg(p.lse + (size_t)(b * p.Hq + hkv * p.G + g) * p.T + t) * kLog2e : 0.f;

    auto load_k = [&](int i) {
      uint64_t* bar = bar_k + (i & 1);
      mbar_expect_tx(bar, kKBytes);
#pragma unroll
      for (int s = 0; s < kSlabs; ++s)
        tma_load_3d(sK + (i & 1) * kKBytes + s * (kKeys * 128), &tm_k, bar, s * 64, i * kKeys, bh);
      k_loaded = i + 1;
    };
    auto issue_s = [&](int i) {
      const uint32_t qa = desc_lo_kmajor(smem_u32(sQ)), ka = desc_lo_kmajor(smem_u32(sK + (i & 1) * kKBytes));
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        const uint32_t slab = kk >> 2, in = (kk & 3) * 32;
        mma_ss(tmem, desc_at(qa, slab * (kRows * 128) + in), desc_at(ka, slab * (kKeys * 128) + in),
               kIdescQK, kk > 0);
      }
      tc_commit(bar_s);
    };
    if (tid == 0) {
      mbar_expect_tx(bar_q, kQBytes);
#pragma unroll
      for (int s = 0; s < kSlabs; ++s)
        tma_load_3d(sQ + s * (kRows * 128), &tm_q, bar_q, s * 64, t0, b * p.Hq + hkv * p.G);
      load_k(0);
      if (n_tiles > 1) load_k(1);
      q_seen = mbar_wait(bar_q, 0, p.status, s_abort, 1);
      if (mbar_wait(bar_k, 0, p.status, s_abort, 2)) k_seen = 1;
      tc_fence_after();
      if (!*s_abort) issue_s(0);
    }

    for (int i = 0; i < n_tiles; ++i) {
      const int key0 = i * kKeys;
      const bool s_ok = mbar_wait(bar_s, i & 1, p.status, s_abort, 4);
      tc_fence_after();
      if (tid == 0 && i + 2 < n_tiles && s_ok) load_k(i + 2);
      __syncwarp();
      uint32_t r[64];
      tmem_ld32(lane_base, r);
      tmem_ld32(lane_base + 32, r + 32);
      tmem_wait_ld();
      tc_fence_before();
      const int hi = row_ok ? min(kKeys - 1, min(p.n_blk, (t + 1) / p.block_size) - 1 - key0) : -1;
      float4* dst = reinterpret_cast<float4*>(sP + tid * kKeys);
#pragma unroll
      for (int c4 = 0; c4 < 16; ++c4) {
        float4 v;
        v.x = (c4 * 4 + 0 <= hi) ? ex2(__uint_as_float(r[c4 * 4 + 0]) * p.scale_log2 - lse2) : 0.f;
        v.y = (c4 * 4 + 1 <= hi) ? ex2(__uint_as_float(r[c4 * 4 + 1]) * p.scale_log2 - lse2) : 0.f;
        v.z = (c4 * 4 + 2 <= hi) ? ex2(__uint_as_float(r[c4 * 4 + 2]) * p.scale_log2 - lse2) : 0.f;
        v.w = (c4 * 4 + 3 <= hi) ? ex2(__uint_as_float(r[c4 * 4 + 3]) * p.scale_log2 - lse2) : 0.f;
        // 16-byte chunk index XOR row: a warp's stores spread over the banks
        dst[c4 ^ (tid & 15)] = v;
      }
      // all of S is read, all of P is in shared memory; one decision for the whole CTA: after a
      // given-up wait nothing more is issued or written
      if (__syncthreads_or(*s_abort)) { aborted = true; break; }
      if (tid == 0 && i + 1 < n_tiles) {
        tc_fence_after();
        if (mbar_wait(bar_k + ((i + 1) & 1), ((i + 1) >> 1) & 1, p.status, s_abort, 2)) {
          k_seen = i + 2;
          issue_s(i + 1);
        }
      }
      // group sums: importance[ql][c] = sum over heads, ascending; four columns per thread
      for (int e = tid; e < p.nq * (kKeys / 4); e += 128) {
        const int qq = e / (kKeys / 4), c4 = e % (kKeys / 4);
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int gg = 0; gg < p.G; ++gg) {
          const int row = gg * p.nq + qq;
          const float4 v = *reinterpret_cast<const float4*>(sP + row * kKeys + ((c4 ^ (row & 15)) << 2));
          acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        *reinterpret_cast<float4*>(sImp + qq * kKeys + c4 * 4) = acc;
        if (p.imp_out && t0 + qq < p.T) {
          const int hq = min(p.n_blk, (t0 + qq + 1) / p.block_size) - 1 - key0;   // last valid column
          float* out = p.imp_out + ((size_t)bh * p.T + t0 + qq) * p.n_blk + key0 + c4 * 4;
          const float vals[4] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
          for (int e = 0; e < 4; ++e)
            if (key0 + c4 * 4 + e < p.n_blk) out[e] = (c4 * 4 + e <= hq) ? vals[e] : 0.f;
        }
      }
      __syncthreads();
      // top-16 update: this thread scans its share of the query's 64 candidates
      {
        const int hq = my_t < p.T ? min(kKeys - 1, min(p.n_blk, (my_t + 1) / p.block_size) - 1 - key0) : -1;
        const int my_cur = my_t / p.block_size;
        const int hf = (forcing && my_t < p.T) ? min(kKeys - 1, my_cur - key0) : -1;
        for (int k = 0; k < per_lane; ++k) {
          const int c = my_sub * per_lane + k;
          if (c > max(hq, hf)) break;
          const int cj = key0 + c;
          float cv = c <= hq ? sImp[my_q * kKeys + c] : -1.f;
          if (forcing) {                     // cj <= my_cur here
            if (cj < p.n_init) cv = kForcedInit - (float)cj;
            else if (cj > my_cur - p.n_local) cv = kForcedLocal - (float)(my_cur - cj);
          }
          if (cv > lv[kList - 1]) {          // beats the list's last entry (empty slots hold -1)
#pragma unroll
            for (int r = kList - 1; r >= 1; --r) {   // strict '>' keeps earlier (lower) indices ahead
              const bool up = cv > lv[r - 1];
              const bool here = cv > lv[r];
              li[r] = up ? li[r - 1] : (here ? cj : li[r]);
              lv[r] = up ? lv[r - 1] : (here ? cv : lv[r]);
            }
            if (cv > lv[0]) { lv[0] = cv; li[0] = cj; }
          }
        }
      }
      __syncthreads();                         // sP / sImp are rewritten by the next tile
    }
    if (!aborted) aborted = __syncthreads_or(*s_abort) != 0;
    if (aborted) {
      // Give-up path: no list is written.  Thread 0 waits (bounded) for the loads still on their
      // way into this CTA's shared memory and for the MMAs already issued, then the tensor memory
      // goes back.
      if (tid == 0) {
        if (!q_seen) mbar_wait_drain(bar_q, 0);
        for (int j = k_seen; j < k_loaded; ++j) mbar_wait_drain(bar_k + (j & 1), (j >> 1) & 1);
        tc_commit(bar_drain);
        mbar_wait_drain(bar_drain, 0);
      }
      tc_fence_before();
      __syncthreads();
      if (warp == 0) tmem_dealloc(tmem, kTmemCols);
      return;
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, kTmemCols);
  }

  // ---- merge the Lq lists of each query: n_sel rounds, each takes the best head ------------------
  for (int r = 0; r < p.n_sel; ++r) {
    float bv = lv[0];
    int bj = li[0];
    for (int o = 1; o < Lq; o <<= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oj = __shfl_xor_sync(0xffffffffu, bj, o);
      if (ov > bv || (ov == bv && oj >= 0 && (bj < 0 || oj < bj))) { bv = ov; bj = oj; }
    }
    if (bj >= 0 && li[0] == bj) {            // this list gave the winner: pop its head
#pragma unroll
      for (int k = 0; k < kList - 1; ++k) { lv[k] = lv[k + 1]; li[k] = li[k + 1]; }
      lv[kList - 1] = -1.f;
      li[kList - 1] = -1;
    }
    if (my_sub == 0 && my_t < p.T) p.block_idx[((size_t)bh * p.T + my_t) * p.n_sel + r] = bj;
  }
  // importance columns no tile covered are zero
  if (p.imp_out && my_t < p.T) {
    float* out = p.imp_out + ((size_t)bh * p.T + my_t) * p.n_blk;
    for (int c = n_tiles * kKeys + my_sub; c < p.n_blk; c += Lq) out[c] = 0.f;
  }
}


// ------------------------------------------------------------------------------------------
// The same for GQA groups of 4, 8 or 16 (padded) heads, without the shared-memory round trip:
// the rows of a tile are ordered query-major (row = query * GP + head, one TMA box from the
// (D, heads, T) view of q), so the GP heads of a query are GP neighbouring lanes of one warp.
// They add their probabilities by a recursive-halving exchange (GP/2, ..., 1 lanes apart), after
// which lane g holds the importance of the tile's blocks [g * 64/GP, (g+1) * 64/GP) and scans
// exactly those for its top-16 list.  64 KB of shared memory: three CTAs per SM.
// ------------------------------------------------------------------------------------------
template <int D, int GP, bool kAligned>
__global__ void __launch_bounds__(128, 3)
tc_score_lanes_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                      const ScoreArgs p) {
  constexpr int kSlabs = D / 64;
  constexpr int kQBytes = kRows * 128 * kSlabs, kKBytes = kKeys * 128 * kSlabs;
  constexpr uint32_t kTmemCols = 64;
  constexpr uint32_t kIdescQK = idesc_bf16(128, kKeys, 0, 0);
  constexpr int NQ = kRows / GP;       // queries per tile
  constexpr int PER = kKeys / GP;      // blocks of a tile each lane ends up owning
  constexpr int kList = 16;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + kQBytes;                        // 2 stages
  uint64_t* bars = (uint64_t*)(sK + 2 * kKBytes);
  uint64_t* bar_q = bars + 0;
  uint64_t* bar_k = bars + 1;   // [2]
  uint64_t* bar_s = bars + 3;
  uint64_t* bar_drain = bars + 4;   // an aborted CTA waits here for its last MMAs
  uint32_t* s_tmem = (uint32_t*)(bars + 5);
  volatile int* s_abort = (volatile int*)(s_tmem + 1);

  const int tid = threadIdx.x, warp = tid >> 5;
  const int qtile = p.n_qtiles - 1 - (int)blockIdx.x;
  const int bh = blockIdx.y;
  const int b = bh / p.Hkv, hkv = bh % p.Hkv;
  const int t0 = qtile * NQ;
  const int t_last = min(p.T - 1, t0 + NQ - 1);
  const int g = tid % GP, ql = tid / GP;
  const int t = t0 + ql;
  const bool row_ok = (g < p.G) && (t < p.T);

  if (tid == 0) {
    *s_abort = (*(volatile int*)p.status != 0) ? 1 : 0;
    mbar_init(bar_q, 1);
    mbar_init(bar_k + 0, 1); mbar_init(bar_k + 1, 1);
    mbar_init(bar_s, 1);
    mbar_init(bar_drain, 1);
    fence_barrier_init();
    prefetch_tensormap(&tm_q); prefetch_tensormap(&tm_k);
  }
  __syncthreads();
  if (*s_abort) return;

  const int hi_last = cmp_visible(t_last, p.block_size, p.stride, p.n_blk) - 1;
  int n_tiles = hi_last < 0 ? 0 : hi_last / kKeys + 1;
  const bool forcing = p.n_init > 0 || p.n_local > 0;
  // forced blocks are candidates whatever their importance: reach the tile whose lanes own the
  // block that holds the last query
  if (forcing) n_tiles = max(n_tiles, (p.r * (t_last / p.sel_block)) / kKeys + 1);

  float lv[kList];
  int li[kList];
#pragma unroll
  for (int k = 0; k < kList; ++k) { lv[k] = -1.f; li[k] = -1; }

  if (n_tiles > 0) {
    if (warp == 0) {
      tmem_alloc(s_tmem, kTmemCols);
      tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *s_tmem;
    bool aborted = false;
    int k_loaded = 0, k_seen = 0;   // thread 0: K tiles whose load was issued / whose arrival was seen
    bool q_seen = false;
    const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);
    const float lse2 = row_ok ? __ldg(p.lse + (size_t)(b * p.Hq + hkv * p.G + g) * p.T + t) * kLog2e : 0.f;
    const int n_vis = t < p.T ? cmp_visible(t, p.block_size, p.stride, p.n_blk) : 0;   // summaries query t sees
    const int my_cur = t / p.sel_block;              // selection block that holds t
    float carry = 0.f;                               // last summary of the previous tile (overlap)

    auto load_k = [&](int i) {
      uint64_t* bar = bar_k + (i & 1);
      mbar_expect_tx(bar, kKBytes);
#pragma unroll
      for (int sl = 0; sl < kSlabs; ++sl)
        tma_load_3d(sK + (i & 1) * kKBytes + sl * (kKeys * 128), &tm_k, bar, sl * 64, i * kKeys, bh);
      k_loaded = i + 1;
    };
    auto issue_s = [&](int i) {
      const uint32_t qa = desc_lo_kmajor(smem_u32(sQ)), ka = desc_lo_kmajor(smem_u32(sK + (i & 1) * kKBytes));
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        const uint32_t slab = kk >> 2, in = (kk & 3) * 32;
        mma_ss(tmem, desc_at(qa, slab * (kRows * 128) + in), desc_at(ka, slab * (kKeys * 128) + in),
               kIdescQK, kk > 0);
      }
      tc_commit(bar_s);
    };
    if (tid == 0) {
      mbar_expect_tx(bar_q, kQBytes);
#pragma unroll
      for (int sl = 0; sl < kSlabs; ++sl)     // box: 64 columns x GP heads x NQ tokens
        tma_load_3d(sQ + sl * (kRows * 128), &tm_q, bar_q, sl * 64, b * p.Hq + hkv * p.G, t0);
      load_k(0);
      if (n_tiles > 1) load_k(1);
      q_seen = mbar_wait(bar_q, 0, p.status, s_abort, 1);
      if (mbar_wait(bar_k, 0, p.status, s_abort, 2)) k_seen = 1;
      tc_fence_after();
      if (!*s_abort) issue_s(0);
    }

    for (int i = 0; i < n_tiles; ++i) {
      const int key0 = i * kKeys;
      mbar_wait(bar_s, i & 1, p.status, s_abort, 4);
      tc_fence_after();
      __syncwarp();
      float v[64];
      {
        uint32_t r[64];
        tmem_ld32(lane_base, r);
        tmem_ld32(lane_base + 32, r + 32);
        tmem_wait_ld();
        tc_fence_before();
        const int hi = row_ok ? min(kKeys - 1, n_vis - 1 - key0) : -1;
#pragma unroll
        for (int c = 0; c < 64; ++c)
          v[c] = (c <= hi) ? ex2(__uint_as_float(r[c]) * p.scale_log2 - lse2) : 0.f;
      }
      // every thread has read S: the next MMA may overwrite it; one decision for the whole CTA:
      // after a given-up wait nothing more is issued or written
      if (__syncthreads_or(*s_abort)) { aborted = true; break; }
      if (tid == 0) {
        if (i + 2 < n_tiles) load_k(i + 2);    // stage i & 1 was read by the MMA that just completed
        if (i + 1 < n_tiles) {
          tc_fence_after();
          if (mbar_wait(bar_k + ((i + 1) & 1), ((i + 1) >> 1) & 1, p.status, s_abort, 2)) {
            k_seen = i + 2;
            issue_s(i + 1);
          }
        }
      }
      __syncwarp();
      // sum over the heads of the query: recursive halving, the lane with the bit set keeps the
      // upper half of the columns
      {
        int width = 64;
#pragma unroll
        for (int o = GP / 2; o >= 1; o >>= 1) {
          width >>= 1;
          const bool upper = (g & o) != 0;
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            if (c < width) {
              const float send = upper ? v[c] : v[c + width];
              const float keep = upper ? v[c + width] : v[c];
              v[c] = keep + __shfl_xor_sync(0xffffffffu, send, o);
            }
          }
        }
      }
      // lane g now holds the summaries key0 + g * PER + k in v[k].  A selection block is r
      // consecutive summaries (plus, when the summaries overlap, the one before them); it is a
      // candidate once its first summary is visible.
      // kAligned: summaries and blocks coincide (r = 1, no overlap), all of it folds away
      const int r_ = kAligned ? 1 : p.r, ov_ = kAligned ? 0 : p.overlap;
      float prev = 0.f;
      if (!kAligned) {
        prev = __shfl_up_sync(0xffffffffu, v[PER - 1], 1);
        if (g == 0) prev = carry;
        carry = __shfl_sync(0xffffffffu, v[PER - 1], (threadIdx.x & 31 & ~(GP - 1)) + GP - 1);
      }
      float* out = (p.imp_out && t < p.T) ? p.imp_out + ((size_t)bh * p.T + t) * p.imp_cols : nullptr;
      // A candidate below entry 16 / GP (counted from 1) of every one of the query's GP lists has
      // at least 16 entries ahead of it, so it cannot reach the merged top 16 and need not enter a
      // list; the bound only rises while the tile is scanned.
      float tau = lv[kList / GP - 1];
#pragma unroll
      for (int o = 1; o < GP; o <<= 1) tau = fminf(tau, __shfl_xor_sync(0xffffffffu, tau, o));
      float accb = 0.f;
#pragma unroll
      for (int k = 0; k < PER; ++k) {
        if ((k & (r_ - 1)) == 0) accb = ov_ ? (k == 0 ? prev : v[k > 0 ? k - 1 : 0]) : 0.f;
        accb += v[k];
        if (((k + 1) & (r_ - 1)) != 0) continue;
        const int cj = (key0 + g * PER + k) / r_;                  // block index
        const bool visible = max(0, r_ * cj - ov_) < n_vis;        // first overlapping summary
        if (out && cj < p.imp_cols) out[cj] = visible ? accb : 0.f;
        float cv = visible ? accb : -1.f;
        if (forcing && cj <= my_cur && t < p.T) {
          if (cj < p.n_init) cv = kForcedInit - (float)cj;
          else if (cj > my_cur - p.n_local) cv = kForcedLocal - (float)(my_cur - cj);
        }
        if (cv > lv[kList - 1] && cv >= tau) {   // beats the list's last entry (empty slots hold -1)
#pragma unroll
          for (int r = kList - 1; r >= 1; --r) {   // strict '>' keeps earlier (lower) indices ahead
            const bool up = cv > lv[r - 1];
            const bool here = cv > lv[r];
            li[r] = up ? li[r - 1] : (here ? cj : li[r]);
            lv[r] = up ? lv[r - 1] : (here ? cv : lv[r]);
          }
          if (cv > lv[0]) { lv[0] = cv; li[0] = cj; }
        }
      }
    }
    if (!aborted) aborted = __syncthreads_or(*s_abort) != 0;
    if (aborted) {
      // Give-up path: no list is written.  Thread 0 waits (bounded) for the loads still on their
      // way into this CTA's shared memory and for the MMAs already issued, then the tensor memory
      // goes back.
      if (tid == 0) {
        if (!q_seen) mbar_wait_drain(bar_q, 0);
        for (int j = k_seen; j < k_loaded; ++j) mbar_wait_drain(bar_k + (j & 1), (j >> 1) & 1);
        tc_commit(bar_drain);
        mbar_wait_drain(bar_drain, 0);
      }
      tc_fence_before();
      __syncthreads();
      if (warp == 0) tmem_dealloc(tmem, kTmemCols);
      return;
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, kTmemCols);
  }

  // ---- merge the GP lists of each query: n_sel rounds, each takes the best head ------------------
  for (int r = 0; r < p.n_sel; ++r) {
    float bv = lv[0];
    int bj = li[0];
#pragma unroll
    for (int o = 1; o < GP; o <<= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oj = __shfl_xor_sync(0xffffffffu, bj, o);
      if (ov > bv || (ov == bv && oj >= 0 && (bj < 0 || oj < bj))) { bv = ov; bj = oj; }
    }
    if (bj >= 0 && li[0] == bj) {            // this list gave the winner: pop its head
#pragma unroll
      for (int k = 0; k < kList - 1; ++k) { lv[k] = lv[k + 1]; li[k] = li[k + 1]; }
      lv[kList - 1] = -1.f;
      li[kList - 1] = -1;
    }
    if (g == 0 && t < p.T) p.block_idx[((size_t)bh * p.T + t) * p.n_sel + r] = bj;
  }
  // importance columns no tile covered are zero
  if (p.imp_out && t < p.T) {
    float* out = p.imp_out + ((size_t)bh * p.T + t) * p.imp_cols;
    for (int c = n_tiles * kKeys / (kAligned ? 1 : p.r) + g; c < p.imp_cols; c += GP) out[c] = 0.f;
  }
}

__host__ inline size_t score_lanes_smem_bytes(int D) {
  return (size_t)(kRows * 128 + 2 * kKeys * 128) * (D / 64) + 256 + 1024;
}

template <int D, int GP>
static int launch_score_lanes(const void* q, const void* k_cmp, const NsaDims& d, int n_blk, ScoreArgs p,
                              cudaStream_t st) {
  p.nq = kRows / GP;
  p.n_qtiles = (d.T + p.nq - 1) / p.nq;
  CUtensorMap tm_q, tm_k;
  int rc = make_map_query_rows(&tm_q, q, d.D, d.T, d.B * d.Hq, GP, p.nq);
  if (rc == NSA_OK) rc = make_map(&tm_k, k_cmp, d.D, n_blk, d.B * d.Hkv, kKeys, 1);
  if (rc != NSA_OK) return rc;
  const size_t smem = score_lanes_smem_bytes(d.D);
  KernelScope ks("tc_score_topn", st);
  if (p.r == 1 && p.overlap == 0) {
    NSA_CUDA_OK(cudaFuncSetAttribute(tc_score_lanes_kernel<D, GP, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    tc_score_lanes_kernel<D, GP, true><<<dim3(p.n_qtiles, d.B * d.Hkv), 128, smem, st>>>(tm_q, tm_k, p);
  } else {
    NSA_CUDA_OK(cudaFuncSetAttribute(tc_score_lanes_kernel<D, GP, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    tc_score_lanes_kernel<D, GP, false><<<dim3(p.n_qtiles, d.B * d.Hkv), 128, smem, st>>>(tm_q, tm_k, p);
  }
  return NSA_OK;
}

}  // namespace tc

bool tc_topn_ok(const NsaDims& d, int n_blk, int n_sel, int cmp_len, int stride, int sel_block) {
  if (d.dtype != NSA_DTYPE_BF16 || (d.D != 64 && d.D != 128)) return false;
  if (n_sel < 1 || n_sel > 16 || n_blk < 1) return false;
  const int G = d.Hq / d.Hkv;
  if (G > 32) return false;   // at least 4 queries per tile, so the lanes of one query sit in one warp
  if (cmp_len == stride && stride == sel_block) return true;
  // summaries and selection blocks on different grids: the lane-exchange kernel only
  const int gp = tc::group_pad(G);
  if (gp != 4 && gp != 8 && gp != 16) return false;
  if (stride <= 0 || sel_block % stride || cmp_len % stride) return false;
  const int r = sel_block / stride, o = cmp_len / stride;
  return (r & (r - 1)) == 0 && r <= tc::kKeys / gp && (o == 1 || o == 2);
}

int tc_topn(const void* q, const void* k_cmp, const float* lse, int32_t* block_idx, float* imp_out,
            const NsaDims& d, int n_blk, int block_size, int n_sel, int n_init, int n_local, int stride,
            int sel_block, int imp_cols, cudaStream_t st) {
  using namespace tc;
  ScoreArgs p;
  p.lse = lse; p.block_idx = block_idx; p.imp_out = imp_out;
  p.status = device_status_ptr();
  if (!p.status) { set_error("device status word unavailable"); return NSA_ERR_CUDA; }
  p.B = d.B; p.Hq = d.Hq; p.Hkv = d.Hkv; p.T = d.T; p.n_blk = n_blk;
  p.G = d.Hq / d.Hkv; p.Gp = group_pad(p.G); p.nq = kRows / p.Gp;
  p.block_size = block_size; p.n_sel = n_sel; p.n_init = n_init; p.n_local = n_local;
  p.stride = stride; p.sel_block = sel_block; p.r = sel_block / stride;
  p.overlap = block_size / stride - 1; p.imp_cols = imp_cols;
  p.n_qtiles = (d.T + p.nq - 1) / p.nq;
  p.scale_log2 = kLog2e / sqrtf((float)d.D);
  if (p.Gp == 4 || p.Gp == 8 || p.Gp == 16) {
    int rc = NSA_ERR_UNSUPPORTED;
    if (d.D == 128) rc = p.Gp == 4 ? launch_score_lanes<128, 4>(q, k_cmp, d, n_blk, p, st)
                       : p.Gp == 8 ? launch_score_lanes<128, 8>(q, k_cmp, d, n_blk, p, st)
                                   : launch_score_lanes<128, 16>(q, k_cmp, d, n_blk, p, st);
    else rc = p.Gp == 4 ? launch_score_lanes<64, 4>(q, k_cmp, d, n_blk, p, st)
            : p.Gp == 8 ? launch_score_lanes<64, 8>(q, k_cmp, d, n_blk, p, st)
                        : launch_score_lanes<64, 16>(q, k_cmp, d, n_blk, p, st);
    if (rc != NSA_OK) return rc;
    NSA_LAUNCH_OK("tc_score_lanes_kernel");
    return NSA_OK;
  }
  CUtensorMap tm_q, tm_k;
  int rc = make_map(&tm_q, q, d.D, d.T, d.B * d.Hq, p.nq, p.Gp);
  if (rc == NSA_OK) rc = make_map(&tm_k, k_cmp, d.D, n_blk, d.B * d.Hkv, kKeys, 1);
  if (rc != NSA_OK) return rc;
  const size_t smem = score_smem_bytes(d.D, p.nq);
  dim3 grid(p.n_qtiles, d.B * d.Hkv);
  if (d.D == 128) {
    NSA_CUDA_OK(cudaFuncSetAttribute(tc_score_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    KernelScope ks("tc_score_topn", st);
    tc_score_kernel<128><<<grid, 128, smem, st>>>(tm_q, tm_k, p);
  } else {
    NSA_CUDA_OK(cudaFuncSetAttribute(tc_score_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    KernelScope ks("tc_score_topn", st);
    tc_score_kernel<64><<<grid, 128, smem, st>>>(tm_q, tm_k, p);
  }
  NSA_LAUNCH_OK("tc_score_kernel");
  return NSA_OK;
}

}  // namespace nsa
