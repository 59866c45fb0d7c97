// tcgen05 / TMEM attention kernels for sm_100a.
//
// One CTA owns a tile of 128 rows = nq consecutive query tokens x the Gp query heads of one
// (batch, kv head) group (row r -> head r / nq, token r % nq), so the heads of a GQA group
// share every K/V tile.  The CTA walks a list of 64-key tiles:
//   window      the tiles covering [t_first - W + 1, t_last]
//   compression the tiles covering summaries [0, (t_last + 1) / Bsz - 1]
//   selection   the union of the 64-token blocks listed for the tile's nq queries, built in
//               shared memory, with a per-(query, block) membership bit
// Per tile: a TMA warp brings K and V (128B-swizzled boxes) into a 2-stage ring; an MMA warp
// issues S = Q K^T (tcgen05.mma, Q held in TMEM as the A operand, accumulator in TMEM); each of
// the 128 softmax threads owns one row of S (tcgen05.ld, lane = row), masks it, runs the online
// softmax in the log2 domain without any cross-thread traffic and writes P as packed bf16 over S
// in TMEM (tcgen05.st); the MMA warp then issues O += P V with P as the TMEM A operand and V as
// an MN-major shared-memory B operand.  The running maximum is only raised when it grows by more
// than 8 (log2 units), so the O accumulator in TMEM is rescaled rarely.
// tc_fwd_kernel takes one row tile per CTA (query-outer selection); tc_fwd_range_kernel is the
// persistent form for window and compression.
#include "tc_common.cuh"
#include "tc_host.cuh"

namespace nsa {
namespace tc {

struct FwdArgs {
  const int32_t* block_idx;
  __nv_bfloat16* o;
  float* lse;
  int* status;
  int B, Hq, Hkv, T, Lk, S, G, Gp, nq;
  int kind, window, block_size;
  const unsigned long long* stats;   // selection: statistics for the variant choice (may be null)
  const int32_t* offsets;            // selection: CSR offsets (pair count at the end)
  int force;
  int debug_starve;          // test only: the V load of the second key tile is never sent
  int n_qtiles, nb_sel;      // nb_sel = ceil(T / 64) blocks a selection list may name
  int nw;                    // 32-bit membership words per block = max(1, nq / 32)
  float scale_log2;
};

template <int D> struct FwdSmem {
  static constexpr int kSlabs = D / 64;
  static constexpr int kQBytes = kRows * 128 * kSlabs;
  static constexpr int kKVBytes = kKeys * 128 * kSlabs;
  static constexpr int kFixed = kQBytes + 4 * kKVBytes;   // Q + 2 K stages + 2 V stages
};

__host__ __device__ inline size_t fwd_smem_bytes(int D, int nb_sel, int nw, int kind) {
  size_t fixed = (size_t)(kRows * 128 + 4 * kKeys * 128) * (D / 64);
  size_t extra = 256 /*barriers etc*/ + 132 * 4 /*scan*/;
  if (kind == 2) extra += (size_t)nb_sel * nw * 4 + (size_t)nb_sel * 2 + 16;
  return fixed + extra + 1024 /*alignment slack*/;
}

// 192 threads in roles.  Warps 0-3 (thread = row = TMEM lane) own the softmax; warp 4 sends the
// TMA loads; warp 5 issues the MMAs.  With the issuing on a softmax warp, as an earlier version
// had it, every tile waited for that warp to get its TMA boxes and a dozen MMAs out between its
// own exponentials.  The Q tile is copied into tensor memory once per CTA, so S = Q K^T takes its
// A operand from there (an MMA of 128 x 64 x 16 that fetches both operands from shared memory is
// bound by that fetch, not by its arithmetic).  Two CTAs per SM.
constexpr int kFwdThreads = 192;
constexpr int kFwdSoftmax = 128;

template <int D>
__global__ void __launch_bounds__(kFwdThreads, 2)
tc_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
              const __grid_constant__ CUtensorMap tm_v, const FwdArgs p) {
  using L = FwdSmem<D>;
  constexpr int kSlabs = L::kSlabs;
  constexpr uint32_t kTmemCols = 256;
  // O in columns 0-127, S in 128-191 (P, bf16, is written over its first 32 columns by the thread
  // that read the row), the Q tile (bf16, D / 2 columns) in 192-255
  constexpr uint32_t kColO = 0, kColS = 128, kColQ = 192;
  constexpr uint32_t kIdescQK = idesc_bf16(128, kKeys, 0, 0);
  constexpr uint32_t kIdescPV = idesc_bf16(128, D, 0, 1);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);   // pointer arithmetic keeps the shared address space
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + L::kQBytes;
  uint8_t* sV = sK + 2 * L::kKVBytes;
  uint64_t* bars = (uint64_t*)(sV + 2 * L::kKVBytes);
  uint64_t* bar_q = bars + 0;        // Q tile landed (TMA bytes)
  uint64_t* bar_k = bars + 1;        // [2] K stage landed
  uint64_t* bar_v = bars + 3;        // [2] V stage landed
  uint64_t* k_free = bars + 5;       // [2] the S MMA that read the stage is done
  uint64_t* v_free = bars + 7;       // [2] the PV MMA that read the stage is done
  uint64_t* bar_s = bars + 9;        // S of a tile is in tensor memory
  uint64_t* bar_p = bars + 10;       // the 128 rows of P are written (and S is read)
  uint64_t* bar_o = bars + 11;       // PV of a tile is done
  uint64_t* bar_qt = bars + 12;      // the 128 rows of Q are in tensor memory
  uint64_t* bar_drain = bars + 13;   // an aborted CTA waits here for its last MMAs
  uint32_t* s_tmem = (uint32_t*)(bars + 14);
  volatile int* s_abort = (volatile int*)(s_tmem + 1);
  int* s_ntiles = (int*)(s_tmem + 2);
  int* s_scan = (int*)(s_tmem + 4);                 // [129]
  uint32_t* s_member = (uint32_t*)(s_scan + 132);   // [nb_sel * nw]   (selection only)
  uint16_t* s_tiles = (uint16_t*)(s_member + (p.kind == 2 ? p.nb_sel * p.nw : 0));

  if (p.kind == 2 && p.stats != nullptr &&
      prefer_pairs(p.stats, p.offsets, p.B * p.Hkv, p.nb_sel, p.nq, p.force))
    return;   // the block-outer variant serves this call: leave before anything is set up
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int qtile = p.n_qtiles - 1 - (int)blockIdx.x;   // long rows first
  const int bh = blockIdx.y;
  const int b = bh / p.Hkv, hkv = bh % p.Hkv;
  const int t0 = qtile * p.nq;
  const int t_last = min(p.T - 1, t0 + p.nq - 1);
  // softmax threads: row of the tile = thread index
  const int row = tid & (kFwdSoftmax - 1);
  const int g = row / p.nq, ql = row % p.nq;
  const int t = t0 + ql;
  const bool row_ok = tid < kFwdSoftmax && (g < p.G) && (t < p.T);
  const int head = hkv * p.G + g;

  if (tid == 0) {
    *s_abort = (*(volatile int*)p.status != 0) ? 1 : 0;
    mbar_init(bar_q, 1);
    for (int k = 1; k <= 8; ++k) mbar_init(bars + k, 1);
    mbar_init(bar_s, 1);
    mbar_init(bar_p, kFwdSoftmax);
    mbar_init(bar_o, 1);
    mbar_init(bar_qt, kFwdSoftmax);
    mbar_init(bar_drain, 1);
    fence_barrier_init();
    prefetch_tensormap(&tm_q); prefetch_tensormap(&tm_k); prefetch_tensormap(&tm_v);
  }
  __syncthreads();
  if (*s_abort) return;

  // ---- tile list ------------------------------------------------------------------------
  int n_tiles = 0, first_key = 0;
  if (p.kind == 0) {
    first_key = max(0, t0 - p.window + 1) & ~(kKeys - 1);
    n_tiles = (min(t_last, p.Lk - 1) - first_key) / kKeys + 1;
  } else if (p.kind == 1) {
    const int hi_last = cmp_visible(t_last, p.block_size, p.window, p.Lk) - 1;   // window: the stride
    n_tiles = hi_last < 0 ? 0 : hi_last / kKeys + 1;
  } else {
    const int nmem = p.nb_sel * p.nw;
    for (int i = tid; i < nmem; i += kFwdThreads) s_member[i] = 0u;
    __syncthreads();
    const int32_t* idx = p.block_idx + ((size_t)bh * p.T + t0) * p.S;
    const int n_entries = (t_last - t0 + 1) * p.S;
    for (int e = tid; e < n_entries; e += kFwdThreads) {
      const int q_local = e / p.S;
      const int blk = __ldg(idx + e);
      if (blk >= 0 && blk < p.nb_sel && blk * kKeys <= t0 + q_local)
        atomicOr(&s_member[blk * p.nw + (q_local >> 5)], 1u << (q_local & 31));
    }
    __syncthreads();
    const int per = (p.nb_sel + 127) / 128;       // the first 128 threads scan `per` blocks each
    const int j0 = tid < 128 ? tid * per : p.nb_sel, j1 = min(p.nb_sel, j0 + per);
    int cnt = 0;
    for (int j = j0; j < j1; ++j) {
      uint32_t any = 0;
      for (int w = 0; w < p.nw; ++w) any |= s_member[j * p.nw + w];
      cnt += any != 0;
    }
    if (tid < 128) s_scan[tid + 1] = cnt;
    __syncthreads();
    if (tid == 0) {
      s_scan[0] = 0;
      for (int i = 1; i <= 128; ++i) s_scan[i] += s_scan[i - 1];
      *s_ntiles = s_scan[128];
    }
    __syncthreads();
    int pos = tid < 128 ? s_scan[tid] : 0;
    for (int j = j0; j < j1; ++j) {
      uint32_t any = 0;
      for (int w = 0; w < p.nw; ++w) any |= s_member[j * p.nw + w];
      if (any) s_tiles[pos++] = (uint16_t)j;
    }
    __syncthreads();
    n_tiles = *s_ntiles;
  }

  float m_used = -INFINITY, l_sum = 0.f;
  __nv_bfloat16* orow = p.o + ((size_t)(b * p.Hq + head) * p.T + t) * D;
  if (n_tiles == 0) {                       // (uniform over the CTA) rows without a key: zeros
    if (row_ok) {
      uint4* dst = reinterpret_cast<uint4*>(orow);
#pragma unroll
      for (int v4 = 0; v4 < D / 8; ++v4) dst[v4] = make_uint4(0, 0, 0, 0);
      p.lse[(size_t)(b * p.Hq + head) * p.T + t] = kLseEmpty;
    }
    return;
  }

  // ---- TMEM ---------------------------------------------------------------------------
  if (warp == 0) {
    tmem_alloc(s_tmem, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *s_tmem;
  const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
  auto key0_of = [&](int i) -> int {
    if (p.kind == 2) return (int)s_tiles[i] * kKeys;
    return first_key + i * kKeys;
  };
  int last_k[2] = {-1, -1}, last_v[2] = {-1, -1};   // producer: last tile sent into each stage

  if (warp == 4) {
    // ---- producer -------------------------------------------------------------------------
    if (lane == 0) {
      auto load_k = [&](int i) {
        uint64_t* bar = bar_k + (i & 1);
        mbar_expect_tx(bar, L::kKVBytes);
#pragma unroll
        for (int s = 0; s < kSlabs; ++s)
          tma_load_3d(sK + (i & 1) * L::kKVBytes + s * (kKeys * 128), &tm_k, bar, s * 64, key0_of(i), bh);
        last_k[i & 1] = i;
      };
      auto load_v = [&](int i) {
        uint64_t* bar = bar_v + (i & 1);
        if (p.debug_starve && i == 1) return;   // test only: this tile's wait has to run out
        mbar_expect_tx(bar, L::kKVBytes);
#pragma unroll
        for (int s = 0; s < kSlabs; ++s)
          tma_load_3d(sV + (i & 1) * L::kKVBytes + s * (kKeys * 128), &tm_v, bar, s * 64, key0_of(i), bh);
        last_v[i & 1] = i;
      };
      mbar_expect_tx(bar_q, L::kQBytes);
#pragma unroll
      for (int s = 0; s < kSlabs; ++s)
        tma_load_3d(sQ + s * (kRows * 128), &tm_q, bar_q, s * 64, t0, b * p.Hq + hkv * p.G);
      load_k(0);
      load_v(0);
      if (n_tiles > 1) { load_k(1); load_v(1); }
      for (int i = 0; i + 2 < n_tiles; ++i) {
        // stage i & 1 is free once the MMAs of tile i that read it are done (a barrier per stage:
        // its next completion needs the very load that waits here, so no phase can be missed)
        if (!mbar_wait(k_free + (i & 1), (i >> 1) & 1, p.status, s_abort, 0x4000)) break;
        load_k(i + 2);
        if (!mbar_wait(v_free + (i & 1), (i >> 1) & 1, p.status, s_abort, 0x4000)) break;
        load_v(i + 2);
      }
    }
  } else if (warp == 5) {
    // ---- MMA issuer ------------------------------------------------------------------------
    if (lane == 0) {
      auto issue_s = [&](int i) {   // S = Q K^T for tile i, Q from tensor memory
        const uint32_t ka = desc_lo_kmajor(smem_u32(sK + (i & 1) * L::kKVBytes));
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t slab = kk >> 2, in = (kk & 3) * 32;
          mma_ts(tmem + kColS, tmem + kColQ + kk * 8, desc_at(ka, slab * (kKeys * 128) + in), kIdescQK, kk > 0);
        }
        tc_commit(bar_s);
        tc_commit(k_free + (i & 1));
      };
      auto issue_pv = [&](int i) {  // O (+)= P V for tile i
        const uint32_t va = desc_lo_mnmajor(smem_u32(sV + (i & 1) * L::kKVBytes), kKeys * 128);
#pragma unroll
        for (int kk = 0; kk < kKeys / 16; ++kk)
          mma_ts(tmem + kColO, tmem + kColS + kk * 8, desc_at(va, kk * 2048), kIdescPV, (i > 0) || (kk > 0));
        tc_commit(bar_o);
        tc_commit(v_free + (i & 1));
      };
      bool ok = mbar_wait(bar_qt, 0, p.status, s_abort, 0x8000) &&
                mbar_wait(bar_k, 0, p.status, s_abort, 2);
      if (ok) {
        tc_fence_after();
        issue_s(0);
      }
      for (int i = 0; ok && i < n_tiles; ++i) {
        ok = mbar_wait(bar_p, i & 1, p.status, s_abort, 0x2000) &&
             mbar_wait(bar_v + (i & 1), (i >> 1) & 1, p.status, s_abort, 16);
        if (!ok) break;
        tc_fence_after();
        issue_pv(i);
        if (i + 1 < n_tiles) {
          // S of the next tile overwrites P of this one: the tensor pipe keeps the order
          ok = mbar_wait(bar_k + ((i + 1) & 1), ((i + 1) >> 1) & 1, p.status, s_abort, 2);
          if (ok) issue_s(i + 1);
        }
      }
      // the tensor pipe is idle before tensor memory is read for the output and given back
      tc_commit(bar_drain);
      if (!mbar_wait(bar_drain, 0, p.status, s_abort, 0x1000)) mbar_wait_drain(bar_drain, 0);
    }
  } else {
    // ---- softmax: thread = row ---------------------------------------------------------------
    // Q: shared memory -> tensor memory, every thread its row
    bool ok = mbar_wait(bar_q, 0, p.status, s_abort, 1);
    {
#pragma unroll
      for (int sl = 0; sl < kSlabs; ++sl) {
        const uint8_t* src = sQ + sl * (kRows * 128) + row * 128;
        uint32_t qv[32];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint4 u = *reinterpret_cast<const uint4*>(src + ((c ^ (row & 7)) << 4));
          qv[4 * c + 0] = u.x; qv[4 * c + 1] = u.y; qv[4 * c + 2] = u.z; qv[4 * c + 3] = u.w;
        }
        tmem_st32(lane_base + kColQ + sl * 32, qv);
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(bar_qt);
    }
    for (int i = 0; i < n_tiles; ++i) {
      const int key0 = key0_of(i);
      ok = mbar_wait(bar_s, i & 1, p.status, s_abort, 4) && ok;
      if (!__all_sync(0xffffffffu, ok)) break;              // the whole warp leaves together
      tc_fence_after();
      uint32_t r[64];
      tmem_ld32(lane_base + kColS, r);
      tmem_ld32(lane_base + kColS + 32, r + 32);
      tmem_wait_ld();

      // valid columns of this row in this tile form one range [lo, hi]
      int lo = 0, hi = -1;
      if (row_ok) {
        if (p.kind == 0) {
          lo = max(0, t - p.window + 1 - key0);
          hi = min(kKeys - 1, t - key0);
        } else if (p.kind == 1) {
          hi = min(kKeys - 1, cmp_visible(t, p.block_size, p.window, p.Lk) - 1 - key0);
        } else {
          const uint32_t w = s_member[(key0 / kKeys) * p.nw + (ql >> 5)];
          if ((w >> (ql & 31)) & 1u) hi = min(kKeys - 1, t - key0);
        }
      }
      float x[64];
      float tmax = -INFINITY;
      if (lo <= 0 && hi >= kKeys - 1) {
#pragma unroll
        for (int c = 0; c < 64; ++c) {
          x[c] = __uint_as_float(r[c]) * p.scale_log2;
          tmax = fmaxf(tmax, x[c]);
        }
      } else {
#pragma unroll
        for (int c = 0; c < 64; ++c) {
          x[c] = (c >= lo && c <= hi) ? __uint_as_float(r[c]) * p.scale_log2 : -INFINITY;
          tmax = fmaxf(tmax, x[c]);
        }
      }
      float alpha = 1.f;
      bool rescale = false;
      if (tmax > m_used + 8.f) {              // also the first finite maximum (m_used = -inf)
        if (m_used != -INFINITY) {
          alpha = ex2(m_used - tmax);
          rescale = true;
          l_sum *= alpha;
        }
        m_used = tmax;
      }
      const float msub = (m_used == -INFINITY) ? 0.f : m_used;
      float psum = 0.f;
      uint32_t pk[32];
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        const float p0 = ex2(x[2 * c] - msub), p1 = ex2(x[2 * c + 1] - msub);
        psum += p0 + p1;
        pk[c] = pack_bf16(p0, p1);
      }
      l_sum += psum;

      // O may be touched once PV of tile i-1 is done; only a warp that has to rescale waits for it
      if (i > 0 && __any_sync(0xffffffffu, rescale)) {
        ok = mbar_wait(bar_o, (i - 1) & 1, p.status, s_abort, 8);
        if (!__all_sync(0xffffffffu, ok)) break;
        tc_fence_after();
#pragma unroll
        for (int cc = 0; cc < D / 32; ++cc) {
          uint32_t o32[32];
          tmem_ld32(lane_base + kColO + cc * 32, o32);
          tmem_wait_ld();
#pragma unroll
          for (int c = 0; c < 32; ++c) o32[c] = __float_as_uint(__uint_as_float(o32[c]) * alpha);
          tmem_st32(lane_base + kColO + cc * 32, o32);
        }
      }
      tmem_st32(lane_base + kColS, pk);        // over the S columns this thread has just read
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(bar_p);
    }
    // the last PV
    if (__all_sync(0xffffffffu, ok)) mbar_wait(bar_o, (n_tiles - 1) & 1, p.status, s_abort, 8);
  }

  // ---- teardown -------------------------------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (*s_abort) {
    // Give-up path: no output is written.  The producer waits (bounded) for the loads still on
    // their way into this CTA's shared memory; the MMA thread has waited for the tensor pipe
    // above; then the tensor memory goes back.
    if (warp == 4 && lane == 0) {
      mbar_wait_drain(bar_q, 0);
#pragma unroll
      for (int st = 0; st < 2; ++st) {
        if (last_k[st] >= 0) mbar_wait_drain(bar_k + st, (last_k[st] >> 1) & 1);
        if (last_v[st] >= 0) mbar_wait_drain(bar_v + st, (last_v[st] >> 1) & 1);
      }
    }
    if (warp == 5 && lane == 0) mbar_wait_drain(bar_drain, 0);
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, kTmemCols);
    return;
  }

  // ---- epilogue ---------------------------------------------------------------------------
  if (tid < kFwdSoftmax) {
    const float inv = l_sum > 0.f ? 1.f / l_sum : 0.f;
#pragma unroll
    for (int cc = 0; cc < D / 32; ++cc) {
      uint32_t o32[32];
      tmem_ld32(lane_base + kColO + cc * 32, o32);
      tmem_wait_ld();
      if (row_ok) {
        uint4* dst = reinterpret_cast<uint4*>(orow + cc * 32);
#pragma unroll
        for (int v4 = 0; v4 < 4; ++v4) {
          uint4 u;
          u.x = pack_bf16(__uint_as_float(o32[v4 * 8 + 0]) * inv, __uint_as_float(o32[v4 * 8 + 1]) * inv);
          u.y = pack_bf16(__uint_as_float(o32[v4 * 8 + 2]) * inv, __uint_as_float(o32[v4 * 8 + 3]) * inv);
          u.z = pack_bf16(__uint_as_float(o32[v4 * 8 + 4]) * inv, __uint_as_float(o32[v4 * 8 + 5]) * inv);
          u.w = pack_bf16(__uint_as_float(o32[v4 * 8 + 6]) * inv, __uint_as_float(o32[v4 * 8 + 7]) * inv);
          if (l_sum > 0.f) dst[v4] = u; else dst[v4] = make_uint4(0, 0, 0, 0);
        }
      }
    }
    if (row_ok)
      p.lse[(size_t)(b * p.Hq + head) * p.T + t] =
          l_sum > 0.f ? (m_used + log2f(l_sum)) * kLn2 : kLseEmpty;
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, kTmemCols);
}

// ---- window / compression forward as a persistent kernel ---------------------------------------
// The same roles and tensor-memory layout as tc_fwd_kernel, but a CTA walks many row tiles (tile
// w, w + gridDim.x, ...), so what a CTA per row tile pays between tiles -- barrier set-up, the
// tensor-memory allocation, the latency of the first Q / K / V loads, the tail of the epilogue --
// is paid once or hidden: the producer runs ahead into the next row tile (its Q lands in shared
// memory while this tile is worked on; the K / V ring never drains), a softmax thread moves its
// row of the next Q into tensor memory right after its last P of this tile, and the next tile's
// first S is computed while the threads write this tile's output.  Every barrier's phase follows
// a running count (of row tiles, or of key tiles over all row tiles) that each role keeps itself.
template <int D>
__global__ void __launch_bounds__(kFwdThreads, 2)
tc_fwd_range_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                    const __grid_constant__ CUtensorMap tm_v, const FwdArgs p) {
  using L = FwdSmem<D>;
  constexpr int kSlabs = L::kSlabs;
  constexpr uint32_t kTmemCols = 256;
  constexpr uint32_t kColO = 0, kColS = 128, kColQ = 192;   // as in tc_fwd_kernel
  constexpr uint32_t kIdescQK = idesc_bf16(128, kKeys, 0, 0);
  constexpr uint32_t kIdescPV = idesc_bf16(128, D, 0, 1);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + L::kQBytes;
  uint8_t* sV = sK + 2 * L::kKVBytes;
  uint64_t* bars = (uint64_t*)(sV + 2 * L::kKVBytes);
  uint64_t* bar_q = bars + 0;        // Q tile landed (TMA bytes); phase = row tile count
  uint64_t* bar_k = bars + 1;        // [2] K stage landed; phase = (key tile count) >> 1
  uint64_t* bar_v = bars + 3;        // [2] V stage landed
  uint64_t* k_free = bars + 5;       // [2] the S MMA that read the stage is done
  uint64_t* v_free = bars + 7;       // [2] the PV MMA that read the stage is done
  uint64_t* bar_s = bars + 9;        // S of a key tile is in tensor memory; phase = key tile count
  uint64_t* bar_p = bars + 10;       // the 128 rows of P are written (and S is read)
  uint64_t* bar_o = bars + 11;       // PV of a key tile is done
  uint64_t* bar_qt = bars + 12;      // the 128 rows of Q are in tensor memory (and its shared-memory tile is free)
  uint64_t* bar_drain = bars + 13;
  uint32_t* s_tmem = (uint32_t*)(bars + 14);
  volatile int* s_abort = (volatile int*)(s_tmem + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    *s_abort = (*(volatile int*)p.status != 0) ? 1 : 0;
    mbar_init(bar_q, 1);
    for (int k = 1; k <= 8; ++k) mbar_init(bars + k, 1);
    mbar_init(bar_s, 1);
    mbar_init(bar_p, kFwdSoftmax);
    mbar_init(bar_o, 1);
    mbar_init(bar_qt, kFwdSoftmax);
    mbar_init(bar_drain, 1);
    fence_barrier_init();
    prefetch_tensormap(&tm_q); prefetch_tensormap(&tm_k); prefetch_tensormap(&tm_v);
  }
  __syncthreads();
  if (*s_abort) return;
  if (warp == 0) {
    tmem_alloc(s_tmem, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *s_tmem;

  // row tile w of the launch: long rows first, the units of one token range next to each other
  const int units = p.B * p.Hkv;
  const int n_work = p.n_qtiles * units;
  struct Tile { int bh, t0, t_last, first_key, n_tiles; };
  auto tile_of = [&](int w) -> Tile {
    Tile x;
    x.bh = w % units;
    const int qtile = p.n_qtiles - 1 - w / units;
    x.t0 = qtile * p.nq;
    x.t_last = min(p.T - 1, x.t0 + p.nq - 1);
    if (p.kind == 0) {
      x.first_key = max(0, x.t0 - p.window + 1) & ~(kKeys - 1);
      x.n_tiles = (min(x.t_last, p.Lk - 1) - x.first_key) / kKeys + 1;
    } else {
      x.first_key = 0;
      const int hi_last = cmp_visible(x.t_last, p.block_size, p.window, p.Lk) - 1;   // window: the stride
      x.n_tiles = hi_last < 0 ? 0 : hi_last / kKeys + 1;
    }
    return x;
  };
  int last_k[2] = {-1, -1}, last_v[2] = {-1, -1};   // producer: running index of the last tile sent into each stage
  int q_sent = 0;                                   // producer: row tiles whose Q was sent

  if (warp == 4) {
    // ---- producer -------------------------------------------------------------------------
    if (lane == 0) {
      int c = 0, it = 0;                              // running key tile / live row tile counts
      bool ok = true;
      for (int w = blockIdx.x; ok && w < n_work; w += gridDim.x) {
        const Tile x = tile_of(w);
        if (x.n_tiles == 0) continue;
        const int b = x.bh / p.Hkv, hkv = x.bh % p.Hkv;
        // the Q tile in shared memory is free once every row of the previous one is in tensor memory
        if (it > 0) ok = mbar_wait(bar_qt, (it - 1) & 1, p.status, s_abort, 0x8000);
        if (!ok) break;
        mbar_expect_tx(bar_q, L::kQBytes);
#pragma unroll
        for (int s = 0; s < kSlabs; ++s)
          tma_load_3d(sQ + s * (kRows * 128), &tm_q, bar_q, s * 64, x.t0, b * p.Hq + hkv * p.G);
        q_sent = it + 1;
        for (int i = 0; i < x.n_tiles; ++i, ++c) {
          const int st = c & 1;
          // a stage is free once the MMAs of the tile two back, which read it, are done
          if (c >= 2) {
            ok = mbar_wait(k_free + st, ((c >> 1) - 1) & 1, p.status, s_abort, 0x4000);
            if (!ok) break;
          }
          mbar_expect_tx(bar_k + st, L::kKVBytes);
#pragma unroll
          for (int s = 0; s < kSlabs; ++s)
            tma_load_3d(sK + st * L::kKVBytes + s * (kKeys * 128), &tm_k, bar_k + st, s * 64,
                        x.first_key + i * kKeys, x.bh);
          last_k[st] = c;
          if (c >= 2) {
            ok = mbar_wait(v_free + st, ((c >> 1) - 1) & 1, p.status, s_abort, 0x4000);
            if (!ok) break;
          }
          if (!(p.debug_starve && c == 1)) {           // test only: this tile's wait has to run out
            mbar_expect_tx(bar_v + st, L::kKVBytes);
#pragma unroll
            for (int s = 0; s < kSlabs; ++s)
              tma_load_3d(sV + st * L::kKVBytes + s * (kKeys * 128), &tm_v, bar_v + st, s * 64,
                          x.first_key + i * kKeys, x.bh);
            last_v[st] = c;
          }
        }
        ++it;
      }
    }
  } else if (warp == 5) {
    // ---- MMA issuer ------------------------------------------------------------------------
    if (lane == 0) {
      int c = 0, it = 0;
      bool ok = true;
      auto issue_s = [&](int cc) {   // S = Q K^T for running key tile cc, Q from tensor memory
        const uint32_t ka = desc_lo_kmajor(smem_u32(sK + (cc & 1) * L::kKVBytes));
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t slab = kk >> 2, in = (kk & 3) * 32;
          mma_ts(tmem + kColS, tmem + kColQ + kk * 8, desc_at(ka, slab * (kKeys * 128) + in), kIdescQK, kk > 0);
        }
        tc_commit(bar_s);
        tc_commit(k_free + (cc & 1));
      };
      for (int w = blockIdx.x; ok && w < n_work; w += gridDim.x) {
        const Tile x = tile_of(w);
        if (x.n_tiles == 0) continue;
        ok = mbar_wait(bar_qt, it & 1, p.status, s_abort, 0x8000) &&
             mbar_wait(bar_k + (c & 1), (c >> 1) & 1, p.status, s_abort, 2);
        if (!ok) break;
        tc_fence_after();
        issue_s(c);                                     // (after the last PV of the previous row tile: P lies over S)
        for (int i = 0; i < x.n_tiles; ++i, ++c) {
          ok = mbar_wait(bar_p, c & 1, p.status, s_abort, 0x2000) &&
               mbar_wait(bar_v + (c & 1), (c >> 1) & 1, p.status, s_abort, 16);
          if (!ok) break;
          tc_fence_after();
          {                                             // O (+)= P V
            const uint32_t va = desc_lo_mnmajor(smem_u32(sV + (c & 1) * L::kKVBytes), kKeys * 128);
#pragma unroll
            for (int kk = 0; kk < kKeys / 16; ++kk)
              mma_ts(tmem + kColO, tmem + kColS + kk * 8, desc_at(va, kk * 2048), kIdescPV, (i > 0) || (kk > 0));
            tc_commit(bar_o);
            tc_commit(v_free + (c & 1));
          }
          if (i + 1 < x.n_tiles) {
            ok = mbar_wait(bar_k + ((c + 1) & 1), ((c + 1) >> 1) & 1, p.status, s_abort, 2);
            if (!ok) break;
            issue_s(c + 1);
          }
        }
        ++it;
      }
      tc_commit(bar_drain);
      if (!mbar_wait(bar_drain, 0, p.status, s_abort, 0x1000)) mbar_wait_drain(bar_drain, 0);
    }
  } else {
    // ---- softmax: thread = row ---------------------------------------------------------------
    const int row = tid;
    const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);
    const int g = row / p.nq, ql = row % p.nq;
    auto q_to_tmem = [&]() {       // this thread's row of the Q tile: shared memory -> tensor memory
#pragma unroll
      for (int sl = 0; sl < kSlabs; ++sl) {
        const uint8_t* src = sQ + sl * (kRows * 128) + row * 128;
        uint32_t qv[32];
#pragma unroll
        for (int cch = 0; cch < 8; ++cch) {
          const uint4 u = *reinterpret_cast<const uint4*>(src + ((cch ^ (row & 7)) << 4));
          qv[4 * cch + 0] = u.x; qv[4 * cch + 1] = u.y; qv[4 * cch + 2] = u.z; qv[4 * cch + 3] = u.w;
        }
        tmem_st32(lane_base + kColQ + sl * 32, qv);
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(bar_qt);
    };
    int c = 0, it = 0;
    bool ok = true;
    // the first live row tile's Q
    int w = blockIdx.x;
    Tile x = tile_of(w < n_work ? w : 0);
    auto skip_empty = [&]() {      // rows without a key: zeros, no barrier is touched
      while (w < n_work && x.n_tiles == 0) {
        const int t = x.t0 + ql;
        if (g < p.G && t < p.T) {
          const int head = (x.bh % p.Hkv) * p.G + g, b = x.bh / p.Hkv;
          uint4* dst = reinterpret_cast<uint4*>(p.o + ((size_t)(b * p.Hq + head) * p.T + t) * D);
#pragma unroll
          for (int v4 = 0; v4 < D / 8; ++v4) dst[v4] = make_uint4(0, 0, 0, 0);
          p.lse[(size_t)(b * p.Hq + head) * p.T + t] = kLseEmpty;
        }
        w += gridDim.x;
        if (w < n_work) x = tile_of(w);
      }
    };
    skip_empty();
    if (w < n_work) {
      ok = mbar_wait(bar_q, 0, p.status, s_abort, 1);
      q_to_tmem();
    }
    while (w < n_work) {
      const int t = x.t0 + ql;
      const bool row_ok = (g < p.G) && (t < p.T);
      const int b = x.bh / p.Hkv, head = (x.bh % p.Hkv) * p.G + g;
      float m_used = -INFINITY, l_sum = 0.f;
      for (int i = 0; i < x.n_tiles; ++i, ++c) {
        const int key0 = x.first_key + i * kKeys;
        ok = mbar_wait(bar_s, c & 1, p.status, s_abort, 4) && ok;
        if (!__all_sync(0xffffffffu, ok)) break;              // the whole warp leaves together
        tc_fence_after();
        uint32_t r[64];
        tmem_ld32(lane_base + kColS, r);
        tmem_ld32(lane_base + kColS + 32, r + 32);
        tmem_wait_ld();
        int lo = 0, hi = -1;
        if (row_ok) {
          if (p.kind == 0) {
            lo = max(0, t - p.window + 1 - key0);
            hi = min(kKeys - 1, t - key0);
          } else {
            hi = min(kKeys - 1, cmp_visible(t, p.block_size, p.window, p.Lk) - 1 - key0);
          }
        }
        float xs[64];
        float tmax = -INFINITY;
        if (lo <= 0 && hi >= kKeys - 1) {
#pragma unroll
          for (int cc = 0; cc < 64; ++cc) {
            xs[cc] = __uint_as_float(r[cc]) * p.scale_log2;
            tmax = fmaxf(tmax, xs[cc]);
          }
        } else {
#pragma unroll
          for (int cc = 0; cc < 64; ++cc) {
            xs[cc] = (cc >= lo && cc <= hi) ? __uint_as_float(r[cc]) * p.scale_log2 : -INFINITY;
            tmax = fmaxf(tmax, xs[cc]);
          }
        }
        float alpha = 1.f;
        bool rescale = false;
        if (tmax > m_used + 8.f) {              // also the first finite maximum (m_used = -inf)
          if (m_used != -INFINITY) {
            alpha = ex2(m_used - tmax);
            rescale = true;
            l_sum *= alpha;
          }
          m_used = tmax;
        }
        const float msub = (m_used == -INFINITY) ? 0.f : m_used;
        float psum = 0.f;
        uint32_t pk[32];
#pragma unroll
        for (int cc = 0; cc < 32; ++cc) {
          const float p0 = ex2(xs[2 * cc] - msub), p1 = ex2(xs[2 * cc + 1] - msub);
          psum += p0 + p1;
          pk[cc] = pack_bf16(p0, p1);
        }
        l_sum += psum;
        // O may be touched once PV of the tile before is done; only a warp that has to rescale waits
        if (i > 0 && __any_sync(0xffffffffu, rescale)) {
          ok = mbar_wait(bar_o, (c - 1) & 1, p.status, s_abort, 8);
          if (!__all_sync(0xffffffffu, ok)) break;
          tc_fence_after();
#pragma unroll
          for (int cc = 0; cc < D / 32; ++cc) {
            uint32_t o32[32];
            tmem_ld32(lane_base + kColO + cc * 32, o32);
            tmem_wait_ld();
#pragma unroll
            for (int e = 0; e < 32; ++e) o32[e] = __float_as_uint(__uint_as_float(o32[e]) * alpha);
            tmem_st32(lane_base + kColO + cc * 32, o32);
          }
        }
        tmem_st32(lane_base + kColS, pk);        // over the S columns this thread has just read
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(bar_p);
      }
      if (!__all_sync(0xffffffffu, ok)) break;
      // next live row tile: its Q goes into tensor memory now (every S of this tile is done: the
      // last one was read above), so that its first S runs while this tile's output is written
      const int w_cur = w;
      const Tile x_cur = x;
      w += gridDim.x;
      if (w < n_work) x = tile_of(w);
      skip_empty();
      ++it;
      if (w < n_work) {
        ok = mbar_wait(bar_q, it & 1, p.status, s_abort, 1);
        if (!__all_sync(0xffffffffu, ok)) break;
        q_to_tmem();
      }
      (void)w_cur;
      // ---- this tile's output: the last PV, then O / l -------------------------------------
      ok = mbar_wait(bar_o, (c - 1) & 1, p.status, s_abort, 8);
      if (!__all_sync(0xffffffffu, ok)) break;
      tc_fence_after();
      {
        const float inv = l_sum > 0.f ? 1.f / l_sum : 0.f;
        __nv_bfloat16* orow = p.o + ((size_t)(b * p.Hq + head) * p.T + t) * D;
#pragma unroll
        for (int cc = 0; cc < D / 32; ++cc) {
          uint32_t o32[32];
          tmem_ld32(lane_base + kColO + cc * 32, o32);
          tmem_wait_ld();
          if (row_ok) {
            uint4* dst = reinterpret_cast<uint4*>(orow + cc * 32);
#pragma unroll
            for (int v4 = 0; v4 < 4; ++v4) {
              uint4 u;
              u.x = pack_bf16(__uint_as_float(o32[v4 * 8 + 0]) * inv, __uint_as_float(o32[v4 * 8 + 1]) * inv);
              u.y = pack_bf16(__uint_as_float(o32[v4 * 8 + 2]) * inv, __uint_as_float(o32[v4 * 8 + 3]) * inv);
              u.z = pack_bf16(__uint_as_float(o32[v4 * 8 + 4]) * inv, __uint_as_float(o32[v4 * 8 + 5]) * inv);
              u.w = pack_bf16(__uint_as_float(o32[v4 * 8 + 6]) * inv, __uint_as_float(o32[v4 * 8 + 7]) * inv);
              if (l_sum > 0.f) dst[v4] = u; else dst[v4] = make_uint4(0, 0, 0, 0);
            }
          }
        }
        if (row_ok)
          p.lse[(size_t)(b * p.Hq + head) * p.T + t] =
              l_sum > 0.f ? (m_used + log2f(l_sum)) * kLn2 : kLseEmpty;
        (void)x_cur;
      }
      tc_fence_before();     // the O columns are read: the next tile's first PV (behind this thread's next P) may overwrite them
    }
  }

  // ---- teardown -------------------------------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (*s_abort) {
    // Give-up path.  The producer waits (bounded) for the loads still on their way into this
    // CTA's shared memory; the MMA thread has waited for the tensor pipe above.
    if (warp == 4 && lane == 0) {
      if (q_sent > 0) mbar_wait_drain(bar_q, (q_sent - 1) & 1);
#pragma unroll
      for (int st = 0; st < 2; ++st) {
        if (last_k[st] >= 0) mbar_wait_drain(bar_k + st, (last_k[st] >> 1) & 1);
        if (last_v[st] >= 0) mbar_wait_drain(bar_v + st, (last_v[st] >> 1) & 1);
      }
    }
    if (warp == 5 && lane == 0) mbar_wait_drain(bar_drain, 0);
    __syncthreads();
  }
  if (warp == 0) tmem_dealloc(tmem, kTmemCols);
}

static const char* const kFwdNames[3] = {"tc_fwd_win", "tc_fwd_cmp", "tc_fwd_slc"};

}  // namespace tc

bool tc_shape_ok(const NsaDims& d, int block_size) {
  if (d.dtype != NSA_DTYPE_BF16) return false;
  if (d.D != 64 && d.D != 128) return false;
  if (block_size != tc::kKeys) return false;
  const int G = d.Hq / d.Hkv;
  if (G < 2 || G > 128) return false;   // the backward tiles hold at most 64 queries
  if (d.T < 1) return false;
  const int nq = tc::kRows / tc::group_pad(G);
  const int nb = (d.T + tc::kKeys - 1) / tc::kKeys;
  if (nb > 65535) return false;
  if (tc::fwd_smem_bytes(d.D, nb, nq >= 32 ? nq / 32 : 1, 2) > 112 * 1024) return false;
  return true;
}

int get_option_debug_starve_load();   // api.cu

static int launch_fwd(const AttnArgs& a, const unsigned long long* stats, const int32_t* offsets,
                      int force, cudaStream_t st) {
  using namespace tc;
  FwdArgs p;
  p.stats = stats; p.offsets = offsets; p.force = force;
  p.debug_starve = get_option_debug_starve_load();
  p.block_idx = a.block_idx;
  p.o = (__nv_bfloat16*)a.o;
  p.lse = a.lse;
  p.status = device_status_ptr();
  if (!p.status) { set_error("device status word unavailable"); return NSA_ERR_CUDA; }
  p.B = a.B; p.Hq = a.Hq; p.Hkv = a.Hkv; p.T = a.T; p.Lk = a.Lk; p.S = a.S;
  p.G = a.Hq / a.Hkv;
  p.Gp = group_pad(p.G);
  p.nq = kRows / p.Gp;
  p.kind = a.kind; p.window = a.window; p.block_size = a.block_size;
  p.n_qtiles = (a.T + p.nq - 1) / p.nq;
  p.nb_sel = (a.T + kKeys - 1) / kKeys;
  p.nw = p.nq >= 32 ? p.nq / 32 : 1;
  p.scale_log2 = a.scale * kLog2e;
  CUtensorMap tm_q, tm_k, tm_v;
  int rc = make_map(&tm_q, a.q, a.D, a.T, a.B * a.Hq, p.nq, p.Gp);
  if (rc == NSA_OK) rc = make_map(&tm_k, a.k, a.D, a.Lk, a.B * a.Hkv, kKeys, 1);
  if (rc == NSA_OK) rc = make_map(&tm_v, a.v, a.D, a.Lk, a.B * a.Hkv, kKeys, 1);
  if (rc != NSA_OK) return rc;
  const size_t smem = fwd_smem_bytes(a.D, p.nb_sel, p.nw, a.kind);
  if (a.kind != 2) {
    // window / compression: persistent CTAs, two per SM, each walking its share of the row tiles
    int dev = 0, sms = 0;
    NSA_CUDA_OK(cudaGetDevice(&dev));
    NSA_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const long long n_work = (long long)p.n_qtiles * a.B * a.Hkv;
    if (n_work == 0) return NSA_OK;
    const unsigned g1 = (unsigned)(n_work < 2LL * sms ? n_work : 2LL * sms);
    KernelScope ks(branch_name(kFwdNames, a.kind), st);
    if (a.D == 128) {
      NSA_CUDA_OK(cudaFuncSetAttribute(tc_fwd_range_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      tc_fwd_range_kernel<128><<<g1, kFwdThreads, smem, st>>>(tm_q, tm_k, tm_v, p);
    } else {
      NSA_CUDA_OK(cudaFuncSetAttribute(tc_fwd_range_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      tc_fwd_range_kernel<64><<<g1, kFwdThreads, smem, st>>>(tm_q, tm_k, tm_v, p);
    }
    NSA_LAUNCH_OK("tc_fwd_range_kernel");
    return NSA_OK;
  }
  dim3 grid(p.n_qtiles, a.B * a.Hkv);
  if (a.D == 128) {
    NSA_CUDA_OK(cudaFuncSetAttribute(tc_fwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    { KernelScope ks(branch_name(kFwdNames, a.kind), st); tc_fwd_kernel<128><<<grid, kFwdThreads, smem, st>>>(tm_q, tm_k, tm_v, p); }
  } else {
    NSA_CUDA_OK(cudaFuncSetAttribute(tc_fwd_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    { KernelScope ks(branch_name(kFwdNames, a.kind), st); tc_fwd_kernel<64><<<grid, kFwdThreads, smem, st>>>(tm_q, tm_k, tm_v, p); }
  }
  NSA_LAUNCH_OK("tc_fwd_kernel");
  return NSA_OK;
}

int tc_attn_fwd(const AttnArgs& a, cudaStream_t st) { return launch_fwd(a, nullptr, nullptr, 0, st); }

int tc_fwd_union_launch(const AttnArgs& a, const unsigned long long* stats, const int32_t* offsets,
                        int force, cudaStream_t st) {
  return launch_fwd(a, stats, offsets, force, st);
}

}  // namespace nsa
