// Selected-block attention forward, key-block outer ("split-K over blocks"): host side, the
// merge of the per-(query, block) partials, the statistics that pick the variant and the work list.
//
// When neighbouring queries list unrelated blocks, a query-outer tile wastes most of every MMA
// on rows that do not attend the block.  The block-outer kernel (tc_fwdpair2.cu) instead gives one
// CTA one 64-token block: K and V of the block are loaded once, the (query, head) rows that list
// the block are gathered from the block -> query CSR, 128 rows at a time, and for each row tile
//   S = Q K^T ,  p = exp2(s*scale*log2e - m) with m the row's maximum over this block,  O_part = P V
// are computed; O_part (bf16), m and the sum of p (fp32) are written per (pair, head).
// sel_combine_kernel merges the partials of each query: o = sum_j 2^(m_j-M) O_j / sum_j 2^(m_j-M) l_j.
// A small statistics kernel counts the distinct blocks per query tile; the launchers of both
// forward variants read it on the device and only the cheaper variant does the work.
#include "tc_common.cuh"
#include "tc_host.cuh"

namespace nsa {
namespace tc {

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
        const float2 st = __ldg(reinterpret_cast<const float2*>(ml + prow * 2));
        m[j] = st.x;
        l[j] = st.y;
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
      const uint32_t h[4] = {u[j].x, u[j].y, u[j].z, u[j].w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {                         // bf16 -> fp32 is a shift
        acc[2 * e] = fmaf(w, __uint_as_float(h[e] << 16), acc[2 * e]);
        acc[2 * e + 1] = fmaf(w, __uint_as_float(h[e] & 0xffff0000u), acc[2 * e + 1]);
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

// The index structures of a block list that the block-outer selection kernels walk: CSR
// (queries of each block), the pair's unit, the block offsets, the (query, slot) -> pair map and
// the work list.  Forward and backward lay them out the same way inside their workspaces, so a
// copy built once ("plan") can be dropped into either instead of building them again.
struct SelRegion { size_t qob, pbh, off, pos, work, total; };
SelRegion sel_region(size_t units, int n_ktiles, size_t cap_pairs, int nq) {
  SelRegion r;
  size_t off = 0;
  r.qob = off; off += align_up(cap_pairs * 4, 256);
  r.pbh = off; off += align_up(cap_pairs * 4, 256);
  r.off = off; off += align_up(units * (n_ktiles + 1) * 4, 256);
  r.pos = off; off += align_up(cap_pairs * 4, 256);
  r.work = off; off += align_up(sel_work_bytes(units, n_ktiles, cap_pairs, nq), 256);
  r.total = off;
  return r;
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
  pl.off_ml = off; off += align_up(pl.cap_pairs * G * 2 * 4, 256);
  pl.off_csr_ws = off; off += align_up(nsa_csr_workspace_bytes(a.B, a.Hkv, pl.n_ktiles * kKeys, a.S, kKeys), 256);
  const SelRegion r = sel_region(units, pl.n_ktiles, pl.cap_pairs, pl.nq);
  pl.off_qob = off + r.qob; pl.off_pbh = off + r.pbh; pl.off_off = off + r.off;
  pl.off_pos = off + r.pos; pl.off_work = off + r.work;
  pl.total = off + r.total;
  return pl;
}

}  // namespace tc

int build_csr_internal(const int32_t* block_idx, int B, int Hkv, int T, int S, int block_size,
                       int n_blk, int32_t* q_of_block, int32_t* block_offsets, int32_t* pair_bh,
                       int32_t* pair_of_slot, void* workspace, size_t workspace_bytes, cudaStream_t st);
int tc_fwd_union_launch(const AttnArgs& a, const unsigned long long* stats, const int32_t* offsets,
                        int force, cudaStream_t st);
int get_option_sel_fwd();
int tc_fwdpair_launch(const AttnArgs& a, const int32_t* q_of_block, const int32_t* offsets, void* o_part,
                       float* ml, const unsigned long long* stats, const void* work, int force, int nq,
                       int n_ktiles, int nq_union, size_t cap_pairs, unsigned grid, cudaStream_t st);

size_t tc_sel_fwd_workspace(const AttnArgs& a) { return tc::plan_pairs(a).total; }

// plan buffer: the region, then the scratch of the CSR build
size_t tc_sel_plan_bytes(const AttnArgs& a) {
  using namespace tc;
  const PairPlan pl = plan_pairs(a);
  const SelRegion r = sel_region((size_t)a.B * a.Hkv, pl.n_ktiles, pl.cap_pairs, pl.nq);
  return r.total + align_up(nsa_csr_workspace_bytes(a.B, a.Hkv, pl.n_ktiles * kKeys, a.S, kKeys), 256);
}

int tc_sel_plan_build(const AttnArgs& a, void* plan, size_t plan_bytes, cudaStream_t st) {
  using namespace tc;
  const PairPlan pl = plan_pairs(a);
  const size_t units = (size_t)a.B * a.Hkv;
  const SelRegion r = sel_region(units, pl.n_ktiles, pl.cap_pairs, pl.nq);
  if (!plan || plan_bytes < tc_sel_plan_bytes(a)) {
    set_error("selection plan buffer too small: need %zu bytes", tc_sel_plan_bytes(a));
    return NSA_ERR_WORKSPACE;
  }
  char* base = (char*)plan;
  int rc = build_csr_internal(a.block_idx, a.B, a.Hkv, a.T, a.S, kKeys, pl.n_ktiles, (int32_t*)(base + r.qob),
                              (int32_t*)(base + r.off), (int32_t*)(base + r.pbh), (int32_t*)(base + r.pos),
                              base + r.total, plan_bytes - r.total, st);
  if (rc != NSA_OK) return rc;
  return sel_build_worklist((const int32_t*)(base + r.off), pl.n_ktiles, units, pl.cap_pairs, pl.nq, base + r.work, st);
}

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
  int rc = NSA_OK;
  if (a.sel_plan) {      // built earlier for this block list: one copy instead of the build
    NSA_CUDA_OK(cudaMemcpyAsync(base + pl.off_qob, a.sel_plan, pl.total - pl.off_qob, cudaMemcpyDeviceToDevice, st));
  } else {
    rc = build_csr_internal(a.block_idx, a.B, a.Hkv, a.T, a.S, kKeys, pl.n_ktiles,
                            (int32_t*)(base + pl.off_qob), offsets, (int32_t*)(base + pl.off_pbh),
                            pair_of_slot, base + pl.off_csr_ws, pl.off_qob - pl.off_csr_ws, st);
    if (rc != NSA_OK) return rc;
    rc = sel_build_worklist(offsets, pl.n_ktiles, (size_t)a.B * a.Hkv, pl.cap_pairs, pl.nq, base + pl.off_work, st);
    if (rc != NSA_OK) return rc;
  }
  const int force = get_option_sel_fwd();
  rc = tc_fwd_union_launch(a, stats, offsets, force, st);
  if (rc != NSA_OK) return rc;

  const unsigned grid = (unsigned)sel_work_max_items((size_t)a.B * a.Hkv, pl.n_ktiles, pl.cap_pairs, pl.nq);
  rc = tc_fwdpair_launch(a, (const int32_t*)(base + pl.off_qob), offsets, base + pl.off_part,
                          (float*)(base + pl.off_ml), stats, base + pl.off_work, force, pl.nq, pl.n_ktiles,
                          nq_union, pl.cap_pairs, grid, st);
  if (rc != NSA_OK) return rc;
  const size_t nthreads = (size_t)a.B * a.Hkv * a.T * G * (a.D / 8);
  const unsigned cgrid = (unsigned)((nthreads + 255) / 256);
  {
    KernelScope ks("sel_combine_kernel", st);
    if (a.D == 128)
      sel_combine_kernel<128><<<cgrid, 256, 0, st>>>((const __nv_bfloat16*)(base + pl.off_part),
                                                    (const float*)(base + pl.off_ml), pair_of_slot, offsets, stats,
                                                    (__nv_bfloat16*)a.o, a.lse, a.B, a.Hq, a.Hkv, a.T, G,
                                                    a.S, pl.n_ktiles, nq_union, force);
    else
      sel_combine_kernel<64><<<cgrid, 256, 0, st>>>((const __nv_bfloat16*)(base + pl.off_part),
                                                   (const float*)(base + pl.off_ml), pair_of_slot, offsets, stats,
                                                   (__nv_bfloat16*)a.o, a.lse, a.B, a.Hq, a.Hkv, a.T, G,
                                                   a.S, pl.n_ktiles, nq_union, force);
  }
  NSA_LAUNCH_OK("sel_combine_kernel");
  return NSA_OK;
}

}  // namespace nsa
