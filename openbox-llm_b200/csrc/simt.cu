// CUDA-core (SIMT) attention kernels: one warp per (batch, query head, query token) row.
// They serve every dtype / head dim / group size / block size the boundary accepts
// (nsa_selection_kernel.py:187-188) and are the fp32 path; the tcgen05 kernels in tc.cu
// take over for the bf16 shapes that fill a tensor-core tile.
//
// The three branches differ only in which keys a row visits:
//   window      keys [max(0,t-W+1), t]                         (nsa_fused_kernel.py:588-589)
//   compression summaries j with (j+1)*Bsz-1 <= t              (nsa_fused_kernel.py:590-592)
//   selection   tokens of the listed blocks with pos <= t      (nsa_selection_kernel.py:144)
#include "common.cuh"

namespace nsa {

namespace {

constexpr int kWarps = 4;
const char* const kFwdNames[3] = {"simt_fwd_win", "simt_fwd_cmp", "simt_fwd_slc"};
const char* const kBwdNames[3] = {"simt_bwd_win", "simt_bwd_cmp", "simt_bwd_slc"};

template <typename T, int D>
__device__ __forceinline__ float dot_row(const T* __restrict__ row, const float* __restrict__ qs);

template <int D>
__device__ __forceinline__ float dot_row_bf16(const __nv_bfloat16* __restrict__ row,
                                              const float* __restrict__ qs) {
  float acc = 0.f;
  const uint4* r4 = reinterpret_cast<const uint4*>(row);
#pragma unroll
  for (int i = 0; i < D / 8; ++i) {
    uint4 u = __ldg(r4 + i);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 f = __bfloat1622float2(h[j]);
      acc = fmaf(f.x, qs[i * 8 + 2 * j], acc);
      acc = fmaf(f.y, qs[i * 8 + 2 * j + 1], acc);
    }
  }
  return acc;
}
template <int D>
__device__ __forceinline__ float dot_row_f32(const float* __restrict__ row,
                                             const float* __restrict__ qs) {
  float acc = 0.f;
  const float4* r4 = reinterpret_cast<const float4*>(row);
#pragma unroll
  for (int i = 0; i < D / 4; ++i) {
    float4 u = __ldg(r4 + i);
    acc = fmaf(u.x, qs[i * 4], acc);
    acc = fmaf(u.y, qs[i * 4 + 1], acc);
    acc = fmaf(u.z, qs[i * 4 + 2], acc);
    acc = fmaf(u.w, qs[i * 4 + 3], acc);
  }
  return acc;
}
template <typename T, int D> struct Dot;
template <int D> struct Dot<__nv_bfloat16, D> {
  static __device__ __forceinline__ float run(const __nv_bfloat16* r, const float* q) {
    return dot_row_bf16<D>(r, q);
  }
};
template <int D> struct Dot<float, D> {
  static __device__ __forceinline__ float run(const float* r, const float* q) {
    return dot_row_f32<D>(r, q);
  }
};

// key range number r of row (b, hkv, t); returns false when the slot is empty
__device__ __forceinline__ bool key_range(const AttnArgs& a, int b, int hkv, int t, int r,
                                          int& lo, int& hi) {
  if (a.kind == 0) {
    lo = max(0, t - a.window + 1);
    hi = min(t, a.Lk - 1);
  } else if (a.kind == 1) {
    lo = 0;
    hi = cmp_visible(t, a.block_size, a.window, a.Lk) - 1;   // compression: window holds the stride
  } else {
    int blk = __ldg(a.block_idx + ((size_t)(b * a.Hkv + hkv) * a.T + t) * a.S + r);
    if (blk < 0) return false;
    lo = blk * a.block_size;
    hi = min(lo + a.block_size - 1, min(t, a.T - 1));
  }
  return hi >= lo;
}

template <typename T, int D>
__global__ void __launch_bounds__(kWarps * 32) simt_fwd_kernel(AttnArgs a) {
  constexpr int DPL = (D + 31) / 32;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const size_t total = (size_t)a.B * a.Hq * a.T;
  const size_t row = (size_t)blockIdx.x * kWarps + warp;
  __shared__ float qs[kWarps][D];
  if (row >= total) return;
  const int t = (int)(row % a.T);
  const int h = (int)((row / a.T) % a.Hq);
  const int b = (int)(row / ((size_t)a.T * a.Hq));
  const int hkv = h / (a.Hq / a.Hkv);
  const T* qrow = reinterpret_cast<const T*>(a.q) + row * D;
  for (int d = lane; d < D; d += 32) qs[warp][d] = to_float(qrow[d]) * a.scale;
  __syncwarp();
  const T* kbase = reinterpret_cast<const T*>(a.k) + (size_t)(b * a.Hkv + hkv) * a.Lk * D;
  const T* vbase = reinterpret_cast<const T*>(a.v) + (size_t)(b * a.Hkv + hkv) * a.Lk * D;

  float m = -INFINITY, l = 0.f, acc[DPL];
#pragma unroll
  for (int i = 0; i < DPL; ++i) acc[i] = 0.f;
  const int nranges = a.kind == 2 ? a.S : 1;
  for (int r = 0; r < nranges; ++r) {
    int lo, hi;
    if (!key_range(a, b, hkv, t, r, lo, hi)) continue;
    for (int c = lo; c <= hi; c += 32) {
      const int key = c + lane;
      const bool valid = key <= hi;
      float s = -INFINITY;
      if (valid) s = Dot<T, D>::run(kbase + (size_t)key * D, qs[warp]);
      const float m_new = fmaxf(m, warp_max(s));
      const float p = valid ? expf(s - m_new) : 0.f;
      const float alpha = expf(m - m_new);
      l = l * alpha + warp_sum(p);
#pragma unroll
      for (int i = 0; i < DPL; ++i) acc[i] *= alpha;
      const int n = min(32, hi - c + 1);
      for (int j = 0; j < n; ++j) {
        const float pj = __shfl_sync(0xffffffffu, p, j);
        const T* vr = vbase + (size_t)(c + j) * D;
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
          const int d = lane + 32 * i;
          if (d < D) acc[i] = fmaf(pj, to_float(vr[d]), acc[i]);
        }
      }
      m = m_new;
    }
  }
  T* orow = reinterpret_cast<T*>(a.o) + row * D;
  const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
  for (int i = 0; i < DPL; ++i) {
    const int d = lane + 32 * i;
    if (d < D) orow[d] = from_float<T>(acc[i] * inv);
  }
  if (lane == 0 && a.lse) a.lse[row] = l > 0.f ? m + logf(l) : kLseEmpty;
}

// backward: dq per row, dk/dv by fp32 atomics into float accumulators
template <typename T, int D>
__global__ void __launch_bounds__(kWarps * 32) simt_bwd_kernel(AttnArgs a) {
  constexpr int DPL = (D + 31) / 32;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const size_t total = (size_t)a.B * a.Hq * a.T;
  const size_t row = (size_t)blockIdx.x * kWarps + warp;
  __shared__ float qs[kWarps][D];
  __shared__ float dos[kWarps][D];
  if (row >= total) return;
  const int t = (int)(row % a.T);
  const int h = (int)((row / a.T) % a.Hq);
  const int b = (int)(row / ((size_t)a.T * a.Hq));
  const int hkv = h / (a.Hq / a.Hkv);
  const T* qrow = reinterpret_cast<const T*>(a.q) + row * D;
  const T* dorow = reinterpret_cast<const T*>(a.d_o) + row * D;
  const T* orow = reinterpret_cast<const T*>(a.o) + row * D;
  // a gated branch receives the op's upstream gradient and its own gate value per row:
  // dO_branch = row_scale * dO and delta = row_scale * row_dot (row_dot = sum_d dO * O_branch)
  const float rs = a.row_scale ? a.row_scale[row] : 1.f;
  float dpart = 0.f;
  for (int d = lane; d < D; d += 32) {
    qs[warp][d] = to_float(qrow[d]) * a.scale;
    const float g = to_float(dorow[d]) * rs;
    dos[warp][d] = g;
    if (!a.row_dot) dpart = fmaf(g, to_float(orow[d]), dpart);
  }
  const float delta = a.row_dot ? rs * a.row_dot[row] : warp_sum(dpart);
  const float lse = a.lse[row];
  __syncwarp();
  const size_t kvoff = (size_t)(b * a.Hkv + hkv) * a.Lk * D;
  const T* kbase = reinterpret_cast<const T*>(a.k) + kvoff;
  const T* vbase = reinterpret_cast<const T*>(a.v) + kvoff;
  float* dkb = a.dk_acc + kvoff;
  float* dvb = a.dv_acc + kvoff;

  float dq[DPL];
#pragma unroll
  for (int i = 0; i < DPL; ++i) dq[i] = 0.f;
  const int nranges = a.kind == 2 ? a.S : 1;
  for (int r = 0; r < nranges; ++r) {
    int lo, hi;
    if (!key_range(a, b, hkv, t, r, lo, hi)) continue;
    for (int c = lo; c <= hi; c += 32) {
      const int key = c + lane;
      const bool valid = key <= hi;
      float p = 0.f, ds = 0.f;
      if (valid) {
        const float s = Dot<T, D>::run(kbase + (size_t)key * D, qs[warp]);
        p = expf(s - lse);
        const float dp = Dot<T, D>::run(vbase + (size_t)key * D, dos[warp]);
        ds = p * (dp - delta);
      }
      const int n = min(32, hi - c + 1);
      for (int j = 0; j < n; ++j) {
        const float pj = __shfl_sync(0xffffffffu, p, j);
        const float dsj = __shfl_sync(0xffffffffu, ds, j);
        const size_t ro = (size_t)(c + j) * D;
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
          const int d = lane + 32 * i;
          if (d < D) {
            dq[i] = fmaf(dsj, to_float(kbase[ro + d]), dq[i]);
            atomicAdd(dkb + ro + d, dsj * qs[warp][d]);      // qs carries the D^-1/2 scale
            atomicAdd(dvb + ro + d, pj * dos[warp][d]);
          }
        }
      }
    }
  }
  T* dqrow = reinterpret_cast<T*>(a.dq) + row * D;
#pragma unroll
  for (int i = 0; i < DPL; ++i) {
    const int d = lane + 32 * i;
    if (d < D) dqrow[d] = from_float<T>(dq[i] * a.scale);
  }
}

template <typename T>
__global__ void cast_kernel(const float* __restrict__ src, T* __restrict__ dst, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) dst[i] = from_float<T>(src[i]);
}

template <typename T>
int launch_fwd(const AttnArgs& a, cudaStream_t st) {
  const size_t rows = (size_t)a.B * a.Hq * a.T;
  const unsigned grid = (unsigned)((rows + kWarps - 1) / kWarps);
  switch (a.D) {
    case 16: { KernelScope ks(branch_name(kFwdNames, a.kind), st); simt_fwd_kernel<T, 16><<<grid, kWarps * 32, 0, st>>>(a); } break;
    case 32: { KernelScope ks(branch_name(kFwdNames, a.kind), st); simt_fwd_kernel<T, 32><<<grid, kWarps * 32, 0, st>>>(a); } break;
    case 64: { KernelScope ks(branch_name(kFwdNames, a.kind), st); simt_fwd_kernel<T, 64><<<grid, kWarps * 32, 0, st>>>(a); } break;
    case 128: { KernelScope ks(branch_name(kFwdNames, a.kind), st); simt_fwd_kernel<T, 128><<<grid, kWarps * 32, 0, st>>>(a); } break;
    default: set_error("head dim %d not in {16,32,64,128}", a.D); return NSA_ERR_UNSUPPORTED;
  }
  NSA_LAUNCH_OK("simt_fwd_kernel");
  return NSA_OK;
}
template <typename T>
int launch_bwd(const AttnArgs& a, cudaStream_t st) {
  const size_t rows = (size_t)a.B * a.Hq * a.T;
  const unsigned grid = (unsigned)((rows + kWarps - 1) / kWarps);
  switch (a.D) {
    case 16: { KernelScope ks(branch_name(kBwdNames, a.kind), st); simt_bwd_kernel<T, 16><<<grid, kWarps * 32, 0, st>>>(a); } break;
    case 32: { KernelScope ks(branch_name(kBwdNames, a.kind), st); simt_bwd_kernel<T, 32><<<grid, kWarps * 32, 0, st>>>(a); } break;
    case 64: { KernelScope ks(branch_name(kBwdNames, a.kind), st); simt_bwd_kernel<T, 64><<<grid, kWarps * 32, 0, st>>>(a); } break;
    case 128: { KernelScope ks(branch_name(kBwdNames, a.kind), st); simt_bwd_kernel<T, 128><<<grid, kWarps * 32, 0, st>>>(a); } break;
    default: set_error("head dim %d not in {16,32,64,128}", a.D); return NSA_ERR_UNSUPPORTED;
  }
  NSA_LAUNCH_OK("simt_bwd_kernel");
  return NSA_OK;
}

}  // namespace

int simt_attn_fwd(const AttnArgs& a, int dtype, cudaStream_t st) {
  if ((size_t)a.B * a.Hq * a.T == 0) return NSA_OK;
  return dtype == NSA_DTYPE_BF16 ? launch_fwd<__nv_bfloat16>(a, st) : launch_fwd<float>(a, st);
}

int simt_attn_bwd(const AttnArgs& a, int dtype, cudaStream_t st) {
  if ((size_t)a.B * a.Hq * a.T == 0) return NSA_OK;
  return dtype == NSA_DTYPE_BF16 ? launch_bwd<__nv_bfloat16>(a, st) : launch_bwd<float>(a, st);
}

int cast_f32_to(const float* src, void* dst, size_t n, int dtype, cudaStream_t st) {
  if (n == 0) return NSA_OK;
  const unsigned grid = (unsigned)min((size_t)148 * 16, (n + 255) / 256);
  if (dtype == NSA_DTYPE_BF16) {
    { KernelScope ks("cast_kernel", st); cast_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(src, reinterpret_cast<__nv_bfloat16*>(dst), n); }
  } else {
    { KernelScope ks("cast_kernel", st); cast_kernel<float><<<grid, 256, 0, st>>>(src, reinterpret_cast<float*>(dst), n); }
  }
  NSA_LAUNCH_OK("cast_kernel");
  return NSA_OK;
}

}  // namespace nsa
