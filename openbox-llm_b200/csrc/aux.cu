// Bandwidth-bound companions of the attention kernels: compression pooling, block scoring +
// top-n, block->query CSR inversion and the sigmoid gate combine.
#include <atomic>

#include "common.cuh"

namespace nsa {
namespace {

// ------------------------------------------------------------------------------------------
// mean pooling (nsa_fused_kernel.py:549-554)
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void mean_pool_fwd_kernel(const T* __restrict__ x, T* __restrict__ out, int T_, int D,
                                     int bs, int n_blk, size_t n_out) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_out) return;
  const int d = (int)(i % D);
  const int j = (int)((i / D) % n_blk);
  const size_t bh = i / ((size_t)D * n_blk);
  const T* p = x + (bh * T_ + (size_t)j * bs) * D + d;
  float s = 0.f;
  for (int r = 0; r < bs; ++r) s += to_float(p[(size_t)r * D]);
  out[i] = from_float<T>(s / (float)bs);
}

template <typename T>
__global__ void mean_pool_bwd_kernel(const T* __restrict__ d_out, T* __restrict__ dx, int T_, int D,
                                     int bs, int n_blk, size_t n_in) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_in) return;
  const int d = (int)(i % D);
  const int t = (int)((i / D) % T_);
  const size_t bh = i / ((size_t)D * T_);
  const int j = t / bs;
  float g = 0.f;
  if (j < n_blk) g = to_float(d_out[(bh * n_blk + j) * D + d]) / (float)bs;
  dx[i] = from_float<T>(g);
}

// ------------------------------------------------------------------------------------------
// learned pooling (nsa_model.py:118-123): one CTA of D threads per (b, hkv, block)
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void compress_fwd_kernel(const T* __restrict__ x, const float* __restrict__ intra,
                                    const float* __restrict__ logits, const float* __restrict__ proj,
                                    T* __restrict__ out, float* __restrict__ pooled_out, int T_,
                                    int D, int bs, int stride, int n_blk) {
  extern __shared__ float sm[];
  float* w = sm;            // [bs]
  float* pooled = sm + bs;  // [D]
  const int j = blockIdx.x % n_blk;
  const size_t bh = blockIdx.x / n_blk;
  const int d = threadIdx.x;
  // softmax over the block positions, every thread redundantly (bs is small)
  float mx = -INFINITY;
  for (int r = 0; r < bs; ++r) mx = fmaxf(mx, logits[r]);
  float den = 0.f;
  for (int r = 0; r < bs; ++r) den += expf(logits[r] - mx);
  for (int r = d; r < bs; r += blockDim.x) w[r] = expf(logits[r] - mx) / den;
  __syncthreads();
  const bool act = d < D;   // the CTA is padded to whole warps
  const T* p = x + (bh * T_ + (size_t)j * stride) * D + d;
  float s = 0.f;
  if (act) {
    for (int r = 0; r < bs; ++r) s = fmaf(w[r], to_float(p[(size_t)r * D]) + intra[r * D + d], s);
    pooled[d] = s;
    if (pooled_out) pooled_out[(bh * n_blk + j) * D + d] = s;
  }
  __syncthreads();
  if (out && act) {
    float o = 0.f;
    const float* pr = proj + (size_t)d * D;   // out[o] = sum_i proj[o][i] * pooled[i]
    for (int i = 0; i < D; ++i) o = fmaf(pr[i], pooled[i], o);
    out[(bh * n_blk + j) * D + d] = from_float<T>(o);
  }
}

// backward stage A: per block.  d_pooled = d_out @ W; dx = w[pos] * d_pooled;
// sum_dpooled[d] += d_pooled[d]; d_w[pos] += sum_d d_pooled[d] * (x[pos][d] + intra[pos][d]).
template <typename T>
__global__ void compress_bwd_block_kernel(const T* __restrict__ x, const float* __restrict__ intra,
                                          const float* __restrict__ logits,
                                          const float* __restrict__ proj,
                                          const T* __restrict__ d_out, T* __restrict__ dx,
                                          float* __restrict__ d_pooled_out,
                                          float* __restrict__ sum_dpooled, float* __restrict__ d_w,
                                          int T_, int D, int bs, int stride, int n_blk) {
  extern __shared__ float sm[];
  float* w = sm;           // [bs]
  float* go = sm + bs;     // [D] d_out row
  float* red = go + D;     // [D] reduction scratch
  const int j = blockIdx.x % n_blk;
  const size_t bh = blockIdx.x / n_blk;
  const int d = threadIdx.x;
  float mx = -INFINITY;
  for (int r = 0; r < bs; ++r) mx = fmaxf(mx, logits[r]);
  float den = 0.f;
  for (int r = 0; r < bs; ++r) den += expf(logits[r] - mx);
  for (int r = d; r < bs; r += blockDim.x) w[r] = expf(logits[r] - mx) / den;
  const bool act = d < D;   // the CTA is padded to whole warps
  if (act) go[d] = to_float(d_out[(bh * n_blk + j) * D + d]);
  __syncthreads();
  float dp = 0.f;   // d_pooled[d] = sum_o d_out[o] * proj[o][d]
  if (act) {
    for (int o = 0; o < D; ++o) dp = fmaf(go[o], proj[(size_t)o * D + d], dp);
    d_pooled_out[(bh * n_blk + j) * D + d] = dp;
    atomicAdd(sum_dpooled + d, dp);
  }
  const size_t xo = (bh * T_ + (size_t)j * stride) * D + d;
  for (int r = 0; r < bs; ++r) {
    float xv = 0.f;
    if (act) {
      xv = to_float(x[xo + (size_t)r * D]) + intra[r * D + d];
      if (stride == bs) dx[xo + (size_t)r * D] = from_float<T>(w[r] * dp);   // else: compress_dx_kernel
    }
    // reduce dp * xv over d for position r
    float part = warp_sum(dp * xv);
    if ((d & 31) == 0) red[d >> 5] = part;
    __syncthreads();
    if (d == 0) {
      float tot = 0.f;
      for (int k = 0; k < (int)(blockDim.x + 31) / 32; ++k) tot += red[k];
      atomicAdd(d_w + r, tot);
    }
    __syncthreads();
  }
}

// ------------------------------------------------------------------------------------------
// bf16 fast path of the learned pooling for D in {16,32,64,128}: one CTA of 256 threads takes
// kCompRows consecutive blocks, streams their tokens with 16-byte loads (D/8 threads per token
// row, 256/(D/8) token rows at a time) and keeps the projection matrix in shared memory
// ------------------------------------------------------------------------------------------
constexpr int kCompRows = 8;
constexpr int kCompThreads = 256;

__device__ __forceinline__ void unpack8(const uint4& u, float* f) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 t = __bfloat1622float2(h[e]);
    f[2 * e] = t.x; f[2 * e + 1] = t.y;
  }
}
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ void pool_weights(const float* __restrict__ logits, float* w, int bs) {
  float mx = -INFINITY;
  for (int r = 0; r < bs; ++r) mx = fmaxf(mx, logits[r]);
  float den = 0.f;
  for (int r = 0; r < bs; ++r) den += expf(logits[r] - mx);
  for (int r = threadIdx.x; r < bs; r += blockDim.x) w[r] = expf(logits[r] - mx) / den;
}

// shared memory: w[bs] | cvec[D] | pooled[kCompRows][D] | part[kCompRows][8][D] | projT[D][D+1]
__global__ void __launch_bounds__(kCompThreads)
compress_fast_fwd_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ intra,
                         const float* __restrict__ logits, const float* __restrict__ proj,
                         __nv_bfloat16* __restrict__ out, float* __restrict__ pooled_out, int T_, int D,
                         int bs, int stride, int n_blk, size_t rows) {
  extern __shared__ float sm[];
  float* w = sm;
  float* cvec = w + bs;
  float* pooled = cvec + D;
  float* part = pooled + kCompRows * D;
  float* projT = part + kCompRows * 8 * D;
  const int tid = threadIdx.x, warp = tid >> 5;
  const int VL = D >> 3, RG = kCompThreads / VL;
  const int vl = tid % VL, rg = tid / VL;
  const size_t row0 = (size_t)blockIdx.x * kCompRows;
  if (out)
    for (int idx = tid; idx < D * D; idx += kCompThreads) projT[(idx % D) * (D + 1) + idx / D] = proj[idx];
  pool_weights(logits, w, bs);
  __syncthreads();
  // the block-independent part: sum_r w[r] * intra[r][:]
  {
    float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int r = rg; r < bs; r += RG) {
      const float4 lo = *reinterpret_cast<const float4*>(intra + (size_t)r * D + vl * 8);
      const float4 hi = *reinterpret_cast<const float4*>(intra + (size_t)r * D + vl * 8 + 4);
      const float wr = w[r];
      a[0] = fmaf(wr, lo.x, a[0]); a[1] = fmaf(wr, lo.y, a[1]); a[2] = fmaf(wr, lo.z, a[2]); a[3] = fmaf(wr, lo.w, a[3]);
      a[4] = fmaf(wr, hi.x, a[4]); a[5] = fmaf(wr, hi.y, a[5]); a[6] = fmaf(wr, hi.z, a[6]); a[7] = fmaf(wr, hi.w, a[7]);
    }
    // threads of a warp that hold the same columns (VL apart) meet by shuffles
    for (int o = 16; o >= VL; o >>= 1)
#pragma unroll
      for (int e = 0; e < 8; ++e) a[e] += __shfl_xor_sync(0xffffffffu, a[e], o);
    if ((tid & 31) < VL)
#pragma unroll
      for (int e = 0; e < 8; ++e) part[warp * D + vl * 8 + e] = a[e];
  }
  __syncthreads();
  if (tid < D) {
    float c = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) c += part[k * D + tid];
    cvec[tid] = c;
  }
  __syncthreads();
#pragma unroll
  for (int b = 0; b < kCompRows; ++b) {
    const size_t row = row0 + b;
    float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (row < rows) {
      const size_t bh = row / n_blk;
      const int j = (int)(row % n_blk);
      const __nv_bfloat16* xb = x + (bh * T_ + (size_t)j * stride) * D + vl * 8;
      for (int r = rg; r < bs; r += RG) {
        const uint4 u = __ldg(reinterpret_cast<const uint4*>(xb + (size_t)r * D));
        float f[8];
        unpack8(u, f);
        const float wr = w[r];
#pragma unroll
        for (int e = 0; e < 8; ++e) a[e] = fmaf(wr, f[e], a[e]);
      }
    }
    for (int o = 16; o >= VL; o >>= 1)
#pragma unroll
      for (int e = 0; e < 8; ++e) a[e] += __shfl_xor_sync(0xffffffffu, a[e], o);
    if ((tid & 31) < VL)
#pragma unroll
      for (int e = 0; e < 8; ++e) part[(b * 8 + warp) * D + vl * 8 + e] = a[e];
  }
  __syncthreads();
  for (int idx = tid; idx < kCompRows * D; idx += kCompThreads) {
    const int b = idx / D, d = idx % D;
    float s = cvec[d];
#pragma unroll
    for (int k = 0; k < 8; ++k) s += part[(b * 8 + k) * D + d];
    pooled[idx] = s;
    if (pooled_out && row0 + b < rows) pooled_out[(row0 + b) * D + d] = s;
  }
  if (!out) return;
  __syncthreads();
  // out[row][o] = sum_i proj[o][i] * pooled[row][i], four rows per thread
  for (int idx = tid; idx < (kCompRows / 4) * D; idx += kCompThreads) {
    const int b0 = (idx / D) * 4, o = idx % D;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int i = 0; i < D; ++i) {
      const float pv = projT[i * (D + 1) + o];
#pragma unroll
      for (int k = 0; k < 4; ++k) acc[k] = fmaf(pv, pooled[(b0 + k) * D + i], acc[k]);
    }
#pragma unroll
    for (int k = 0; k < 4; ++k)
      if (row0 + b0 + k < rows) out[(row0 + b0 + k) * D + o] = __float2bfloat16(acc[k]);
  }
}

// backward of the same: d_pooled = d_out @ W, dx = w[pos] * d_pooled, sum_dpooled += d_pooled,
// d_w[pos] += sum_d d_pooled[d] * x[pos][d] (the intra_pos share of d_w is added by the final
// kernel from sum_dpooled).  shared memory: w[bs] | dw[bs] | go[rows][D] | dp[rows][D] | proj[D][D]
__global__ void __launch_bounds__(kCompThreads)
compress_fast_bwd_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ logits,
                         const float* __restrict__ proj, const __nv_bfloat16* __restrict__ d_out,
                         __nv_bfloat16* __restrict__ dx, float* __restrict__ d_pooled_out,
                         float* __restrict__ sum_dpooled, float* __restrict__ d_w, int T_, int D, int bs,
                         int stride, int n_blk, size_t rows) {
  extern __shared__ float sm[];
  float* w = sm;
  float* dw = w + bs;
  float* go = dw + bs;
  float* dp = go + kCompRows * D;
  float* pj = dp + kCompRows * D;
  const int tid = threadIdx.x;
  const int VL = D >> 3, RG = kCompThreads / VL;
  const int vl = tid % VL, rg = tid / VL;
  const size_t row0 = (size_t)blockIdx.x * kCompRows;
  for (int idx = tid; idx < D * D; idx += kCompThreads) pj[idx] = proj[idx];
  for (int idx = tid; idx < kCompRows * D; idx += kCompThreads)
    go[idx] = row0 + idx / D < rows ? __bfloat162float(d_out[row0 * D + idx]) : 0.f;
  for (int r = tid; r < bs; r += kCompThreads) dw[r] = 0.f;
  pool_weights(logits, w, bs);
  __syncthreads();
  for (int idx = tid; idx < (kCompRows / 4) * D; idx += kCompThreads) {
    const int b0 = (idx / D) * 4, d = idx % D;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int o = 0; o < D; ++o) {
      const float pv = pj[o * D + d];
#pragma unroll
      for (int k = 0; k < 4; ++k) acc[k] = fmaf(go[(b0 + k) * D + o], pv, acc[k]);
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      dp[(b0 + k) * D + d] = acc[k];
      if (row0 + b0 + k < rows) d_pooled_out[(row0 + b0 + k) * D + d] = acc[k];
    }
  }
  __syncthreads();
  if (tid < D) {
    float s = 0.f;
#pragma unroll
    for (int b = 0; b < kCompRows; ++b) s += dp[b * D + tid];   // rows past the end hold zeros
    atomicAdd(sum_dpooled + tid, s);
  }
#pragma unroll 2
  for (int b = 0; b < kCompRows; ++b) {
    const size_t row = row0 + b;
    if (row >= rows) break;
    const size_t bh = row / n_blk;
    const int j = (int)(row % n_blk);
    const size_t base = (bh * T_ + (size_t)j * stride) * D + vl * 8;
    const bool write_dx = stride == bs;               // overlapping windows: compress_dx_kernel
    float g[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) g[e] = dp[b * D + vl * 8 + e];
    for (int r0 = 0; r0 < bs; r0 += RG) {
      const int r = r0 + rg;
      float dot = 0.f;
      if (r < bs) {
        const uint4 u = __ldg(reinterpret_cast<const uint4*>(x + base + (size_t)r * D));
        float f[8];
        unpack8(u, f);
        const float wr = w[r];
        uint4 o;
        o.x = pack2(wr * g[0], wr * g[1]); o.y = pack2(wr * g[2], wr * g[3]);
        o.z = pack2(wr * g[4], wr * g[5]); o.w = pack2(wr * g[6], wr * g[7]);
        if (write_dx) *reinterpret_cast<uint4*>(dx + base + (size_t)r * D) = o;
#pragma unroll
        for (int e = 0; e < 8; ++e) dot = fmaf(g[e], f[e], dot);
      }
      for (int o = VL >> 1; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
      if (vl == 0 && r < bs) atomicAdd(dw + r, dot);
    }
  }
  __syncthreads();
  for (int r = tid; r < bs; r += kCompThreads) atomicAdd(d_w + r, dw[r]);
}

bool compress_fast_ok(int D, int bs, int dtype) {
  return dtype == NSA_DTYPE_BF16 && (D == 16 || D == 32 || D == 64 || D == 128) && bs >= 1 && bs <= 1024;
}
size_t compress_fast_fwd_smem(int D, int bs, bool with_proj) {
  return ((size_t)bs + D + kCompRows * D + kCompRows * 8 * D + (with_proj ? (size_t)D * (D + 1) : 0)) * sizeof(float);
}
size_t compress_fast_bwd_smem(int D, int bs) {
  return (2 * (size_t)bs + 2 * kCompRows * D + (size_t)D * D) * sizeof(float);
}

// dx for overlapping windows (stride < length): token pos of (b, hkv) collects
// w[pos - j*stride] * d_pooled[j] from every window j that holds it; tokens in no window get 0
template <typename T>
__global__ void compress_dx_kernel(const float* __restrict__ d_pooled, const float* __restrict__ logits,
                                   T* __restrict__ dx, int T_, int D, int bs, int stride, int n_blk,
                                   size_t n_elems) {
  extern __shared__ float w[];
  pool_weights(logits, w, bs);
  __syncthreads();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_elems) return;
  const int d = (int)(i % D);
  const int pos = (int)((i / D) % T_);
  const size_t bh = i / ((size_t)D * T_);
  const int j_hi = min(n_blk - 1, pos / stride);
  const int j_lo = max(0, (pos - bs + stride) / stride);   // ceil((pos - bs + 1) / stride) for pos >= bs - 1
  float acc = 0.f;
  for (int j = j_lo; j <= j_hi; ++j) acc = fmaf(w[pos - j * stride], d_pooled[(bh * n_blk + j) * D + d], acc);
  dx[i] = from_float<T>(acc);
}

// the same for bf16 rows of D = 8 * k elements: one thread per 8 columns, 16-byte stores
__global__ void compress_dx_vec_kernel(const float* __restrict__ d_pooled, const float* __restrict__ logits,
                                       __nv_bfloat16* __restrict__ dx, int T_, int D, int bs, int stride,
                                       int n_blk, size_t n_vec) {
  extern __shared__ float w[];
  pool_weights(logits, w, bs);
  __syncthreads();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_vec) return;
  const int VL = D >> 3;
  const int vl = (int)(i % VL);
  const int pos = (int)((i / VL) % T_);
  const size_t bh = i / ((size_t)VL * T_);
  const int j_hi = min(n_blk - 1, pos / stride);
  const int j_lo = max(0, (pos - bs + stride) / stride);
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int j = j_lo; j <= j_hi; ++j) {
    const float wj = w[pos - j * stride];
    const float4 lo = *reinterpret_cast<const float4*>(d_pooled + (bh * n_blk + j) * D + vl * 8);
    const float4 hi = *reinterpret_cast<const float4*>(d_pooled + (bh * n_blk + j) * D + vl * 8 + 4);
    acc[0] = fmaf(wj, lo.x, acc[0]); acc[1] = fmaf(wj, lo.y, acc[1]); acc[2] = fmaf(wj, lo.z, acc[2]); acc[3] = fmaf(wj, lo.w, acc[3]);
    acc[4] = fmaf(wj, hi.x, acc[4]); acc[5] = fmaf(wj, hi.y, acc[5]); acc[6] = fmaf(wj, hi.z, acc[6]); acc[7] = fmaf(wj, hi.w, acc[7]);
  }
  uint4 o;
  o.x = pack2(acc[0], acc[1]); o.y = pack2(acc[2], acc[3]); o.z = pack2(acc[4], acc[5]); o.w = pack2(acc[6], acc[7]);
  *reinterpret_cast<uint4*>(dx + i * 8) = o;
}

// tail tokens past the last complete block get zero gradient
template <typename T>
__global__ void zero_tail_kernel(T* __restrict__ dx, int T_, int D, int t_first, size_t n_bh) {
  const size_t per = (size_t)(T_ - t_first) * D;
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= per * n_bh) return;
  const size_t bh = i / per, r = i % per;
  dx[(bh * T_ + t_first) * D + r] = from_float<T>(0.f);
}

// stage B: d_proj[o][i] = sum_rows d_out[row][o] * pooled[row][i]; CTA (o, chunk of rows),
// chunks meet through atomicAdd on the zero-initialised output
template <typename T>
__global__ void compress_bwd_proj_kernel(const T* __restrict__ d_out, const float* __restrict__ pooled,
                                         float* __restrict__ d_proj, size_t rows, int D) {
  const int o = blockIdx.x, i = threadIdx.x;
  if (i >= D) return;
  const size_t per = (rows + gridDim.y - 1) / gridDim.y;
  const size_t r0 = (size_t)blockIdx.y * per, r1 = r0 + per < rows ? r0 + per : rows;
  float s = 0.f;
  for (size_t r = r0; r < r1; ++r) s = fmaf(to_float(d_out[r * D + o]), pooled[r * D + i], s);
  if (r1 > r0) atomicAdd(d_proj + (size_t)o * D + i, s);
}

// stage C: d_intra[pos][d] = w[pos] * sum_dpooled[d]; d_logits = w * (d_w - sum(d_w * w))
__global__ void compress_bwd_final_kernel(const float* __restrict__ logits,
                                          const float* __restrict__ sum_dpooled,
                                          float* __restrict__ d_w, const float* __restrict__ intra,
                                          float* __restrict__ d_intra,
                                          float* __restrict__ d_logits, int D, int bs) {
  extern __shared__ float w[];
  if (intra) {   // the streaming kernel left out sum_d sum_dpooled[d] * intra_pos[pos][d]
    for (int r = threadIdx.x; r < bs; r += blockDim.x) {
      float s = 0.f;
      for (int d = 0; d < D; ++d) s = fmaf(sum_dpooled[d], intra[(size_t)r * D + d], s);
      d_w[r] += s;
    }
    __syncthreads();
  }
  float mx = -INFINITY;
  for (int r = 0; r < bs; ++r) mx = fmaxf(mx, logits[r]);
  float den = 0.f;
  for (int r = 0; r < bs; ++r) den += expf(logits[r] - mx);
  for (int r = threadIdx.x; r < bs; r += blockDim.x) w[r] = expf(logits[r] - mx) / den;
  __syncthreads();
  float dot = 0.f;
  for (int r = 0; r < bs; ++r) dot = fmaf(d_w[r], w[r], dot);
  for (int r = threadIdx.x; r < bs; r += blockDim.x) d_logits[r] = w[r] * (d_w[r] - dot);
  for (int i = threadIdx.x; i < bs * D; i += blockDim.x) d_intra[i] = w[i / D] * sum_dpooled[i % D];
}

// ------------------------------------------------------------------------------------------
// block scoring + top-n (nsa_model.py:343-355): one warp per (b, hkv, t)
// ------------------------------------------------------------------------------------------
template <typename T, int D>
__global__ void __launch_bounds__(128) topn_kernel(const T* __restrict__ q, const T* __restrict__ kc,
                                                   const float* __restrict__ lse,
                                                   int32_t* __restrict__ block_idx,
                                                   float* __restrict__ imp_out, int B, int Hq, int Hkv,
                                                   int T_, int n_blk, int bs, int n_sel, int n_init,
                                                   int n_local, float scale, int stride, int sel_block,
                                                   int n_sblk, int imp_cols) {
  // n_blk summaries of bs tokens every `stride` tokens; n_sblk selection blocks of sel_block
  // tokens.  A selection block takes the sum of the summaries that overlap it and is a candidate
  // once the first of them is visible; with bs == stride == sel_block blocks and summaries coincide.
  extern __shared__ float sm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* qs = sm + (size_t)warp * (D + n_blk + n_sblk + 1);   // [D]
  float* sums = qs + D;                                       // [n_blk] importance of the summaries
  float* imp = sums + n_blk;                                  // [n_sblk + 1] importance of the blocks
  const size_t total = (size_t)B * Hkv * T_;
  const size_t unit = (size_t)blockIdx.x * 4 + warp;
  if (unit >= total) return;
  const int t = (int)(unit % T_);
  const int hkv = (int)((unit / T_) % Hkv);
  const int b = (int)(unit / ((size_t)T_ * Hkv));
  const int G = Hq / Hkv;
  const int n_valid = cmp_visible(t, bs, stride, n_blk);
  for (int j = lane; j < n_blk; j += 32) sums[j] = 0.f;
  const T* kbase = kc + (size_t)(b * Hkv + hkv) * n_blk * D;
  for (int g = 0; g < G; ++g) {
    const size_t row = ((size_t)(b * Hq + hkv * G + g)) * T_ + t;
    __syncwarp();
    for (int d = lane; d < D; d += 32) qs[d] = to_float(q[row * D + d]) * scale;
    __syncwarp();
    const float l = lse[row];
    for (int j = lane; j < n_valid; j += 32) {
      float s;
      if constexpr (sizeof(T) == 2) {
        float acc = 0.f;
        const uint4* r4 = reinterpret_cast<const uint4*>(kbase + (size_t)j * D);
#pragma unroll
        for (int i = 0; i < D / 8; ++i) {
          uint4 u = __ldg(r4 + i);
          const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            float2 f = __bfloat1622float2(h2[c]);
            acc = fmaf(f.x, qs[i * 8 + 2 * c], acc);
            acc = fmaf(f.y, qs[i * 8 + 2 * c + 1], acc);
          }
        }
        s = acc;
      } else {
        float acc = 0.f;
        const float* kr = reinterpret_cast<const float*>(kbase) + (size_t)j * D;
        for (int i = 0; i < D; ++i) acc = fmaf(kr[i], qs[i], acc);
        s = acc;
      }
      sums[j] += expf(s - l);
    }
  }
  __syncwarp();
  // selection blocks up to the one holding t: importance, -1 when no overlapping summary is visible
  const int r_ = sel_block / stride, o_ = bs / stride;
  const int cur = t / sel_block;
  for (int bb = lane; bb <= cur; bb += 32) {
    const int j0 = max(0, r_ * bb - o_ + 1), j1 = min(n_valid - 1, r_ * bb + r_ - 1);
    float v = -1.f;
    if (j0 < n_valid) {
      v = 0.f;
      for (int j = j0; j <= j1; ++j) v += sums[j];
    }
    imp[bb] = v;
  }
  __syncwarp();
  if (imp_out) {
    float* dst = imp_out + unit * imp_cols;
    for (int j = lane; j < imp_cols; j += 32) dst[j] = (j <= cur && imp[j] >= 0.f) ? imp[j] : 0.f;
  }
  int32_t* out = block_idx + unit * n_sel;
  // forced blocks: the first n_init blocks and the n_local most recent ones (the block holding
  // t included) rank ahead of every importance (<= G); other invisible blocks do not compete
  const int n_cand = cur + 1;
  if (n_init > 0 || n_local > 0) {
    __syncwarp();
    for (int j = lane; j <= cur; j += 32) {
      if (j < n_init) imp[j] = kForcedInit - (float)j;
      else if (j > cur - n_local) imp[j] = kForcedLocal - (float)(cur - j);
    }
    __syncwarp();
  }
  for (int s = 0; s < n_sel; ++s) {
    float best = -1.f;
    int bj = 0x7fffffff;
    for (int j = lane; j < n_cand; j += 32) {
      const float v = imp[j];
      if (v > best) { best = v; bj = j; }        // ascending j: first maximum wins
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oj = __shfl_xor_sync(0xffffffffu, bj, o);
      if (ov > best || (ov == best && oj < bj)) { best = ov; bj = oj; }
    }
    const bool found = best >= 0.f;
    if (lane == 0) out[s] = found ? bj : -1;
    if (found && lane == (bj & 31)) imp[bj] = -2.f;   // taken
    __syncwarp();
  }
}

// ------------------------------------------------------------------------------------------
// block -> query CSR (nsa_fsa.py:14-64) through a [B*Hkv, n_blk, T] bitmap
// ------------------------------------------------------------------------------------------
__global__ void csr_mark_kernel(const int32_t* __restrict__ idx, uint32_t* __restrict__ bitmap,
                                int T_, int S, int bs, int n_blk, int words, size_t n_entries) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_entries) return;
  const int j = idx[i];
  const int t = (int)((i / S) % T_);
  const size_t bh = i / ((size_t)S * T_);
  if (j < 0 || j >= n_blk || (long long)j * bs > t) return;
  atomicOr(bitmap + (bh * n_blk + j) * words + (t >> 5), 1u << (t & 31));
}

// one warp per (bh, block) row: population count, and for every bitmap word the number of set
// bits before it in the row
__global__ void csr_count_kernel(const uint32_t* __restrict__ bitmap, int32_t* __restrict__ counts,
                                 int32_t* __restrict__ prefix, int words, size_t rows) {
  const size_t row = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  int run = 0;
  for (int w0 = 0; w0 < words; w0 += 32) {
    const int w = w0 + lane;
    const int c = w < words ? __popc(bitmap[row * words + w]) : 0;
    int incl = c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    if (w < words) prefix[row * words + w] = run + incl - c;
    run += __shfl_sync(0xffffffffu, incl, 31);
  }
  if (lane == 0) counts[row] = run;
}

// single CTA exclusive scan of counts[rows] into block_offsets laid out [BH][n_blk+1]
__global__ void csr_scan_kernel(const int32_t* __restrict__ counts, int32_t* __restrict__ offsets,
                                int32_t* __restrict__ row_start, int n_blk, size_t rows) {
  __shared__ int part[1024];
  __shared__ int carry;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (size_t base = 0; base < rows; base += 1024) {
    const size_t r = base + threadIdx.x;
    const int c = r < rows ? counts[r] : 0;
    part[threadIdx.x] = c;
    __syncthreads();
    for (int o = 1; o < 1024; o <<= 1) {
      int v = threadIdx.x >= o ? part[threadIdx.x - o] : 0;
      __syncthreads();
      part[threadIdx.x] += v;
      __syncthreads();
    }
    const int incl = part[threadIdx.x] + carry;
    if (r < rows) {
      const size_t bh = r / n_blk, j = r % n_blk;
      row_start[r] = incl - c;
      offsets[bh * (n_blk + 1) + j] = incl - c;
      offsets[bh * (n_blk + 1) + j + 1] = incl;   // last block of a group; else overwritten equal
    }
    __syncthreads();
    if (threadIdx.x == 1023) carry = incl;
    __syncthreads();
  }
}

// one thread per (b, hkv, t, slot) entry: its pair index is the row start plus the rank of t
// among the set bits of row (b, hkv, block); a block listed twice by one query keeps its first slot
__global__ void csr_fill_kernel(const int32_t* __restrict__ idx, const uint32_t* __restrict__ bitmap,
                                const int32_t* __restrict__ prefix, const int32_t* __restrict__ row_start,
                                int32_t* __restrict__ q_of_block, int32_t* __restrict__ pair_bh,
                                int32_t* __restrict__ pair_of_slot, int T_, int S, int bs, int n_blk,
                                int words, size_t n_entries) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_entries) return;
  const int j = idx[i];
  const int slot = (int)(i % S);
  const int t = (int)((i / S) % T_);
  const size_t bh = i / ((size_t)S * T_);
  int p = -1;
  if (j >= 0 && j < n_blk && (long long)j * bs <= t) {
    bool dup = false;
    for (int s2 = 0; s2 < slot; ++s2) dup |= idx[i - slot + s2] == j;
    if (!dup) {
      const size_t row = bh * n_blk + j;
      const uint32_t bits = bitmap[row * words + (t >> 5)];
      p = row_start[row] + prefix[row * words + (t >> 5)] + __popc(bits & ((1u << (t & 31)) - 1u));
      q_of_block[p] = t;
      pair_bh[p] = (int)bh;
    }
  }
  if (pair_of_slot) pair_of_slot[i] = p;
}

// ------------------------------------------------------------------------------------------
// gate combine (nsa_model.py:366-368)
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + expf(-x)); }

// one warp per (b,h,t) row
template <typename T>
__global__ void gate_fwd_kernel(const T* __restrict__ oc, const T* __restrict__ os,
                                const T* __restrict__ ow, const T* __restrict__ gate,
                                T* __restrict__ out, size_t rows, int D) {
  const size_t row = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const float g0 = sigmoidf_(to_float(gate[row * 3 + 0]));
  const float g1 = sigmoidf_(to_float(gate[row * 3 + 1]));
  const float g2 = sigmoidf_(to_float(gate[row * 3 + 2]));
  for (int d = lane; d < D; d += 32) {
    const size_t i = row * D + d;
    out[i] = from_float<T>(g0 * to_float(oc[i]) + g1 * to_float(os[i]) + g2 * to_float(ow[i]));
  }
}

template <typename T>
__global__ void gate_bwd_kernel(const T* __restrict__ oc, const T* __restrict__ os,
                                const T* __restrict__ ow, const T* __restrict__ gate,
                                const T* __restrict__ d_out, T* __restrict__ dc, T* __restrict__ ds,
                                T* __restrict__ dw, T* __restrict__ d_gate, size_t rows, int D) {
  const size_t row = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const float g0 = sigmoidf_(to_float(gate[row * 3 + 0]));
  const float g1 = sigmoidf_(to_float(gate[row * 3 + 1]));
  const float g2 = sigmoidf_(to_float(gate[row * 3 + 2]));
  float a0 = 0.f, a1 = 0.f, a2 = 0.f;
  for (int d = lane; d < D; d += 32) {
    const size_t i = row * D + d;
    const float g = to_float(d_out[i]);
    a0 = fmaf(g, to_float(oc[i]), a0);
    a1 = fmaf(g, to_float(os[i]), a1);
    a2 = fmaf(g, to_float(ow[i]), a2);
    dc[i] = from_float<T>(g0 * g);
    ds[i] = from_float<T>(g1 * g);
    dw[i] = from_float<T>(g2 * g);
  }
  a0 = warp_sum(a0); a1 = warp_sum(a1); a2 = warp_sum(a2);
  if (lane == 0) {
    d_gate[row * 3 + 0] = from_float<T>(a0 * g0 * (1.f - g0));
    d_gate[row * 3 + 1] = from_float<T>(a1 * g1 * (1.f - g1));
    d_gate[row * 3 + 2] = from_float<T>(a2 * g2 * (1.f - g2));
  }
}

// bf16 rows of D = 8 * VL elements (VL a power of two <= 32): VL threads per row, 16 bytes each
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float* f) {
  const uint4 u = __ldg(reinterpret_cast<const uint4*>(p));
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 t = __bfloat1622float2(h[e]);
    f[2 * e] = t.x; f[2 * e + 1] = t.y;
  }
}

__global__ void gate_fwd_vec_kernel(const __nv_bfloat16* __restrict__ oc, const __nv_bfloat16* __restrict__ os,
                                    const __nv_bfloat16* __restrict__ ow, const __nv_bfloat16* __restrict__ gate,
                                    __nv_bfloat16* __restrict__ out, size_t rows, int VL) {
  const size_t gid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t row = gid / VL;
  if (row >= rows) return;
  const size_t i = gid * 8;
  float a[8], b[8], c[8];
  load8(oc + i, a); load8(os + i, b); load8(ow + i, c);
  const float g0 = sigmoidf_(__bfloat162float(gate[row * 3 + 0]));
  const float g1 = sigmoidf_(__bfloat162float(gate[row * 3 + 1]));
  const float g2 = sigmoidf_(__bfloat162float(gate[row * 3 + 2]));
  uint4 r;
  __nv_bfloat162* rs = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
  for (int e = 0; e < 4; ++e)
    rs[e] = __floats2bfloat162_rn(g0 * a[2 * e] + g1 * b[2 * e] + g2 * c[2 * e],
                                  g0 * a[2 * e + 1] + g1 * b[2 * e + 1] + g2 * c[2 * e + 1]);
  *reinterpret_cast<uint4*>(out + i) = r;
}

__global__ void gate_bwd_rows_vec_kernel(const __nv_bfloat16* __restrict__ oc, const __nv_bfloat16* __restrict__ os,
                                         const __nv_bfloat16* __restrict__ ow, const __nv_bfloat16* __restrict__ gate,
                                         const __nv_bfloat16* __restrict__ d_out, float* __restrict__ row_scale,
                                         float* __restrict__ row_dot, __nv_bfloat16* __restrict__ d_gate,
                                         size_t rows, int VL) {
  const size_t gid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t row = gid / VL;                    // the grid is padded to whole warps: no early return
  const bool live = row < rows;
  float a0 = 0.f, a1 = 0.f, a2 = 0.f;
  if (live) {
    const size_t i = gid * 8;
    float g[8], a[8], b[8], c[8];
    load8(d_out + i, g); load8(oc + i, a); load8(os + i, b); load8(ow + i, c);
#pragma unroll
    for (int e = 0; e < 8; ++e) { a0 = fmaf(g[e], a[e], a0); a1 = fmaf(g[e], b[e], a1); a2 = fmaf(g[e], c[e], a2); }
  }
  for (int o = VL >> 1; o > 0; o >>= 1) {
    a0 += __shfl_xor_sync(0xffffffffu, a0, o);
    a1 += __shfl_xor_sync(0xffffffffu, a1, o);
    a2 += __shfl_xor_sync(0xffffffffu, a2, o);
  }
  if (live && gid % VL == 0) {
    const float g0 = sigmoidf_(__bfloat162float(gate[row * 3 + 0]));
    const float g1 = sigmoidf_(__bfloat162float(gate[row * 3 + 1]));
    const float g2 = sigmoidf_(__bfloat162float(gate[row * 3 + 2]));
    row_scale[row] = g0; row_scale[rows + row] = g1; row_scale[2 * rows + row] = g2;
    row_dot[row] = a0; row_dot[rows + row] = a1; row_dot[2 * rows + row] = a2;
    d_gate[row * 3 + 0] = __float2bfloat16(a0 * g0 * (1.f - g0));
    d_gate[row * 3 + 1] = __float2bfloat16(a1 * g1 * (1.f - g1));
    d_gate[row * 3 + 2] = __float2bfloat16(a2 * g2 * (1.f - g2));
  }
}

inline bool gate_vec_ok(int D, int dtype) {
  return dtype == NSA_DTYPE_BF16 && D >= 8 && D <= 256 && (D & (D - 1)) == 0;
}

// out = a + b + c, fp32 accumulation, 8 elements per thread (bf16) or 4 (fp32)
__global__ void sum3_bf16_kernel(const uint4* __restrict__ a, const uint4* __restrict__ b,
                                 const uint4* __restrict__ c, uint4* __restrict__ out, size_t n8) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  const uint4 x = __ldg(a + i), y = __ldg(b + i), z = __ldg(c + i);
  const __nv_bfloat162* xs = reinterpret_cast<const __nv_bfloat162*>(&x);
  const __nv_bfloat162* ys = reinterpret_cast<const __nv_bfloat162*>(&y);
  const __nv_bfloat162* zs = reinterpret_cast<const __nv_bfloat162*>(&z);
  uint4 r;
  __nv_bfloat162* rs = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 fx = __bfloat1622float2(xs[e]), fy = __bfloat1622float2(ys[e]), fz = __bfloat1622float2(zs[e]);
    rs[e] = __floats2bfloat162_rn(fx.x + fy.x + fz.x, fx.y + fy.y + fz.y);
  }
  out[i] = r;
}
__global__ void sum3_f32_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                const float* __restrict__ c, float* __restrict__ out, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = a[i] + b[i] + c[i];
}

// per row: gate values, <dO, o_branch> and d_gate; the branch backward kernels then work from the
// op's upstream gradient directly
template <typename T>
__global__ void gate_bwd_rows_kernel(const T* __restrict__ oc, const T* __restrict__ os,
                                     const T* __restrict__ ow, const T* __restrict__ gate,
                                     const T* __restrict__ d_out, float* __restrict__ row_scale,
                                     float* __restrict__ row_dot, T* __restrict__ d_gate, size_t rows, int D) {
  const size_t row = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  float a0 = 0.f, a1 = 0.f, a2 = 0.f;
  for (int d = lane; d < D; d += 32) {
    const size_t i = row * D + d;
    const float g = to_float(d_out[i]);
    a0 = fmaf(g, to_float(oc[i]), a0);
    a1 = fmaf(g, to_float(os[i]), a1);
    a2 = fmaf(g, to_float(ow[i]), a2);
  }
  a0 = warp_sum(a0); a1 = warp_sum(a1); a2 = warp_sum(a2);
  if (lane == 0) {
    const float g0 = sigmoidf_(to_float(gate[row * 3 + 0]));
    const float g1 = sigmoidf_(to_float(gate[row * 3 + 1]));
    const float g2 = sigmoidf_(to_float(gate[row * 3 + 2]));
    row_scale[row] = g0; row_scale[rows + row] = g1; row_scale[2 * rows + row] = g2;
    row_dot[row] = a0; row_dot[rows + row] = a1; row_dot[2 * rows + row] = a2;
    d_gate[row * 3 + 0] = from_float<T>(a0 * g0 * (1.f - g0));
    d_gate[row * 3 + 1] = from_float<T>(a1 * g1 * (1.f - g1));
    d_gate[row * 3 + 2] = from_float<T>(a2 * g2 * (1.f - g2));
  }
}

inline unsigned blocks_for(size_t n, int per) { return (unsigned)((n + per - 1) / per); }

}  // namespace
}  // namespace nsa

using namespace nsa;

extern "C" int nsa_block_mean_pool_fwd(const void* x, void* out, int B, int Hkv, int T, int D,
                                       int block_size, int dtype, void* stream) {
  NSA_CHECK_ARG(block_size > 0 && D > 0, "bad block_size/D");
  const int n_blk = T / block_size;
  const size_t n = (size_t)B * Hkv * n_blk * D;
  if (n == 0) return NSA_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == NSA_DTYPE_BF16)
    { KernelScope ks("mean_pool_fwd_kernel", st); mean_pool_fwd_kernel<<<blocks_for(n, 256), 256, 0, st>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)out, T, D, block_size, n_blk, n); }
  else
    { KernelScope ks("mean_pool_fwd_kernel", st); mean_pool_fwd_kernel<<<blocks_for(n, 256), 256, 0, st>>>((const float*)x, (float*)out, T, D, block_size, n_blk, n); }
  NSA_LAUNCH_OK("mean_pool_fwd_kernel");
  return NSA_OK;
}

extern "C" int nsa_block_mean_pool_bwd(const void* d_out, void* dx, int B, int Hkv, int T, int D,
                                       int block_size, int dtype, void* stream) {
  NSA_CHECK_ARG(block_size > 0 && D > 0, "bad block_size/D");
  const int n_blk = T / block_size;
  const size_t n = (size_t)B * Hkv * T * D;
  if (n == 0) return NSA_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == NSA_DTYPE_BF16)
    { KernelScope ks("mean_pool_bwd_kernel", st); mean_pool_bwd_kernel<<<blocks_for(n, 256), 256, 0, st>>>((const __nv_bfloat16*)d_out, (__nv_bfloat16*)dx, T, D, block_size, n_blk, n); }
  else
    { KernelScope ks("mean_pool_bwd_kernel", st); mean_pool_bwd_kernel<<<blocks_for(n, 256), 256, 0, st>>>((const float*)d_out, (float*)dx, T, D, block_size, n_blk, n); }
  NSA_LAUNCH_OK("mean_pool_bwd_kernel");
  return NSA_OK;
}

static int n_windows(int T, int len, int stride) { return T >= len ? (T - len) / stride + 1 : 0; }

extern "C" int nsa_block_compress_fwd(const void* x, const float* intra_pos, const float* pool_logits,
                                      const float* proj_w, void* out, int B, int Hkv, int T, int D,
                                      int block_size, int dtype, void* stream) {
  return nsa_block_compress_strided_fwd(x, intra_pos, pool_logits, proj_w, out, B, Hkv, T, D, block_size,
                                        block_size, dtype, stream);
}

extern "C" int nsa_block_compress_strided_fwd(const void* x, const float* intra_pos,
                                              const float* pool_logits, const float* proj_w, void* out,
                                              int B, int Hkv, int T, int D, int block_size, int stride,
                                              int dtype, void* stream) {
  NSA_CHECK_ARG(block_size > 0 && D > 0 && D <= 1024, "bad block_size/D");
  NSA_CHECK_ARG(stride > 0 && stride <= block_size, "stride must be in [1, block_size]");
  const int n_blk = n_windows(T, block_size, stride);
  const size_t ctas = (size_t)B * Hkv * n_blk;
  if (ctas == 0) return NSA_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const size_t sm = (size_t)(block_size + D) * sizeof(float);
  if (compress_fast_ok(D, block_size, dtype)) {
    const size_t fsm = compress_fast_fwd_smem(D, block_size, true);
    NSA_CUDA_OK(cudaFuncSetAttribute(compress_fast_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fsm));
    KernelScope ks("compress_fast_fwd_kernel", st);
    compress_fast_fwd_kernel<<<(unsigned)((ctas + kCompRows - 1) / kCompRows), kCompThreads, fsm, st>>>(
        (const __nv_bfloat16*)x, intra_pos, pool_logits, proj_w, (__nv_bfloat16*)out, (float*)nullptr, T, D,
        block_size, stride, n_blk, ctas);
  } else if (dtype == NSA_DTYPE_BF16)
    { KernelScope ks("compress_fwd_kernel", st); compress_fwd_kernel<<<(unsigned)ctas, (D + 31) / 32 * 32, sm, st>>>((const __nv_bfloat16*)x, intra_pos, pool_logits, proj_w, (__nv_bfloat16*)out, (float*)nullptr, T, D, block_size, stride, n_blk); }
  else
    { KernelScope ks("compress_fwd_kernel", st); compress_fwd_kernel<<<(unsigned)ctas, (D + 31) / 32 * 32, sm, st>>>((const float*)x, intra_pos, pool_logits, proj_w, (float*)out, (float*)nullptr, T, D, block_size, stride, n_blk); }
  NSA_LAUNCH_OK("compress_fwd_kernel");
  return NSA_OK;
}

extern "C" size_t nsa_block_compress_bwd_workspace_bytes(int B, int Hkv, int T, int D, int block_size) {
  return nsa_block_compress_strided_bwd_workspace_bytes(B, Hkv, T, D, block_size, block_size);
}

extern "C" size_t nsa_block_compress_strided_bwd_workspace_bytes(int B, int Hkv, int T, int D,
                                                                 int block_size, int stride) {
  const size_t rows = (size_t)B * Hkv * (block_size > 0 && stride > 0 ? n_windows(T, block_size, stride) : 0);
  // pooled[rows,D] + d_pooled[rows,D] + sum_dpooled[D] + d_w[block_size]
  return align_up((2 * rows * D + D + block_size) * sizeof(float), 256);
}

extern "C" int nsa_block_compress_bwd(const void* x, const float* intra_pos, const float* pool_logits,
                                      const float* proj_w, const void* d_out, void* dx,
                                      float* d_intra_pos, float* d_pool_logits, float* d_proj_w,
                                      int B, int Hkv, int T, int D, int block_size, int dtype,
                                      void* workspace, size_t workspace_bytes, void* stream) {
  return nsa_block_compress_strided_bwd(x, intra_pos, pool_logits, proj_w, d_out, dx, d_intra_pos,
                                        d_pool_logits, d_proj_w, B, Hkv, T, D, block_size, block_size,
                                        dtype, workspace, workspace_bytes, stream);
}

extern "C" int nsa_block_compress_strided_bwd(const void* x, const float* intra_pos,
                                              const float* pool_logits, const float* proj_w,
                                              const void* d_out, void* dx, float* d_intra_pos,
                                              float* d_pool_logits, float* d_proj_w, int B, int Hkv,
                                              int T, int D, int block_size, int stride, int dtype,
                                              void* workspace, size_t workspace_bytes, void* stream) {
  NSA_CHECK_ARG(block_size > 0 && D > 0 && D <= 1024, "bad block_size/D");
  NSA_CHECK_ARG(stride > 0 && stride <= block_size, "stride must be in [1, block_size]");
  const int n_blk = n_windows(T, block_size, stride);
  const size_t rows = (size_t)B * Hkv * n_blk;
  cudaStream_t st = (cudaStream_t)stream;
  if (workspace_bytes < nsa_block_compress_strided_bwd_workspace_bytes(B, Hkv, T, D, block_size, stride) || !workspace) {
    set_error("compress bwd workspace too small");
    return NSA_ERR_WORKSPACE;
  }
  float* pooled = (float*)workspace;
  float* d_pooled = pooled + rows * D;
  float* sum_dp = d_pooled + rows * D;
  float* d_w = sum_dp + D;
  NSA_CUDA_OK(cudaMemsetAsync(sum_dp, 0, (size_t)(D + block_size) * sizeof(float), st));
  const size_t sm_f = (size_t)(block_size + D) * sizeof(float);
  const size_t sm_b = (size_t)(block_size + D + 32) * sizeof(float);
  const bool overlap = stride < block_size;
  const size_t tail = overlap ? 0 : (size_t)(T - n_blk * block_size) * D * B * Hkv;
  NSA_CUDA_OK(cudaMemsetAsync(d_proj_w, 0, (size_t)D * D * sizeof(float), st));
  const dim3 pgrid(D, (unsigned)(rows >= 4096 ? 64 : (rows >= 64 ? rows / 64 : 1)));
  const bool fast = compress_fast_ok(D, block_size, dtype);
  if (rows > 0) {
    if (fast) {
      const size_t fsm = compress_fast_fwd_smem(D, block_size, false), bsm = compress_fast_bwd_smem(D, block_size);
      NSA_CUDA_OK(cudaFuncSetAttribute(compress_fast_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)compress_fast_fwd_smem(D, block_size, true)));
      NSA_CUDA_OK(cudaFuncSetAttribute(compress_fast_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bsm));
      const unsigned grid = (unsigned)((rows + kCompRows - 1) / kCompRows);
      { KernelScope ks("compress_fast_fwd_kernel", st);
        compress_fast_fwd_kernel<<<grid, kCompThreads, fsm, st>>>((const __nv_bfloat16*)x, intra_pos, pool_logits, proj_w,
                                                                 (__nv_bfloat16*)nullptr, pooled, T, D, block_size, stride, n_blk, rows); }
      { KernelScope ks("compress_fast_bwd_kernel", st);
        compress_fast_bwd_kernel<<<grid, kCompThreads, bsm, st>>>((const __nv_bfloat16*)x, pool_logits, proj_w,
                                                                 (const __nv_bfloat16*)d_out, (__nv_bfloat16*)dx, d_pooled,
                                                                 sum_dp, d_w, T, D, block_size, stride, n_blk, rows); }
      { KernelScope ks("compress_bwd_proj_kernel", st); compress_bwd_proj_kernel<<<pgrid, (D + 31) / 32 * 32, 0, st>>>((const __nv_bfloat16*)d_out, pooled, d_proj_w, rows, D); }
    } else if (dtype == NSA_DTYPE_BF16) {
      { KernelScope ks("compress_fwd_kernel", st); compress_fwd_kernel<<<(unsigned)rows, (D + 31) / 32 * 32, sm_f, st>>>((const __nv_bfloat16*)x, intra_pos, pool_logits, proj_w, (__nv_bfloat16*)nullptr, pooled, T, D, block_size, stride, n_blk); }
      { KernelScope ks("compress_bwd_block_kernel", st); compress_bwd_block_kernel<<<(unsigned)rows, (D + 31) / 32 * 32, sm_b, st>>>((const __nv_bfloat16*)x, intra_pos, pool_logits, proj_w, (const __nv_bfloat16*)d_out, (__nv_bfloat16*)dx, d_pooled, sum_dp, d_w, T, D, block_size, stride, n_blk); }
      { KernelScope ks("compress_bwd_proj_kernel", st); compress_bwd_proj_kernel<<<pgrid, (D + 31) / 32 * 32, 0, st>>>((const __nv_bfloat16*)d_out, pooled, d_proj_w, rows, D); }
    } else {
      { KernelScope ks("compress_fwd_kernel", st); compress_fwd_kernel<<<(unsigned)rows, (D + 31) / 32 * 32, sm_f, st>>>((const float*)x, intra_pos, pool_logits, proj_w, (float*)nullptr, pooled, T, D, block_size, stride, n_blk); }
      { KernelScope ks("compress_bwd_block_kernel", st); compress_bwd_block_kernel<<<(unsigned)rows, (D + 31) / 32 * 32, sm_b, st>>>((const float*)x, intra_pos, pool_logits, proj_w, (const float*)d_out, (float*)dx, d_pooled, sum_dp, d_w, T, D, block_size, stride, n_blk); }
      { KernelScope ks("compress_bwd_proj_kernel", st); compress_bwd_proj_kernel<<<pgrid, (D + 31) / 32 * 32, 0, st>>>((const float*)d_out, pooled, d_proj_w, rows, D); }
    }
    NSA_LAUNCH_OK("compress_bwd kernels");
  }
  if (overlap) {   // every token of dx is written here (tokens in no window: 0)
    const size_t n = (size_t)B * Hkv * T * D;
    if (n && rows == 0) NSA_CUDA_OK(cudaMemsetAsync(dx, 0, n * (dtype == NSA_DTYPE_BF16 ? 2 : 4), st));
    if (n && rows) {
      KernelScope ks("compress_dx_kernel", st);
      if (dtype == NSA_DTYPE_BF16 && D % 8 == 0)
        compress_dx_vec_kernel<<<blocks_for(n / 8, 256), 256, block_size * sizeof(float), st>>>(d_pooled, pool_logits, (__nv_bfloat16*)dx, T, D, block_size, stride, n_blk, n / 8);
      else if (dtype == NSA_DTYPE_BF16)
        compress_dx_kernel<<<blocks_for(n, 256), 256, block_size * sizeof(float), st>>>(d_pooled, pool_logits, (__nv_bfloat16*)dx, T, D, block_size, stride, n_blk, n);
      else
        compress_dx_kernel<<<blocks_for(n, 256), 256, block_size * sizeof(float), st>>>(d_pooled, pool_logits, (float*)dx, T, D, block_size, stride, n_blk, n);
      NSA_LAUNCH_OK("compress_dx_kernel");
    }
  }
  if (tail > 0) {
    if (dtype == NSA_DTYPE_BF16)
      { KernelScope ks("zero_tail_kernel", st); zero_tail_kernel<<<blocks_for(tail, 256), 256, 0, st>>>((__nv_bfloat16*)dx, T, D, n_blk * block_size, (size_t)B * Hkv); }
    else
      { KernelScope ks("zero_tail_kernel", st); zero_tail_kernel<<<blocks_for(tail, 256), 256, 0, st>>>((float*)dx, T, D, n_blk * block_size, (size_t)B * Hkv); }
    NSA_LAUNCH_OK("zero_tail_kernel");
  }
  { KernelScope ks("compress_bwd_final_kernel", st); compress_bwd_final_kernel<<<1, 256, block_size * sizeof(float), st>>>(pool_logits, sum_dp, d_w, fast && rows > 0 ? intra_pos : nullptr, d_intra_pos, d_pool_logits, D, block_size); }
  NSA_LAUNCH_OK("compress_bwd_final_kernel");
  return NSA_OK;
}

namespace nsa {
bool tc_topn_ok(const NsaDims& d, int n_blk, int n_sel, int cmp_len, int stride, int sel_block);
int tc_topn(const void* q, const void* k_cmp, const float* lse, int32_t* block_idx, float* imp_out,
            const NsaDims& d, int n_blk, int block_size, int n_sel, int n_init, int n_local, int stride,
            int sel_block, int imp_cols, cudaStream_t st);
}

extern "C" int nsa_topn_blocks(const void* q, const void* k_cmp, const float* lse_cmp,
                               int32_t* block_idx, float* importance_out, const NsaDims* dims,
                               int n_blk, int block_size, int n_sel, int impl, void* stream) {
  return nsa_topn_blocks_forced(q, k_cmp, lse_cmp, block_idx, importance_out, dims, n_blk, block_size,
                                n_sel, 0, 0, impl, stream);
}

extern "C" int nsa_topn_blocks_forced(const void* q, const void* k_cmp, const float* lse_cmp,
                                      int32_t* block_idx, float* importance_out, const NsaDims* dims,
                                      int n_blk, int block_size, int n_sel, int n_init, int n_local,
                                      int impl, void* stream) {
  return nsa_topn_blocks_general(q, k_cmp, lse_cmp, block_idx, importance_out, dims, n_blk, block_size,
                                 block_size, block_size, n_sel, n_init, n_local, impl, stream);
}

extern "C" int nsa_topn_blocks_general(const void* q, const void* k_cmp, const float* lse_cmp,
                                       int32_t* block_idx, float* importance_out, const NsaDims* dims,
                                       int n_cmp, int cmp_len, int cmp_stride, int sel_block, int n_sel,
                                       int n_init, int n_local, int impl, void* stream) {
  const int n_blk = n_cmp, block_size = cmp_len;
  NSA_CHECK_ARG(dims && q && lse_cmp && block_idx && (k_cmp || n_blk == 0), "null argument");
  NSA_CHECK_ARG(n_init >= 0 && n_local >= 0 && n_init < (1 << 18) && n_local < (1 << 18), "bad forced block counts");
  NSA_CHECK_ARG(dims->Hkv > 0 && dims->Hq % dims->Hkv == 0, "Hq must be a multiple of Hkv");
  NSA_CHECK_ARG(block_size > 0 && n_sel > 0 && n_blk >= 0, "bad block_size/n_sel/n_blk");
  NSA_CHECK_ARG(cmp_stride > 0 && cmp_stride <= cmp_len && cmp_len % cmp_stride == 0 && sel_block > 0 &&
                sel_block % cmp_stride == 0, "summary length and selection block must be multiples of the stride");
  const bool aligned = cmp_len == cmp_stride && cmp_stride == sel_block;
  const int n_sblk = (dims->T + sel_block - 1) / sel_block;
  const int imp_cols = aligned ? n_blk : n_sblk;     // the aligned call keeps its [.., n_blk] layout
  const int D = dims->D;
  cudaStream_t st = (cudaStream_t)stream;
  const size_t units = (size_t)dims->B * dims->Hkv * dims->T;
  if (units == 0) return NSA_OK;
  if (impl != NSA_IMPL_SIMT) {
    if (tc_topn_ok(*dims, n_blk, n_sel, cmp_len, cmp_stride, sel_block))
      return tc_topn(q, k_cmp, lse_cmp, block_idx, importance_out, *dims, n_blk, block_size, n_sel, n_init,
                     n_local, cmp_stride, sel_block, imp_cols, st);
    if (impl == NSA_IMPL_TC) {
      set_error("scoring shape not served by the tcgen05 kernel");
      return NSA_ERR_UNSUPPORTED;
    }
  }
  const size_t sm = (size_t)4 * (D + n_blk + n_sblk + 1) * sizeof(float);
  NSA_CHECK_ARG(sm <= 200 * 1024, "n_blk %d too large for the scoring kernel", n_blk);
  const float scale = 1.0f / sqrtf((float)D);
  const unsigned grid = blocks_for(units, 4);
#define NSA_TOPN(TT, DD)                                                                        \
  do {                                                                                          \
    if (sm > 48 * 1024)                                                                         \
      NSA_CUDA_OK(cudaFuncSetAttribute(topn_kernel<TT, DD>,                                     \
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm));  \
    KernelScope ks("topn_kernel", st);                                                          \
    topn_kernel<TT, DD><<<grid, 128, sm, st>>>((const TT*)q, (const TT*)k_cmp, lse_cmp,         \
        block_idx, importance_out, dims->B, dims->Hq, dims->Hkv, dims->T, n_blk, block_size,    \
        n_sel, n_init, n_local, scale, cmp_stride, sel_block, n_sblk, imp_cols);                \
  } while (0)
  if (dims->dtype == NSA_DTYPE_BF16) {
    switch (D) {
      case 16: NSA_TOPN(__nv_bfloat16, 16); break;
      case 32: NSA_TOPN(__nv_bfloat16, 32); break;
      case 64: NSA_TOPN(__nv_bfloat16, 64); break;
      case 128: NSA_TOPN(__nv_bfloat16, 128); break;
      default: set_error("head dim %d unsupported", D); return NSA_ERR_UNSUPPORTED;
    }
  } else {
    switch (D) {
      case 16: NSA_TOPN(float, 16); break;
      case 32: NSA_TOPN(float, 32); break;
      case 64: NSA_TOPN(float, 64); break;
      case 128: NSA_TOPN(float, 128); break;
      default: set_error("head dim %d unsupported", D); return NSA_ERR_UNSUPPORTED;
    }
  }
#undef NSA_TOPN
  NSA_LAUNCH_OK("topn_kernel");
  return NSA_OK;
}

extern "C" size_t nsa_csr_workspace_bytes(int B, int Hkv, int T, int S, int block_size) {
  (void)S;
  const size_t n_blk = block_size > 0 ? (T + block_size - 1) / block_size : 0;
  const size_t rows = (size_t)B * Hkv * n_blk;
  const size_t words = (T + 31) / 32;
  return 2 * align_up(rows * words * 4, 256) + 2 * align_up(rows * 4, 256);
}

namespace nsa {
// CSR over n_blk blocks (the public entry point uses T / block_size, as the reference does;
// the tcgen05 backward also counts a ragged tail block).  pair_of_slot, when given, receives
// for every (b, hkv, t, slot) the pair index of that selection or -1.
int build_csr_internal(const int32_t* block_idx, int B, int Hkv, int T, int S, int block_size,
                       int n_blk, int32_t* q_of_block, int32_t* block_offsets, int32_t* pair_bh,
                       int32_t* pair_of_slot, void* workspace, size_t workspace_bytes, cudaStream_t st) {
  const size_t rows = (size_t)B * Hkv * n_blk;
  const int words = (T + 31) / 32;
  if ((size_t)B * Hkv == 0) return NSA_OK;
  if (rows == 0) {
    NSA_CUDA_OK(cudaMemsetAsync(block_offsets, 0, (size_t)B * Hkv * sizeof(int32_t), st));
    return NSA_OK;
  }
  const size_t need = 2 * align_up(rows * words * 4, 256) + 2 * align_up(rows * 4, 256);
  if (!workspace || workspace_bytes < need) {
    set_error("csr workspace too small");
    return NSA_ERR_WORKSPACE;
  }
  uint32_t* bitmap = (uint32_t*)workspace;
  int32_t* prefix = (int32_t*)((char*)workspace + align_up(rows * words * 4, 256));
  int32_t* counts = (int32_t*)((char*)prefix + align_up(rows * words * 4, 256));
  int32_t* row_start = (int32_t*)((char*)counts + align_up(rows * 4, 256));
  NSA_CUDA_OK(cudaMemsetAsync(bitmap, 0, rows * words * 4, st));
  const size_t n_entries = (size_t)B * Hkv * T * S;
  if (n_entries) {
    KernelScope ks("csr_mark_kernel", st);
    csr_mark_kernel<<<blocks_for(n_entries, 256), 256, 0, st>>>(block_idx, bitmap, T, S, block_size, n_blk, words, n_entries);
  }
  { KernelScope ks("csr_count_kernel", st); csr_count_kernel<<<blocks_for(rows, 8), 256, 0, st>>>(bitmap, counts, prefix, words, rows); }
  { KernelScope ks("csr_scan_kernel", st); csr_scan_kernel<<<1, 1024, 0, st>>>(counts, block_offsets, row_start, n_blk, rows); }
  if (n_entries) {
    KernelScope ks("csr_fill_kernel", st);
    csr_fill_kernel<<<blocks_for(n_entries, 256), 256, 0, st>>>(block_idx, bitmap, prefix, row_start, q_of_block, pair_bh, pair_of_slot, T, S, block_size, n_blk, words, n_entries);
  }
  NSA_LAUNCH_OK("csr kernels");
  return NSA_OK;
}
}  // namespace nsa

extern "C" int nsa_build_block_to_query_csr(const int32_t* block_idx, int B, int Hkv, int T, int S,
                                            int block_size, int32_t* q_of_block,
                                            int32_t* block_offsets, int32_t* pair_bh, void* workspace,
                                            size_t workspace_bytes, void* stream) {
  NSA_CHECK_ARG(block_size > 0 && B >= 0 && Hkv >= 0 && T >= 0 && S >= 0, "bad sizes");
  return build_csr_internal(block_idx, B, Hkv, T, S, block_size, T / block_size, q_of_block,
                            block_offsets, pair_bh, nullptr, workspace, workspace_bytes,
                            (cudaStream_t)stream);
}

// ---- CSR without caller-provided scratch -----------------------------------------------------
// The scratch of the CSR build (bitmap, bit-rank prefixes, counts, row starts) lives in this fixed
// device array.
// In host code the array's name is only a handle: the device address is looked up once per
// device with cudaGetSymbolAddress and that pointer is what the kernels receive.
constexpr size_t kCsrBuiltinScratchBytes = (size_t)8 << 20;
static __device__ __align__(256) unsigned char g_csr_builtin_scratch[kCsrBuiltinScratchBytes];

extern "C" size_t nsa_csr_builtin_scratch_bytes(void) { return kCsrBuiltinScratchBytes; }

extern "C" int nsa_build_block_to_query_csr_noalloc(const int32_t* block_idx, int B, int Hkv, int T,
                                                    int S, int block_size, int32_t* q_of_block,
                                                    int32_t* block_offsets, int32_t* pair_bh,
                                                    void* stream) {
  NSA_CHECK_ARG(block_size > 0 && B >= 0 && Hkv >= 0 && T >= 0 && S >= 0, "bad sizes");
  const size_t need = nsa_csr_workspace_bytes(B, Hkv, T, S, block_size);
  if (need > kCsrBuiltinScratchBytes) {
    set_error("this CSR needs %zu bytes of scratch but the built-in scratch holds %zu: use "
              "nsa_build_block_to_query_csr with a caller-provided workspace", need,
              kCsrBuiltinScratchBytes);
    return NSA_ERR_WORKSPACE;
  }
  // one address per device, published with release / acquire so that threads of a multi-threaded
  // host may race on the first call (each would look up the same address)
  static std::atomic<void*> scratch_of_device[64];
  int dev = 0;
  NSA_CUDA_OK(cudaGetDevice(&dev));
  NSA_CHECK_ARG(dev >= 0 && dev < 64, "device ordinal %d out of range", dev);
  void* scratch = scratch_of_device[dev].load(std::memory_order_acquire);
  if (scratch == nullptr) {   // first call on this device, with it current
    NSA_CUDA_OK(cudaGetSymbolAddress(&scratch, g_csr_builtin_scratch));
    scratch_of_device[dev].store(scratch, std::memory_order_release);
  }
  return build_csr_internal(block_idx, B, Hkv, T, S, block_size, T / block_size, q_of_block,
                            block_offsets, pair_bh, nullptr, scratch,
                            kCsrBuiltinScratchBytes, (cudaStream_t)stream);
}

extern "C" int nsa_gate_combine_bwd_rows(const void* o_cmp, const void* o_slc, const void* o_win,
                                         const void* gate_logits, const void* d_out, float* row_scale,
                                         float* row_dot, void* d_gate_logits, const NsaDims* dims,
                                         void* stream) {
  NSA_CHECK_ARG(dims && row_scale && row_dot && d_gate_logits, "null argument");
  const size_t rows = (size_t)dims->B * dims->Hq * dims->T;
  if (rows == 0) return NSA_OK;
  cudaStream_t st = (cudaStream_t)stream;
  KernelScope ks("gate_bwd_rows_kernel", st);
  if (gate_vec_ok(dims->D, dims->dtype))
    gate_bwd_rows_vec_kernel<<<blocks_for(rows * (dims->D / 8), 256), 256, 0, st>>>((const __nv_bfloat16*)o_cmp, (const __nv_bfloat16*)o_slc, (const __nv_bfloat16*)o_win, (const __nv_bfloat16*)gate_logits, (const __nv_bfloat16*)d_out, row_scale, row_dot, (__nv_bfloat16*)d_gate_logits, rows, dims->D / 8);
  else if (dims->dtype == NSA_DTYPE_BF16)
    gate_bwd_rows_kernel<<<blocks_for(rows, 8), 256, 0, st>>>((const __nv_bfloat16*)o_cmp, (const __nv_bfloat16*)o_slc, (const __nv_bfloat16*)o_win, (const __nv_bfloat16*)gate_logits, (const __nv_bfloat16*)d_out, row_scale, row_dot, (__nv_bfloat16*)d_gate_logits, rows, dims->D);
  else
    gate_bwd_rows_kernel<<<blocks_for(rows, 8), 256, 0, st>>>((const float*)o_cmp, (const float*)o_slc, (const float*)o_win, (const float*)gate_logits, (const float*)d_out, row_scale, row_dot, (float*)d_gate_logits, rows, dims->D);
  NSA_LAUNCH_OK("gate_bwd_rows_kernel");
  return NSA_OK;
}

extern "C" int nsa_sum3(const void* a, const void* b, const void* c, void* out, size_t n, int dtype,
                        void* stream) {
  if (n == 0) return NSA_OK;
  NSA_CHECK_ARG(a && b && c && out, "null tensor");
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == NSA_DTYPE_BF16) {
    NSA_CHECK_ARG(n % 8 == 0, "element count must be a multiple of 8");
    KernelScope ks("sum3_kernel", st);
    sum3_bf16_kernel<<<blocks_for(n / 8, 256), 256, 0, st>>>((const uint4*)a, (const uint4*)b, (const uint4*)c, (uint4*)out, n / 8);
  } else {
    KernelScope ks("sum3_kernel", st);
    sum3_f32_kernel<<<blocks_for(n, 256), 256, 0, st>>>((const float*)a, (const float*)b, (const float*)c, (float*)out, n);
  }
  NSA_LAUNCH_OK("sum3_kernel");
  return NSA_OK;
}

// ---- projection glue: one pass between the fused projection's [B,T,W] rows and the head-major
// tensors the attention kernels take ------------------------------------------------------------
namespace nsa {
namespace {
// A row of the fused projection holds, for one token: q (Hq*D), then kc, vc, ks, vs, kw, vw (Hkv*D
// each), then the gate logits (3*Hq, padded to a multiple of 8 elements).  `to_heads`: rows -> q
// [B,Hq,T,D], kv [6][B,Hkv,T,D], gate [B,Hq,T,3]; else the other way (gradients), the padding zeroed.
template <typename T, typename V>   // V: the 16-byte vector of T
__global__ void split_heads_kernel(T* __restrict__ y, T* __restrict__ q, T* __restrict__ kv, T* __restrict__ gate,
                                   int B, int Tn, int Hq, int Hkv, int D, int W, int to_heads, size_t n_vec) {
  constexpr int kPer = 16 / (int)sizeof(T);                 // elements per vector
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_vec) return;
  const int wv = W / kPer;
  const int col = (int)(i % wv) * kPer;
  const size_t bt = i / wv;
  const int t = (int)(bt % Tn), b = (int)(bt / Tn);
  V* row = reinterpret_cast<V*>(y + bt * W + col);
  const int n_attn = (Hq + 6 * Hkv) * D;
  if (col < n_attn) {
    T* dst;
    if (col < Hq * D) {
      const int h = col / D, d = col % D;
      dst = q + (((size_t)b * Hq + h) * Tn + t) * D + d;
    } else {
      const int c2 = col - Hq * D;
      const int which = c2 / (Hkv * D), c3 = c2 % (Hkv * D);
      const int h = c3 / D, d = c3 % D;
      dst = kv + ((((size_t)which * B + b) * Hkv + h) * Tn + t) * D + d;
    }
    if (to_heads) *reinterpret_cast<V*>(dst) = *row;
    else *row = *reinterpret_cast<const V*>(dst);
  } else {
    T tmp[kPer];
    if (to_heads) *reinterpret_cast<V*>(tmp) = *row;
#pragma unroll
    for (int e = 0; e < kPer; ++e) {
      const int c = col - n_attn + e;                       // h * 3 + branch
      if (c < 3 * Hq) {
        T* g = gate + ((((size_t)b * Hq + c / 3) * Tn + t) * 3 + c % 3);
        if (to_heads) *g = tmp[e]; else tmp[e] = *g;
      } else if (!to_heads) {
        tmp[e] = T(0.f);
      }
    }
    if (!to_heads) *row = *reinterpret_cast<const V*>(tmp);
  }
}

// [B,H,T,D] <-> [B,T,H,D], 16 bytes per thread
template <typename V>
__global__ void swap_heads_tokens_kernel(const V* __restrict__ src, V* __restrict__ dst, int H, int Tn, int Dv,
                                         int to_tokens, size_t n_vec) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;    // over dst vectors
  if (i >= n_vec) return;
  const int d = (int)(i % Dv);
  const size_t r = i / Dv;
  size_t s;
  if (to_tokens) {                                          // dst [B,T,H,D]
    const int h = (int)(r % H);
    const size_t bt = r / H;
    const int t = (int)(bt % Tn);
    const size_t b = bt / Tn;
    s = ((b * H + h) * Tn + t) * Dv + d;
  } else {                                                  // dst [B,H,T,D]
    const int t = (int)(r % Tn);
    const size_t bh = r / Tn;
    const int h = (int)(bh % H);
    const size_t b = bh / H;
    s = ((b * Tn + t) * H + h) * Dv + d;
  }
  dst[i] = __ldg(src + s);
}
}  // namespace
}  // namespace nsa

extern "C" int nsa_fused_projection_width(int Hq, int Hkv, int D) {
  return (Hq + 6 * Hkv) * D + (3 * Hq + 7) / 8 * 8;
}

static int split_or_merge(void* y, void* q, void* kv, void* gate, int B, int T, int Hq, int Hkv, int D, int dtype,
                          int to_heads, void* stream) {
  NSA_CHECK_ARG(B >= 0 && T >= 0 && Hq > 0 && Hkv > 0 && D > 0 && D % 8 == 0, "bad sizes");
  NSA_CHECK_ARG(dtype == NSA_DTYPE_BF16 || dtype == NSA_DTYPE_F32, "bad dtype %d", dtype);
  const int W = nsa_fused_projection_width(Hq, Hkv, D);
  const size_t rows = (size_t)B * T;
  if (rows == 0) return NSA_OK;
  NSA_CHECK_ARG(y && q && kv && gate, "null tensor");
  cudaStream_t st = (cudaStream_t)stream;
  KernelScope ks(to_heads ? "split_heads_kernel" : "merge_heads_kernel", st);
  if (dtype == NSA_DTYPE_BF16) {
    const size_t n = rows * (W / 8);
    split_heads_kernel<__nv_bfloat16, uint4><<<blocks_for(n, 256), 256, 0, st>>>(
        (__nv_bfloat16*)y, (__nv_bfloat16*)q, (__nv_bfloat16*)kv, (__nv_bfloat16*)gate, B, T, Hq, Hkv, D, W, to_heads, n);
  } else {
    const size_t n = rows * (W / 4);
    split_heads_kernel<float, float4><<<blocks_for(n, 256), 256, 0, st>>>(
        (float*)y, (float*)q, (float*)kv, (float*)gate, B, T, Hq, Hkv, D, W, to_heads, n);
  }
  NSA_LAUNCH_OK("split_heads_kernel");
  return NSA_OK;
}

extern "C" int nsa_split_heads(const void* y, void* q, void* kv, void* gate, int B, int T, int Hq, int Hkv, int D,
                               int dtype, void* stream) {
  return split_or_merge(const_cast<void*>(y), q, kv, gate, B, T, Hq, Hkv, D, dtype, 1, stream);
}

extern "C" int nsa_merge_heads(const void* dq, const void* dkv, const void* dgate, void* dy, int B, int T, int Hq,
                               int Hkv, int D, int dtype, void* stream) {
  return split_or_merge(dy, const_cast<void*>(dq), const_cast<void*>(dkv), const_cast<void*>(dgate), B, T, Hq, Hkv,
                        D, dtype, 0, stream);
}

extern "C" int nsa_swap_heads_tokens(const void* src, void* dst, int B, int H, int T, int D, int dtype,
                                     int to_tokens, void* stream) {
  NSA_CHECK_ARG(B >= 0 && T >= 0 && H > 0 && D > 0 && D % 8 == 0, "bad sizes");
  NSA_CHECK_ARG(dtype == NSA_DTYPE_BF16 || dtype == NSA_DTYPE_F32, "bad dtype %d", dtype);
  const int Dv = dtype == NSA_DTYPE_BF16 ? D / 8 : D / 4;
  const size_t n = (size_t)B * H * T * Dv;
  if (n == 0) return NSA_OK;
  NSA_CHECK_ARG(src && dst, "null tensor");
  cudaStream_t st = (cudaStream_t)stream;
  KernelScope ks("swap_heads_tokens_kernel", st);
  swap_heads_tokens_kernel<uint4><<<blocks_for(n, 256), 256, 0, st>>>((const uint4*)src, (uint4*)dst, H, T, Dv,
                                                                       to_tokens, n);
  NSA_LAUNCH_OK("swap_heads_tokens_kernel");
  return NSA_OK;
}

extern "C" int nsa_gate_combine_fwd(const void* o_cmp, const void* o_slc, const void* o_win,
                                    const void* gate_logits, void* out, const NsaDims* dims,
                                    void* stream) {
  NSA_CHECK_ARG(dims, "null dims");
  const size_t rows = (size_t)dims->B * dims->Hq * dims->T;
  if (rows == 0) return NSA_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (gate_vec_ok(dims->D, dims->dtype))
    { KernelScope ks("gate_fwd_kernel", st); gate_fwd_vec_kernel<<<blocks_for(rows * (dims->D / 8), 256), 256, 0, st>>>((const __nv_bfloat16*)o_cmp, (const __nv_bfloat16*)o_slc, (const __nv_bfloat16*)o_win, (const __nv_bfloat16*)gate_logits, (__nv_bfloat16*)out, rows, dims->D / 8); }
  else if (dims->dtype == NSA_DTYPE_BF16)
    { KernelScope ks("gate_fwd_kernel", st); gate_fwd_kernel<<<blocks_for(rows, 8), 256, 0, st>>>((const __nv_bfloat16*)o_cmp, (const __nv_bfloat16*)o_slc, (const __nv_bfloat16*)o_win, (const __nv_bfloat16*)gate_logits, (__nv_bfloat16*)out, rows, dims->D); }
  else
    { KernelScope ks("gate_fwd_kernel", st); gate_fwd_kernel<<<blocks_for(rows, 8), 256, 0, st>>>((const float*)o_cmp, (const float*)o_slc, (const float*)o_win, (const float*)gate_logits, (float*)out, rows, dims->D); }
  NSA_LAUNCH_OK("gate_fwd_kernel");
  return NSA_OK;
}

extern "C" int nsa_gate_combine_bwd(const void* o_cmp, const void* o_slc, const void* o_win,
                                    const void* gate_logits, const void* d_out, void* do_cmp,
                                    void* do_slc, void* do_win, void* d_gate_logits,
                                    const NsaDims* dims, void* stream) {
  NSA_CHECK_ARG(dims, "null dims");
  const size_t rows = (size_t)dims->B * dims->Hq * dims->T;
  if (rows == 0) return NSA_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (dims->dtype == NSA_DTYPE_BF16)
    { KernelScope ks("gate_bwd_kernel", st); gate_bwd_kernel<<<blocks_for(rows, 8), 256, 0, st>>>((const __nv_bfloat16*)o_cmp, (const __nv_bfloat16*)o_slc, (const __nv_bfloat16*)o_win, (const __nv_bfloat16*)gate_logits, (const __nv_bfloat16*)d_out, (__nv_bfloat16*)do_cmp, (__nv_bfloat16*)do_slc, (__nv_bfloat16*)do_win, (__nv_bfloat16*)d_gate_logits, rows, dims->D); }
  else
    { KernelScope ks("gate_bwd_kernel", st); gate_bwd_kernel<<<blocks_for(rows, 8), 256, 0, st>>>((const float*)o_cmp, (const float*)o_slc, (const float*)o_win, (const float*)gate_logits, (const float*)d_out, (float*)do_cmp, (float*)do_slc, (float*)do_win, (float*)d_gate_logits, rows, dims->D); }
  NSA_LAUNCH_OK("gate_bwd_kernel");
  return NSA_OK;
}
