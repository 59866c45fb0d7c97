// Optimizer step of the data-parallel training step: the squared gradient norm, the clip factor
// and AdamW over flat fp32 buffers, with no host synchronisation in between (the reference's
// step is torch.nn.utils.clip_grad_norm_ + torch.optim.AdamW, train.py:148-149 and :262-264).
// Streaming kernels: 16 bytes read and 12 written per parameter.
#include "common.cuh"

namespace nsa {
namespace {

__global__ void sumsq_kernel(const float* __restrict__ x, size_t n, float* __restrict__ out) {
  float acc = 0.f;
  const size_t n4 = n / 4;
  const float4* x4 = reinterpret_cast<const float4*>(x);
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
    const float4 v = __ldg(x4 + i);
    acc = fmaf(v.x, v.x, acc); acc = fmaf(v.y, v.y, acc); acc = fmaf(v.z, v.z, acc); acc = fmaf(v.w, v.w, acc);
  }
  if (blockIdx.x == 0 && threadIdx.x < (int)(n - n4 * 4)) {
    const float v = x[n4 * 4 + threadIdx.x];
    acc = fmaf(v, v, acc);
  }
  acc = warp_sum(acc);
  __shared__ float part[32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) part[warp] = acc;
  __syncthreads();
  if (warp == 0) {
    float v = lane < (int)(blockDim.x >> 5) ? part[lane] : 0.f;
    v = warp_sum(v);
    if (lane == 0) atomicAdd(out, v);
  }
}

// torch.optim.AdamW semantics (decoupled weight decay, bias-corrected moments); the gradient is
// first multiplied by grad_scale (1 / world size after a summing all-reduce) and by the clip factor
// min(1, max_norm / (grad_scale * sqrt(sumsq) + 1e-6)) of torch.nn.utils.clip_grad_norm_.
__global__ void adamw_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m,
                             float* __restrict__ v, size_t n, float lr, float beta1, float beta2,
                             float eps, float weight_decay, float bc1, float bc2_sqrt,
                             const float* __restrict__ sumsq, float max_norm, float grad_scale) {
  float clip = 1.f;
  if (sumsq && max_norm > 0.f) {
    const float norm = grad_scale * sqrtf(__ldg(sumsq));
    clip = fminf(1.f, max_norm / (norm + 1e-6f));
  }
  const float gs = grad_scale * clip;
  const float step_size = lr / bc1;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const float gi = g[i] * gs;
    float pi = p[i] * (1.f - lr * weight_decay);
    const float mi = beta1 * m[i] + (1.f - beta1) * gi;
    const float vi = beta2 * v[i] + (1.f - beta2) * gi * gi;
    pi -= step_size * mi / (sqrtf(vi) / bc2_sqrt + eps);
    p[i] = pi; m[i] = mi; v[i] = vi;
  }
}

}  // namespace
}  // namespace nsa

using namespace nsa;

extern "C" int nsa_sumsq_f32(const float* x, size_t n, float* accum, void* stream) {
  if (n == 0) return NSA_OK;
  NSA_CHECK_ARG(x && accum, "null argument");
  NSA_CHECK_ARG(((uintptr_t)x & 15) == 0, "x must be 16-byte aligned");
  cudaStream_t st = (cudaStream_t)stream;
  const unsigned grid = (unsigned)std::min<size_t>((n / 4 + 255) / 256 + 1, 148 * 8);
  KernelScope ks("sumsq_kernel", st);
  sumsq_kernel<<<grid, 256, 0, st>>>(x, n, accum);
  NSA_LAUNCH_OK("sumsq_kernel");
  return NSA_OK;
}

extern "C" int nsa_adamw_step_f32(float* p, const float* g, float* m, float* v, size_t n, float lr,
                                  float beta1, float beta2, float eps, float weight_decay, int step,
                                  const float* sumsq, float max_norm, float grad_scale, void* stream) {
  if (n == 0) return NSA_OK;
  NSA_CHECK_ARG(p && g && m && v, "null argument");
  NSA_CHECK_ARG(step >= 1, "step counts from 1");
  cudaStream_t st = (cudaStream_t)stream;
  const float bc1 = 1.f - powf(beta1, (float)step);
  const float bc2_sqrt = sqrtf(1.f - powf(beta2, (float)step));
  const unsigned grid = (unsigned)std::min<size_t>((n + 255) / 256, 148 * 16);
  KernelScope ks("adamw_kernel", st);
  adamw_kernel<<<grid, 256, 0, st>>>(p, g, m, v, n, lr, beta1, beta2, eps, weight_decay, bc1, bc2_sqrt, sumsq,
                                     max_norm, grad_scale);
  NSA_LAUNCH_OK("adamw_kernel");
  return NSA_OK;
}
