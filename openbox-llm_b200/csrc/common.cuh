// Shared host/device helpers of libnsa_b200: error reporting, dtype loads, launch checks.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/nsa_b200.h"

namespace nsa {
// Compression summaries: summary j covers tokens [j * stride, j * stride + len); query t sees
// the summaries that end at or before t (nsa_model.py:233-235 for stride == len).
__host__ __device__ __forceinline__ int cmp_visible(int t, int len, int stride, int n_summaries) {
  if (t + 1 < len) return 0;
  const int n = (t + 1 - len) / stride + 1;
  return n < n_summaries ? n : n_summaries;
}

// Rank keys of forced selection blocks: above every importance (a sum of at most G <= 128
// probabilities), initial blocks ahead of local ones, exact in fp32 for counts below 2^18.
constexpr float kForcedInit = 1048576.f;    // - block index
constexpr float kForcedLocal = 524288.f;    // - distance from the block holding the query

void set_error(const char* fmt, ...);

#define NSA_CHECK_ARG(cond, ...)            \
  do {                                      \
    if (!(cond)) {                          \
      nsa::set_error(__VA_ARGS__);          \
      return NSA_ERR_BAD_ARG;               \
    }                                       \
  } while (0)

#define NSA_CUDA_OK(expr)                                                        \
  do {                                                                           \
    cudaError_t _e = (expr);                                                     \
    if (_e != cudaSuccess) {                                                     \
      nsa::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e),     \
                     __FILE__, __LINE__);                                        \
      return NSA_ERR_CUDA;                                                       \
    }                                                                            \
  } while (0)

#define NSA_LAUNCH_OK(name)                                                      \
  do {                                                                           \
    cudaError_t _e = cudaGetLastError();                                         \
    if (_e != cudaSuccess) {                                                     \
      nsa::set_error("launch of %s failed: %s", name, cudaGetErrorString(_e));   \
      return NSA_ERR_CUDA;                                                       \
    }                                                                            \
  } while (0)

constexpr float kLseEmpty = -1.0e9f;  // nsa_selection_kernel.py:134,171
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

__device__ __forceinline__ float to_float(float x) { return x; }
__device__ __forceinline__ float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }
template <typename T> __device__ __forceinline__ T from_float(float x);
template <> __device__ __forceinline__ float from_float<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float x) {
  return __float2bfloat16_rn(x);
}

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}
__device__ __forceinline__ float warp_max(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
  return x;
}

// error word raised by kernels whose bounded waits run out; defined in api.cu
int* device_status_ptr();

// Per-kernel accounting (api.cu): every kernel launch of the library sits inside a KernelScope,
// which counts it and, when profiling is on, brackets it with CUDA events on its stream.
void kernel_begin(const char* name, cudaStream_t st);
void kernel_end(cudaStream_t st);
struct KernelScope {
  cudaStream_t st;
  KernelScope(const char* name, cudaStream_t s) : st(s) { kernel_begin(name, s); }
  ~KernelScope() { kernel_end(st); }
};

// kernel names carry the branch they serve: <prefix>_win / _cmp / _slc
inline const char* branch_name(const char* const names[3], int kind) { return names[kind == 0 ? 0 : (kind == 1 ? 1 : 2)]; }

// ---- SIMT kernel family (simt.cu) ---------------------------------------------------------
struct AttnArgs {
  const void* q; const void* k; const void* v; const int32_t* block_idx;
  void* o; float* lse;
  const void* d_o; void* dq; float* dk_acc; float* dv_acc;   // backward
  const float* row_scale; const float* row_dot;   // backward of a gated branch (may be null)
  float* dq_acc;     // tcgen05 window / compression backward: fp32 accumulator [B*Hkv][T][G][D] that takes dQ (or null)
  const void* sel_plan;   // tcgen05 selection: CSR + pair map + work list built earlier (tc_sel_plan_build), or null
  int B, Hq, Hkv, T, Lk, D, S;
  int kind;          // 0 window, 1 compress, 2 selection
  int window, block_size;
  float scale;
};
int simt_attn_fwd(const AttnArgs& a, int dtype, cudaStream_t st);
int simt_attn_bwd(const AttnArgs& a, int dtype, cudaStream_t st);
int cast_f32_to(const float* src, void* dst, size_t n, int dtype, cudaStream_t st);

// ---- tcgen05 kernel family (tc.cu) ----------------------------------------------------------
bool tc_shape_ok(const NsaDims& d, int block_size);
int tc_attn_fwd(const AttnArgs& a, cudaStream_t st);
size_t tc_sel_fwd_workspace(const AttnArgs& a);
int tc_sel_fwd(const AttnArgs& a, void* ws, size_t ws_bytes, cudaStream_t st);
size_t tc_sel_plan_bytes(const AttnArgs& a);
int tc_sel_plan_build(const AttnArgs& a, void* plan, size_t plan_bytes, cudaStream_t st);
size_t tc_attn_bwd_workspace(const AttnArgs& a);
int tc_attn_bwd(const AttnArgs& a, void* ws, size_t ws_bytes, cudaStream_t st);
int tc_dq_reduce3(const AttnArgs& base, int Lk_cmp, int cmp_len, int cmp_stride, int S, int block_size,
                  int window, const void* ws_cmp, const void* ws_slc, const void* ws_win,
                  const float* dq_acc, void* dq, cudaStream_t st);

}  // namespace nsa
