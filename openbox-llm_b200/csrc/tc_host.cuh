// Host-side helpers of the tcgen05 kernels: TMA tensor-map creation through the driver entry
// point (no link-time dependency on libcuda) and the row-tile geometry.
#pragma once

#include "tc_common.cuh"

namespace nsa {
namespace tc {

// ---- host side -------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) ==
            cudaSuccess && qres == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)ptr;
  }
  return fn;
}

// 3-D map over a [heads, rows, D] bf16 tensor: box = 64 elements x box_rows x box_heads
static inline int make_map(CUtensorMap* m, const void* base, int D, int rows, int heads, int box_rows,
                    int box_heads) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) { set_error("cuTensorMapEncodeTiled is not available"); return NSA_ERR_CUDA; }
  cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)rows, (cuuint64_t)heads};
  cuuint64_t strides[2] = {(cuuint64_t)D * 2, (cuuint64_t)rows * D * 2};
  cuuint32_t box[3] = {64u, (cuuint32_t)box_rows, (cuuint32_t)box_heads};
  cuuint32_t estr[3] = {1u, 1u, 1u};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled failed with %d", (int)r); return NSA_ERR_CUDA; }
  return NSA_OK;
}

// 3-D map over the same [heads, T, D] tensor with the head index as second dimension and the
// token index as third: a box of 64 elements x G heads x 1 token brings the G rows of one query
// of a GQA group into G consecutive 128-byte rows of shared memory.
static inline int make_map_query_rows(CUtensorMap* m, const void* base, int D, int T, int heads, int G,
                                      int box_tokens = 1) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) { set_error("cuTensorMapEncodeTiled is not available"); return NSA_ERR_CUDA; }
  cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)heads, (cuuint64_t)T};
  cuuint64_t strides[2] = {(cuuint64_t)T * D * 2, (cuuint64_t)D * 2};
  cuuint32_t box[3] = {64u, (cuuint32_t)G, (cuuint32_t)box_tokens};
  cuuint32_t estr[3] = {1u, 1u, 1u};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled (query rows) failed with %d", (int)r); return NSA_ERR_CUDA; }
  return NSA_OK;
}

// 5-D map over a [heads, T, D] bf16 tensor (D = 128, heads a multiple of 8) whose box brings ALL of one
// query's rows in one go: 64 elements x 8 heads x 2 column slabs x 1 token x G/8 head groups.  In
// shared memory the box is laid out [head group][slab][8 heads][128 bytes]: every (head group, slab)
// is one 1024-byte swizzle atom, the two slabs of an 8-row group are neighbours and consecutive
// 8-row groups are 2048 bytes apart.
static inline int make_map_query_both_slabs(CUtensorMap* m, const void* base, int T, int heads, int G) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) { set_error("cuTensorMapEncodeTiled is not available"); return NSA_ERR_CUDA; }
  const cuuint64_t row = 128 * 2;
  cuuint64_t dims[5] = {64u, 8u, 2u, (cuuint64_t)T, (cuuint64_t)(heads / 8)};
  cuuint64_t strides[4] = {(cuuint64_t)T * row, 128u, row, (cuuint64_t)8 * T * row};
  cuuint32_t box[5] = {64u, 8u, 2u, 1u, (cuuint32_t)(G / 8)};
  cuuint32_t estr[5] = {1u, 1u, 1u, 1u, 1u};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled (query, both slabs) failed with %d", (int)r); return NSA_ERR_CUDA; }
  return NSA_OK;
}

// 5-D map over a bf16 partial buffer [outer][mid][slots][G][D] for stores of boxes
// 64 elements x G x 1 x box_mid x 1: the G rows of box_mid consecutive `mid` entries of one slot.
static inline int make_map_partial(CUtensorMap* m, void* base, int D, int G, size_t slots, size_t mid,
                                   size_t outer, int box_mid) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) { set_error("cuTensorMapEncodeTiled is not available"); return NSA_ERR_CUDA; }
  cuuint64_t dims[5] = {(cuuint64_t)D, (cuuint64_t)G, (cuuint64_t)slots, (cuuint64_t)mid, (cuuint64_t)outer};
  const cuuint64_t row = (cuuint64_t)D * 2;
  cuuint64_t strides[4] = {row, row * G, row * G * slots, row * G * slots * mid};
  cuuint32_t box[5] = {64u, (cuuint32_t)G, 1u, (cuuint32_t)box_mid, 1u};
  cuuint32_t estr[5] = {1u, 1u, 1u, 1u, 1u};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, base, dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled (partials) failed with %d", (int)r); return NSA_ERR_CUDA; }
  return NSA_OK;
}

// 4-D map over the fp32 dQ accumulator [units][T][G][D] for reductions of boxes
// 32 floats x G x box_tokens x 1: the G rows of box_tokens consecutive queries, one 128-byte
// column slab at a time.
static inline int make_map_dq_acc(CUtensorMap* m, void* base, int D, int G, size_t T, size_t units,
                                  int box_tokens) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) { set_error("cuTensorMapEncodeTiled is not available"); return NSA_ERR_CUDA; }
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)G, (cuuint64_t)T, (cuuint64_t)units};
  const cuuint64_t row = (cuuint64_t)D * 4;
  cuuint64_t strides[3] = {row, row * G, row * G * T};
  cuuint32_t box[4] = {32u, (cuuint32_t)G, (cuuint32_t)box_tokens, 1u};
  cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, base, dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled (dq accumulator) failed with %d", (int)r); return NSA_ERR_CUDA; }
  return NSA_OK;
}

static inline int group_pad(int G) {
  int gp = 1;
  while (gp < G) gp <<= 1;
  return gp;
}


}  // namespace tc
}  // namespace nsa
