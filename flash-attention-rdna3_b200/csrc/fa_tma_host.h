// Host-side construction of the TMA tensor maps the tcgen05 kernels read their operands through.
// cuTensorMapEncodeTiled is looked up at run time through the CUDA runtime, so the library does not
// link against the driver library.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "fa_common.cuh"

namespace fa {

typedef CUresult (*TensorMapEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                      const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                      CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline TensorMapEncodeFn tensor_map_encoder() {
  static TensorMapEncodeFn fn = []() -> TensorMapEncodeFn {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess) return nullptr;
    if (q != cudaDriverEntryPointSuccess) return nullptr;
    return reinterpret_cast<TensorMapEncodeFn>(ptr);
  }();
  return fn;
}

// A 16-bit operand (batch, head, row, dim) can be read by TMA when its inner stride is one element,
// its base is 16-byte aligned and every other stride is a multiple of 16 bytes.
// sizes = (batch, heads, rows): a dimension of size one may carry any stride.
inline bool tma_operand_ok(const void* ptr, const int64_t strides[4], const int64_t sizes[3]) {
  if (ptr == nullptr || (reinterpret_cast<uintptr_t>(ptr) & 15)) return false;
  if (strides[3] != 1) return false;
  for (int i = 0; i < 3; ++i) {
    if (sizes[i] <= 1) continue;
    if (strides[i] <= 0 || (strides[i] % 8) != 0) return false;
  }
  return true;
}

// Tensor map over (dim, rows, heads, batch) with a box of 64 elements x box_rows rows and the 128-byte
// swizzle; out-of-range rows read as zero. Strides are in elements.
inline int make_tile_map(CUtensorMap* map, const void* ptr, int dtype, int head_dim, int64_t rows, int64_t heads,
                         int64_t batch, int64_t stride_row, int64_t stride_head, int64_t stride_batch,
                         int box_rows = 128) {
  TensorMapEncodeFn enc = tensor_map_encoder();
  if (enc == nullptr) return set_error(FA_ERR_DEVICE, "cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t dims[4] = {(cuuint64_t)head_dim, (cuuint64_t)rows, (cuuint64_t)heads, (cuuint64_t)batch};
  // a size-1 dimension never advances; give it any legal stride
  const int64_t legal = (int64_t)head_dim;
  auto bytes = [&](int64_t s, int64_t n) { return (cuuint64_t)((n > 1 && s > 0) ? s : legal) * 2; };
  const cuuint64_t strides[3] = {bytes(stride_row, rows), bytes(stride_head, heads), bytes(stride_batch, batch)};
  const cuuint32_t box[4] = {64, (cuuint32_t)box_rows, 1, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUtensorMapDataType dt = (dtype == FA_BF16) ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUresult r = enc(map, dt, 4, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_error(FA_ERR_LAUNCH, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  return 0;
}

// The same for fp32 operands: a box of 32 elements (128 bytes) x box_rows rows. Base 16-byte aligned, strides (in
// elements) multiples of 4.
inline int make_tile_map_f32(CUtensorMap* map, const void* ptr, int head_dim, int64_t rows, int64_t heads, int64_t batch,
                             int64_t stride_row, int64_t stride_head, int64_t stride_batch, int box_rows = 128) {
  TensorMapEncodeFn enc = tensor_map_encoder();
  if (enc == nullptr) return set_error(FA_ERR_DEVICE, "cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t dims[4] = {(cuuint64_t)head_dim, (cuuint64_t)rows, (cuuint64_t)heads, (cuuint64_t)batch};
  const int64_t legal = (int64_t)head_dim;
  auto bytes = [&](int64_t s, int64_t n) { return (cuuint64_t)((n > 1 && s > 0) ? s : legal) * 4; };
  const cuuint64_t strides[3] = {bytes(stride_row, rows), bytes(stride_head, heads), bytes(stride_batch, batch)};
  const cuuint32_t box[4] = {32, (cuuint32_t)box_rows, 1, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_error(FA_ERR_LAUNCH, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  return 0;
}

}  // namespace fa
