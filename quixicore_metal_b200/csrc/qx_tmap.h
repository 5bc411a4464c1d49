// Host-side construction of the TMA tensor maps the kernels use for packed weight matrices.
#pragma once

#include <cstdint>

#include <cuda.h>
#include <cuda_runtime.h>

namespace qx {

// Tensor map over a packed weight matrix seen as V rows of 32-bit words, box = (box_bytes / 4) words x
// box_rows rows; rows past the end read as zeros.  The driver entry point is looked up at run time, so the library does not link libcuda.
typedef CUresult (*TensorMapEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                      const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                      CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                      CUtensorMapFloatOOBfill);
inline TensorMapEncodeFn tensor_map_encode_fn() {
  static TensorMapEncodeFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess) {
      cudaGetLastError();
      return (TensorMapEncodeFn) nullptr;
    }
    return (TensorMapEncodeFn)p;
  }();
  return fn;
}
inline bool make_weight_map(CUtensorMap* map, const void* w, int64_t V, size_t row_bytes, int box_bytes,
                            int box_rows = 128) {
  TensorMapEncodeFn enc = tensor_map_encode_fn();
  if (!enc) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)(row_bytes / 4), (cuuint64_t)V};
  const cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
  const cuuint32_t box[2] = {(cuuint32_t)(box_bytes / 4), (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1u, 1u};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(w), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// The same through a small cache keyed by (device, base, rows, row bytes, box): see qx_scratch.cu.
bool cached_weight_map(CUtensorMap* map, const void* w, int64_t rows, size_t row_bytes, int box_bytes,
                       int box_rows = 128);

}  // namespace qx
