// Host-side construction of TMA tensor maps without linking libcuda: the encode function is
// looked up through the runtime (cudaGetDriverEntryPoint), so the library still loads on a
// machine without a driver.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace flare {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode_tiled() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// Map of a 16-bit [d3][d2][rows][D] tensor (unit stride on D, byte strides for the others) with a
// box of {D, box_rows, 1, 1} and the swizzle that matches a row of 2*D bytes.
// dtype16: 0 = fp16, 1 = bf16.  Returns false when the driver rejects the description.
inline bool make_tile_map(CUtensorMap* map, const void* base, int dtype16, int D, uint64_t rows, uint64_t d2,
                          uint64_t d3, uint64_t stride_row_b, uint64_t stride_d2_b, uint64_t stride_d3_b,
                          uint32_t box_rows) {
  EncodeTiledFn enc = get_encode_tiled();
  if (!enc) return false;
  cuuint64_t dims[4] = {(cuuint64_t)D, rows, d2, d3};
  cuuint64_t strides[3] = {stride_row_b, stride_d2_b, stride_d3_b};
  cuuint32_t box[4] = {(cuuint32_t)D, box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  const int rowb = 2 * D;
  CUtensorMapSwizzle sw = rowb == 32 ? CU_TENSOR_MAP_SWIZZLE_32B
                          : rowb == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B;
  CUresult r = enc(map, dtype16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                   const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// Same tensor, but a box of `box_cols` of its D columns (a multiple of 8; 2 * box_cols bytes per tile row, which picks the
// swizzle): rows wider than one 128-byte swizzle span are fetched as several column blocks, each a tile of its own.
inline bool make_tile_map_cols(CUtensorMap* map, const void* base, int dtype16, int D, int box_cols, uint64_t rows,
                               uint64_t d2, uint64_t d3, uint64_t stride_row_b, uint64_t stride_d2_b,
                               uint64_t stride_d3_b, uint32_t box_rows) {
  EncodeTiledFn enc = get_encode_tiled();
  if (!enc) return false;
  cuuint64_t dims[4] = {(cuuint64_t)D, rows, d2, d3};
  cuuint64_t strides[3] = {stride_row_b, stride_d2_b, stride_d3_b};
  cuuint32_t box[4] = {(cuuint32_t)box_cols, box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  const int rowb = 2 * box_cols;
  if (rowb != 32 && rowb != 64 && rowb != 128) return false;
  CUtensorMapSwizzle sw = rowb == 32 ? CU_TENSOR_MAP_SWIZZLE_32B
                          : rowb == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B;
  CUresult r = enc(map, dtype16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                   const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

}  // namespace flare
