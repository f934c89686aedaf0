// Host-side construction of TMA tensor maps.  The driver entry point is resolved at run time
// through the CUDA runtime, so the library has no link-time dependency on libcuda and can be
// loaded (for symbol checks) on a machine without a GPU driver.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace mpsa {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn resolve_encode_tiled() {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
      q == cudaDriverEntryPointSuccess)
    return (EncodeTiledFn)p;
  return nullptr;
}
inline EncodeTiledFn get_encode_tiled() {
  static const EncodeTiledFn fn = resolve_encode_tiled();   // initialised once, thread-safe
  return fn;
}

// 2-D byte tensor [rows, row_bytes] with pitch `pitch_bytes`, boxes of box_rows x box_bytes.
// Returns 0 on success.  The base must be 16-byte aligned, the pitch a multiple of 16, and
// box_bytes at most the swizzle span.
inline int make_tmap_2d_bytes(CUtensorMap* m, const void* base, uint64_t row_bytes, uint64_t rows,
                              uint64_t pitch_bytes, uint32_t box_bytes, uint32_t box_rows, CUtensorMapSwizzle sw) {
  EncodeTiledFn fn = get_encode_tiled();
  if (!fn) return -1;
  cuuint64_t dims[2] = {row_bytes, rows};
  cuuint64_t strides[1] = {pitch_bytes};
  cuuint32_t box[2] = {box_bytes, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

// 2-D tensor of 16-bit elements [rows, cols] with pitch in bytes; box_cols*2 <= swizzle span.
inline int make_tmap_2d_b16(CUtensorMap* m, const void* base, uint64_t cols, uint64_t rows, uint64_t pitch_bytes,
                            uint32_t box_cols, uint32_t box_rows, CUtensorMapSwizzle sw) {
  EncodeTiledFn fn = get_encode_tiled();
  if (!fn) return -1;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {pitch_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

}  // namespace mpsa
