// Host-side construction of TMA tensor maps.  The driver entry point is resolved at run time
// through the CUDA runtime, so the library links against no driver stub.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace nx {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// Row-major tensor [d2][d1][d0] (d0 innermost), 128-byte swizzle, zero fill out of bounds.
// `ld1` = elements between consecutive d1 rows, `ld2` = elements between d2 slices (0 when d2 == 1).
// The box is {box0, box1, 1}; box0 * elem_bytes must be 128.
inline int make_tensor_map_3d(CUtensorMap* out, CUtensorMapDataType dt, int elem_bytes, const void* base,
                              uint64_t d0, uint64_t d1, uint64_t d2, uint64_t ld1, uint64_t ld2, uint32_t box0,
                              uint32_t box1, CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return -3;
  if (d2 <= 1) {
    d2 = 1;
    ld2 = ld1 * d1;
  }
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {ld1 * elem_bytes, ld2 * elem_bytes};
  cuuint32_t box[3] = {box0, box1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -4;
}

// General 4-D map [d3][d2][d1][d0] with explicit element strides for d1..d3; box {box0, box1, box2, 1}.
inline int make_tensor_map_4d(CUtensorMap* out, CUtensorMapDataType dt, int elem_bytes, const void* base,
                              uint64_t d0, uint64_t d1, uint64_t d2, uint64_t d3, uint64_t ld1, uint64_t ld2,
                              uint64_t ld3, uint32_t box0, uint32_t box1, uint32_t box2,
                              CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return -3;
  cuuint64_t dims[4] = {d0, d1, d2, d3};
  cuuint64_t strides[3] = {ld1 * elem_bytes, ld2 * elem_bytes, ld3 * elem_bytes};
  cuuint32_t box[4] = {box0, box1, box2, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(out, dt, 4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -4;
}

}  // namespace nx
