// Host-side construction of TMA tensor maps (CUtensorMap) without a link-time dependency on
// libcuda: the encoder entry point is resolved through the CUDA runtime.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>
#include <stdexcept>
#include <string>
#include <unordered_map>

namespace tb {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || p == nullptr)
      throw std::runtime_error("cuTensorMapEncodeTiled is not available from the CUDA driver");
    fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// 3-D tiled map over a [d2][d1][d0] array (d0 contiguous). Strides in BYTES for d1 and d2 (multiples of
// 16). Boxes are {b0, b1, 1}. 128-byte swizzle when b0 * elem_bytes == 128, 64-byte swizzle when it is 64, none otherwise.
inline CUtensorMap make_tmap_3d(const void* base, CUtensorMapDataType dt, int elem_bytes, uint64_t d0, uint64_t d1,
                                uint64_t d2, uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t b0,
                                uint32_t b1) {
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) throw std::runtime_error("TMA base must be 16-byte aligned");
  if ((stride1_bytes & 15) != 0 || (stride2_bytes & 15) != 0)
    throw std::runtime_error("TMA strides must be multiples of 16 bytes");
  if (b0 > 256 || b1 > 256) throw std::runtime_error("TMA box dims must be <= 256");
  CUtensorMap m;
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
  cuuint32_t box[3] = {b0, b1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUtensorMapSwizzle sw = (b0 * elem_bytes == 128) ? CU_TENSOR_MAP_SWIZZLE_128B
                          : (b0 * elem_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_NONE);
  CUresult r = get_encode_fn()(&m, dt, 3, const_cast<void*>(base), dims, strides, box, estr,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) throw std::runtime_error("cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
  return m;
}

}  // namespace tb
