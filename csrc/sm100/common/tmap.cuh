// Host-side construction of TMA tensor maps without linking libcuda: the driver entry
// point is fetched through the runtime once per process.
#pragma once

#include <cstdint>
#include <cstdio>
#include <cuda.h>
#include <cuda_runtime.h>

namespace ka {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

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

// Row-major [rows, cols] matrix of 2-byte elements; box = [box_rows, box_cols] with the
// 128-byte swizzle (box_cols * 2 bytes must be 128). Out-of-range elements read as zero.
// `row_stride_elems` is the distance between rows in elements (>= cols, multiple of 8).
inline int make_tmap_2d_16bit_sw128(CUtensorMap* map, CUtensorMapDataType dt, const void* base,
                                    uint64_t rows, uint64_t cols, uint64_t row_stride_elems,
                                    uint32_t box_rows, uint32_t box_cols) {
  EncodeTiledFn fn = get_encode_tiled();
  if (!fn) return -1;
  // The encode call is a driver entry point and needs the tensor's context current on this
  // thread. A host thread that has not touched CUDA yet (an autograd worker, for one) has
  // none: bind the device the tensor lives on.
  {
    cudaPointerAttributes at;
    if (cudaPointerGetAttributes(&at, base) == cudaSuccess && at.type == cudaMemoryTypeDevice)
      cudaSetDevice(at.device);
    else
      cudaGetLastError();
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0 || (row_stride_elems * 2) % 16 != 0) return -2;
  cuuint64_t gdim[2] = {cols, rows};
  cuuint64_t gstride[1] = {row_stride_elems * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, dt, 2, const_cast<void*>(base), gdim, gstride, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -100 - static_cast<int>(r);
}

}  // namespace ka
