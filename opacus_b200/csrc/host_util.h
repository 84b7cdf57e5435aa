// Host-side helpers shared by the kernel launchers: TMA tensor-map encoding
// (the driver entry point is looked up at run time, so nothing links against
// libcuda) and a cached SM count.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cudaTypedefs.h>
#include <stdint.h>

namespace dpk {

inline PFN_cuTensorMapEncodeTiled_v12000 tmap_encoder() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  }
  return fn;
}

// [d2][d1][d0] tensor of 16-bit elements, d0 contiguous; box = (b0, b1, 1); 128-byte swizzle; zero fill.
inline int make_tmap_3d_bf16(CUtensorMap* map, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint32_t b0,
                             uint32_t b1) {
  auto enc = tmap_encoder();
  if (!enc) return cudaErrorNotSupported;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || ((d0 * 2) & 15) != 0) return cudaErrorInvalidValue;
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {d0 * 2, d0 * d1 * 2};
  cuuint32_t box[3] = {b0, b1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : cudaErrorInvalidValue;
}

// [d1][d0] tensor of 16-bit elements, d0 contiguous; box = (b0, b1).
inline int make_tmap_2d_bf16(CUtensorMap* map, const void* base, uint64_t d0, uint64_t d1, uint32_t b0, uint32_t b1) {
  auto enc = tmap_encoder();
  if (!enc) return cudaErrorNotSupported;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || ((d0 * 2) & 15) != 0) return cudaErrorInvalidValue;
  cuuint64_t dims[2] = {d0, d1};
  cuuint64_t strides[1] = {d0 * 2};
  cuuint32_t box[2] = {b0, b1};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : cudaErrorInvalidValue;
}

// [d3][d2][d1][d0] tensor of 16-bit elements, d0 contiguous (an NHWC image batch: d0 = channels, d1 = width,
// d2 = height, d3 = sample).  The box takes 64 channels and n1 x n2 pixels that are s1 / s2 elements apart
// (a strided convolution's input positions); 128-byte swizzle; zero fill outside the tensor.
inline int make_tmap_4d_bf16(CUtensorMap* map, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t d3,
                             uint32_t n1, uint32_t n2, uint32_t s1, uint32_t s2) {
  auto enc = tmap_encoder();
  if (!enc) return cudaErrorNotSupported;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || ((d0 * 2) & 15) != 0) return cudaErrorInvalidValue;
  if (n1 * s1 > 256 || n2 * s2 > 256 || s1 < 1 || s2 < 1 || s1 > 8 || s2 > 8) return cudaErrorInvalidValue;
  cuuint64_t dims[4] = {d0, d1, d2, d3};
  cuuint64_t strides[3] = {d0 * 2, d0 * d1 * 2, d0 * d1 * d2 * 2};
  cuuint32_t box[4] = {64, n1 * s1, n2 * s2, 1};
  cuuint32_t estr[4] = {1, s1, s2, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : cudaErrorInvalidValue;
}

inline int num_sms() {
  static int cached[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (cached[dev] == 0) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    cached[dev] = n > 0 ? n : 1;
  }
  return cached[dev];
}

}  // namespace dpk
