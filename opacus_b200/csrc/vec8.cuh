// 8-wide typed loads and stores for the streaming kernels: KIND 0 = fp32 (two 16-byte accesses),
// 1 = bf16, 2 = fp16 (one 16-byte access).  Indices are in elements; the address must be 16-byte aligned.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace dpk {

template <int KIND>
__device__ __forceinline__ void vload8(const void* base, int64_t idx, float (&v)[8]) {
  if constexpr (KIND == 0) {
    const float4* p = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + idx);
    const float4 a = p[0], b = p[1];
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  } else {
    const uint4 raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(base) + idx);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      if constexpr (KIND == 1) {
        const __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162*>(&w[q]);
        v[2 * q] = __bfloat162float(h.x); v[2 * q + 1] = __bfloat162float(h.y);
      } else {
        const __half2 h = *reinterpret_cast<const __half2*>(&w[q]);
        v[2 * q] = __half2float(h.x); v[2 * q + 1] = __half2float(h.y);
      }
    }
  }
}
template <int KIND>
__device__ __forceinline__ void vstore8(void* base, int64_t idx, const float (&v)[8]) {
  if constexpr (KIND == 0) {
    float4* p = reinterpret_cast<float4*>(reinterpret_cast<float*>(base) + idx);
    p[0] = make_float4(v[0], v[1], v[2], v[3]);
    p[1] = make_float4(v[4], v[5], v[6], v[7]);
  } else {
    uint4 pk;
    uint32_t* w = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      if constexpr (KIND == 1) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * q], v[2 * q + 1]);
        w[q] = *reinterpret_cast<const uint32_t*>(&h);
      } else {
        const __half2 h = __floats2half2_rn(v[2 * q], v[2 * q + 1]);
        w[q] = *reinterpret_cast<const uint32_t*>(&h);
      }
    }
    *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(base) + idx) = pk;
  }
}

template <int KIND>
__device__ __forceinline__ float vload1(const void* base, int64_t idx) {
  if constexpr (KIND == 0) return reinterpret_cast<const float*>(base)[idx];
  else if constexpr (KIND == 1) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[idx]);
  else return __half2float(reinterpret_cast<const __half*>(base)[idx]);
}
template <int KIND>
__device__ __forceinline__ void vstore1(void* base, int64_t idx, float v) {
  if constexpr (KIND == 0) reinterpret_cast<float*>(base)[idx] = v;
  else if constexpr (KIND == 1) reinterpret_cast<__nv_bfloat16*>(base)[idx] = __float2bfloat16(v);
  else reinterpret_cast<__half*>(base)[idx] = __float2half(v);
}

}  // namespace dpk
