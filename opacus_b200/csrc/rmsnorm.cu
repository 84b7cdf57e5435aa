// Residual add fused with RMSNorm, one pass each way (rows of up to 8192 elements, a multiple of 8):
//
//   forward : h = x + delta   (delta may be absent: h = x, not rewritten)
//             y = h * rsqrt(mean(h^2) + eps) * w ,  rstd kept per row
//   backward: dh = dres + rstd * (dy*w) - h * rstd^3 * <dy*w, h> / D     (dres may be absent)
//
// h is rounded to the storage type before the statistics are taken, so forward and backward see the same values.
// Replaces the separate add / rms_norm / rms_norm_backward / gradient-accumulation kernels around every norm
// of the decoder.  Part of this package's Llama model, not of the DP machinery.
#include "api.h"
#include "common.cuh"
#include "vec8.cuh"

namespace dpk {
namespace {

constexpr int RN_THREADS = 256;
constexpr int RN_MAX_ITERS = 4;       // 256 threads x 8 elements x 4 = 8192

__device__ __forceinline__ float rn_block_sum(float v, float* sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) sh[w] = v;
  __syncthreads();
  float t = l < RN_THREADS / 32 ? sh[l] : 0.f;
#pragma unroll
  for (int o = 4; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  return __shfl_sync(0xffffffffu, t, 0);
}

template <int KIND>
__device__ __forceinline__ float rn_round(float v) {
  if constexpr (KIND == 1) return __bfloat162float(__float2bfloat16(v));
  else if constexpr (KIND == 2) return __half2float(__float2half(v));
  else return v;
}

template <int KIND>
__global__ void __launch_bounds__(RN_THREADS)
add_rmsnorm_fwd_kernel(const void* x, const void* delta, const void* w, void* h_out, void* y_out, float* rstd_out,
                       int64_t D, float eps) {
  __shared__ float sh[RN_THREADS / 32];
  const int64_t base = (int64_t)blockIdx.x * D;
  float h[RN_MAX_ITERS][8];
  float ss = 0.f;
#pragma unroll
  for (int it = 0; it < RN_MAX_ITERS; ++it) {
    const int64_t i = ((int64_t)it * RN_THREADS + threadIdx.x) * 8;
    if (i < D) {
      vload8<KIND>(x, base + i, h[it]);
      if (delta != nullptr) {
        float d[8];
        vload8<KIND>(delta, base + i, d);
#pragma unroll
        for (int q = 0; q < 8; ++q) h[it][q] = rn_round<KIND>(h[it][q] + d[q]);
        vstore8<KIND>(h_out, base + i, h[it]);
      }
#pragma unroll
      for (int q = 0; q < 8; ++q) ss = fmaf(h[it][q], h[it][q], ss);
    }
  }
  ss = rn_block_sum(ss, sh);
  const float rstd = rsqrtf(ss / (float)D + eps);
  if (threadIdx.x == 0) rstd_out[blockIdx.x] = rstd;
#pragma unroll
  for (int it = 0; it < RN_MAX_ITERS; ++it) {
    const int64_t i = ((int64_t)it * RN_THREADS + threadIdx.x) * 8;
    if (i < D) {
      float wv[8], y[8];
      vload8<KIND>(w, i, wv);
#pragma unroll
      for (int q = 0; q < 8; ++q) y[q] = h[it][q] * rstd * wv[q];
      vstore8<KIND>(y_out, base + i, y);
    }
  }
}

template <int KIND>
__global__ void __launch_bounds__(RN_THREADS)
add_rmsnorm_bwd_kernel(const void* dy, const void* dres, const void* h, const float* rstd_in, const void* w,
                       void* dh_out, int64_t D) {
  __shared__ float sh[RN_THREADS / 32];
  const int64_t base = (int64_t)blockIdx.x * D;
  float g[RN_MAX_ITERS][8], hv[RN_MAX_ITERS][8];
  float dot = 0.f;
#pragma unroll
  for (int it = 0; it < RN_MAX_ITERS; ++it) {
    const int64_t i = ((int64_t)it * RN_THREADS + threadIdx.x) * 8;
    if (i < D) {
      float wv[8];
      vload8<KIND>(dy, base + i, g[it]);
      vload8<KIND>(h, base + i, hv[it]);
      vload8<KIND>(w, i, wv);
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        g[it][q] *= wv[q];
        dot = fmaf(g[it][q], hv[it][q], dot);
      }
    }
  }
  dot = rn_block_sum(dot, sh);
  const float rstd = rstd_in[blockIdx.x];
  const float k = rstd * rstd * rstd * dot / (float)D;
#pragma unroll
  for (int it = 0; it < RN_MAX_ITERS; ++it) {
    const int64_t i = ((int64_t)it * RN_THREADS + threadIdx.x) * 8;
    if (i < D) {
      float out[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) out[q] = rstd * g[it][q] - hv[it][q] * k;
      if (dres != nullptr) {
        float r[8];
        vload8<KIND>(dres, base + i, r);
#pragma unroll
        for (int q = 0; q < 8; ++q) out[q] += r[q];
      }
      vstore8<KIND>(dh_out, base + i, out);
    }
  }
}

}  // namespace
}  // namespace dpk

extern "C" int dpk_add_rmsnorm_forward(const void* x, const void* delta, const void* w, void* h_out, void* y_out,
                                       float* rstd_out, int kind, int64_t rows, int64_t D, float eps,
                                       cudaStream_t stream) {
  using namespace dpk;
  if (rows <= 0) return 0;
  if (D <= 0 || (D & 7) || D > RN_THREADS * 8 * RN_MAX_ITERS || kind < 0 || kind > 2 || rows > 0x7fffffffLL)
    return cudaErrorInvalidValue;
  if (delta != nullptr && h_out == nullptr) return cudaErrorInvalidValue;
  if (kind == 0) add_rmsnorm_fwd_kernel<0><<<(unsigned)rows, RN_THREADS, 0, stream>>>(x, delta, w, h_out, y_out, rstd_out, D, eps);
  else if (kind == 1) add_rmsnorm_fwd_kernel<1><<<(unsigned)rows, RN_THREADS, 0, stream>>>(x, delta, w, h_out, y_out, rstd_out, D, eps);
  else add_rmsnorm_fwd_kernel<2><<<(unsigned)rows, RN_THREADS, 0, stream>>>(x, delta, w, h_out, y_out, rstd_out, D, eps);
  return cudaGetLastError();
}

extern "C" int dpk_add_rmsnorm_backward(const void* dy, const void* dres, const void* h, const float* rstd,
                                        const void* w, void* dh_out, int kind, int64_t rows, int64_t D,
                                        cudaStream_t stream) {
  using namespace dpk;
  if (rows <= 0) return 0;
  if (D <= 0 || (D & 7) || D > RN_THREADS * 8 * RN_MAX_ITERS || kind < 0 || kind > 2 || rows > 0x7fffffffLL)
    return cudaErrorInvalidValue;
  if (kind == 0) add_rmsnorm_bwd_kernel<0><<<(unsigned)rows, RN_THREADS, 0, stream>>>(dy, dres, h, rstd, w, dh_out, D);
  else if (kind == 1) add_rmsnorm_bwd_kernel<1><<<(unsigned)rows, RN_THREADS, 0, stream>>>(dy, dres, h, rstd, w, dh_out, D);
  else add_rmsnorm_bwd_kernel<2><<<(unsigned)rows, RN_THREADS, 0, stream>>>(dy, dres, h, rstd, w, dh_out, D);
  return cudaGetLastError();
}
