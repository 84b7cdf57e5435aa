// Rotary position embedding, optionally fused with the head transpose around attention:
//
//   y[.., :hd/2] = x1 cos - x2 sin,  y[.., hd/2:] = x2 cos + x1 sin,  angle = t * theta^(-2j/hd)
//   source and destination are each either token-major [B, T, H, hd] (the projection output viewed per
//   head) or head-major [B, H, T, hd]; sign = -1 applies the inverse rotation (the gradient).
//
// One read and one write of the tensor; sines and cosines are evaluated in fp32 in the kernel.  The
// composition it replaces (slices, four multiplies, negate, concatenate on strided views, separate
// cos/sin tables) makes about ten passes.  Part of this package's Llama model, not of the DP machinery.
#include "api.h"
#include "common.cuh"
#include "vec8.cuh"

namespace dpk {
namespace {

template <int KIND>
__global__ void __launch_bounds__(256)
rope_kernel(const void* in, void* out, int64_t B, int64_t T, int64_t H, int hd, float log2_theta, int src_heads,
            int dst_heads, float sign) {
  const int half = hd >> 1;
  const int cpr = half >> 3;                         // 8-element chunks per half row
  const int64_t total = B * T * H * cpr;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % cpr);
    int64_t r = i / cpr;
    const int64_t h = r % H;
    r /= H;
    const int64_t t = r % T;
    const int64_t b = r / T;
    const int64_t tok_major = ((b * T + t) * H + h) * hd;      // [B, T, H, hd]
    const int64_t head_major = ((b * H + h) * T + t) * hd;     // [B, H, T, hd]
    const int64_t src = src_heads ? head_major : tok_major;
    const int64_t dst = dst_heads ? head_major : tok_major;
    float x1[8], x2[8], y1[8], y2[8];
    vload8<KIND>(in, src + c * 8, x1);
    vload8<KIND>(in, src + half + c * 8, x2);
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const int j = c * 8 + q;
      const float inv = exp2f(-(2.f * j / hd) * log2_theta);
      float sn, cs;
      sincosf((float)t * inv, &sn, &cs);
      sn *= sign;
      y1[q] = x1[q] * cs - x2[q] * sn;
      y2[q] = x2[q] * cs + x1[q] * sn;
    }
    vstore8<KIND>(out, dst + c * 8, y1);
    vstore8<KIND>(out, dst + half + c * 8, y2);
  }
}

}  // namespace
}  // namespace dpk

extern "C" int dpk_rope(const void* in, void* out, int kind, int64_t B, int64_t T, int64_t H, int hd, float theta,
                        int src_heads, int dst_heads, float sign, cudaStream_t stream) {
  using namespace dpk;
  if (B <= 0 || T <= 0 || H <= 0) return 0;
  if (hd <= 0 || (hd % 16) != 0 || kind < 0 || kind > 2 || theta <= 0.f) return cudaErrorInvalidValue;
  if (((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15) != 0) return cudaErrorInvalidValue;
  const int64_t total = B * T * H * (hd / 16);
  int64_t blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  const float l2 = log2f(theta);
  if (kind == 0) rope_kernel<0><<<(unsigned)blocks, 256, 0, stream>>>(in, out, B, T, H, hd, l2, src_heads, dst_heads, sign);
  else if (kind == 1) rope_kernel<1><<<(unsigned)blocks, 256, 0, stream>>>(in, out, B, T, H, hd, l2, src_heads, dst_heads, sign);
  else rope_kernel<2><<<(unsigned)blocks, 256, 0, stream>>>(in, out, B, T, H, hd, l2, src_heads, dst_heads, sign);
  return cudaGetLastError();
}
