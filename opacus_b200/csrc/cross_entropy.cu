// Token-wise cross entropy over a large vocabulary straight from 16-bit logits.
//
//   forward : loss[r] = logsumexp(x[r, :]) - x[r, target[r]]   (one read of the logits, online softmax)
//   backward: dx[r, :] = (exp(x[r, :] - lse[r]) - onehot(target[r])) * g[r]   (one read, one 16-bit write)
//
// The composition this replaces -- logits.float(), log_softmax forward and backward in fp32, the cast
// of the gradient back to bf16 -- moves ~12 bytes per logit each way; here it is 2 in the forward and
// 4 in the backward pass.  For DP training the per-token losses (no reduction) are what the clipping
// loss wrapper needs (opacus/utils/fast_gradient_clipping_utils.py:224-262 calls the criterion with
// reduction="none").  Rows whose target equals ignore_index give loss 0 and gradient 0.
#include "api.h"
#include "common.cuh"
#include "vec8.cuh"

namespace dpk {

namespace {

constexpr int CE_THREADS = 512;

// (m, s) <- combination of two partial softmax states: value = s * exp(m)
__device__ __forceinline__ void ce_merge(float& m, float& s, float m2, float s2) {
  const float mn = fmaxf(m, m2);
  s = (m == -INFINITY ? 0.f : s * __expf(m - mn)) + (m2 == -INFINITY ? 0.f : s2 * __expf(m2 - mn));
  m = mn;
}

template <int KIND>
__global__ void __launch_bounds__(CE_THREADS)
ce_forward_kernel(const void* x, const int64_t* target, int64_t V, int64_t ignore_index, float* loss, float* lse) {
  __shared__ float sh_m[CE_THREADS / 32], sh_s[CE_THREADS / 32];
  const int64_t row = blockIdx.x;
  const int64_t base = row * V;
  const bool vec = (V & 7) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0;
  float m = -INFINITY, s = 0.f;
  if (vec) {
    for (int64_t i = (int64_t)threadIdx.x * 8; i < V; i += (int64_t)CE_THREADS * 8) {
      float v[8];
      vload8<KIND>(x, base + i, v);
      float mx = v[0];
#pragma unroll
      for (int q = 1; q < 8; ++q) mx = fmaxf(mx, v[q]);
      if (mx > m) { s *= __expf(m - mx); m = mx; }
#pragma unroll
      for (int q = 0; q < 8; ++q) s += __expf(v[q] - m);
    }
  } else {
    for (int64_t i = threadIdx.x; i < V; i += CE_THREADS) {
      const float v = vload1<KIND>(x, base + i);
      if (v > m) { s *= __expf(m - v); m = v; }
      s += __expf(v - m);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
    ce_merge(m, s, m2, s2);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) { sh_m[warp] = m; sh_s[warp] = s; }
  __syncthreads();
  if (warp == 0) {
    m = lane < CE_THREADS / 32 ? sh_m[lane] : -INFINITY;
    s = lane < CE_THREADS / 32 ? sh_s[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
      ce_merge(m, s, m2, s2);
    }
    if (lane == 0) {
      const float l = m + __logf(s);
      const int64_t t = target[row];
      lse[row] = l;
      loss[row] = (t == ignore_index || t < 0 || t >= V) ? 0.f : l - vload1<KIND>(x, base + t);
    }
  }
}

template <int KIND>
__global__ void __launch_bounds__(CE_THREADS)
ce_backward_kernel(const void* x, const int64_t* target, const float* lse, const float* g, int64_t V,
                   int64_t ignore_index, void* dx) {
  const int64_t row = blockIdx.x;
  const int64_t base = row * V;
  const int64_t t = target[row];
  const bool live = !(t == ignore_index || t < 0 || t >= V);
  const float gr = live ? g[row] : 0.f;
  const float l = lse[row];
  const bool vec = (V & 7) == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dx)) & 15) == 0;
  if (vec) {
    for (int64_t i = (int64_t)threadIdx.x * 8; i < V; i += (int64_t)CE_THREADS * 8) {
      float v[8];
      vload8<KIND>(x, base + i, v);
#pragma unroll
      for (int q = 0; q < 8; ++q) v[q] = (__expf(v[q] - l) - ((i + q == t) ? 1.f : 0.f)) * gr;
      vstore8<KIND>(dx, base + i, v);
    }
  } else {
    for (int64_t i = threadIdx.x; i < V; i += CE_THREADS)
      vstore1<KIND>(dx, base + i, (__expf(vload1<KIND>(x, base + i) - l) - ((i == t) ? 1.f : 0.f)) * gr);
  }
}

}  // namespace
}  // namespace dpk

extern "C" int dpk_cross_entropy_forward(const void* logits, int kind, const int64_t* target, int64_t rows, int64_t V,
                                         int64_t ignore_index, float* loss, float* lse, cudaStream_t stream) {
  using namespace dpk;
  if (rows <= 0) return 0;
  if (V <= 0 || kind < 0 || kind > 2 || rows > 0x7fffffffLL) return cudaErrorInvalidValue;
  if (kind == 0) ce_forward_kernel<0><<<(unsigned)rows, CE_THREADS, 0, stream>>>(logits, target, V, ignore_index, loss, lse);
  else if (kind == 1) ce_forward_kernel<1><<<(unsigned)rows, CE_THREADS, 0, stream>>>(logits, target, V, ignore_index, loss, lse);
  else ce_forward_kernel<2><<<(unsigned)rows, CE_THREADS, 0, stream>>>(logits, target, V, ignore_index, loss, lse);
  return cudaGetLastError();
}

extern "C" int dpk_cross_entropy_backward(const void* logits, int kind, const int64_t* target, const float* lse,
                                          const float* grad_loss, int64_t rows, int64_t V, int64_t ignore_index,
                                          void* dlogits, cudaStream_t stream) {
  using namespace dpk;
  if (rows <= 0) return 0;
  if (V <= 0 || kind < 0 || kind > 2 || rows > 0x7fffffffLL) return cudaErrorInvalidValue;
  if (kind == 0) ce_backward_kernel<0><<<(unsigned)rows, CE_THREADS, 0, stream>>>(logits, target, lse, grad_loss, V, ignore_index, dlogits);
  else if (kind == 1) ce_backward_kernel<1><<<(unsigned)rows, CE_THREADS, 0, stream>>>(logits, target, lse, grad_loss, V, ignore_index, dlogits);
  else ce_backward_kernel<2><<<(unsigned)rows, CE_THREADS, 0, stream>>>(logits, target, lse, grad_loss, V, ignore_index, dlogits);
  return cudaGetLastError();
}
