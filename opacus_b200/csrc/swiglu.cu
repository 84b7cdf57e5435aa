// SwiGLU gate of a Llama MLP in one pass each way:
//   forward : h = silu(gate) * up
//   backward: dgate = dh * up * silu'(gate),  dup = dh * silu(gate)     (silu recomputed, nothing saved)
// Three tensor passes forward and five backward instead of five and about nine for the separate
// silu / multiply / silu_backward kernels.  Part of this package's Llama model.
#include "api.h"
#include "common.cuh"
#include "vec8.cuh"

namespace dpk {
namespace {

template <int KIND>
__global__ void __launch_bounds__(256) swiglu_fwd_kernel(const void* gate, const void* up, void* h, int64_t nvec) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
    float g[8], u[8], o[8];
    vload8<KIND>(gate, i << 3, g);
    vload8<KIND>(up, i << 3, u);
#pragma unroll
    for (int q = 0; q < 8; ++q) o[q] = g[q] / (1.f + __expf(-g[q])) * u[q];
    vstore8<KIND>(h, i << 3, o);
  }
}

template <int KIND>
__global__ void __launch_bounds__(256)
swiglu_bwd_kernel(const void* gate, const void* up, const void* dh, void* dgate, void* dup, int64_t nvec) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
    float g[8], u[8], d[8], dg[8], du[8];
    vload8<KIND>(gate, i << 3, g);
    vload8<KIND>(up, i << 3, u);
    vload8<KIND>(dh, i << 3, d);
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const float s = 1.f / (1.f + __expf(-g[q]));
      du[q] = d[q] * g[q] * s;
      dg[q] = d[q] * u[q] * s * (1.f + g[q] * (1.f - s));
    }
    vstore8<KIND>(dgate, i << 3, dg);
    vstore8<KIND>(dup, i << 3, du);
  }
}

inline unsigned grid_of(int64_t nvec) {
  int64_t b = (nvec + 255) / 256;
  return (unsigned)(b > 148 * 16 ? 148 * 16 : (b < 1 ? 1 : b));
}

}  // namespace
}  // namespace dpk

extern "C" int dpk_swiglu_forward(const void* gate, const void* up, void* h, int kind, int64_t n, cudaStream_t stream) {
  using namespace dpk;
  if (n <= 0) return 0;
  if ((n & 7) != 0 || kind < 0 || kind > 2) return cudaErrorInvalidValue;
  const int64_t nvec = n >> 3;
  if (kind == 0) swiglu_fwd_kernel<0><<<grid_of(nvec), 256, 0, stream>>>(gate, up, h, nvec);
  else if (kind == 1) swiglu_fwd_kernel<1><<<grid_of(nvec), 256, 0, stream>>>(gate, up, h, nvec);
  else swiglu_fwd_kernel<2><<<grid_of(nvec), 256, 0, stream>>>(gate, up, h, nvec);
  return cudaGetLastError();
}

extern "C" int dpk_swiglu_backward(const void* gate, const void* up, const void* dh, void* dgate, void* dup, int kind,
                                   int64_t n, cudaStream_t stream) {
  using namespace dpk;
  if (n <= 0) return 0;
  if ((n & 7) != 0 || kind < 0 || kind > 2) return cudaErrorInvalidValue;
  const int64_t nvec = n >> 3;
  if (kind == 0) swiglu_bwd_kernel<0><<<grid_of(nvec), 256, 0, stream>>>(gate, up, dh, dgate, dup, nvec);
  else if (kind == 1) swiglu_bwd_kernel<1><<<grid_of(nvec), 256, 0, stream>>>(gate, up, dh, dgate, dup, nvec);
  else swiglu_bwd_kernel<2><<<grid_of(nvec), 256, 0, stream>>>(gate, up, dh, dgate, dup, nvec);
  return cudaGetLastError();
}
