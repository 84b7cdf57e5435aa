// See gram_pair_static.h: the ghost-norm kernel with its scratch in a static
// device array, for callers that cannot allocate.
#include "gram_pair_static.h"

#include <stdio.h>

#include <mutex>

#include "api.h"

// defined in gram_pair.cu
int dpk_gram_pair_launch(const void* x, const int64_t* ids, const void* g, int B, int T, int d_x, int d_g, float scale,
                         float* scratch, float* out_w, float* out_b, int accumulate, uint32_t* status,
                         cudaStream_t stream);

namespace {

// One item of the kernel writes two floats here; see the header for the sizing rule.
static __device__ __align__(256) float g_static_scratch[DPK_GRAM_STATIC_MAX_FLOATS];

constexpr int kMaxDevices = 64;
float* g_scratch_addr[kMaxDevices] = {nullptr};   // device address of g_static_scratch, per device
std::mutex g_setup_mutex;

// `g_static_scratch` as written in host code is only a handle for the runtime,
// not an address a kernel can use; the device address has to be asked for, on
// the device it is wanted for.
int scratch_for_current_device(float** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_addr[dev] == nullptr) {
    float* ptr = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_static_scratch);
    if (e != cudaSuccess) return e;
    if (ptr == nullptr) return cudaErrorInvalidSymbol;
    g_scratch_addr[dev] = ptr;
  }
  *out = g_scratch_addr[dev];
  return 0;
}

}  // namespace

extern "C" int dpk_gram_pair_norm_static(const void* x, const int64_t* ids, const void* g, int B, int T, int d_x,
                                         int d_g, float scale, float* out_w, float* out_b, int accumulate,
                                         uint32_t* status, cudaStream_t stream) {
  if (B <= 0 || T <= 0) return cudaErrorInvalidValue;
  const size_t need = dpk_gram_pair_scratch_floats(B, T);
  if (need > static_cast<size_t>(DPK_GRAM_STATIC_MAX_FLOATS)) {
    fprintf(stderr,
            "dpk_gram_pair_norm_static: B=%d, T=%d needs %zu scratch floats, the built-in array holds %d; "
            "use dpk_gram_pair_norm with a caller-provided buffer\n",
            B, T, need, DPK_GRAM_STATIC_MAX_FLOATS);
    return cudaErrorInvalidValue;
  }
  float* scratch = nullptr;
  int rc = scratch_for_current_device(&scratch);
  if (rc != 0) return rc;
  // Left-overs of the previous call must not be mistaken for results: all-ones bytes are a NaN.
  cudaError_t e = cudaMemsetAsync(scratch, 0xFF, need * sizeof(float), stream);
  if (e != cudaSuccess) return e;
  return dpk_gram_pair_launch(x, ids, g, B, T, d_x, d_g, scale, scratch, out_w, out_b, accumulate, status, stream);
}
