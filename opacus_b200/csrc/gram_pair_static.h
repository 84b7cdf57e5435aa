// Ghost-norm entry point for callers that must not allocate device memory.
//
// This function has no counterpart in the reference library; it exists for
// embedders of these kernels that run where cudaMalloc is off limits: code
// that executes inside another framework's memory plan (a fixed arena handed
// out at start-up), real-time or safety-rated host loops where an allocation
// may block or fail, and plug-ins that are only given input and output
// buffers.  The regular entry point, dpk_gram_pair_norm (api.h), needs a
// scratch buffer from its caller; this one brings its own.
//
// The scratch lives in a file-scope `static __device__` array of
// DPK_GRAM_STATIC_MAX_FLOATS floats (1 MiB).  Every GPU that loads this
// library holds that megabyte until the process exits.  A problem needs
// 2 * B * n * (n + 1) / 2 floats with n = ceil(T / 128); larger problems are
// rejected with cudaErrorInvalidValue and a message on stderr that states the
// need and the limit (B = 8 sequences of 1024 tokens need 576 floats; the
// limit admits e.g. B = 32 at T = 8192, which needs 133,120).
//
// Set-up: the first call on each device looks up the array's device address
// (cudaGetSymbolAddress, with that device current).  Make that first call
// outside of any stream capture.  The call itself performs no cudaMalloc,
// cudaFree or any other allocating routine; it enqueues a fill of the used
// part of the array, the tensor-core kernel and the per-sample reduction on
// `stream`.
//
// Sharing: all calls on a device use the same array, and it keeps whatever the
// previous call left in it.  The part a call is going to use is therefore first
// overwritten with a NaN pattern, so a work item the kernel failed to finish
// shows up as NaN instead of passing for a result.  Two calls whose GPU work
// can overlap (different streams, or different host threads without ordering)
// race on the array; order them on one stream or with events.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define DPK_GRAM_STATIC_MAX_FLOATS (1 << 18)

#ifdef __cplusplus
extern "C" {
#endif

// Same arguments and results as dpk_gram_pair_norm, minus the scratch pointer:
//   x   [B, T, d_x] bf16 or NULL;  ids [B, T] int64 or NULL (used when x is NULL);  g [B, T, d_g] bf16
//   out_w[n] (+)= scale * <X_n X_n^T, G_n G_n^T>,  out_b[n] (+)= scale * sum(G_n G_n^T)   (either may be NULL)
//   status: four zeroed 32-bit words in device-visible memory, or NULL
// Returns 0 or a cudaError_t value.
int dpk_gram_pair_norm_static(const void* x, const int64_t* ids, const void* g, int B, int T, int d_x, int d_g,
                              float scale, float* out_w, float* out_b, int accumulate, uint32_t* status,
                              cudaStream_t stream);

#ifdef __cplusplus
}
#endif
