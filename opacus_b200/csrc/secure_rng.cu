// ChaCha20 keystream on the GPU for secure-mode noise: the same stream as utils/secure_rng.py computes on the CPU
// (original ChaCha20: 20 rounds, 256-bit key, 64-bit block counter in words 12-13, 64-bit nonce in words 14-15).
// One thread computes one 64-byte block in registers and turns it into raw words, or into Gaussians by Box-Muller.
// The reference takes its secure generator from the torchcsprng package (opacus/privacy_engine.py:86-96) and sums four
// draws per element (opacus/optimizers/optimizer.py:143-160); `draws == 4` is that rule.
#include "api.h"

namespace dpk {

struct ChaChaKey {
  uint32_t k[8];
};

__device__ __forceinline__ uint32_t rotl32(uint32_t x, int n) { return __funnelshift_l(x, x, n); }

#define DPK_QR(a, b, c, d)                      \
  a += b; d ^= a; d = rotl32(d, 16);            \
  c += d; b ^= c; b = rotl32(b, 12);            \
  a += b; d ^= a; d = rotl32(d, 8);             \
  c += d; b ^= c; b = rotl32(b, 7);

__device__ __forceinline__ void chacha20_block(const ChaChaKey& key, uint64_t counter, uint64_t nonce, uint32_t (&x)[16]) {
  uint32_t s[16];
  s[0] = 0x61707865u; s[1] = 0x3320646eu; s[2] = 0x79622d32u; s[3] = 0x6b206574u;     // "expand 32-byte k"
#pragma unroll
  for (int i = 0; i < 8; ++i) s[4 + i] = key.k[i];
  s[12] = (uint32_t)counter; s[13] = (uint32_t)(counter >> 32);
  s[14] = (uint32_t)nonce;   s[15] = (uint32_t)(nonce >> 32);
#pragma unroll
  for (int i = 0; i < 16; ++i) x[i] = s[i];
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    DPK_QR(x[0], x[4], x[8], x[12]) DPK_QR(x[1], x[5], x[9], x[13])
    DPK_QR(x[2], x[6], x[10], x[14]) DPK_QR(x[3], x[7], x[11], x[15])
    DPK_QR(x[0], x[5], x[10], x[15]) DPK_QR(x[1], x[6], x[11], x[12])
    DPK_QR(x[2], x[7], x[8], x[13]) DPK_QR(x[3], x[4], x[9], x[14])
  }
#pragma unroll
  for (int i = 0; i < 16; ++i) x[i] += s[i];
}

// Box-Muller on one word pair: u1 = (w0 + 1) / 2^32 in (0, 1], u2 = w1 / 2^32; returns (r cos, r sin).
__device__ __forceinline__ float2 normal_pair(uint32_t w0, uint32_t w1) {
  const float u1 = ((float)w0 + 1.0f) * 2.3283064365386963e-10f;
  const float u2 = (float)w1 * 2.3283064365386963e-10f;
  const float r = sqrtf(-2.0f * logf(u1));
  float s, c;
  sincosf(6.2831853071795865f * u2, &s, &c);
  return make_float2(r * c, r * s);
}

__global__ void __launch_bounds__(256) chacha_words_kernel(uint32_t* __restrict__ out, int64_t n_blocks, ChaChaKey key,
                                                           uint64_t nonce, uint64_t first) {
  const int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= n_blocks) return;
  uint32_t x[16];
  chacha20_block(key, first + (uint64_t)b, nonce, x);
  uint4* dst = reinterpret_cast<uint4*>(out + b * 16);
#pragma unroll
  for (int i = 0; i < 4; ++i) dst[i] = make_uint4(x[4 * i], x[4 * i + 1], x[4 * i + 2], x[4 * i + 3]);
}

// draws == 4: element i = std * (sum of the four normals of words [4i, 4i+4)) / 2; a block gives 4 elements.
// draws == 1: element i = std * (cosine normal of words [2i, 2i+2)); a block gives 8 elements.
template <int DRAWS>
__global__ void __launch_bounds__(256) chacha_normal_kernel(float* __restrict__ out, int64_t n, ChaChaKey key,
                                                            uint64_t nonce, uint64_t first, float std) {
  constexpr int PER = DRAWS == 4 ? 4 : 8;                 // elements per block
  const int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t base = b * PER;
  if (base >= n) return;
  uint32_t x[16];
  chacha20_block(key, first + (uint64_t)b, nonce, x);
  float v[PER];
  if (DRAWS == 4) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 p = normal_pair(x[4 * e], x[4 * e + 1]);
      const float2 q = normal_pair(x[4 * e + 2], x[4 * e + 3]);
      v[e] = (((p.x + p.y) + q.x) + q.y) * 0.5f * std;
    }
  } else {
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = normal_pair(x[2 * e], x[2 * e + 1]).x * std;
  }
  if (base + PER <= n) {
    float4* dst = reinterpret_cast<float4*>(out + base);          // out is 16-byte aligned, base a multiple of 4
#pragma unroll
    for (int i = 0; i < PER / 4; ++i) dst[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
  } else {
#pragma unroll
    for (int e = 0; e < PER; ++e)
      if (base + e < n) out[base + e] = v[e];
  }
}

}  // namespace dpk

extern "C" int dpk_chacha_words(uint32_t* out, int64_t n_blocks, const uint32_t* key8_host, uint64_t nonce,
                                uint64_t first_block, cudaStream_t stream) {
  using namespace dpk;
  if (n_blocks <= 0) return 0;
  if (out == nullptr || key8_host == nullptr || (reinterpret_cast<uintptr_t>(out) & 15) != 0) return cudaErrorInvalidValue;
  ChaChaKey key;
  for (int i = 0; i < 8; ++i) key.k[i] = key8_host[i];
  const int64_t grid = (n_blocks + 255) / 256;
  chacha_words_kernel<<<(unsigned)grid, 256, 0, stream>>>(out, n_blocks, key, nonce, first_block);
  return (int)cudaGetLastError();
}

extern "C" int dpk_chacha_normal(float* out, int64_t n, const uint32_t* key8_host, uint64_t nonce, uint64_t first_block,
                                 float std, int draws, cudaStream_t stream) {
  using namespace dpk;
  if (n <= 0) return 0;
  if (out == nullptr || key8_host == nullptr || (draws != 1 && draws != 4) ||
      (reinterpret_cast<uintptr_t>(out) & 15) != 0)
    return cudaErrorInvalidValue;
  ChaChaKey key;
  for (int i = 0; i < 8; ++i) key.k[i] = key8_host[i];
  const int per = draws == 4 ? 4 : 8;
  const int64_t blocks = (n + per - 1) / per;
  const int64_t grid = (blocks + 255) / 256;
  if (grid > 0x7FFFFFFF) return cudaErrorInvalidValue;
  if (draws == 4)
    chacha_normal_kernel<4><<<(unsigned)grid, 256, 0, stream>>>(out, n, key, nonce, first_block, std);
  else
    chacha_normal_kernel<1><<<(unsigned)grid, 256, 0, stream>>>(out, n, key, nonce, first_block, std);
  return (int)cudaGetLastError();
}
