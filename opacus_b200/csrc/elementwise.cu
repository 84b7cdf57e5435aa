// Bandwidth-bound kernels of the DP step: row scaling, clip factors, per-sample
// squared norms, clip-weighted sums, normalisation-layer per-sample gradients,
// embedding scatter, and the fused "noise + scale + optimiser update" pass with
// an in-kernel Philox generator.  All of them stream their inputs once with
// 16-byte accesses; none uses shared-memory tiling because there is no reuse.
#include "api.h"
#include "common.cuh"
#include "host_util.h"
#include <cuda_fp16.h>

namespace dpk {

// ---------------------------------------------------------------- typed 8-wide loads
template <int KIND> struct Elem;                       // 0 fp32, 1 bf16, 2 fp16
template <> struct Elem<0> { using T = float; };
template <> struct Elem<1> { using T = __nv_bfloat16; };
template <> struct Elem<2> { using T = __half; };

template <int KIND>
__device__ __forceinline__ void load8(const void* base, int64_t idx, float (&v)[8]) {
  if constexpr (KIND == 0) {
    const float4* p = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + idx);
    float4 a = p[0], b = p[1];
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  } else {
    uint4 raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(base) + idx);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      if constexpr (KIND == 1) {
        __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162*>(&w[q]);
        v[2 * q] = __bfloat162float(h.x); v[2 * q + 1] = __bfloat162float(h.y);
      } else {
        __half2 h = *reinterpret_cast<const __half2*>(&w[q]);
        v[2 * q] = __half2float(h.x); v[2 * q + 1] = __half2float(h.y);
      }
    }
  }
}
template <int KIND>
__device__ __forceinline__ float load1(const void* base, int64_t idx) {
  if constexpr (KIND == 0) return reinterpret_cast<const float*>(base)[idx];
  else if constexpr (KIND == 1) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[idx]);
  else return __half2float(reinterpret_cast<const __half*>(base)[idx]);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
// Sum over a block of up to 1024 threads; result valid in every thread.
__device__ __forceinline__ float block_sum(float v, float* sh) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (l == 0) sh[w] = v;
  __syncthreads();
  float t = (threadIdx.x < nw) ? sh[threadIdx.x] : 0.f;
  if (w == 0) t = warp_sum(t);
  if (threadIdx.x == 0) sh[0] = t;
  __syncthreads();
  return sh[0];
}

// ---------------------------------------------------------------- scale_rows
template <int KIND>
__global__ void scale_rows_kernel(const void* x, const float* c, __nv_bfloat16* y, int64_t rows, int64_t cols,
                                  int64_t rps, float scale) {
  const int64_t vec_per_row = cols >> 3;
  const int64_t total = rows * vec_per_row;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / vec_per_row;
    const float f = (c ? c[r / rps] : 1.f) * scale;
    float v[8];
    load8<KIND>(x, i << 3, v);
    uint4 out;
    uint32_t* ow = reinterpret_cast<uint32_t*>(&out);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * q] * f, v[2 * q + 1] * f);
      ow[q] = *reinterpret_cast<uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(y + (i << 3)) = out;
  }
}

// ---------------------------------------------------------------- fp32 operand as three bf16 planes
// v = x * c * scale is written as hi = bf16(v), lo = bf16(v - hi): hi + lo carries 16 mantissa bits.  For a product
// of two such operands the tensor cores run on the planes (hi, hi, lo) of the left one against (hi, lo, hi) of the
// right one, stacked along the contraction axis: hi*hi + hi*lo + lo*hi, i.e. the fp32 product up to the
// lo*lo term (relative 2^-16).  Row r of sample b = r / T lands in rows (3 b + j) * T + r % T, j = 0, 1, 2.
__global__ void split3_rows_kernel(const float* x, const float* c, __nv_bfloat16* y, int64_t rows, int64_t cols,
                                   int64_t T, float scale, int right) {
  const int64_t vec_per_row = cols >> 3;
  const int64_t total = rows * vec_per_row;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / vec_per_row;
    const int64_t col = (i - r * vec_per_row) << 3;
    const int64_t b = r / T, t = r - b * T;
    const float f = (c ? c[b] : 1.f) * scale;
    float v[8];
    load8<0>(x, i << 3, v);
    uint4 hi, lo;
    uint32_t* hw = reinterpret_cast<uint32_t*>(&hi);
    uint32_t* lw = reinterpret_cast<uint32_t*>(&lo);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float v0 = v[2 * q] * f, v1 = v[2 * q + 1] * f;
      const __nv_bfloat162 h = __floats2bfloat162_rn(v0, v1);
      const __nv_bfloat162 l = __floats2bfloat162_rn(v0 - __bfloat162float(h.x), v1 - __bfloat162float(h.y));
      hw[q] = *reinterpret_cast<const uint32_t*>(&h);
      lw[q] = *reinterpret_cast<const uint32_t*>(&l);
    }
    __nv_bfloat16* base = y + ((b * 3) * T + t) * cols + col;
    const int64_t plane = T * cols;
    *reinterpret_cast<uint4*>(base) = hi;
    *reinterpret_cast<uint4*>(base + plane) = right ? lo : hi;
    *reinterpret_cast<uint4*>(base + 2 * plane) = right ? hi : lo;
  }
}

// ---------------------------------------------------------------- clip factor
// A NaN norm (a producer that marked unfinished work, an overflow upstream) gives a NaN factor, never 1:
// clipping must not fail open.  fmaxf / fminf would drop the NaN.
__global__ void clip_factor_kernel(const float* n2, float* c, int64_t B, float C) {
  const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i < B) c[i] = clip_factor_of(n2[i], C);
}

// ---------------------------------------------------------------- per-row squared norm
template <int KIND>
__global__ void row_norm_sq_kernel(const void* x, int64_t cols, float* out) {
  __shared__ float sh[32];
  const int64_t row = blockIdx.y;
  const int64_t base = row * cols;
  float acc = 0.f;
  const bool vec_ok = (cols & 7) == 0;
  if (vec_ok) {
    const int64_t nvec = cols >> 3;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
      float v[8];
      load8<KIND>(x, base + (i << 3), v);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc = fmaf(v[j], v[j], acc);
    }
  } else {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < cols; i += (int64_t)gridDim.x * blockDim.x) {
      const float v = load1<KIND>(x, base + i);
      acc = fmaf(v, v, acc);
    }
  }
  const float tot = block_sum(acc, sh);
  if (threadIdx.x == 0) atomicAdd(out + row, tot);
}

// ---------------------------------------------------------------- weighted sum over samples
template <int KIND>
__global__ void weighted_sum_kernel(const void* x, const float* c, int64_t B, int64_t cols, float* out) {
  const int64_t j = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  const int64_t b0 = blockIdx.y, bstep = gridDim.y;
  if ((cols & 7) == 0) {
    if ((j << 3) >= cols) return;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int64_t n = b0; n < B; n += bstep) {
      float v[8];
      load8<KIND>(x, n * cols + (j << 3), v);
      const float w = c[n];
#pragma unroll
      for (int q = 0; q < 8; ++q) acc[q] = fmaf(w, v[q], acc[q]);
    }
    if (bstep == 1) {
#pragma unroll
      for (int q = 0; q < 8; ++q) out[(j << 3) + q] = acc[q];
    } else {
#pragma unroll
      for (int q = 0; q < 8; ++q) atomicAdd(out + (j << 3) + q, acc[q]);
    }
  } else {
    if (j >= cols) return;
    float acc = 0.f;
    for (int64_t n = b0; n < B; n += bstep) acc = fmaf(c[n], load1<KIND>(x, n * cols + j), acc);
    if (bstep == 1) out[j] = acc; else atomicAdd(out + j, acc);
  }
}

// ---------------------------------------------------------------- 2-d input ghost norm
template <int KIND>
__global__ void outer_norm_sq_kernel(const void* a, const void* g, int64_t d_a, int64_t d_g, float scale, float* out_w,
                                     float* out_b, int accumulate) {
  __shared__ float sh[32];
  const int64_t n = blockIdx.x;
  float sa = 0.f, sg = 0.f;
  if (a) for (int64_t i = threadIdx.x; i < d_a; i += blockDim.x) { const float v = load1<KIND>(a, n * d_a + i); sa = fmaf(v, v, sa); }
  for (int64_t i = threadIdx.x; i < d_g; i += blockDim.x) { const float v = load1<KIND>(g, n * d_g + i); sg = fmaf(v, v, sg); }
  sa = block_sum(sa, sh);
  sg = block_sum(sg, sh);
  if (threadIdx.x == 0) {
    if (out_w) out_w[n] = (accumulate ? out_w[n] : 0.f) + sa * sg * scale;
    if (out_b) out_b[n] = (accumulate ? out_b[n] : 0.f) + sg * scale;
  }
}

// ---------------------------------------------------------------- LayerNorm / RMSNorm
// stats[row] = (mean, rstd) over the last dimension (mean = 0 for RMSNorm).
template <int KIND>
__global__ void row_stats_kernel(int kind, const void* x, int64_t nrows, int64_t d, float eps, float2* stats) {
  const int warps = blockDim.x >> 5;
  const int64_t row = blockIdx.x * (int64_t)warps + (threadIdx.x >> 5);
  if (row >= nrows) return;
  const int lane = threadIdx.x & 31;
  float s = 0.f, ss = 0.f;
  for (int64_t i = lane; i < d; i += 32) {
    const float v = load1<KIND>(x, row * d + i);
    s += v; ss = fmaf(v, v, ss);
  }
  s = warp_sum(s); ss = warp_sum(ss);
  if (lane == 0) {
    if (kind == 0) {
      const float mean = s / d;
      const float var = fmaxf(ss / d - mean * mean, 0.f);
      stats[row] = make_float2(mean, rsqrtf(var + eps));
    } else {
      stats[row] = make_float2(0.f, rsqrtf(ss / d + eps));
    }
  }
}
// gw[n, j] += sum_r (x[n,r,j]-mean)*rstd*g[n,r,j];  gb[n, j] += sum_r g[n,r,j]
template <int KIND>
__global__ void lastdim_grad_kernel(const void* x, const void* g, const float2* stats, int64_t rows, int64_t d,
                                    int64_t rows_per_block, float* gw, float* gb) {
  const int64_t j = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (j >= d) return;
  const int64_t n = blockIdx.z;
  const int64_t r0 = blockIdx.y * rows_per_block;
  const int64_t r1 = min(rows, r0 + rows_per_block);
  float aw = 0.f, ab = 0.f;
  for (int64_t r = r0; r < r1; ++r) {
    const int64_t row = n * rows + r;
    const float2 st = stats[row];
    const float xv = load1<KIND>(x, row * d + j);
    const float gv = load1<KIND>(g, row * d + j);
    aw = fmaf((xv - st.x) * st.y, gv, aw);
    ab += gv;
  }
  if (gw) atomicAdd(gw + n * d + j, aw);
  if (gb) atomicAdd(gb + n * d + j, ab);
}

// ---------------------------------------------------------------- LayerNorm / RMSNorm, one launch
// Per-sample affine gradients AND their squared norms in one kernel (d a multiple of 8, d <= 256 * NV * ... see
// the launcher).  grid = (chunks, B); a block takes rows [r0, r1) of sample n, one row per warp at a time:
//   pass 1 over the row gives mean / rstd, pass 2 (the row is in L1 by then) accumulates xhat * g (and g) in
//   registers, lane l holding columns 8 * (l + 32 * i) .. + 8;
// the warps of a block are added in shared memory, every block writes its partial [d] vector to scratch, and the
// last block of a sample to finish (a ticket counter per sample) adds the partial vectors in a fixed order into
// gw / gb and squares and sums them: n2w[n] / n2b[n] (+= when accumulate).  The counter is left at zero again.
template <int KIND, int NV, bool BIAS>
__global__ void __launch_bounds__(256)
lastdim_psg_fused_kernel(int norm_kind, const void* x, const void* g, int64_t rows, int64_t d, int64_t rows_per_block,
                         float eps, float* gw, float* gb, float* n2w, float* n2b, int accumulate,
                         unsigned int* tickets, float* part) {
  extern __shared__ float red[];               // [d] (+ [d] with BIAS)
  __shared__ float sh[32];
  __shared__ unsigned int sh_last;
  const int64_t n = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t r0 = blockIdx.x * rows_per_block;
  const int64_t r1 = min(rows, r0 + rows_per_block);
  float aw[NV][8];
  float ab[BIAS ? NV : 1][8];
#pragma unroll
  for (int i = 0; i < NV; ++i)
#pragma unroll
    for (int q = 0; q < 8; ++q) { aw[i][q] = 0.f; if (BIAS) ab[i][q] = 0.f; }
  for (int64_t r = r0 + warp; r < r1; r += 8) {
    const int64_t base = (n * rows + r) * d;
    float s = 0.f, ss = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int64_t col = (int64_t)(lane + 32 * i) * 8;
      if (col < d) {
        float v[8];
        load8<KIND>(x, base + col, v);
#pragma unroll
        for (int q = 0; q < 8; ++q) { s += v[q]; ss = fmaf(v[q], v[q], ss); }
      }
    }
    s = warp_sum(s); ss = warp_sum(ss);
    float mean = 0.f, rstd;
    if (norm_kind == 0) {
      mean = s / d;
      rstd = rsqrtf(fmaxf(ss / d - mean * mean, 0.f) + eps);
    } else {
      rstd = rsqrtf(ss / d + eps);
    }
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int64_t col = (int64_t)(lane + 32 * i) * 8;
      if (col < d) {
        float xv[8], gv[8];
        load8<KIND>(x, base + col, xv);
        load8<KIND>(g, base + col, gv);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          aw[i][q] = fmaf((xv[q] - mean) * rstd, gv[q], aw[i][q]);
          if (BIAS) ab[i][q] += gv[q];
        }
      }
    }
  }
  // warps -> block (one warp at a time adds its registers into shared memory), block -> global
  for (int64_t j = threadIdx.x; j < (BIAS ? 2 * d : d); j += blockDim.x) red[j] = 0.f;
  __syncthreads();
  for (int w = 0; w < 8; ++w) {
    if (warp == w) {
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int64_t col = (int64_t)(lane + 32 * i) * 8;
        if (col < d) {
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            red[col + q] += aw[i][q];
            if (BIAS) red[d + col + q] += ab[i][q];
          }
        }
      }
    }
    __syncthreads();
  }
  // block -> global: this block's partial sums go to its own row of `part` ([B, chunks, d] (x2 with BIAS)); the last
  // block of the sample to finish adds the rows in chunk order -- no atomics on the result, same bits on every run
  const int64_t width = BIAS ? 2 * d : d;
  float* mine = part + (n * gridDim.x + blockIdx.x) * width;
  for (int64_t j = threadIdx.x; j < width; j += blockDim.x) mine[j] = red[j];
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int t = atomicAdd(tickets + n, 1u);
    sh_last = (t == gridDim.x - 1) ? 1u : 0u;
  }
  __syncthreads();
  if (!sh_last) return;
  __threadfence();
  float qw = 0.f, qb = 0.f;
  const float* all = part + n * gridDim.x * width;
  // width is a multiple of 8: 16-byte loads, four partial rows in flight per thread
  for (int64_t j4 = threadIdx.x; j4 < (width >> 2); j4 += blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    unsigned int c = 0;
    for (; c + 4 <= gridDim.x; c += 4) {
      const float4 v0 = __ldcg(reinterpret_cast<const float4*>(all + (c + 0) * width) + j4);
      const float4 v1 = __ldcg(reinterpret_cast<const float4*>(all + (c + 1) * width) + j4);
      const float4 v2 = __ldcg(reinterpret_cast<const float4*>(all + (c + 2) * width) + j4);
      const float4 v3 = __ldcg(reinterpret_cast<const float4*>(all + (c + 3) * width) + j4);
      acc.x += v0.x; acc.y += v0.y; acc.z += v0.z; acc.w += v0.w;       // chunk order: same bits on every run
      acc.x += v1.x; acc.y += v1.y; acc.z += v1.z; acc.w += v1.w;
      acc.x += v2.x; acc.y += v2.y; acc.z += v2.z; acc.w += v2.w;
      acc.x += v3.x; acc.y += v3.y; acc.z += v3.z; acc.w += v3.w;
    }
    for (; c < gridDim.x; ++c) {
      const float4 v = __ldcg(reinterpret_cast<const float4*>(all + c * width) + j4);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    const int64_t j = j4 << 2;
    const float sq = acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
    if (!BIAS || j < d) {
      *reinterpret_cast<float4*>(gw + n * d + j) = acc;
      qw += sq;
    } else {
      *reinterpret_cast<float4*>(gb + n * d + (j - d)) = acc;
      qb += sq;
    }
  }
  qw = block_sum(qw, sh);
  if (BIAS) qb = block_sum(qb, sh);
  if (threadIdx.x == 0) {
    if (n2w) n2w[n] = (accumulate ? n2w[n] : 0.f) + qw;
    if (BIAS && n2b) n2b[n] = (accumulate ? n2b[n] : 0.f) + qb;
    tickets[n] = 0;
  }
}

// ---------------------------------------------------------------- GroupNorm / InstanceNorm
// One block per (sample, group).  x, g: [B, C, S].  The group's statistics come from one 8-wide sweep
// of its (contiguous) data; then each warp takes whole channels, so the per-channel sums need no block barrier
// and the second read of x hits L1/L2.
template <int KIND>
__global__ void __launch_bounds__(256)
channel_grad_kernel(const void* x, const void* g, int64_t C, int64_t S, int groups, float eps, float* gw, float* gb) {
  __shared__ float sh[32];
  const int64_t n = blockIdx.x / groups;
  const int grp = blockIdx.x % groups;
  const int64_t cpg = C / groups;
  const int64_t base = (n * C + grp * cpg) * S;
  const int64_t cnt = cpg * S;
  // 8-wide loads need every channel row to start on a 16-byte boundary
  const bool vec = (S & 7) == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(g)) & 15) == 0;
  float s = 0.f, ss = 0.f;
  if (vec) {
    for (int64_t i = (int64_t)threadIdx.x * 8; i < cnt; i += (int64_t)blockDim.x * 8) {
      float v[8];
      load8<KIND>(x, base + i, v);
#pragma unroll
      for (int q = 0; q < 8; ++q) { s += v[q]; ss = fmaf(v[q], v[q], ss); }
    }
  } else {
    for (int64_t i = threadIdx.x; i < cnt; i += blockDim.x) {
      const float v = load1<KIND>(x, base + i);
      s += v; ss = fmaf(v, v, ss);
    }
  }
  s = block_sum(s, sh);
  ss = block_sum(ss, sh);
  const float mean = s / cnt;
  const float rstd = rsqrtf(fmaxf(ss / cnt - mean * mean, 0.f) + eps);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  for (int64_t c = warp; c < cpg; c += nwarps) {
    const int64_t row = base + c * S;
    float aw = 0.f, ab = 0.f;
    if (vec) {
      for (int64_t i = (int64_t)lane * 8; i < S; i += 32 * 8) {
        float xv[8], gv[8];
        load8<KIND>(x, row + i, xv);
        load8<KIND>(g, row + i, gv);
#pragma unroll
        for (int q = 0; q < 8; ++q) { aw = fmaf((xv[q] - mean) * rstd, gv[q], aw); ab += gv[q]; }
      }
    } else {
      for (int64_t i = lane; i < S; i += 32) {
        const float gv = load1<KIND>(g, row + i);
        aw = fmaf((load1<KIND>(x, row + i) - mean) * rstd, gv, aw);
        ab += gv;
      }
    }
    aw = warp_sum(aw);
    ab = warp_sum(ab);
    if (lane == 0) {
      if (gw) gw[n * C + grp * cpg + c] = aw;
      if (gb) gb[n * C + grp * cpg + c] = ab;
    }
  }
}

// ---------------------------------------------------------------- embedding scatter
template <int KIND>
__global__ void embedding_scatter_kernel(const int64_t* ids, const void* g, const float* c, int64_t rows, int64_t T,
                                         int64_t D, int64_t V, int64_t padding_idx, float scale, float* out) {
  const int64_t vec_per_row = (D + 3) >> 2;
  const int64_t total = rows * vec_per_row;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / vec_per_row;
    const int64_t col = (i - r * vec_per_row) << 2;
    const int64_t id = ids[r];
    if (id < 0 || id >= V || id == padding_idx) continue;
    const float f = c[r / T] * scale;
#pragma unroll
    for (int q = 0; q < 4; ++q)
      if (col + q < D) atomicAdd(out + id * D + col + q, f * load1<KIND>(g, r * D + col + q));
  }
}

// ---------------------------------------------------------------- fused DP step
constexpr int kStepChunk = 4096;        // elements per block
constexpr int kStepThreads = 256;       // 4 per thread per iteration

__global__ void __launch_bounds__(kStepThreads)
fused_dp_step_kernel(const DpkTensorEntry* table, int n_tensors, const int64_t* chunk_prefix, DpkStepHyper h) {
  // locate the tensor owning this chunk: chunk_prefix[t] <= blockIdx.x < chunk_prefix[t+1]
  int lo = 0, hi = n_tensors;
  const int64_t b = blockIdx.x;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (chunk_prefix[mid] <= b) lo = mid; else hi = mid;
  }
  const DpkTensorEntry e = table[lo];
  const int64_t start = (b - chunk_prefix[lo]) * kStepChunk;
  const int64_t end = min(e.numel, start + kStepChunk);
  const Philox rng(h.seed);
  float* pf = reinterpret_cast<float*>(e.param);
  __nv_bfloat16* pb = reinterpret_cast<__nv_bfloat16*>(e.param);

  // 16-byte accesses whenever every array of this tensor is 16-byte aligned (the usual case)
  const bool vec = (((reinterpret_cast<uintptr_t>(e.grad) | reinterpret_cast<uintptr_t>(e.state0) |
                      reinterpret_cast<uintptr_t>(e.state1) | reinterpret_cast<uintptr_t>(e.master)) & 15) == 0) &&
                   ((reinterpret_cast<uintptr_t>(e.param) & (e.param_bf16 ? 7 : 15)) == 0);
  const bool use_m = h.kind != 0 || h.momentum != 0.f;
  for (int64_t i0 = start + 4 * (int64_t)threadIdx.x; i0 < end; i0 += 4 * kStepThreads) {
    float z[4] = {0.f, 0.f, 0.f, 0.f};
    if (h.noise_std != 0.f) {
      const uint4 u = rng(static_cast<uint64_t>(e.rng_offset + i0) >> 2, h.offset);
      const float2 n01 = box_muller(u.x, u.y), n23 = box_muller(u.z, u.w);
      z[0] = n01.x * h.noise_std; z[1] = n01.y * h.noise_std; z[2] = n23.x * h.noise_std; z[3] = n23.y * h.noise_std;
    }
    const bool full = vec && i0 + 4 <= end;
    float g[4], w[4], m[4] = {0, 0, 0, 0}, v[4] = {0, 0, 0, 0};
    if (full) {
      const float4 gv = *reinterpret_cast<const float4*>(e.grad + i0);
      g[0] = gv.x; g[1] = gv.y; g[2] = gv.z; g[3] = gv.w;
      if (e.master) {
        const float4 t = *reinterpret_cast<const float4*>(e.master + i0);
        w[0] = t.x; w[1] = t.y; w[2] = t.z; w[3] = t.w;
      } else if (e.param_bf16) {
        const uint2 t = *reinterpret_cast<const uint2*>(pb + i0);
        const __nv_bfloat162 lo2 = *reinterpret_cast<const __nv_bfloat162*>(&t.x);
        const __nv_bfloat162 hi2 = *reinterpret_cast<const __nv_bfloat162*>(&t.y);
        w[0] = __bfloat162float(lo2.x); w[1] = __bfloat162float(lo2.y);
        w[2] = __bfloat162float(hi2.x); w[3] = __bfloat162float(hi2.y);
      } else {
        const float4 t = *reinterpret_cast<const float4*>(pf + i0);
        w[0] = t.x; w[1] = t.y; w[2] = t.z; w[3] = t.w;
      }
      if (use_m && !(h.kind == 0 && h.first_step)) {
        const float4 t = *reinterpret_cast<const float4*>(e.state0 + i0);
        m[0] = t.x; m[1] = t.y; m[2] = t.z; m[3] = t.w;
      }
      if (h.kind != 0) {
        const float4 t = *reinterpret_cast<const float4*>(e.state1 + i0);
        v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
      }
    } else {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int64_t i = i0 + q;
        if (i >= end) { g[q] = 0.f; w[q] = 0.f; continue; }
        g[q] = e.grad[i];
        w[q] = e.master ? e.master[i] : (e.param_bf16 ? __bfloat162float(pb[i]) : pf[i]);
        if (use_m && !(h.kind == 0 && h.first_step)) m[q] = e.state0[i];
        if (h.kind != 0) v[q] = e.state1[i];
      }
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      float grad = (g[q] + z[q]) * h.inv_scale;
      g[q] = grad;
      float pv = w[q];
      if (h.kind == 0) {
        if (h.weight_decay != 0.f) grad = fmaf(h.weight_decay, pv, grad);
        if (h.momentum != 0.f) {
          const float buf = h.first_step ? grad : fmaf(h.momentum, m[q], (1.f - h.dampening) * grad);
          m[q] = buf;
          grad = h.nesterov ? fmaf(h.momentum, buf, grad) : buf;
        }
        pv = fmaf(-h.lr, grad, pv);
      } else {
        if (h.weight_decay != 0.f) {
          if (h.kind == 2) pv *= (1.f - h.lr * h.weight_decay);
          else grad = fmaf(h.weight_decay, pv, grad);
        }
        m[q] = fmaf(h.beta1, m[q], (1.f - h.beta1) * grad);
        v[q] = fmaf(h.beta2, v[q], (1.f - h.beta2) * grad * grad);
        pv -= (h.lr / h.bias_c1) * (m[q] / (sqrtf(v[q]) / h.bias_c2_sqrt + h.eps));
      }
      w[q] = pv;
    }
    if (full) {
      *reinterpret_cast<float4*>(e.grad + i0) = make_float4(g[0], g[1], g[2], g[3]);
      if (use_m) *reinterpret_cast<float4*>(e.state0 + i0) = make_float4(m[0], m[1], m[2], m[3]);
      if (h.kind != 0) *reinterpret_cast<float4*>(e.state1 + i0) = make_float4(v[0], v[1], v[2], v[3]);
      if (e.master) *reinterpret_cast<float4*>(e.master + i0) = make_float4(w[0], w[1], w[2], w[3]);
      if (e.param_bf16) {
        __nv_bfloat162 lo2 = __floats2bfloat162_rn(w[0], w[1]), hi2 = __floats2bfloat162_rn(w[2], w[3]);
        uint2 t;
        t.x = *reinterpret_cast<uint32_t*>(&lo2);
        t.y = *reinterpret_cast<uint32_t*>(&hi2);
        *reinterpret_cast<uint2*>(pb + i0) = t;
      } else {
        *reinterpret_cast<float4*>(pf + i0) = make_float4(w[0], w[1], w[2], w[3]);
      }
    } else {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int64_t i = i0 + q;
        if (i >= end) break;
        e.grad[i] = g[q];
        if (use_m) e.state0[i] = m[q];
        if (h.kind != 0) e.state1[i] = v[q];
        if (e.master) e.master[i] = w[q];
        if (e.param_bf16) pb[i] = __float2bfloat16_rn(w[q]); else pf[i] = w[q];
      }
    }
  }
}

__global__ void philox_normal_kernel(float* out, int64_t n, uint64_t seed, uint64_t offset, float std) {
  const Philox rng(seed);
  for (int64_t i0 = 4 * (blockIdx.x * (int64_t)blockDim.x + threadIdx.x); i0 < n; i0 += 4 * (int64_t)gridDim.x * blockDim.x) {
    const uint4 u = rng(static_cast<uint64_t>(i0) >> 2, offset);
    const float2 a = box_muller(u.x, u.y), b = box_muller(u.z, u.w);
    const float z[4] = {a.x, a.y, b.x, b.y};
    for (int q = 0; q < 4 && i0 + q < n; ++q) out[i0 + q] = z[q] * std;
  }
}

inline int grid_for(int64_t work, int threads, int max_blocks) {
  int64_t b = (work + threads - 1) / threads;
  if (b < 1) b = 1;
  return (int)(b > max_blocks ? max_blocks : b);
}

}  // namespace dpk

using namespace dpk;

#define DISPATCH_KIND(kind, ...)                         \
  switch (kind) {                                        \
    case 0: { constexpr int KIND = 0; __VA_ARGS__; break; } \
    case 1: { constexpr int KIND = 1; __VA_ARGS__; break; } \
    case 2: { constexpr int KIND = 2; __VA_ARGS__; break; } \
    default: return cudaErrorInvalidValue;               \
  }

extern "C" int dpk_scale_rows(const void* x, int x_is_fp32, const float* c, void* y, int64_t rows, int64_t cols,
                              int64_t rps, float scale, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0 || (cols & 7) || rps <= 0) return cudaErrorInvalidValue;
  const int grid = grid_for(rows * (cols >> 3), 256, num_sms() * 16);
  if (x_is_fp32) scale_rows_kernel<0><<<grid, 256, 0, stream>>>(x, c, (__nv_bfloat16*)y, rows, cols, rps, scale);
  else scale_rows_kernel<1><<<grid, 256, 0, stream>>>(x, c, (__nv_bfloat16*)y, rows, cols, rps, scale);
  return cudaGetLastError();
}

extern "C" int dpk_split3_rows(const float* x, const float* c, void* y, int64_t rows, int64_t cols, int64_t T,
                               float scale, int right, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0 || (cols & 7) || T <= 0 || rows % T) return cudaErrorInvalidValue;
  const int grid = grid_for(rows * (cols >> 3), 256, num_sms() * 16);
  split3_rows_kernel<<<grid, 256, 0, stream>>>(x, c, (__nv_bfloat16*)y, rows, cols, T, scale, right);
  return cudaGetLastError();
}

extern "C" int dpk_clip_factor(const float* n2, float* c, int64_t B, float C, cudaStream_t stream) {
  if (B <= 0) return 0;
  clip_factor_kernel<<<(int)((B + 255) / 256), 256, 0, stream>>>(n2, c, B, C);
  return cudaGetLastError();
}

extern "C" int dpk_row_norm_sq(const void* x, int kind, int64_t B, int64_t cols, float* out, int accumulate,
                               cudaStream_t stream) {
  if (B <= 0 || cols <= 0) return 0;
  if (!accumulate) cudaMemsetAsync(out, 0, sizeof(float) * B, stream);
  int64_t per_row = (cols + 8 * 256 - 1) / (8 * 256);
  int64_t want = (int64_t)num_sms() * 8 / (B > 0 ? B : 1) + 1;
  int gx = (int)(per_row < want ? per_row : want);
  if (gx < 1) gx = 1;
  dim3 grid(gx, (unsigned)B);
  if (B > 65535) return cudaErrorInvalidValue;
  DISPATCH_KIND(kind, (row_norm_sq_kernel<KIND><<<grid, 256, 0, stream>>>(x, cols, out)));
  return cudaGetLastError();
}

extern "C" int dpk_weighted_sum(const void* x, int kind, const float* c, int64_t B, int64_t cols, float* out,
                                cudaStream_t stream) {
  if (cols <= 0) return 0;
  const int64_t lanes = (cols & 7) == 0 ? (cols >> 3) : cols;
  const int gx = (int)((lanes + 127) / 128);
  int gy = 1;
  if (gx < num_sms() * 2 && B >= 16) {
    gy = (int)((num_sms() * 4 + gx - 1) / gx);
    if (gy > B / 4) gy = (int)(B / 4);
    if (gy < 1) gy = 1;
    if (gy > 1024) gy = 1024;
  }
  if (gy > 1) cudaMemsetAsync(out, 0, sizeof(float) * cols, stream);
  dim3 grid(gx, gy);
  DISPATCH_KIND(kind, (weighted_sum_kernel<KIND><<<grid, 128, 0, stream>>>(x, c, B, cols, out)));
  return cudaGetLastError();
}

extern "C" int dpk_outer_norm_sq(const void* a, const void* g, int kind, int64_t B, int64_t d_a, int64_t d_g,
                                 float scale, float* out_w, float* out_b, int accumulate, cudaStream_t stream) {
  if (B <= 0) return 0;
  DISPATCH_KIND(kind, (outer_norm_sq_kernel<KIND><<<(unsigned)B, 256, 0, stream>>>(a, g, d_a, d_g, scale, out_w, out_b,
                                                                                 accumulate)));
  return cudaGetLastError();
}

extern "C" int dpk_norm_lastdim_grad(int norm_kind, const void* x, const void* g, int kind, int64_t B, int64_t rows,
                                     int64_t d, float eps, float* stats_scratch, float* gw, float* gb,
                                     cudaStream_t stream) {
  if (B <= 0 || rows <= 0 || d <= 0) return 0;
  float2* stats = reinterpret_cast<float2*>(stats_scratch);  // [B*rows] (mean, rstd)
  if (gw) cudaMemsetAsync(gw, 0, sizeof(float) * B * d, stream);
  if (gb) cudaMemsetAsync(gb, 0, sizeof(float) * B * d, stream);
  const int64_t nrows = B * rows;
  DISPATCH_KIND(kind, (row_stats_kernel<KIND><<<(unsigned)((nrows + 7) / 8), 256, 0, stream>>>(norm_kind, x, nrows, d, eps, stats)));
  int64_t rpb = rows;
  const int gx = (int)((d + 127) / 128);
  int64_t want_y = ((int64_t)num_sms() * 8) / ((int64_t)gx * B) + 1;
  if (want_y > rows) want_y = rows;
  rpb = (rows + want_y - 1) / want_y;
  const int gy = (int)((rows + rpb - 1) / rpb);
  if (B > 65535 || gy > 65535) return cudaErrorInvalidValue;
  dim3 grid(gx, gy, (unsigned)B);
  DISPATCH_KIND(kind, (lastdim_grad_kernel<KIND><<<grid, 128, 0, stream>>>(x, g, stats, rows, d, rpb, gw, gb)));
  return cudaGetLastError();
}

// One-launch form: tickets [B] must be ZERO on entry; part is scratch of dpk_norm_lastdim_psg_scratch_floats() floats.  Returns cudaErrorNotSupported when the shape is outside what the kernel covers
// (d % 8, d > 4096, or d > 2048 with a bias) so that the caller can take the two-kernel path.
// Blocks per sample: two blocks per SM over the whole batch, at least 16 rows (two per warp) per block.
static int64_t psg_chunks(int64_t B, int64_t rows) {
  int64_t chunks = ((int64_t)dpk::num_sms() * 2 + B - 1) / B;
  if (chunks > (rows + 15) / 16) chunks = (rows + 15) / 16;
  return chunks < 1 ? 1 : chunks;
}

extern "C" int64_t dpk_norm_lastdim_psg_scratch_floats(int64_t B, int64_t rows, int64_t d, int with_bias) {
  return B * psg_chunks(B, rows) * d * (with_bias ? 2 : 1);
}

extern "C" int dpk_norm_lastdim_psg_fused(int norm_kind, const void* x, const void* g, int kind, int64_t B,
                                          int64_t rows, int64_t d, float eps, float* gw, float* gb, float* n2w,
                                          float* n2b, int accumulate, unsigned int* tickets, float* part,
                                          cudaStream_t stream) {
  if (B <= 0 || rows <= 0 || d <= 0) return 0;
  const bool bias = gb != nullptr;
  if ((d & 7) || d > 4096 || (bias && d > 2048) || B > 65535 || gw == nullptr || part == nullptr)
    return cudaErrorNotSupported;
  if (((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(g)) & 15) != 0) return cudaErrorNotSupported;
  int64_t chunks = psg_chunks(B, rows);
  const int64_t rpb = (rows + chunks - 1) / chunks;
  chunks = (rows + rpb - 1) / rpb;
  dim3 grid((unsigned)chunks, (unsigned)B);
  const size_t smem = sizeof(float) * d * (bias ? 2 : 1);
  const int nv = (int)((d + 255) / 256);
#define PSG_LAUNCH(NV_, BIAS_)                                                                                   \
  DISPATCH_KIND(kind, (lastdim_psg_fused_kernel<KIND, NV_, BIAS_><<<grid, 256, smem, stream>>>(                  \
                          norm_kind, x, g, rows, d, rpb, eps, gw, gb, n2w, n2b, accumulate, tickets, part)))
  if (bias) {
    if (nv <= 1) { PSG_LAUNCH(1, true); } else if (nv <= 2) { PSG_LAUNCH(2, true); }
    else if (nv <= 4) { PSG_LAUNCH(4, true); } else { PSG_LAUNCH(8, true); }
  } else {
    if (nv <= 1) { PSG_LAUNCH(1, false); } else if (nv <= 2) { PSG_LAUNCH(2, false); }
    else if (nv <= 4) { PSG_LAUNCH(4, false); } else if (nv <= 8) { PSG_LAUNCH(8, false); }
    else { PSG_LAUNCH(16, false); }
  }
#undef PSG_LAUNCH
  return cudaGetLastError();
}

extern "C" int dpk_norm_channel_grad(const void* x, const void* g, int kind, int64_t B, int64_t C, int64_t S,
                                     int groups, float eps, float* gw, float* gb, cudaStream_t stream) {
  if (B <= 0 || C <= 0 || S <= 0 || groups <= 0 || C % groups) return cudaErrorInvalidValue;
  DISPATCH_KIND(kind, (channel_grad_kernel<KIND><<<(unsigned)(B * groups), 256, 0, stream>>>(x, g, C, S, groups, eps, gw, gb)));
  return cudaGetLastError();
}

extern "C" int dpk_embedding_scatter(const int64_t* ids, const void* g, int kind, const float* c, int64_t rows,
                                     int64_t T, int64_t D, int64_t V, int64_t padding_idx, float scale, float* out,
                                     cudaStream_t stream) {
  if (rows <= 0) return 0;
  const int grid = grid_for(rows * ((D + 3) >> 2), 256, num_sms() * 16);
  DISPATCH_KIND(kind, (embedding_scatter_kernel<KIND><<<grid, 256, 0, stream>>>(ids, g, c, rows, T, D, V, padding_idx,
                                                                               scale, out)));
  return cudaGetLastError();
}

extern "C" int dpk_fused_dp_step(const DpkTensorEntry* table, int n_tensors, int64_t total_chunks,
                                 const int64_t* chunk_prefix, DpkStepHyper h, cudaStream_t stream) {
  if (n_tensors <= 0 || total_chunks <= 0) return 0;
  if (total_chunks > 0x7fffffffLL) return cudaErrorInvalidValue;
  fused_dp_step_kernel<<<(unsigned)total_chunks, kStepThreads, 0, stream>>>(table, n_tensors, chunk_prefix, h);
  return cudaGetLastError();
}

extern "C" int dpk_philox_normal(float* out, int64_t n, uint64_t seed, uint64_t offset, float std, cudaStream_t stream) {
  if (n <= 0) return 0;
  philox_normal_kernel<<<grid_for((n + 3) / 4, 256, num_sms() * 8), 256, 0, stream>>>(out, n, seed, offset, std);
  return cudaGetLastError();
}
