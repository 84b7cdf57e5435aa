// Per-sample weight gradient of a 1-d / 2-d convolution without an unfolded copy of
// the input (implicit GEMM on tcgen05):
//
//   gs[b][o][i][j][c] = sum_{oh, ow} G[b][oh][ow][o] * X[b][oh*sh + i*dh - ph][ow*sw + j*dw - pw][c]
//
// with X and G channels-last (NHWC).  The reference materialises unfold(X) -- kh*kw
// times the input -- and calls einsum on it (opacus/grad_sample/conv.py:97-117,
// opacus/utils/tensor_utils.py:116-287).  Here the contraction index is the output
// pixel; a TMA box of bh x bw output pixels x 64 channels is, for both operands, 64
// swizzled 128-byte rows, i.e. the canonical MN-major tile of the tensor core.  For
// X the box is simply started at the pixel shifted by the filter tap (zero fill
// outside the image gives the padding; the map's element strides give the
// convolution stride), so every (tap, 64-channel block) is one more 64-column chunk
// of the N operand and nothing is ever unfolded in memory.
//
// Modes:
//   per sample   out[b][O][taps][C] (bf16 or fp32) and/or norm_sq[b] += ||gs_b||^2
//                (out == nullptr: norm only, the ghost-clipping norm of a conv layer)
//   batch sum    out[O][taps][C] = beta*out + sum_b (...), G pre-scaled by the clip
//                factors: the clipped gradient sum as ONE GEMM with K = B * pixels,
//                split along K over CTAs (fp32 vector atomics)
//
// Persistent CTAs; warp 0 = TMA producer, warp 1 = MMA issuer, warp 2 = TMEM
// allocation, warps 4-7 = epilogue; two TMEM accumulators so the epilogue of one
// tile overlaps the MMAs of the next.  Every wait is bounded.
#include "api.h"
#include "common.cuh"
#include "host_util.h"

namespace dpk {

constexpr int CV_BK = 64;                  // output pixels per stage
constexpr int CV_BOX_BYTES = CV_BK * 128;  // one 64-column chunk
constexpr int CV_BM = 128;                 // output channels per tile
constexpr int CV_MAXCH = 4;                // chunks per tile (N <= 256)
constexpr int CV_STAGES = 3;
constexpr int CV_ABYTES = 2 * CV_BOX_BYTES;
constexpr int CV_STAGE_BYTES = CV_ABYTES + CV_MAXCH * CV_BOX_BYTES;
constexpr int CV_THREADS = 256;
constexpr int CV_EPI_BYTES = 32 * 128;     // one staged 32-row x 64-channel bf16 block (128-byte swizzled rows)
constexpr int CV_EPI_TOTAL = 4 * CV_MAXCH * CV_EPI_BYTES;   // four epilogue warps x one whole tile row-block each

struct CvParams {
  int B, C, O, OH, OW;
  int kh, kw, sh, sw, ph, pw, dh, dw;
  int bh, bw, hblocks, wblocks;  // pixel block bh x bw = 64; blocks per sample
  int cblocks, chunks, nchunk;   // ceil(C/64); kh*kw*cblocks; chunks per tile
  int mt, nt;
  int reduce_batch, splits, kpb, ktotal, items;
  void* out;
  int out_bf16;
  float beta;
  float* norm_sq;
  uint32_t* status;
};

struct __align__(8) CvBarriers {
  uint64_t full[CV_STAGES];
  uint64_t empty[CV_STAGES];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  uint32_t abort_flag;
};

struct CvItem {
  int b, m0, nc0, k0, k1;
};

__device__ __forceinline__ CvItem cv_decode(const CvParams& p, int item) {
  CvItem w;
  const int tiles = p.mt * p.nt;
  if (p.reduce_batch) {
    const int split = item / tiles;
    const int tile = item - split * tiles;
    w.b = 0;
    w.m0 = (tile % p.mt) * CV_BM;
    w.nc0 = (tile / p.mt) * p.nchunk;
    const int per = (p.ktotal + p.splits - 1) / p.splits;
    w.k0 = split * per;
    w.k1 = min(p.ktotal, w.k0 + per);
  } else {
    w.b = item / tiles;
    const int tile = item - w.b * tiles;
    w.m0 = (tile % p.mt) * CV_BM;
    w.nc0 = (tile / p.mt) * p.nchunk;
    w.k0 = 0;
    w.k1 = p.kpb;
  }
  return w;
}

__global__ void __launch_bounds__(CV_THREADS, 1)
conv_psg_kernel(const __grid_constant__ CUtensorMap map_g, const __grid_constant__ CUtensorMap map_x,
                const __grid_constant__ CUtensorMap map_o, CvParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi = smem + CV_STAGES * CV_STAGE_BYTES;            // staging rows of the bf16 epilogue
  auto* bars = reinterpret_cast<CvBarriers*>(epi + CV_EPI_TOTAL);
  volatile uint32_t* abort_flag = &bars->abort_flag;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t stage_tx = CV_ABYTES + p.nchunk * CV_BOX_BYTES;

  if (threadIdx.x == 0) {
    for (int s = 0; s < CV_STAGES; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&bars->acc_full[a], 1);
      mbar_init(&bars->acc_empty[a], 4);
    }
    bars->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 2) {
    tmem_alloc(&bars->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      tma_prefetch_desc(&map_g);
      tma_prefetch_desc(&map_x);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < p.items && ok; item += gridDim.x) {
        const CvItem w = cv_decode(p, item);
        for (int kk = w.k0; kk < w.k1; ++kk) {
          int b = w.b, pb = kk;
          if (p.reduce_batch) { b = kk / p.kpb; pb = kk - b * p.kpb; }
          const int hb = pb / p.wblocks;
          const int oh0 = hb * p.bh;
          const int ow0 = (pb - hb * p.wblocks) * p.bw;
          if (!mbar_wait(&bars->empty[stage], phase ^ 1, abort_flag, p.status, 21)) { ok = false; break; }
          uint8_t* dst = smem + stage * CV_STAGE_BYTES;
          mbar_expect_tx(&bars->full[stage], stage_tx);
          // a box that lies wholly outside the tensor (o >= O, c >= C) is filled with zeros
          tma_load_4d(dst, &map_g, &bars->full[stage], w.m0, ow0, oh0, b);
          tma_load_4d(dst + CV_BOX_BYTES, &map_g, &bars->full[stage], w.m0 + 64, ow0, oh0, b);
          for (int j = 0; j < p.nchunk; ++j) {
            const int chunk = w.nc0 + j;
            int c0 = p.cblocks * 64, ih0 = 0, iw0 = 0;
            if (chunk < p.chunks) {
              const int tap = chunk / p.cblocks;
              c0 = (chunk - tap * p.cblocks) * 64;
              const int ti = tap / p.kw;
              ih0 = oh0 * p.sh + ti * p.dh - p.ph;
              iw0 = ow0 * p.sw + (tap - ti * p.kw) * p.dw - p.pw;
            }
            tma_load_4d(dst + CV_ABYTES + j * CV_BOX_BYTES, &map_x, &bars->full[stage], c0, iw0, ih0, b);
          }
          if (++stage == CV_STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {  // let loads that are still in flight land before the CTA exits
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 200000ull) {}
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      const uint32_t idesc = make_idesc(1, 1, 1, CV_BM, p.nchunk * 64);
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < p.items && ok; item += gridDim.x, ++local) {
        const CvItem w = cv_decode(p, item);
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        if (!mbar_wait(&bars->acc_empty[acc], acc_phase ^ 1, abort_flag, p.status, 22)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d0 = tmem_base + acc * 256;
        for (int kk = w.k0; kk < w.k1; ++kk) {
          if (!mbar_wait(&bars->full[stage], phase, abort_flag, p.status, 23)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + stage * CV_STAGE_BYTES);
          const uint32_t b_addr = a_addr + CV_ABYTES;
#pragma unroll
          for (int k = 0; k < CV_BK / 16; ++k) {
            const uint64_t da = smem_desc_sw128(a_addr + k * 2048, CV_BOX_BYTES, 1024);
            const uint64_t db = smem_desc_sw128(b_addr + k * 2048, CV_BOX_BYTES, 1024);
            umma_f16(d0, da, db, idesc, (kk != w.k0 || k != 0) ? 1u : 0u);
          }
          umma_commit(&bars->empty[stage]);
          if (++stage == CV_STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(&bars->acc_full[acc]);
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ epilogue
    const int ew = warp - 4;
    const int taps = p.kh * p.kw;
    int local = 0;
    for (int item = blockIdx.x; item < p.items; item += gridDim.x, ++local) {
      const CvItem w = cv_decode(p, item);
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      if (!mbar_wait(&bars->acc_full[acc], acc_phase, abort_flag, p.status, 24)) break;
      tc_fence_after();
      float sq = 0.f;
      const int row = w.m0 + ew * 32 + lane;      // output channel o
      const uint32_t taddr = tmem_base + acc * 256 + (static_cast<uint32_t>(ew * 32) << 16);
      const int64_t row_base = ((int64_t)w.b * p.O + row) * taps;
      const bool atomic_out = p.reduce_batch && p.splits > 1;
      if (p.out != nullptr && p.out_bf16) {
        // bf16 gradients: every 32-row x 64-channel block is staged in shared memory in the 128-byte-swizzle
        // pattern and written with ONE tensor store, so global memory sees whole 128-byte rows instead of
        // 16-byte fragments.  The map clips rows >= O and channels >= C.
        const int o0 = w.m0 + ew * 32;
        uint8_t* stage0 = epi + ew * (CV_MAXCH * CV_EPI_BYTES);
        if (lane == 0) bulk_wait_read<0>();            // the previous tile's stores have left the staging rows
        __syncwarp();
        int nstore = 0;
#pragma unroll 1
        for (int j = 0; j < p.nchunk; ++j) {
          if (w.nc0 + j >= p.chunks) break;
          uint8_t* stage = stage0 + j * CV_EPI_BYTES;
          uint32_t r[2][32];                           // both halves of the 64-column chunk in flight at once
          tmem_ld_32x32(taddr + j * 64, r[0]);
          tmem_ld_32x32(taddr + j * 64 + 32, r[1]);
          tmem_ld_wait();
#pragma unroll
          for (int hlf = 0; hlf < 2; ++hlf) {
#pragma unroll
            for (int q8 = 0; q8 < 4; ++q8) {
              uint4 pk;
              uint32_t* pw = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const float v0 = __uint_as_float(r[hlf][q8 * 8 + 2 * q]), v1 = __uint_as_float(r[hlf][q8 * 8 + 2 * q + 1]);
                sq = fmaf(v0, v0, fmaf(v1, v1, sq));
                __nv_bfloat162 nv = __floats2bfloat162_rn(v0, v1);
                pw[q] = *reinterpret_cast<uint32_t*>(&nv);
              }
              const int c16 = hlf * 4 + q8;              // 16-byte column of the 128-byte row
              *reinterpret_cast<uint4*>(stage + lane * 128 + ((c16 ^ (lane & 7)) << 4)) = pk;
            }
          }
          ++nstore;
        }
        tc_fence_before();                             // the accumulator can be reused while the stores go out
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->acc_empty[acc]);
        fence_proxy_async();                           // ONE proxy fence per tile
        __syncwarp();
        if (lane == 0 && o0 < p.O) {
          for (int j = 0; j < nstore; ++j) {
            const int chunk = w.nc0 + j;
            const int tap = chunk / p.cblocks;
            tma_store_4d(&map_o, stage0 + j * CV_EPI_BYTES, (chunk - tap * p.cblocks) * 64, tap, o0, w.b);
          }
          bulk_commit();
        }
        if (p.norm_sq != nullptr) {
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
          if (lane == 0) atomicAdd(p.norm_sq + w.b, sq);
        }
        continue;
      }
#pragma unroll 1
      for (int c0 = 0; c0 < p.nchunk * 64; c0 += 32) {
        const int chunk = w.nc0 + (c0 >> 6);
        if (chunk >= p.chunks) break;
        uint32_t r[32];
        tmem_ld_32x32(taddr + c0, r);
        tmem_ld_wait();
        if (p.out == nullptr) {  // norm only: rows / channels outside the tensor are exact zeros
#pragma unroll
          for (int j = 0; j < 32; ++j) sq = fmaf(__uint_as_float(r[j]), __uint_as_float(r[j]), sq);
          continue;
        }
        if (row >= p.O) continue;
        const int tap = chunk / p.cblocks;
        const int ch = (chunk - tap * p.cblocks) * 64 + (c0 & 63);
        const int64_t off = (row_base + tap) * p.C + ch;
        if (p.out_bf16) {
          __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + off;
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            if (ch + j < p.C) {
              uint4 pk;
              uint32_t* pw = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const float v0 = __uint_as_float(r[j + 2 * q]), v1 = __uint_as_float(r[j + 2 * q + 1]);
                sq = fmaf(v0, v0, fmaf(v1, v1, sq));
                __nv_bfloat162 nv = __floats2bfloat162_rn(v0, v1);
                pw[q] = *reinterpret_cast<uint32_t*>(&nv);
              }
              *reinterpret_cast<uint4*>(o + j) = pk;
            }
          }
        } else {
          float* o = reinterpret_cast<float*>(p.out) + off;
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            if (ch + j < p.C) {
              float4 v = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]),
                                     __uint_as_float(r[j + 3]));
              sq = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, sq))));
              if (atomic_out) {
                asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(o + j), "f"(v.x), "f"(v.y),
                             "f"(v.z), "f"(v.w)
                             : "memory");
              } else {
                if (p.beta != 0.f) {
                  const float4 old = *reinterpret_cast<const float4*>(o + j);
                  v.x += p.beta * old.x; v.y += p.beta * old.y; v.z += p.beta * old.z; v.w += p.beta * old.w;
                }
                *reinterpret_cast<float4*>(o + j) = v;
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->acc_empty[acc]);
      if (p.norm_sq != nullptr && !p.reduce_batch) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
        if (lane == 0) atomicAdd(p.norm_sq + w.b, sq);
      }
    }
  }

  if (warp >= 4 && lane == 0) bulk_wait<0>();        // tensor stores of this warp have completed
  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace dpk

extern "C" int dpk_conv_psg(const void* x, const void* g, int B, int C, int H, int W, int O, int OH, int OW, int kh,
                            int kw, int sh, int sw, int ph, int pw, int dh, int dw, int reduce_batch, void* out,
                            int out_bf16, float beta, float* norm_sq, uint32_t* status, cudaStream_t stream) {
  using namespace dpk;
  if (B <= 0 || C <= 0 || O <= 0 || OH <= 0 || OW <= 0 || H <= 0 || W <= 0 || kh <= 0 || kw <= 0) return cudaErrorInvalidValue;
  if ((C % 8) != 0 || (O % 8) != 0 || sh < 1 || sw < 1 || sh > 8 || sw > 8) return cudaErrorInvalidValue;
  if (reduce_batch && (out == nullptr || out_bf16 || (beta != 0.f && beta != 1.f))) return cudaErrorInvalidValue;
  if (!reduce_batch && out != nullptr && out_bf16 && beta != 0.f) return cudaErrorInvalidValue;
  CvParams p{};
  p.B = B; p.C = C; p.O = O; p.OH = OH; p.OW = OW;
  p.kh = kh; p.kw = kw; p.sh = sh; p.sw = sw; p.ph = ph; p.pw = pw; p.dh = dh; p.dw = dw;
  int bw = 1;
  while (bw < OW && bw < 64) bw *= 2;
  p.bw = bw;
  p.bh = 64 / bw;
  p.wblocks = (OW + p.bw - 1) / p.bw;
  p.hblocks = (OH + p.bh - 1) / p.bh;
  p.kpb = p.wblocks * p.hblocks;
  p.cblocks = (C + 63) / 64;
  p.chunks = kh * kw * p.cblocks;
  p.mt = (O + CV_BM - 1) / CV_BM;
  // chunks per tile: the largest of 4..1 that wastes the fewest columns
  int best = 1, best_waste = 1 << 30;
  for (int n = CV_MAXCH; n >= 1; --n) {
    const int waste = (p.chunks + n - 1) / n * n - p.chunks;
    if (waste < best_waste) { best_waste = waste; best = n; }
  }
  p.nchunk = best;
  p.nt = (p.chunks + p.nchunk - 1) / p.nchunk;
  p.reduce_batch = reduce_batch ? 1 : 0;
  p.out = out; p.out_bf16 = out_bf16; p.beta = beta; p.norm_sq = norm_sq; p.status = status;
  const int sms = num_sms();
  if (p.reduce_batch) {
    p.ktotal = p.kpb * B;
    const int tiles = p.mt * p.nt;
    int s = (2 * sms + tiles - 1) / tiles;          // about two waves of CTAs
    const int max_s = p.ktotal / 8 > 0 ? p.ktotal / 8 : 1;
    if (s > max_s) s = max_s;
    if (s < 1) s = 1;
    p.splits = s;
    p.items = tiles * s;
  } else {
    p.ktotal = p.kpb;
    p.splits = 1;
    p.items = p.mt * p.nt * B;
  }
  CUtensorMap map_g, map_x;
  int rc = make_tmap_4d_bf16(&map_g, g, O, OW, OH, B, p.bw, p.bh, 1, 1);
  if (rc) return rc;
  rc = make_tmap_4d_bf16(&map_x, x, C, W, H, B, p.bw, p.bh, sw, sh);
  if (rc) return rc;
  CUtensorMap map_o = map_g;     // only read by the bf16 per-sample epilogue
  if (out != nullptr && out_bf16 && !reduce_batch) {
    rc = make_tmap_4d_bf16(&map_o, out, C, kh * kw, O, B, 1, 32, 1, 1);
    if (rc) return rc;
  }
  const size_t smem = 1024 + CV_STAGES * CV_STAGE_BYTES + CV_EPI_TOTAL + sizeof(CvBarriers);
  static_assert(1024 + CV_STAGES * CV_STAGE_BYTES + CV_EPI_TOTAL + sizeof(CvBarriers) <= 227 * 1024, "shared memory");
  cudaError_t e = cudaSuccess;
  {
    static bool attr_done[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !attr_done[dev]) {
      e = cudaFuncSetAttribute(conv_psg_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return e;
      if (dev >= 0 && dev < 64) attr_done[dev] = true;
    }
  }
  if (p.reduce_batch && p.splits > 1 && beta == 0.f) {
    e = cudaMemsetAsync(out, 0, sizeof(float) * (size_t)O * kh * kw * C, stream);
    if (e != cudaSuccess) return e;
  }
  const int grid = p.items < sms ? p.items : sms;
  conv_psg_kernel<<<grid, CV_THREADS, smem, stream>>>(map_g, map_x, map_o, p);
  return cudaGetLastError();
}
