// Ghost norm on tcgen05: per sample n,
//     out_w[n] = sum_{t,s} (X_n X_n^T)[t,s] * (G_n G_n^T)[t,s]   ( = ||G_n^T X_n||_F^2 )
//     out_b[n] = sum_{t,s} (G_n G_n^T)[t,s]                        ( = ||sum_t g_t||^2  )
// without ever storing a T x T matrix: each CTA walks over (sample, t-block, s-block)
// work items with s-block >= t-block (both Grams are symmetric; off-diagonal
// blocks count twice), accumulates the two 128x128 Gram tiles side by side in
// TMEM (K = d_x for X, K = d_g for G), and the epilogue multiplies and sums them.
// In "mask" mode X X^T is replaced by the indicator [id_t == id_s], which gives
// the embedding-layer norm with no sort or unique.
//
// Roles (256 threads): warp 0 = TMA producer, warp 1 = MMA issuer, warp 2 = TMEM
// allocator, warps 4-7 = epilogue.  A ring of kStages shared-memory stages feeds
// the MMAs; two TMEM accumulator sets let the epilogue of item i overlap the MMAs
// of item i+1.  Each item's result goes to scratch[item]; a second, tiny kernel
// adds them per sample in a fixed order, so results are bit-reproducible.
//
// Counterpart in the reference: opacus/grad_sample/linear.py:83-92 (two bmm's that
// materialise [B,T,T] each) and opacus/grad_sample/embedding_norm_sample.py:103-150.
#include "api.h"
#include "common.cuh"
#include "host_util.h"

namespace dpk {

constexpr int kTile = 128;                 // rows of a t- or s-block
constexpr int kBK = 64;                    // bf16 elements per k-block = 128 bytes = one swizzle row
constexpr int kStages = 6;
constexpr int kTileBytes = kTile * kBK * 2;        // 16 KB
constexpr int kStageBytes = 2 * kTileBytes;        // X-rows tile + X-cols tile
constexpr int kThreads = 256;
constexpr int kTmemCols = 512;
constexpr uint32_t kIdesc = make_idesc(/*bf16*/ 1, /*A K-major*/ 0, /*B K-major*/ 0, kTile, kTile);

struct GramParams {
  int B, T, nT, pairs, items;
  int kb_x, kb_g;          // k-blocks for the two Grams (kb_x == 0: no X operand)
  int mask_mode;           // X X^T := [id_t == id_s]
  int cross_mode;          // tied embedding / output layer: rows from map_x (G_E), columns from map_g (A_H),
                           // every (t-block, s-block) pair, product weighted by gather_src[n, s, ids[n, t]]
  const void* gather_src;  // [B, T, V] output-layer gradient (cross_mode)
  int64_t V;
  int gather_fp32;
  int want_w, want_b;
  int right_off;           // > 0: the column tiles are read right_off rows further down (the operands hold a "left"
                           // block of rows followed by a "right" block per sample: split fp32 operands)
  float* scratch;          // [items][2]
  const int64_t* ids;      // [B, T] when mask_mode
  uint32_t* status;
};

struct __align__(8) GramBarriers {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  uint32_t abort_flag;
  float warp_sum[4][2];
  int64_t col_ids[2][kTile];
};

// true iff `mine` is true for all 128 threads of the epilogue group (named barrier 1).
__device__ __forceinline__ bool group_all_ok(bool mine) {
  uint32_t any_bad;
  asm volatile(
      "{\n\t"
      ".reg .pred p, q;\n\t"
      "setp.eq.u32 p, %1, 0;\n\t"
      "bar.red.or.pred q, 1, 128, p;\n\t"
      "selp.u32 %0, 1, 0, q;\n\t"
      "}\n"
      : "=r"(any_bad)
      : "r"(mine ? 1u : 0u)
      : "memory");
  return any_bad == 0;
}

__device__ __forceinline__ void decode_item(int item, int pairs, int nT, int cross, int& n, int& tb, int& sb) {
  n = item / pairs;
  int p = item - n * pairs;
  if (cross) {
    tb = p / nT;
    sb = p - tb * nT;
    return;
  }
  tb = 0;
  while (p >= nT - tb) {
    p -= nT - tb;
    ++tb;
  }
  sb = tb + p;
}

__global__ void __launch_bounds__(kThreads, 1)
gram_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_g, GramParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  GramBarriers* bars = reinterpret_cast<GramBarriers*>(smem + kStages * kStageBytes);
  volatile uint32_t* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
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
    tmem_alloc(&bars->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;
  const int kb_total = p.kb_x + p.kb_g;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      if (p.kb_x) tma_prefetch_desc(&map_x);
      tma_prefetch_desc(&map_g);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < p.items && ok; item += gridDim.x) {
        int n, tb, sb;
        decode_item(item, p.pairs, p.nT, p.cross_mode, n, tb, sb);
        for (int kb = 0; kb < kb_total; ++kb) {
          if (!mbar_wait(&bars->empty[stage], phase ^ 1, abort_flag, p.status, 1)) { ok = false; break; }
          const CUtensorMap* map = kb < p.kb_x ? &map_x : &map_g;
          const int k0 = (kb < p.kb_x ? kb : kb - p.kb_x) * kBK;
          uint8_t* dst = smem + stage * kStageBytes;
          mbar_expect_tx(&bars->full[stage], kStageBytes);
          tma_load_3d(dst, map, &bars->full[stage], k0, tb * kTile, n);
          tma_load_3d(dst + kTileBytes, p.cross_mode ? &map_g : map, &bars->full[stage], k0,
                      sb * kTile + (p.cross_mode ? 0 : p.right_off), n);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
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
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < p.items && ok; item += gridDim.x, ++local) {
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        if (!mbar_wait(&bars->acc_empty[acc], acc_phase ^ 1, abort_flag, p.status, 2)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_x = tmem_base + acc * 256;
        const uint32_t d_g = d_x + 128;
        for (int kb = 0; kb < kb_total; ++kb) {
          if (!mbar_wait(&bars->full[stage], phase, abort_flag, p.status, 3)) { ok = false; break; }
          tc_fence_after();
          const bool is_x = kb < p.kb_x;
          const uint32_t d = is_x ? d_x : d_g;
          const int kfirst = is_x ? 0 : p.kb_x;
          const uint32_t a_addr = smem_u32(smem + stage * kStageBytes);
          const uint32_t b_addr = a_addr + kTileBytes;
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            const uint64_t da = smem_desc_sw128(a_addr + k * 32, 16, 1024);
            const uint64_t db = smem_desc_sw128(b_addr + k * 32, 16, 1024);
            umma_f16(d, da, db, kIdesc, (kb != kfirst || k != 0) ? 1u : 0u);
          }
          umma_commit(&bars->empty[stage]);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(&bars->acc_full[acc]);
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ epilogue
    const int ew = warp - 4;                     // TMEM lanes [32*ew, 32*ew+32)
    const int row = ew * 32 + lane;              // row of the t-block owned by this thread
    int local = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < p.items && ok; item += gridDim.x, ++local) {
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      int n, tb, sb;
      decode_item(item, p.pairs, p.nT, p.cross_mode, n, tb, sb);
      int64_t my_id = -1;
      if (p.cross_mode) {
        const int t = tb * kTile + row;
        my_id = t < p.T ? p.ids[(int64_t)n * p.T + t] : -1;
        if (my_id >= p.V) my_id = -1;
      } else if (p.mask_mode) {
        const int t = tb * kTile + row;
        const int s = sb * kTile + row;
        my_id = t < p.T ? p.ids[(int64_t)n * p.T + t] : -1 - (int64_t)t;
        bars->col_ids[acc][row] = s < p.T ? p.ids[(int64_t)n * p.T + s] : -2 - (int64_t)p.T - s;
        asm volatile("bar.sync 1, 128;" ::: "memory");
      }
      // The verdict of the bounded wait is made uniform over the 128 epilogue
      // threads, so that none of them is left alone at a later named barrier.
      ok = group_all_ok(mbar_wait(&bars->acc_full[acc], acc_phase, abort_flag, p.status, 4));
      if (!ok) break;
      tc_fence_after();
      const uint32_t t_x = tmem_base + acc * 256 + (static_cast<uint32_t>(ew * 32) << 16);
      const uint32_t t_g = t_x + 128;
      float sum_w = 0.f, sum_b = 0.f;
#pragma unroll 1
      for (int c0 = 0; c0 < kTile; c0 += 32) {
        uint32_t rg[32];
        if (p.cross_mode) {
          tmem_ld_32x32(t_x + c0, rg);
          tmem_ld_wait();
          if (my_id >= 0) {
            const int s0 = sb * kTile + c0;
            const int64_t base = ((int64_t)n * p.T + s0) * p.V + my_id;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if (s0 + j < p.T) {
                const float w = p.gather_fp32
                                    ? reinterpret_cast<const float*>(p.gather_src)[base + (int64_t)j * p.V]
                                    : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.gather_src)[base + (int64_t)j * p.V]);
                sum_w = fmaf(__uint_as_float(rg[j]), w, sum_w);
              }
            }
          }
          continue;
        }
        tmem_ld_32x32(t_g + c0, rg);
        if (p.mask_mode) {
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float q = __uint_as_float(rg[j]);
            sum_b += q;
            sum_w += (bars->col_ids[acc][c0 + j] == my_id) ? q : 0.f;
          }
        } else if (p.kb_x) {
          uint32_t rx[32];
          tmem_ld_32x32(t_x + c0, rx);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float q = __uint_as_float(rg[j]);
            sum_b += q;
            sum_w = fmaf(__uint_as_float(rx[j]), q, sum_w);
          }
        } else {
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) sum_b += __uint_as_float(rg[j]);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->acc_empty[acc]);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        sum_w += __shfl_xor_sync(0xffffffffu, sum_w, o);
        sum_b += __shfl_xor_sync(0xffffffffu, sum_b, o);
      }
      if (lane == 0) {
        bars->warp_sum[ew][0] = sum_w;
        bars->warp_sum[ew][1] = sum_b;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (ew == 0 && lane == 0) {
        const float wgt = (tb == sb || p.cross_mode) ? 1.f : 2.f;
        float w = 0.f, b = 0.f;
        for (int i = 0; i < 4; ++i) {
          w += bars->warp_sum[i][0];
          b += bars->warp_sum[i][1];
        }
        p.scratch[2 * (int64_t)item] = w * wgt;
        p.scratch[2 * (int64_t)item + 1] = b * wgt;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// out[n] (+)= scale * sum over the sample's items, in item order.
__global__ void gram_reduce_kernel(const float* scratch, int B, int pairs, float scale, float* out_w, float* out_b,
                                   int accumulate, const uint32_t* status, int signed_sum = 0) {
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= B) return;
  float w = 0.f, b = 0.f;
  for (int j = 0; j < pairs; ++j) {
    w += scratch[2 * ((int64_t)n * pairs + j)];
    b += scratch[2 * ((int64_t)n * pairs + j) + 1];
  }
  if (status != nullptr && status[0] != 0) { w = nanf(""); b = nanf(""); }
  if (out_w) out_w[n] = (accumulate ? out_w[n] : 0.f) + (signed_sum ? w : fmaxf(w, 0.f)) * scale + (w != w ? w : 0.f);
  if (out_b) out_b[n] = (accumulate ? out_b[n] : 0.f) + fmaxf(b, 0.f) * scale + (b != b ? b : 0.f);
}

}  // namespace dpk

using namespace dpk;

extern "C" size_t dpk_gram_pair_scratch_floats(int B, int T) {
  const size_t nT = (T + kTile - 1) / kTile;
  return 2 * static_cast<size_t>(B) * (nT * (nT + 1) / 2);
}

int dpk_gram_pair_launch_lr(const void* x, const int64_t* ids, const void* g, int B, int T, int d_x, int d_g,
                            int right_off, float scale, float* scratch, float* out_w, float* out_b, int accumulate,
                            uint32_t* status, cudaStream_t stream);

int dpk_gram_pair_launch(const void* x, const int64_t* ids, const void* g, int B, int T, int d_x, int d_g, float scale,
                         float* scratch, float* out_w, float* out_b, int accumulate, uint32_t* status,
                         cudaStream_t stream) {
  return dpk_gram_pair_launch_lr(x, ids, g, B, T, d_x, d_g, 0, scale, scratch, out_w, out_b, accumulate, status, stream);
}

// right_off > 0: x and g are [B, 2 * right_off, d] with rows [0, T) the left operand and rows
// [right_off, right_off + T) the right operand of each Gram product (rows in between zero); right_off is a
// multiple of 128 and at least T.  The products L R^T must be symmetric (they are for split fp32 operands).
int dpk_gram_pair_launch_lr(const void* x, const int64_t* ids, const void* g, int B, int T, int d_x, int d_g,
                            int right_off, float scale, float* scratch, float* out_w, float* out_b, int accumulate,
                            uint32_t* status, cudaStream_t stream) {
  if (B <= 0 || T <= 0 || d_g <= 0 || (d_g % 8) != 0 || (x != nullptr && (d_x <= 0 || (d_x % 8) != 0)))
    return cudaErrorInvalidValue;
  if (right_off < 0 || (right_off > 0 && ((right_off % kTile) != 0 || right_off < T))) return cudaErrorInvalidValue;
  const int rows = right_off > 0 ? 2 * right_off : T;
  GramParams p{};
  p.right_off = right_off;
  p.B = B;
  p.T = T;
  p.nT = (T + kTile - 1) / kTile;
  p.pairs = p.nT * (p.nT + 1) / 2;
  p.items = B * p.pairs;
  p.kb_x = x ? (d_x + kBK - 1) / kBK : 0;
  p.kb_g = (d_g + kBK - 1) / kBK;
  p.mask_mode = (x == nullptr && ids != nullptr) ? 1 : 0;
  p.want_w = out_w != nullptr;
  p.want_b = out_b != nullptr;
  p.scratch = scratch;
  p.ids = ids;
  p.status = status;

  CUtensorMap map_x, map_g;
  int rc = make_tmap_3d_bf16(&map_g, g, d_g, rows, B, kBK, kTile);
  if (rc) return rc;
  if (x) {
    rc = make_tmap_3d_bf16(&map_x, x, d_x, rows, B, kBK, kTile);
    if (rc) return rc;
  } else {
    map_x = map_g;
  }
  const size_t smem = 1024 + kStages * kStageBytes + sizeof(GramBarriers);
  {
    static bool attr_done[64] = {false};   // per device; the attribute only has to be set once
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !attr_done[dev]) {
      cudaError_t e = cudaFuncSetAttribute(gram_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return e;
      if (dev >= 0 && dev < 64) attr_done[dev] = true;
    }
  }
  const int grid = p.items < num_sms() ? p.items : num_sms();
  gram_pair_kernel<<<grid, kThreads, smem, stream>>>(map_x, map_g, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  gram_reduce_kernel<<<(B + 127) / 128, 128, 0, stream>>>(scratch, B, p.pairs, scale, out_w, out_b, accumulate, status);
  return cudaGetLastError();
}

extern "C" int dpk_gram_pair_norm(const void* x, const int64_t* ids, const void* g, int B, int T, int d_x, int d_g,
                                  float scale, float* scratch, float* out_w, float* out_b, int accumulate,
                                  uint32_t* status, cudaStream_t stream) {
  return dpk_gram_pair_launch(x, ids, g, B, T, d_x, d_g, scale, scratch, out_w, out_b, accumulate, status, stream);
}

extern "C" int dpk_gram_pair_norm_lr(const void* x, const int64_t* ids, const void* g, int B, int T, int d_x, int d_g,
                                     int right_off, float scale, float* scratch, float* out_w, float* out_b,
                                     int accumulate, uint32_t* status, cudaStream_t stream) {
  return dpk_gram_pair_launch_lr(x, ids, g, B, T, d_x, d_g, right_off, scale, scratch, out_w, out_b, accumulate, status,
                                 stream);
}

// 2 <g_E, g_H> of a weight shared by an embedding (ids, output gradient g_e [B, T, D]) and an output projection
// (input a_h [B, T, D], output gradient g_h [B, T, V]):  out[n] (+)= scale * sum_{t,s} g_h[n, s, ids[n, t]] * <g_e[n, t], a_h[n, s]>.
// scratch: 2 * B * ceil(T/128)^2 floats.
extern "C" int dpk_tied_cross_norm(const int64_t* ids, const void* g_e, const void* a_h, const void* g_h, int g_h_fp32,
                                   int B, int T, int D, int64_t V, float scale, float* scratch, float* out,
                                   int accumulate, uint32_t* status, cudaStream_t stream) {
  if (B <= 0 || T <= 0 || D <= 0 || (D % 8) != 0 || V <= 0) return cudaErrorInvalidValue;
  GramParams p{};
  p.B = B;
  p.T = T;
  p.nT = (T + kTile - 1) / kTile;
  p.pairs = p.nT * p.nT;
  p.items = B * p.pairs;
  p.kb_x = (D + kBK - 1) / kBK;
  p.kb_g = 0;
  p.cross_mode = 1;
  p.want_w = 1;
  p.scratch = scratch;
  p.ids = ids;
  p.gather_src = g_h;
  p.gather_fp32 = g_h_fp32;
  p.V = V;
  p.status = status;
  CUtensorMap map_x, map_g;
  int rc = make_tmap_3d_bf16(&map_x, g_e, D, T, B, kBK, kTile);
  if (rc) return rc;
  rc = make_tmap_3d_bf16(&map_g, a_h, D, T, B, kBK, kTile);
  if (rc) return rc;
  const size_t smem = 1024 + kStages * kStageBytes + sizeof(GramBarriers);
  cudaError_t e = cudaFuncSetAttribute(gram_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  const int grid = p.items < num_sms() ? p.items : num_sms();
  gram_pair_kernel<<<grid, kThreads, smem, stream>>>(map_x, map_g, p);
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  gram_reduce_kernel<<<(B + 127) / 128, 128, 0, stream>>>(scratch, B, p.pairs, scale, out, nullptr, accumulate, status, 1);
  return cudaGetLastError();
}
