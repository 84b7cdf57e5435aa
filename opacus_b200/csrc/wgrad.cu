// Transposed-operand GEMM on tcgen05 for the two gradient products of DP training:
//
//   clipped sum      out[M, N]      = beta * out + Gs^T A        Gs [K, M], A [K, N], K = B*T (all tokens)
//   per-sample grads out[b][M, N]   = G_b^T A_b  (+ ||.||_F^2)   G [B, T, M], A [B, T, N], K = T
//
// The first replaces the whole second backward pass of two-pass ghost clipping
// (opacus/utils/fast_gradient_clipping_utils.py:194-201); the second is the
// "hooks" mode per-sample gradient of a Linear layer with the per-sample norm
// of opacus/optimizers/optimizer.py:444-446 fused into its epilogue
// (opacus/grad_sample/linear.py:47).
//
// Both operands have the contraction index as their *outer* dimension, i.e. they
// are "MN-major" for the tensor core: a TMA box of 64 rows (K) x 64 columns lands
// in shared memory as 64 swizzled 128-byte rows, which is exactly the canonical
// MN-major 128B-swizzle layout (8-row groups 1024 bytes apart, next block of 64
// columns one box further).  No transpose is ever materialised.
//
// Persistent CTAs (one per SM) walk over work items (batch, m-tile, n-tile, k-split)
// in an order that keeps concurrently running tiles inside a compact block of the
// output (L2 reuse of both operands).  Warp 0 feeds a ring of shared-memory stages
// with TMA, warp 1 issues the MMAs, warps 4-7 drain TMEM to global memory.
//   BM = 128: two TMEM accumulators, the epilogue of one tile overlaps the MMAs of the next;
//   BM = 256: two 128-row accumulators share every A panel (half the operand bytes
//             per FLOP); the epilogue is not overlapped.
// Small outputs with a long contraction are split along K; the partial tiles are
// added with fp32 atomics (the summation order is then not fixed).
#include "api.h"
#include "common.cuh"
#include "host_util.h"

namespace dpk {

constexpr int WG_BK = 64;              // rows (contraction) per stage
constexpr int WG_BOX = 64;             // columns per TMA box = 128 bytes
constexpr int WG_BOX_BYTES = WG_BK * 128;
constexpr int WG_THREADS = 256;
constexpr int WG_GROUP_M = 8;          // m-tiles per raster group

template <int BM, int BN>
struct WgCfg {
  static constexpr int kHalves = BM / 128;                           // accumulators per tile
  static constexpr int kABytes = (BM / WG_BOX) * WG_BOX_BYTES;       // Gs tile
  static constexpr int kBBytes = (BN / WG_BOX) * WG_BOX_BYTES;       // A tile
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = (200 * 1024) / kStageBytes > 6 ? 6 : (200 * 1024) / kStageBytes;
  static constexpr int kAccSets = BM == 128 ? 2 : 1;                 // double buffering only for BM = 128
  static constexpr int kTmemCols = (kHalves * kAccSets * BN) <= 256 ? 256 : 512;
  static constexpr uint32_t kIdesc = make_idesc(1, 1, 1, 128, BN);
};

struct WgParams {
  int K, M, N, batch;
  int mt, nt, splits, kblocks, items;
  void* out;
  float* norm_sq;        // [batch] or null
  int out_bf16;
  int atomic_out;        // splits > 1
  float beta;
  uint32_t* status;
};

template <int STAGES>
struct __align__(8) WgBarriers {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  uint32_t abort_flag;
};

struct WgItem {
  int b, m0, n0, kb0, kb1;
};

template <int BM, int BN>
__device__ __forceinline__ WgItem wg_decode(const WgParams& p, int item) {
  WgItem w;
  const int tiles_per_batch = p.mt * p.nt;
  const int per_b = tiles_per_batch * p.splits;
  w.b = item / per_b;
  int r = item - w.b * per_b;
  const int split = r / tiles_per_batch;
  int tile = r - split * tiles_per_batch;
  const int per_group = WG_GROUP_M * p.nt;
  const int group = tile / per_group;
  const int first_m = group * WG_GROUP_M;
  const int gsize = min(p.mt - first_m, WG_GROUP_M);
  const int in_group = tile - group * per_group;
  w.m0 = (first_m + in_group % gsize) * BM;
  w.n0 = (in_group / gsize) * BN;
  const int per_split = (p.kblocks + p.splits - 1) / p.splits;
  w.kb0 = split * per_split;
  w.kb1 = min(p.kblocks, w.kb0 + per_split);
  return w;
}

template <int BM, int BN>
__global__ void __launch_bounds__(WG_THREADS, 1)
wgrad_tn_kernel(const __grid_constant__ CUtensorMap map_g, const __grid_constant__ CUtensorMap map_a, WgParams p) {
  using Cfg = WgCfg<BM, BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  auto* bars = reinterpret_cast<WgBarriers<Cfg::kStages>*>(smem + Cfg::kStages * Cfg::kStageBytes);
  volatile uint32_t* abort_flag = &bars->abort_flag;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; ++s) {
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
    tmem_alloc(&bars->tmem_base, Cfg::kTmemCols);
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
      tma_prefetch_desc(&map_a);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < p.items && ok; item += gridDim.x) {
        const WgItem w = wg_decode<BM, BN>(p, item);
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          if (!mbar_wait(&bars->empty[stage], phase ^ 1, abort_flag, p.status, 11)) { ok = false; break; }
          uint8_t* dst = smem + stage * Cfg::kStageBytes;
          mbar_expect_tx(&bars->full[stage], Cfg::kStageBytes);
#pragma unroll
          for (int j = 0; j < BM / WG_BOX; ++j)
            tma_load_3d(dst + j * WG_BOX_BYTES, &map_g, &bars->full[stage], w.m0 + j * WG_BOX, kb * WG_BK, w.b);
#pragma unroll
          for (int j = 0; j < BN / WG_BOX; ++j)
            tma_load_3d(dst + Cfg::kABytes + j * WG_BOX_BYTES, &map_a, &bars->full[stage], w.n0 + j * WG_BOX,
                        kb * WG_BK, w.b);
          if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
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
        const WgItem w = wg_decode<BM, BN>(p, item);
        const int acc = Cfg::kAccSets == 2 ? (local & 1) : 0;
        const uint32_t acc_phase = Cfg::kAccSets == 2 ? ((local >> 1) & 1) : (local & 1);
        if (!mbar_wait(&bars->acc_empty[acc], acc_phase ^ 1, abort_flag, p.status, 12)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d0 = tmem_base + acc * (Cfg::kHalves * BN);
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          if (!mbar_wait(&bars->full[stage], phase, abort_flag, p.status, 13)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + stage * Cfg::kStageBytes);
          const uint32_t b_addr = a_addr + Cfg::kABytes;
#pragma unroll
          for (int k = 0; k < WG_BK / 16; ++k) {
            // 16 contraction rows = 2048 bytes further into every 64-column box
            const uint64_t db = smem_desc_sw128(b_addr + k * 2048, WG_BOX_BYTES, 1024);
#pragma unroll
            for (int h = 0; h < Cfg::kHalves; ++h) {
              const uint64_t da = smem_desc_sw128(a_addr + h * 2 * WG_BOX_BYTES + k * 2048, WG_BOX_BYTES, 1024);
              umma_f16(d0 + h * BN, da, db, Cfg::kIdesc, (kb != w.kb0 || k != 0) ? 1u : 0u);
            }
          }
          umma_commit(&bars->empty[stage]);
          if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(&bars->acc_full[acc]);
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ epilogue
    const int ew = warp - 4;
    int local = 0;
    for (int item = blockIdx.x; item < p.items; item += gridDim.x, ++local) {
      const WgItem w = wg_decode<BM, BN>(p, item);
      const int acc = Cfg::kAccSets == 2 ? (local & 1) : 0;
      const uint32_t acc_phase = Cfg::kAccSets == 2 ? ((local >> 1) & 1) : (local & 1);
      if (!mbar_wait(&bars->acc_full[acc], acc_phase, abort_flag, p.status, 14)) break;
      tc_fence_after();
      float sq = 0.f;
      const int64_t out_base = (int64_t)w.b * p.M * p.N;
#pragma unroll 1
      for (int h = 0; h < Cfg::kHalves; ++h) {
        const int row = w.m0 + h * 128 + ew * 32 + lane;
        const uint32_t taddr = tmem_base + acc * (Cfg::kHalves * BN) + h * BN + (static_cast<uint32_t>(ew * 32) << 16);
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          uint32_t r[32];
          tmem_ld_32x32(taddr + c0, r);
          tmem_ld_wait();
          const int col = w.n0 + c0;
          if (p.out == nullptr) {          // norm only: rows/columns outside the matrix are exact zeros
#pragma unroll
            for (int j = 0; j < 32; ++j) sq = fmaf(__uint_as_float(r[j]), __uint_as_float(r[j]), sq);
          } else if (row < p.M && col < p.N) {
            if (p.out_bf16) {
              __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + out_base + (int64_t)row * p.N + col;
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                if (col + j < p.N) {
                  uint4 pk;
                  uint32_t* pw = reinterpret_cast<uint32_t*>(&pk);
                  if (p.beta != 0.f) pk = *reinterpret_cast<const uint4*>(o + j);
#pragma unroll
                  for (int q = 0; q < 4; ++q) {
                    float v0 = __uint_as_float(r[j + 2 * q]), v1 = __uint_as_float(r[j + 2 * q + 1]);
                    sq = fmaf(v0, v0, fmaf(v1, v1, sq));
                    if (p.beta != 0.f) {
                      __nv_bfloat162 old = *reinterpret_cast<__nv_bfloat162*>(&pw[q]);
                      v0 += p.beta * __bfloat162float(old.x);
                      v1 += p.beta * __bfloat162float(old.y);
                    }
                    __nv_bfloat162 nv = __floats2bfloat162_rn(v0, v1);
                    pw[q] = *reinterpret_cast<uint32_t*>(&nv);
                  }
                  *reinterpret_cast<uint4*>(o + j) = pk;
                }
              }
            } else {
              float* o = reinterpret_cast<float*>(p.out) + out_base + (int64_t)row * p.N + col;
              if (p.atomic_out) {
#pragma unroll
                for (int j = 0; j < 32; j += 4)
                  if (col + j < p.N)
                    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(o + j),
                                 "f"(__uint_as_float(r[j])), "f"(__uint_as_float(r[j + 1])),
                                 "f"(__uint_as_float(r[j + 2])), "f"(__uint_as_float(r[j + 3]))
                                 : "memory");
              } else {
#pragma unroll
                for (int j = 0; j < 32; j += 4) {
                  if (col + j < p.N) {
                    float4 v = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]),
                                           __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
                    sq = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, sq))));
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
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->acc_empty[acc]);
      if (p.norm_sq != nullptr) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
        if (lane == 0) atomicAdd(p.norm_sq + w.b, sq);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

// [d2][d1][d0] tensor of 16-bit elements; box = (64, 64, 1)
template <int BM, int BN>
int launch_wgrad(const void* gs, const void* a, int K, int M, int N, int batch, int splits, void* out, int out_bf16,
                 float beta, float* norm_sq, uint32_t* status, cudaStream_t stream) {
  using Cfg = WgCfg<BM, BN>;
  WgParams p{};
  p.K = K; p.M = M; p.N = N; p.batch = batch;
  p.mt = (M + BM - 1) / BM;
  p.nt = (N + BN - 1) / BN;
  p.kblocks = (K + WG_BK - 1) / WG_BK;
  p.splits = splits;
  p.items = p.mt * p.nt * splits * batch;
  p.out = out; p.out_bf16 = out_bf16; p.beta = beta; p.status = status;
  p.norm_sq = norm_sq;
  p.atomic_out = splits > 1 ? 1 : 0;
  CUtensorMap map_g, map_a;
  int rc = make_tmap_3d_bf16(&map_g, gs, M, K, batch, WG_BOX, WG_BK);
  if (rc) return rc;
  rc = make_tmap_3d_bf16(&map_a, a, N, K, batch, WG_BOX, WG_BK);
  if (rc) return rc;
  const size_t smem = 1024 + Cfg::kStages * Cfg::kStageBytes + sizeof(WgBarriers<Cfg::kStages>);
  cudaError_t e = cudaSuccess;
  {
    static bool attr_done[64] = {false};   // per device and per tile shape (this function is a template)
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !attr_done[dev]) {
      e = cudaFuncSetAttribute(wgrad_tn_kernel<BM, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return e;
      if (dev >= 0 && dev < 64) attr_done[dev] = true;
    }
  }
  if (p.atomic_out && beta == 0.f) {
    e = cudaMemsetAsync(out, 0, sizeof(float) * (size_t)M * N * batch, stream);
    if (e != cudaSuccess) return e;
  }
  const int grid = p.items < num_sms() ? p.items : num_sms();
  wgrad_tn_kernel<BM, BN><<<grid, WG_THREADS, smem, stream>>>(map_g, map_a, p);
  return cudaGetLastError();
}

// Picks tile shape and K split for the given problem; `force` (bm*1000+bn*... ) is for tests.
int wgrad_dispatch(const void* gs, const void* a, int K, int M, int N, int batch, void* out, int out_bf16, float beta,
                   float* norm_sq, int force_bm, int force_bn, int force_splits, uint32_t* status,
                   cudaStream_t stream) {
  if (K <= 0 || M <= 0 || N <= 0 || batch <= 0 || (M % 8) != 0 || (N % 8) != 0) return cudaErrorInvalidValue;
  const int sms = num_sms();
  const int kblocks = (K + WG_BK - 1) / WG_BK;
  const bool may_split = batch == 1 && norm_sq == nullptr && out != nullptr && !out_bf16 && (beta == 0.f || beta == 1.f);
  struct Cand { int bm, bn; double w; };
  const Cand cands[3] = {{256, 256, 1.0}, {128, 256, 0.8}, {128, 128, 0.62}};
  int best_bm = 128, best_bn = 128, best_s = 1;
  double best = -1.0;
  for (const Cand& c : cands) {
    if (force_bm && (c.bm != force_bm || c.bn != force_bn)) continue;
    if (!force_bm && ((c.bm == 256 && M < 192) || (c.bn == 256 && N < 192))) continue;
    const long tiles = (long)((M + c.bm - 1) / c.bm) * ((N + c.bn - 1) / c.bn) * batch;
    for (int s = 1; s <= 8; s *= 2) {
      if (force_splits && s != force_splits) continue;
      if (s > 1 && (!may_split || kblocks < 8 * s)) continue;
      const long items = tiles * s;
      const long waves = (items + sms - 1) / sms;
      double score = c.w * (double)items / (double)(waves * sms);
      for (int q = s; q > 1; q >>= 1) score *= 0.85;   // atomics and the zero-fill are not free
      if (score > best) { best = score; best_bm = c.bm; best_bn = c.bn; best_s = s; }
    }
  }
  if (best < 0) return cudaErrorInvalidValue;
#define WG_CASE(BM_, BN_)                                                                                       \
  if (best_bm == BM_ && best_bn == BN_)                                                                          \
    return launch_wgrad<BM_, BN_>(gs, a, K, M, N, batch, best_s, out, out_bf16, beta, norm_sq, status, stream);
  WG_CASE(256, 256)
  WG_CASE(128, 256)
  WG_CASE(128, 128)
#undef WG_CASE
  return cudaErrorInvalidValue;
}

}  // namespace dpk

extern "C" int dpk_wgrad_tn(const void* gs, const void* a, int K, int M, int N, void* out, int out_bf16, float beta,
                            uint32_t* status, cudaStream_t stream) {
  return dpk::wgrad_dispatch(gs, a, K, M, N, 1, out, out_bf16, beta, nullptr, 0, 0, 0, status, stream);
}

extern "C" int dpk_wgrad_tn_ex(const void* gs, const void* a, int K, int M, int N, int batch, void* out, int out_bf16,
                               float beta, float* norm_sq, int force_bm, int force_bn, int force_splits,
                               uint32_t* status, cudaStream_t stream) {
  return dpk::wgrad_dispatch(gs, a, K, M, N, batch, out, out_bf16, beta, norm_sq, force_bm, force_bn, force_splits,
                             status, stream);
}
