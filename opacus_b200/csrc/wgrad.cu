// Clipped weight gradient on tcgen05:  out[M, N] = beta * out + Gs^T A  with
// Gs = diag(c) G of shape [K, M] and A of shape [K, N], K = B*T rows (all samples
// and positions), both row-major bf16.  One ordinary GEMM with contraction over
// every token replaces the whole second backward pass of two-pass ghost clipping
// (opacus/utils/fast_gradient_clipping_utils.py:194-201).
//
// Both operands have the contraction index as their *outer* dimension, i.e. they
// are "MN-major" for the tensor core: a TMA box of 64 rows (K) x 64 columns lands
// in shared memory as 64 swizzled 128-byte rows, which is exactly the canonical
// MN-major 128B-swizzle layout (8-row groups 1024 bytes apart, next block of 64
// columns one box further).  No transpose is ever materialised.
//
// Persistent CTAs (one per SM) walk over 128 x BN output tiles; warp 0 feeds a
// ring of shared-memory stages with TMA, warp 1 issues the MMAs into one of two
// TMEM accumulators, warps 4-7 drain the other one to global memory.
#include "api.h"
#include "common.cuh"
#include "host_util.h"

namespace dpk {

constexpr int WG_BM = 128;
constexpr int WG_BK = 64;              // rows (contraction) per stage
constexpr int WG_BOX = 64;             // columns per TMA box = 128 bytes
constexpr int WG_BOX_BYTES = WG_BK * 128;
constexpr int WG_THREADS = 256;

template <int BN>
struct WgCfg {
  static constexpr int kABytes = (WG_BM / WG_BOX) * WG_BOX_BYTES;   // Gs tile
  static constexpr int kBBytes = (BN / WG_BOX) * WG_BOX_BYTES;      // A tile
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = BN == 256 ? 4 : 6;
  static constexpr int kTmemCols = 2 * BN;                          // two accumulators
  static constexpr uint32_t kIdesc = make_idesc(1, 1, 1, WG_BM, BN);
};

struct WgParams {
  int K, M, N;
  int mt, nt, tiles, kblocks;
  void* out;
  int out_bf16;
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

template <int BN>
__global__ void __launch_bounds__(WG_THREADS, 1)
wgrad_tn_kernel(const __grid_constant__ CUtensorMap map_g, const __grid_constant__ CUtensorMap map_a, WgParams p) {
  using Cfg = WgCfg<BN>;
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
    if (elect_one()) {
      tma_prefetch_desc(&map_g);
      tma_prefetch_desc(&map_a);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < p.tiles && ok; tile += gridDim.x) {
        const int m0 = (tile % p.mt) * WG_BM;
        const int n0 = (tile / p.mt) * BN;
        for (int kb = 0; kb < p.kblocks; ++kb) {
          if (!mbar_wait(&bars->empty[stage], phase ^ 1, abort_flag, p.status, 11)) { ok = false; break; }
          uint8_t* dst = smem + stage * Cfg::kStageBytes;
          mbar_expect_tx(&bars->full[stage], Cfg::kStageBytes);
#pragma unroll
          for (int j = 0; j < WG_BM / WG_BOX; ++j)
            tma_load_2d(dst + j * WG_BOX_BYTES, &map_g, &bars->full[stage], m0 + j * WG_BOX, kb * WG_BK);
#pragma unroll
          for (int j = 0; j < BN / WG_BOX; ++j)
            tma_load_2d(dst + Cfg::kABytes + j * WG_BOX_BYTES, &map_a, &bars->full[stage], n0 + j * WG_BOX,
                        kb * WG_BK);
          if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 200000ull) {}
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < p.tiles && ok; tile += gridDim.x, ++local) {
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        if (!mbar_wait(&bars->acc_empty[acc], acc_phase ^ 1, abort_flag, p.status, 12)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d = tmem_base + acc * BN;
        for (int kb = 0; kb < p.kblocks; ++kb) {
          if (!mbar_wait(&bars->full[stage], phase, abort_flag, p.status, 13)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + stage * Cfg::kStageBytes);
          const uint32_t b_addr = a_addr + Cfg::kABytes;
#pragma unroll
          for (int k = 0; k < WG_BK / 16; ++k) {
            // 16 contraction rows = 2048 bytes further into every 64-column box
            const uint64_t da = smem_desc_sw128(a_addr + k * 2048, WG_BOX_BYTES, 1024);
            const uint64_t db = smem_desc_sw128(b_addr + k * 2048, WG_BOX_BYTES, 1024);
            umma_f16(d, da, db, Cfg::kIdesc, (kb | k) ? 1u : 0u);
          }
          umma_commit(&bars->empty[stage]);
          if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(&bars->acc_full[acc]);
      }
    }
  } else if (warp >= 4) {
    const int ew = warp - 4;
    int local = 0;
    for (int tile = blockIdx.x; tile < p.tiles; tile += gridDim.x, ++local) {
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      const int m0 = (tile % p.mt) * WG_BM;
      const int n0 = (tile / p.mt) * BN;
      if (!mbar_wait(&bars->acc_full[acc], acc_phase, abort_flag, p.status, 14)) break;
      tc_fence_after();
      const int row = m0 + ew * 32 + lane;
      const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(ew * 32) << 16);
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c0, r);
        tmem_ld_wait();
        const int col = n0 + c0;
        if (row < p.M && col < p.N) {
          if (p.out_bf16) {
            __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + (int64_t)row * p.N + col;
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              if (col + j < p.N) {
                uint4 pk;
                uint32_t* pw = reinterpret_cast<uint32_t*>(&pk);
                if (p.beta != 0.f) pk = *reinterpret_cast<const uint4*>(o + j);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  float v0 = __uint_as_float(r[j + 2 * q]), v1 = __uint_as_float(r[j + 2 * q + 1]);
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
            float* o = reinterpret_cast<float*>(p.out) + (int64_t)row * p.N + col;
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              if (col + j < p.N) {
                float4 v = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]),
                                       __uint_as_float(r[j + 3]));
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
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

template <int BN>
int launch_wgrad(const void* gs, const void* a, int K, int M, int N, void* out, int out_bf16, float beta,
                 uint32_t* status, cudaStream_t stream) {
  using Cfg = WgCfg<BN>;
  WgParams p{};
  p.K = K; p.M = M; p.N = N;
  p.mt = (M + WG_BM - 1) / WG_BM;
  p.nt = (N + BN - 1) / BN;
  p.tiles = p.mt * p.nt;
  p.kblocks = (K + WG_BK - 1) / WG_BK;
  p.out = out; p.out_bf16 = out_bf16; p.beta = beta; p.status = status;
  CUtensorMap map_g, map_a;
  int rc = make_tmap_2d_bf16(&map_g, gs, M, K, WG_BOX, WG_BK);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&map_a, a, N, K, WG_BOX, WG_BK);
  if (rc) return rc;
  const size_t smem = 1024 + Cfg::kStages * Cfg::kStageBytes + sizeof(WgBarriers<Cfg::kStages>);
  cudaError_t e = cudaFuncSetAttribute(wgrad_tn_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  const int grid = p.tiles < num_sms() ? p.tiles : num_sms();
  wgrad_tn_kernel<BN><<<grid, WG_THREADS, smem, stream>>>(map_g, map_a, p);
  return cudaGetLastError();
}

}  // namespace dpk

extern "C" int dpk_wgrad_tn(const void* gs, const void* a, int K, int M, int N, void* out, int out_bf16, float beta,
                            uint32_t* status, cudaStream_t stream) {
  using namespace dpk;
  if (K <= 0 || M <= 0 || N <= 0 || (M % 8) != 0 || (N % 8) != 0) return cudaErrorInvalidValue;
  // Pick the tile width that wastes fewer SM-waves.
  const int sms = num_sms();
  auto waves = [&](int bn) {
    const long tiles = (long)((M + WG_BM - 1) / WG_BM) * ((N + bn - 1) / bn);
    const long w = (tiles + sms - 1) / sms;
    return (double)w * bn;  // time ~ waves * tile width
  };
  if (N > 128 && waves(256) <= waves(128)) return launch_wgrad<256>(gs, a, K, M, N, out, out_bf16, beta, status, stream);
  return launch_wgrad<128>(gs, a, K, M, N, out, out_bf16, beta, status, stream);
}
