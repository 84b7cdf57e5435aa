// Clipped weight gradient  out[M, N] = beta * out + Gs^T A  on a PAIR of SMs (tcgen05 cta_group::2):
// a cluster of two CTAs computes one 256 x 256 tile.  CTA r of the pair stages rows [128 r, 128 r + 128) of the M
// side (Gs) and columns [128 r, 128 r + 128) of the N side (A) -- each operand byte is fetched once per pair, so a
// CTA moves 32 KB per 64-deep k-block where the one-CTA 256 x 256 tile moves 64 KB -- and holds the 128 x 256 fp32
// accumulator of its rows in tensor memory.  That is half of an SM's 512 columns, so accumulators are double
// buffered: the epilogue of tile i (TMEM -> registers -> global, or vector atomics when K is split) overlaps the
// MMAs of tile i + 1, which the one-CTA 256 x 256 tile cannot do.
//
// Roles per CTA (256 threads): warp 0 = TMA producer (one elected thread), warp 1 = MMA issuer (leader CTA only),
// warp 2 = TMEM allocator, warps 4-7 = epilogue.  Synchronisation:
//   full[s]      (leader's copy is the one used): both CTAs' TMA loads complete their bytes on the LEADER's barrier
//                (cta_group::2 loads may signal the peer's barrier); the leader's producer announces 64 KB per stage;
//   empty[s]     both copies: tcgen05.commit of the leader, delivered to both CTAs, frees the stage in both;
//   acc_full[a]  both copies: the same commit mechanism tells both epilogues that an accumulator is complete;
//   acc_empty[a] leader's copy: 4 local + 4 remote epilogue warps arrive.
// No TMA load uses multicast.  Every wait is bounded (common.cuh); both CTAs meet at a cluster barrier before the
// first remote signal and before they exit, whichever way they leave their loops.
//
// Same operand layout as wgrad.cu (both operands MN-major straight from row-major [K, M] / [K, N]); the reference
// computes this product with a second backward pass (opacus/utils/fast_gradient_clipping_utils.py:194-201).
#include "api.h"
#include "common.cuh"
#include "host_util.h"

namespace dpk {

constexpr int W2_BK = 64;                    // contraction rows per stage
constexpr int W2_BOX = 64;                   // columns per TMA box = 128 bytes
constexpr int W2_BOX_BYTES = W2_BK * 128;    // 8 KB
constexpr int W2_THREADS = 256;
constexpr int W2_TILE = 256;                 // pair tile is 256 x 256
constexpr int W2_HALF = 128;                 // rows (and operand columns) per CTA
constexpr int W2_STAGE_BYTES = 4 * W2_BOX_BYTES;   // 2 boxes of Gs + 2 boxes of A = 32 KB per CTA
constexpr int W2_STAGES = 6;
constexpr int W2_GROUP_M = 8;
constexpr uint32_t W2_IDESC = make_idesc(1, 1, 1, W2_TILE, W2_TILE);   // bf16, both MN-major, M = N = 256 per pair

struct W2Params {
  int K, M, N;
  int mt, nt, splits, kblocks, items;
  float* out;
  int atomic_out;
  float beta;
  uint32_t* status;
};

struct __align__(8) W2Barriers {
  uint64_t full[W2_STAGES];
  uint64_t empty[W2_STAGES];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  uint32_t abort_flag;
};

// ---- cluster / cta_group::2 primitives
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `local` (an address in this CTA's shared memory) inside CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local, uint32_t rank) {
  uint32_t a;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(local), "r"(rank));
  return a;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Tiled load whose completion bytes are counted on a barrier that may live in the peer CTA of the pair.
__device__ __forceinline__ void tma_load_3d_pair(void* smem_dst, const CUtensorMap* map, uint32_t bar_cluster_addr,
                                                 int32_t x, int32_t y, int32_t z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// D[tmem of both CTAs] (+)= A[smem of both CTAs] * B[smem of both CTAs]; issued by ONE thread of the leader CTA.
__device__ __forceinline__ void umma2_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// All MMAs issued so far by this thread arrive, when complete, on the barrier at this offset in BOTH CTAs.
__device__ __forceinline__ void umma2_commit_both(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"(mask)
               : "memory");
}

struct W2Item {
  int m0, n0, kb0, kb1;
};

__device__ __forceinline__ W2Item w2_decode(const W2Params& p, int item) {
  W2Item w;
  const int tiles = p.mt * p.nt;
  const int split = item / tiles;
  const int tile = item - split * tiles;
  const int per_group = W2_GROUP_M * p.nt;
  const int group = tile / per_group;
  const int first_m = group * W2_GROUP_M;
  const int gsize = min(p.mt - first_m, W2_GROUP_M);
  const int in_group = tile - group * per_group;
  w.m0 = (first_m + in_group % gsize) * W2_TILE;
  w.n0 = (in_group / gsize) * W2_TILE;
  const int per_split = (p.kblocks + p.splits - 1) / p.splits;
  w.kb0 = split * per_split;
  w.kb1 = min(p.kblocks, w.kb0 + per_split);
  return w;
}

__global__ void __launch_bounds__(W2_THREADS, 1)
wgrad2_tn_kernel(const __grid_constant__ CUtensorMap map_g, const __grid_constant__ CUtensorMap map_a, W2Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  auto* bars = reinterpret_cast<W2Barriers*>(smem + W2_STAGES * W2_STAGE_BYTES);
  volatile uint32_t* abort_flag = &bars->abort_flag;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();          // 0 = leader of the pair
  const int pair = blockIdx.x >> 1;
  const int pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < W2_STAGES; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&bars->acc_full[a], 1);
      mbar_init(&bars->acc_empty[a], 8);           // 4 epilogue warps of each CTA (used in the leader only)
    }
    bars->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 2) {
    tmem_alloc2(&bars->tmem_base, 512);
    tmem_relinquish2();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                              // the peer's barriers exist before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (elect_one()) {
      tma_prefetch_desc(&map_g);
      tma_prefetch_desc(&map_a);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int item = pair; item < p.items && ok; item += pairs) {
        const W2Item w = w2_decode(p, item);
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          if (!mbar_wait(&bars->empty[stage], phase ^ 1, abort_flag, p.status, 61)) { ok = false; break; }
          uint8_t* dst = smem + stage * W2_STAGE_BYTES;
          // bytes of BOTH CTAs' loads are counted on the leader's barrier of this stage
          const uint32_t full_leader = map_to_cta(smem_u32(&bars->full[stage]), 0);
          if (cta == 0) mbar_expect_tx(&bars->full[stage], 2 * W2_STAGE_BYTES);
          const int mcol = w.m0 + (int)cta * W2_HALF;
          const int ncol = w.n0 + (int)cta * W2_HALF;
#pragma unroll
          for (int j = 0; j < 2; ++j)
            tma_load_3d_pair(dst + j * W2_BOX_BYTES, &map_g, full_leader, mcol + j * W2_BOX, kb * W2_BK, 0);
#pragma unroll
          for (int j = 0; j < 2; ++j)
            tma_load_3d_pair(dst + (2 + j) * W2_BOX_BYTES, &map_a, full_leader, ncol + j * W2_BOX, kb * W2_BK, 0);
          if (++stage == W2_STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {  // let loads that are still in flight land before the CTA exits
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 200000ull) {}
      }
    }
  } else if (warp == 1 && cta == 0) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA)
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      for (int item = pair; item < p.items && ok; item += pairs, ++local) {
        const W2Item w = w2_decode(p, item);
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        if (!mbar_wait(&bars->acc_empty[acc], acc_phase ^ 1, abort_flag, p.status, 62)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d0 = tmem_base + acc * W2_TILE;
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          if (!mbar_wait(&bars->full[stage], phase, abort_flag, p.status, 63)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + stage * W2_STAGE_BYTES);
          const uint32_t b_addr = a_addr + 2 * W2_BOX_BYTES;
#pragma unroll
          for (int k = 0; k < W2_BK / 16; ++k) {
            // 16 contraction rows = 2048 bytes further into every 64-column box; the same offsets hold in the peer
            const uint64_t da = smem_desc_sw128(a_addr + k * 2048, W2_BOX_BYTES, 1024);
            const uint64_t db = smem_desc_sw128(b_addr + k * 2048, W2_BOX_BYTES, 1024);
            umma2_f16(d0, da, db, W2_IDESC, (kb != w.kb0 || k != 0) ? 1u : 0u);
          }
          umma2_commit_both(&bars->empty[stage]);
          if (++stage == W2_STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) umma2_commit_both(&bars->acc_full[acc]);
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ epilogue (both CTAs, own 128 rows)
    const int ew = warp - 4;
    const uint32_t acc_empty_leader[2] = {map_to_cta(smem_u32(&bars->acc_empty[0]), 0),
                                          map_to_cta(smem_u32(&bars->acc_empty[1]), 0)};
    int local = 0;
    for (int item = pair; item < p.items; item += pairs, ++local) {
      const W2Item w = w2_decode(p, item);
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      if (!mbar_wait(&bars->acc_full[acc], acc_phase, abort_flag, p.status, 64)) break;
      tc_fence_after();
      const int row = w.m0 + (int)cta * W2_HALF + ew * 32 + lane;
      const uint32_t taddr = tmem_base + acc * W2_TILE + (static_cast<uint32_t>(ew * 32) << 16);
#pragma unroll 1
      for (int c0 = 0; c0 < W2_TILE; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c0, r);
        tmem_ld_wait();
        const int col = w.n0 + c0;
        if (row < p.M && col < p.N) {
          float* o = p.out + (int64_t)row * p.N + col;
          if (p.atomic_out) {
#pragma unroll
            for (int j = 0; j < 32; j += 4)
              if (col + j < p.N)
                asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(o + j), "f"(__uint_as_float(r[j])),
                             "f"(__uint_as_float(r[j + 1])), "f"(__uint_as_float(r[j + 2])),
                             "f"(__uint_as_float(r[j + 3]))
                             : "memory");
          } else {
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
      if (lane == 0) mbar_arrive_cluster(acc_empty_leader[acc]);
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                              // neither CTA leaves while the other may still signal it
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc2(tmem_base, 512);
  }
}

}  // namespace dpk

// out [M, N] fp32 = beta * out + gs^T a with gs [K, M], a [K, N] bf16 row-major; beta in {0, 1} when splits > 1.
// M, N multiples of 8.  Returns cudaErrorNotSupported where cluster launches are not available.
extern "C" int dpk_wgrad2_tn(const void* gs, const void* a, int K, int M, int N, float* out, float beta, int splits,
                             uint32_t* status, cudaStream_t stream) {
  using namespace dpk;
  if (K <= 0 || M <= 0 || N <= 0 || (M % 8) != 0 || (N % 8) != 0 || out == nullptr || splits < 1)
    return cudaErrorInvalidValue;
  if (splits > 1 && beta != 0.f && beta != 1.f) return cudaErrorInvalidValue;
  W2Params p{};
  p.K = K; p.M = M; p.N = N;
  p.mt = (M + W2_TILE - 1) / W2_TILE;
  p.nt = (N + W2_TILE - 1) / W2_TILE;
  p.kblocks = (K + W2_BK - 1) / W2_BK;
  p.splits = splits;
  p.items = p.mt * p.nt * splits;
  p.out = out; p.beta = beta; p.status = status;
  p.atomic_out = splits > 1 ? 1 : 0;
  CUtensorMap map_g, map_a;
  int rc = make_tmap_3d_bf16(&map_g, gs, M, K, 1, W2_BOX, W2_BK);
  if (rc) return rc;
  rc = make_tmap_3d_bf16(&map_a, a, N, K, 1, W2_BOX, W2_BK);
  if (rc) return rc;
  const size_t smem = 1024 + W2_STAGES * W2_STAGE_BYTES + sizeof(W2Barriers);
  cudaError_t e = cudaSuccess;
  {
    static bool attr_done[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !attr_done[dev]) {
      e = cudaFuncSetAttribute(wgrad2_tn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return e;
      if (dev >= 0 && dev < 64) attr_done[dev] = true;
    }
  }
  if (p.atomic_out && beta == 0.f) {
    e = cudaMemsetAsync(out, 0, sizeof(float) * (size_t)M * N, stream);
    if (e != cudaSuccess) return e;
  }
  const int max_pairs = num_sms() / 2;
  const int pairs = p.items < max_pairs ? p.items : max_pairs;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(2 * pairs);
  cfg.blockDim = dim3(W2_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  e = cudaLaunchKernelEx(&cfg, wgrad2_tn_kernel, map_g, map_a, p);
  return e;
}
