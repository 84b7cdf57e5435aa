// C[M, N] = A[M, K] B[N, K]^T on tcgen05 (bf16 in, fp32 accumulate in tensor memory, bf16 out),
// alone or fused with the collective that tensor / sharded parallelism puts next to it:
//
//   mode 0  plain GEMM
//   mode 1  all-gather(A rows) -> GEMM      sequence-sharded activations into a column-parallel layer
//   mode 2  all-gather(B rows) -> GEMM      row-sharded weights (ZeRO-3 / FSDP) into their first use
//   mode 3  GEMM -> reduce-scatter(C rows)  row-parallel layer producing sequence-sharded output
//
// Gather modes: warp 3 of every CTA is a copier.  Together the copiers pull the peers' shards over
// NVLink with untiled bulk copies (global -> shared -> global through a small ring, 8 KB pieces dealt
// round-robin to the CTAs) into a local buffer that holds the whole operand, unit by unit (a unit =
// the rows of one tile), own shard first, then the peers in ring order, and count every finished
// piece on its unit's ready counter.  The GEMM warps walk the tiles in the same unit order and wait
// (bounded) for a unit to be complete before their TMA touches it, so every byte crosses NVLink once,
// no SM is given up to copying, and the transfer of unit u+1.. overlaps the math on unit u.  The
// gathered operand stays in the local buffer for the per-sample-gradient kernels of the backward pass.
//
// Reduce-scatter mode: each tile's epilogue stores its bf16 partial straight into the row owner's
// slot buffer (peer stores; tiles of remote owners are computed first); after a grid barrier and a
// bounded meeting of the ranks, all CTAs add the `world` slots of the locally owned rows in rank
// order with fp32 accumulation.  Slots are double-buffered by call parity.
//
// Replaces NCCL all-gather / reduce-scatter followed or preceded by a cuBLAS GEMM (DTensor
// ColwiseParallel / RowwiseParallel in examples/tensor_parallelism_llama.py:104-152 and FSDP2's
// all-gather in opacus/utils/fsdp_utils.py:52-60).  No TMA load is multicast and no tensor map
// points at peer memory; peers are reached only by untiled bulk loads and plain stores.
//
// Modes 1-3 need all CTAs resident at once (they wait on one another): cooperative launch, one CTA
// per SM.  Every wait is bounded by a timer; a CTA that gives up records it and falls through.
#include "api.h"
#include "common.cuh"
#include "host_util.h"

namespace dpk {

constexpr int TG_BM = 128, TG_BN = 256, TG_BK = 64;
constexpr int TG_STAGES = 4;
constexpr int TG_ABYTES = TG_BM * TG_BK * 2;     // 16 KB
constexpr int TG_BBYTES = TG_BN * TG_BK * 2;     // 32 KB
constexpr int TG_STAGE_BYTES = TG_ABYTES + TG_BBYTES;
constexpr int TG_THREADS = 256;
constexpr uint32_t TG_IDESC = make_idesc(1, 0, 0, TG_BM, TG_BN);
// copier ring (after the stages in shared memory)
constexpr int TG_PIECE = 8 * 1024;
constexpr int TG_SLOTS = 4;
constexpr int TG_LOOKAHEAD = 2;
constexpr int TG_RING_BYTES = TG_SLOTS * TG_PIECE;
constexpr int TG_EPI_PITCH = 144;          // bytes per staged row: 64 bf16 + 16 bytes of padding (mode 3 epilogue)
static_assert(4 * 32 * TG_EPI_PITCH <= TG_RING_BYTES, "the mode-3 staging rows reuse the copier ring");
// flag words (per rank, symmetric)
constexpr int TG_F_START = 0, TG_F_DONE = 8, TG_F_GO = 16, TG_F_COUNT = 17, TG_F_GO2 = 18, TG_F_COUNT2 = 19;

struct __align__(8) TgBarriers {
  uint64_t full[TG_STAGES];
  uint64_t empty[TG_STAGES];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint64_t piece[TG_SLOTS];
  uint32_t tmem_base;
  uint32_t abort_flag;
};

struct TgTile {
  int m0, n0, unit, owner;
};

// Tile number `s` in this rank's processing order.  The "major" tile index is the one the collective
// works along (m, or n in mode 2); majors are taken in arrival order (gather: own shard first, then the
// peers in ring order; reduce-scatter: rows of remote owners first) and in groups of TG_GROUP, inside
// which the tiles that run at the same time form a compact block of C (both operands reused from L2).
constexpr int TG_GROUP = 8;

__device__ __forceinline__ TgTile tg_decode(const DpkTpGemm& p, int s, int mt, int nt) {
  TgTile t;
  const int nmaj = p.mode == 2 ? nt : mt, nmin = p.mode == 2 ? mt : nt;
  const int per_group = TG_GROUP * nmin;
  const int g = s / per_group;
  const int gfirst = g * TG_GROUP;
  const int gsize = min(TG_GROUP, nmaj - gfirst);
  const int in = s - g * per_group;
  const int useq = gfirst + in % gsize;
  const int minor = in / gsize;
  int major = useq;
  if (p.mode != 0) {
    const int upr = nmaj / p.world;
    int r = p.rank + (p.mode == 3 ? 1 : 0) + useq / upr;
    if (r >= p.world) r -= p.world;
    major = r * upr + useq % upr;
  }
  const int mi = p.mode == 2 ? minor : major, ni = p.mode == 2 ? major : minor;
  t.unit = major;
  t.m0 = mi * TG_BM;
  t.n0 = ni * TG_BN;
  t.owner = p.mode == 3 ? t.m0 / (p.M / p.world) : 0;
  return t;
}

// ------------------------------------------------------------------------------------------------ copier warp
// Run by warp 3 of every CTA in the gather modes.  Pieces are numbered in arrival order (unit by unit,
// own shard first); CTA c moves pieces c, c + grid, c + 2 grid, ...
__device__ void tg_copy_warp(const DpkTpGemm& p, uint8_t* ring, TgBarriers* bars) {
  volatile uint32_t* my_flags = p.flags[p.rank];
  const int lane = threadIdx.x & 31;
  // meeting #1 (CTA 0): every rank's shard is final before anybody pulls it
  if (blockIdx.x == 0) {
    bool ok = true;
    if (lane < p.world) {
      __threadfence_system();
      volatile uint32_t* theirs = p.flags[lane] + TG_F_START + p.rank;
      *theirs = p.epoch;
      ok = spin_until_epoch(my_flags + TG_F_START + lane, p.epoch, p.status, 41);
    }
    ok = __all_sync(0xffffffffu, ok);
    if (lane == 0) {
      __threadfence_system();
      my_flags[TG_F_GO] = ok ? p.epoch : (p.epoch | kAbortBit);
    }
  }
  if (lane == 0) {
    const int unit_rows = p.mode == 1 ? TG_BM : TG_BN;
    const int rows = p.mode == 1 ? p.M : p.N;
    const int units = rows / unit_rows;
    const int upr = units / p.world;
    const int64_t unit_bytes = (int64_t)unit_rows * p.K * 2;
    const int ppu = (int)(unit_bytes / TG_PIECE);                 // the launcher checked divisibility
    const int total = units * ppu;
    const int G = (int)gridDim.x;
    const int mine = total > (int)blockIdx.x ? (total - (int)blockIdx.x + G - 1) / G : 0;
    uint8_t* full = reinterpret_cast<uint8_t*>(const_cast<void*>(p.mode == 1 ? p.a : p.b));
    bool ok = true, went = false;
    // j-th piece of this CTA -> addresses and unit; returns whether it comes from a peer
    auto locate = [&](int j, const uint8_t*& src, uint8_t*& dst, int& unit) -> bool {
      const int i = (int)blockIdx.x + j * G;
      const int useq = i / ppu, k = i - useq * ppu;
      int r = p.rank + useq / upr;
      if (r >= p.world) r -= p.world;
      const int in_owner = useq % upr;
      unit = r * upr + in_owner;
      src = reinterpret_cast<const uint8_t*>(p.shard[r]) + (int64_t)in_owner * unit_bytes + (int64_t)k * TG_PIECE;
      dst = full + (int64_t)unit * unit_bytes + (int64_t)k * TG_PIECE;
      return r != p.rank;
    };
    auto issue_load = [&](int j) {
      const uint8_t* src; uint8_t* dst; int unit;
      const bool remote = locate(j, src, dst, unit);
      if (remote && !went) {               // first pull from a peer: meeting #1 must be over
        ok = spin_until_epoch(my_flags + TG_F_GO, p.epoch, p.status, 42);
        went = true;
      }
      if (!ok) return;
      const int slot = j % TG_SLOTS;
      mbar_expect_tx(&bars->piece[slot], TG_PIECE);
      bulk_load(ring + slot * TG_PIECE, src, TG_PIECE, &bars->piece[slot]);
    };
    auto signal = [&](int j) {             // piece j has been written completely
      const uint8_t* src; uint8_t* dst; int unit;
      locate(j, src, dst, unit);
      fence_proxy_async();
      __threadfence();
      atomicAdd(p.ready + unit, 1u);
    };
    int loaded = 0;
    for (; loaded < mine && loaded < TG_LOOKAHEAD && ok; ++loaded) issue_load(loaded);
    for (int j = 0; j < mine && ok; ++j) {
      const int slot = j % TG_SLOTS;
      if (!mbar_wait(&bars->piece[slot], (j / TG_SLOTS) & 1, &bars->abort_flag, p.status, 43)) { ok = false; break; }
      const uint8_t* src; uint8_t* dst; int unit;
      locate(j, src, dst, unit);
      bulk_store(dst, ring + slot * TG_PIECE, TG_PIECE);
      bulk_commit();
      // at most SLOTS - LOOKAHEAD groups pending: the slot that load (j + LOOKAHEAD) reuses is drained,
      // and piece j - (SLOTS - LOOKAHEAD) is completely written
      bulk_wait<TG_SLOTS - TG_LOOKAHEAD>();
      if (j >= TG_SLOTS - TG_LOOKAHEAD) signal(j - (TG_SLOTS - TG_LOOKAHEAD));
      if (loaded < mine) { issue_load(loaded); ++loaded; }
    }
    bulk_wait<0>();
    if (ok)
      for (int j = max(0, mine - (TG_SLOTS - TG_LOOKAHEAD)); j < mine; ++j) signal(j);
    if (!ok) {                             // let loads in flight land, then make the waiting tiles give up
      const uint64_t t0 = global_timer_ns();
      while (global_timer_ns() - t0 < 200000ull) {}
      for (int u = 0; u < units; ++u) atomicOr(p.ready + u, kAbortBit);
    }
  }
  __syncwarp();
  // meeting #2 (the last CTA to finish copying): nobody leaves while a peer may still be pulling its shard
  uint32_t last = 0;
  if (lane == 0) {
    __threadfence_system();
    const uint32_t old = atomicAdd(const_cast<uint32_t*>(my_flags + TG_F_COUNT), 1u);
    last = old == gridDim.x - 1 ? 1u : 0u;
    if (last) my_flags[TG_F_COUNT] = 0;
  }
  last = __shfl_sync(0xffffffffu, last, 0);
  if (last && lane < p.world) {
    __threadfence_system();
    volatile uint32_t* theirs = p.flags[lane] + TG_F_DONE + p.rank;
    *theirs = p.epoch;
    spin_until_epoch(my_flags + TG_F_DONE + lane, p.epoch, p.status, 44);
  }
}

// ------------------------------------------------------------------------------------------------ kernel
__global__ void __launch_bounds__(TG_THREADS, 1)
tp_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, DpkTpGemm p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* ring = smem + TG_STAGES * TG_STAGE_BYTES;
  auto* bars = reinterpret_cast<TgBarriers*>(ring + TG_RING_BYTES);
  volatile uint32_t* abort_flag = &bars->abort_flag;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const bool gather = p.mode == 1 || p.mode == 2;

  if (threadIdx.x == 0) {
    for (int s = 0; s < TG_STAGES; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&bars->acc_full[a], 1);
      mbar_init(&bars->acc_empty[a], 4);
    }
    for (int s = 0; s < TG_SLOTS; ++s) mbar_init(&bars->piece[s], 1);
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

  const int mt = (p.M + TG_BM - 1) / TG_BM, nt = (p.N + TG_BN - 1) / TG_BN;
  const int tiles = mt * nt;
  const int kblocks = (p.K + TG_BK - 1) / TG_BK;
  const int first = (int)blockIdx.x, stride = (int)gridDim.x;
  // pieces per unit of the gathered operand: a unit is complete when its counter reaches epoch * ppu
  const uint32_t ppu = gather ? (uint32_t)(((int64_t)(p.mode == 1 ? TG_BM : TG_BN) * p.K * 2) / TG_PIECE) : 0u;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      tma_prefetch_desc(&map_a);
      tma_prefetch_desc(&map_b);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int s = first; s < tiles && ok; s += stride) {
        const TgTile t = tg_decode(p, s, mt, nt);
        if (gather) {                      // the unit must have arrived in the local buffer
          if (!spin_until_epoch(p.ready + t.unit, p.epoch * ppu, p.status, 45)) { ok = false; *abort_flag = 1; break; }
          fence_proxy_async();
        }
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(&bars->empty[stage], phase ^ 1, abort_flag, p.status, 46)) { ok = false; break; }
          uint8_t* dst = smem + stage * TG_STAGE_BYTES;
          mbar_expect_tx(&bars->full[stage], TG_STAGE_BYTES);
          tma_load_2d(dst, &map_a, &bars->full[stage], kb * TG_BK, t.m0);
          tma_load_2d(dst + TG_ABYTES, &map_b, &bars->full[stage], kb * TG_BK, t.n0);
          if (++stage == TG_STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
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
      for (int s = first; s < tiles && ok; s += stride, ++local) {
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        if (!mbar_wait(&bars->acc_empty[acc], acc_phase ^ 1, abort_flag, p.status, 47)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d0 = tmem_base + acc * TG_BN;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(&bars->full[stage], phase, abort_flag, p.status, 48)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + stage * TG_STAGE_BYTES);
          const uint32_t b_addr = a_addr + TG_ABYTES;
#pragma unroll
          for (int k = 0; k < TG_BK / 16; ++k) {
            const uint64_t da = smem_desc_sw128(a_addr + k * 32, 16, 1024);
            const uint64_t db = smem_desc_sw128(b_addr + k * 32, 16, 1024);
            umma_f16(d0, da, db, TG_IDESC, (kb != 0 || k != 0) ? 1u : 0u);
          }
          umma_commit(&bars->empty[stage]);
          if (++stage == TG_STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(&bars->acc_full[acc]);
      }
    }
  } else if (warp == 3) {
    if (gather) tg_copy_warp(p, ring, bars);
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ epilogue
    const int ew = warp - 4;
    const int rpr = p.M / p.world;                                  // rows per rank (mode 3)
    const int64_t slot_elems = (int64_t)rpr * p.N;
    int local = 0;
    for (int s = first; s < tiles; s += stride, ++local) {
      const TgTile t = tg_decode(p, s, mt, nt);
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      if (!mbar_wait(&bars->acc_full[acc], acc_phase, abort_flag, p.status, 49)) break;
      tc_fence_after();
      const int row = t.m0 + ew * 32 + lane;
      const uint32_t taddr = tmem_base + acc * TG_BN + (static_cast<uint32_t>(ew * 32) << 16);
      __nv_bfloat16* orow;
      if (p.mode == 3)
        orow = reinterpret_cast<__nv_bfloat16*>(p.slots[t.owner]) +
               ((int64_t)(p.epoch & 1u) * p.world + p.rank) * slot_elems + (int64_t)(row - t.owner * rpr) * p.N;
      else
        orow = reinterpret_cast<__nv_bfloat16*>(p.out) + (int64_t)row * p.N;
      if (p.mode == 3) {
        // Through shared memory, then one bulk store of a 128-byte row segment per lane: NVLink carries
        // full packets instead of 16-byte fragments.  Row pitch 144 bytes keeps the writes at 4-way conflicts.
        uint8_t* stage = ring + ew * (32 * TG_EPI_PITCH);
#pragma unroll 1
        for (int c0 = 0; c0 < TG_BN; c0 += 64) {
          const int col = t.n0 + c0;
          if (col >= p.N) break;
          bulk_wait_read<0>();               // the previous pass has been read out of the staging rows
          __syncwarp();
#pragma unroll
          for (int hlf = 0; hlf < 2; ++hlf) {
            uint32_t r[32];
            tmem_ld_32x32(taddr + c0 + hlf * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              uint4 pk;
              uint32_t* pw = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                __nv_bfloat162 nv = __floats2bfloat162_rn(__uint_as_float(r[j + 2 * q]), __uint_as_float(r[j + 2 * q + 1]));
                pw[q] = *reinterpret_cast<uint32_t*>(&nv);
              }
              *reinterpret_cast<uint4*>(stage + lane * TG_EPI_PITCH + (hlf * 32 + j) * 2) = pk;
            }
          }
          fence_proxy_async();
          __syncwarp();
          const int ncols = min(64, p.N - col);
          if (row < p.M) bulk_store(orow + col, stage + lane * TG_EPI_PITCH, (uint32_t)ncols * 2);
          bulk_commit();
        }
        bulk_wait_read<0>();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->acc_empty[acc]);
        continue;
      }
#pragma unroll 1
      for (int c0 = 0; c0 < TG_BN; c0 += 32) {
        const int col = t.n0 + c0;
        if (col >= p.N) break;
        uint32_t r[32];
        tmem_ld_32x32(taddr + c0, r);
        tmem_ld_wait();
        if (row < p.M) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            if (col + j < p.N) {
              uint4 pk;
              uint32_t* pw = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                __nv_bfloat162 nv = __floats2bfloat162_rn(__uint_as_float(r[j + 2 * q]), __uint_as_float(r[j + 2 * q + 1]));
                pw[q] = *reinterpret_cast<uint32_t*>(&nv);
              }
              *reinterpret_cast<uint4*>(orow + col + j) = pk;
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->acc_empty[acc]);
    }
  }

  if (p.mode == 3 && warp >= 4) bulk_wait<0>();      // this thread's row segments have been written
  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
  if (p.mode != 3) return;

  // ------------------------------------------------------------------ reduce-scatter: meet, then add the slots
  volatile uint32_t* my_flags = p.flags[p.rank];
  __shared__ uint32_t sh_last, sh_ok;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t old = atomicAdd(const_cast<uint32_t*>(my_flags + TG_F_COUNT2), 1u);
    sh_last = old == gridDim.x - 1 ? 1u : 0u;
    if (sh_last) my_flags[TG_F_COUNT2] = 0;
    sh_ok = 1;
  }
  __syncthreads();
  if (sh_last) {
    if (threadIdx.x < p.world) {
      __threadfence_system();
      volatile uint32_t* theirs = p.flags[threadIdx.x] + TG_F_DONE + p.rank;
      *theirs = p.epoch;
      if (!spin_until_epoch(my_flags + TG_F_DONE + threadIdx.x, p.epoch, p.status, 50)) sh_ok = 0;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence_system();
      my_flags[TG_F_GO2] = (sh_ok && !*abort_flag) ? p.epoch : (p.epoch | kAbortBit);
    }
  }
  if (threadIdx.x == 0) sh_ok = spin_until_epoch(my_flags + TG_F_GO2, p.epoch, p.status, 51) ? 1u : 0u;
  __syncthreads();
  if (!sh_ok) return;
  __threadfence_system();
  {
    const int rpr = p.M / p.world;
    const int64_t slot_elems = (int64_t)rpr * p.N;
    const __nv_bfloat16* base = reinterpret_cast<const __nv_bfloat16*>(p.slots[p.rank]) +
                                (int64_t)(p.epoch & 1u) * p.world * slot_elems;
    __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.out);
    const int64_t nvec = slot_elems >> 3;
    for (int64_t v = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; v < nvec; v += (int64_t)gridDim.x * blockDim.x) {
      float acc8[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int r = 0; r < p.world; ++r) {
        const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(base + (int64_t)r * slot_elems + (v << 3)));
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162*>(&w[q]);
          acc8[2 * q] += __bfloat162float(h.x);
          acc8[2 * q + 1] += __bfloat162float(h.y);
        }
      }
      uint4 pk;
      uint32_t* pw = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        __nv_bfloat162 nv = __floats2bfloat162_rn(acc8[2 * q], acc8[2 * q + 1]);
        pw[q] = *reinterpret_cast<uint32_t*>(&nv);
      }
      *reinterpret_cast<uint4*>(out + (v << 3)) = pk;
    }
  }
}

}  // namespace dpk

extern "C" int dpk_tp_gemm(const DpkTpGemm* ph, cudaStream_t stream) {
  using namespace dpk;
  DpkTpGemm p = *ph;
  if (p.M <= 0 || p.N <= 0 || p.K <= 0 || (p.K % 8) != 0 || (p.N % 8) != 0 || p.mode < 0 || p.mode > 3)
    return cudaErrorInvalidValue;
  if (p.world < 1 || p.world > 8 || p.rank < 0 || p.rank >= p.world) return cudaErrorInvalidValue;
  const int sms = num_sms();
  if (p.mode == 1 || p.mode == 2) {
    const int unit_rows = p.mode == 1 ? TG_BM : TG_BN;
    const int rows = p.mode == 1 ? p.M : p.N;
    if (rows % (unit_rows * p.world) != 0) return cudaErrorInvalidValue;
    if (((int64_t)unit_rows * p.K * 2) % TG_PIECE != 0) return cudaErrorInvalidValue;   // K % 32 (A) / K % 16 (B)
    if (p.ready == nullptr) return cudaErrorInvalidValue;
  }
  if (p.mode == 3 && p.M % (TG_BM * p.world) != 0) return cudaErrorInvalidValue;
  CUtensorMap map_a, map_b;
  int rc = make_tmap_2d_bf16(&map_a, p.a, p.K, p.M, TG_BK, TG_BM);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&map_b, p.b, p.K, p.N, TG_BK, TG_BN);
  if (rc) return rc;
  const size_t smem = 1024 + TG_STAGES * TG_STAGE_BYTES + TG_RING_BYTES + sizeof(TgBarriers);
  static_assert(1024 + TG_STAGES * TG_STAGE_BYTES + TG_RING_BYTES + sizeof(TgBarriers) <= 227 * 1024, "shared memory");
  cudaError_t e = cudaSuccess;
  {
    static bool attr_done[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !attr_done[dev]) {
      e = cudaFuncSetAttribute(tp_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return e;
      if (dev >= 0 && dev < 64) attr_done[dev] = true;
    }
  }
  const int tiles = ((p.M + TG_BM - 1) / TG_BM) * ((p.N + TG_BN - 1) / TG_BN);
  if (p.mode == 0) {
    const int grid = tiles < sms ? tiles : sms;
    tp_gemm_kernel<<<grid, TG_THREADS, smem, stream>>>(map_a, map_b, p);
    return cudaGetLastError();
  }
  // CTAs wait on one another: all of them must be resident
  int per_sm = 0;
  e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, tp_gemm_kernel, TG_THREADS, smem);
  if (e != cudaSuccess) return e;
  if (per_sm < 1) return cudaErrorLaunchOutOfResources;
  void* args[] = {(void*)&map_a, (void*)&map_b, (void*)&p};
  return cudaLaunchCooperativeKernel((void*)tp_gemm_kernel, dim3(sms), dim3(TG_THREADS), args, smem, stream);
}
