// Sharded data-parallel DP step in ONE kernel per rank, over NVLink peer memory:
//
//   reduce-scatter : every rank sums, for the slice of the flat gradient it owns,
//                    the clipped gradient sums of all ranks (plain peer loads)
//   noise          : the owner draws the single N(0, (sigma*C)^2) sample of each
//                    element (Philox counter = global element index, so no two
//                    ranks ever draw for the same element)
//   update         : scale, then SGD / Adam / AdamW on the fp32 master weights and
//                    optimiser state of the owned slice (never replicated)
//   all-gather     : the new weights are stored, in compute precision, straight
//                    into every rank's parameter buffer (plain peer stores)
//
// When the buffers are bound to an NVLink multicast object (NVLS), the reduce is ONE
// multimem.ld_reduce per 16 bytes -- the switch adds the eight copies and returns the sum,
// so a rank receives 1/world of the bytes the peer-load loop pulls and needs 1/world of
// the loads in flight -- and the publish is ONE multimem.st per 16 bytes, replicated by
// the switch, instead of world - 1 stores that each cross this GPU's link.
//
// A launch covers any 8-aligned range of the rank's share, so the host can step the flat
// space in pieces, each as soon as its gradients are final on every rank, beside the
// weight-gradient GEMMs that are still running; every launch is one flag epoch.
//
// Parameter groups with their own learning rate / weight decay are ranges of the flat
// space listed in a small device table (segment ends, ascending), searched per 8 elements.
//
// Ranks meet twice through flag words in symmetric memory: before the first peer
// access (everyone's gradients are final, nobody still reads the old weights) and
// after the last store (everyone's weights are complete when the kernel ends).
// Both waits are bounded; a rank that gives up records it and returns.
//
// Replaces, for the sharded (FSDP-style) path, two reduce-scatters, three
// all-gathers and the per-parameter noise/scale/step kernels of the reference
// (opacus/optimizers/fsdpoptimizer_fast_gradient_clipping.py:138-181 on top of
// torch FSDP2), and for plain data parallelism the per-parameter all-reduce of
// opacus/optimizers/ddpoptimizer.py:64-70.
#include "api.h"
#include "common.cuh"
#include "host_util.h"

namespace dpk {

constexpr int kSlotStart = 0;     // flags[kSlotStart + r]  : rank r reached the kernel (epoch)
constexpr int kSlotDone = 8;      // flags[kSlotDone + r]   : rank r finished its stores (epoch)
constexpr int kSlotGo = 16;       // local: block 0 -> other blocks
constexpr int kSlotCount = 17;    // local: finished-block counter
constexpr int kShThreads = 512;

// Sum over all ranks' copies of 4 consecutive floats, formed inside the NVSwitch.
__device__ __forceinline__ float4 multimem_ld_reduce_f32x4(const float* mc_addr) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(mc_addr)
               : "memory");
  return v;
}
// 16 bytes stored into every rank's copy (the payload is opaque bits; .f32 only names the vector shape).
__device__ __forceinline__ void multimem_st_b128(void* mc_addr, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "f"(__uint_as_float(v.x)),
               "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
               : "memory");
}

// WORLD > 0: the number of ranks is a compile-time constant and all peer loads of a vector are issued before the
// first one is used (one NVLink round trip per vector instead of one per rank); WORLD == 0: any number of ranks,
// one rank after the other.
// 8 bytes stored into every rank's copy.
__device__ __forceinline__ void multimem_st_b64(void* mc_addr, uint2 v) {
  asm volatile("multimem.st.relaxed.sys.global.v2.f32 [%0], {%1, %2};" ::"l"(mc_addr), "f"(__uint_as_float(v.x)),
               "f"(__uint_as_float(v.y))
               : "memory");
}

template <int WORLD>
__global__ void __launch_bounds__(kShThreads, WORLD == 1 ? 2 : 1) sharded_step_kernel(DpkShardedStep p) {
  __shared__ uint32_t sh_ok;
  volatile uint32_t* my_flags = p.flags[p.rank];

  // ---------------------------------------------------------------- meet #1
  if (blockIdx.x == 0) {
    if (threadIdx.x == 0) sh_ok = 1;
    __syncthreads();
    if (threadIdx.x < p.world) {
      __threadfence_system();
      volatile uint32_t* theirs = p.flags[threadIdx.x] + kSlotStart + p.rank;
      *theirs = p.epoch;
      if (!spin_until_epoch(my_flags + kSlotStart + threadIdx.x, p.epoch, p.status, 21)) sh_ok = 0;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence_system();
      my_flags[kSlotGo] = sh_ok ? p.epoch : (p.epoch | kAbortBit);
    }
  }
  if (threadIdx.x == 0) sh_ok = spin_until_epoch(my_flags + kSlotGo, p.epoch, p.status, 22) ? 1 : 0;
  __syncthreads();
  const bool go = sh_ok != 0;

  // ---------------------------------------------------------------- reduce, noise, update, publish
  // A thread owns 8 elements per iteration as two groups of 4.  When the range allows it (lengths multiples of
  // 256) the groups of a warp interleave -- lane l takes elements [4l, 4l + 4) and [128 + 4l, 128 + 4l + 4) of the
  // warp's 256 -- so that every load and store instruction of a warp covers one contiguous run of whole 32-byte
  // sectors: a peer read moves a sector over NVLink, and the 16-bytes-per-lane-at-a-32-byte-stride pattern of
  // "8 consecutive elements per thread" would fetch every remote sector twice.
  if (go) {
    __threadfence_system();          // the peers' gradient stores, published by their flags, before any read here
    DpkStepHyper h = p.h;
    const Philox rng(h.seed);
    const int64_t nvec = p.slice_len >> 3;
    // (with one rank everything is local and cached: consecutive elements per thread are slightly faster there)
    const bool wide = WORLD != 1 && ((p.slice_len | p.stripe_len) & 255) == 0;
    const bool has_m = p.state0 != nullptr && (h.kind != 0 || h.momentum != 0.f);
    for (int64_t v = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; v < nvec; v += (int64_t)gridDim.x * blockDim.x) {
      int64_t li[2], gi[2];            // index inside the owned share covered by this launch / in the flat space
      li[0] = wide ? ((v >> 5) << 8) + ((v & 31) << 2) : (v << 3);
      li[1] = li[0] + (wide ? 128 : 4);
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        gi[hf] = p.slice_begin + li[hf];
        if (p.stripe_len > 0)          // the share is one stripe of every piece: stripes are stripe_stride apart
          gi[hf] += (li[hf] / p.stripe_len) * (p.stripe_stride - p.stripe_len);
      }
      float4 g[2];
      if (p.grad_mc != nullptr) {
        g[0] = multimem_ld_reduce_f32x4(p.grad_mc + gi[0]);
        g[1] = multimem_ld_reduce_f32x4(p.grad_mc + gi[1]);
      } else if constexpr (WORLD > 0) {
        float4 a[WORLD], b[WORLD];
#pragma unroll
        for (int q = 0; q < WORLD; ++q) {         // rank order is fixed (0, 1, ...): the sum has the same bits on
          a[q] = __ldcg(reinterpret_cast<const float4*>(p.grad[q] + gi[0]));   // whichever rank owns the element
          b[q] = __ldcg(reinterpret_cast<const float4*>(p.grad[q] + gi[1]));
        }
        g[0] = a[0]; g[1] = b[0];
#pragma unroll
        for (int q = 1; q < WORLD; ++q) {
          g[0].x += a[q].x; g[0].y += a[q].y; g[0].z += a[q].z; g[0].w += a[q].w;
          g[1].x += b[q].x; g[1].y += b[q].y; g[1].z += b[q].z; g[1].w += b[q].w;
        }
      } else {
        g[0] = g[1] = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int q = 0; q < p.world; ++q) {
          const float4 a = __ldcg(reinterpret_cast<const float4*>(p.grad[q] + gi[0]));
          const float4 b = __ldcg(reinterpret_cast<const float4*>(p.grad[q] + gi[1]));
          g[0].x += a.x; g[0].y += a.y; g[0].z += a.z; g[0].w += a.w;
          g[1].x += b.x; g[1].y += b.y; g[1].z += b.z; g[1].w += b.w;
        }
      }
      float4 w[2], m[2], s[2];
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        w[hf] = *reinterpret_cast<const float4*>(p.master + li[hf]);
        if (has_m) m[hf] = *reinterpret_cast<const float4*>(p.state0 + li[hf]);
        if (h.kind != 0) s[hf] = *reinterpret_cast<const float4*>(p.state1 + li[hf]);
      }
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        if (p.nseg > 1) {
          // first segment whose end lies beyond the group (parameters start on multiples of 64: one segment per group)
          int lo = 0, hi = p.nseg - 1;
          while (lo < hi) {
            const int mid = (lo + hi) >> 1;
            if (__ldg(&p.segs[mid].end) > gi[hf]) hi = mid; else lo = mid + 1;
          }
          h.lr = __ldg(&p.segs[lo].lr);
          h.weight_decay = __ldg(&p.segs[lo].weight_decay);
        }
        float gv[4] = {g[hf].x, g[hf].y, g[hf].z, g[hf].w};
        float wv[4] = {w[hf].x, w[hf].y, w[hf].z, w[hf].w};
        float mv[4] = {0.f, 0.f, 0.f, 0.f}, sv[4] = {0.f, 0.f, 0.f, 0.f};
        if (has_m) { mv[0] = m[hf].x; mv[1] = m[hf].y; mv[2] = m[hf].z; mv[3] = m[hf].w; }
        if (h.kind != 0) { sv[0] = s[hf].x; sv[1] = s[hf].y; sv[2] = s[hf].z; sv[3] = s[hf].w; }
        if (h.noise_std != 0.f) {
          const uint64_t ni = static_cast<uint64_t>(gi[hf] >= p.noise_split ? gi[hf] + p.noise_shift : gi[hf]);
          const uint4 u = rng(ni >> 2, h.offset);          // one counter per 4 elements of the flat space
          const float2 z0 = box_muller(u.x, u.y), z1 = box_muller(u.z, u.w);
          gv[0] += z0.x * h.noise_std; gv[1] += z0.y * h.noise_std;
          gv[2] += z1.x * h.noise_std; gv[3] += z1.y * h.noise_std;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float grad = gv[j] * h.inv_scale;
          float pv = wv[j];
          if (h.kind == 0) {
            if (h.weight_decay != 0.f) grad = fmaf(h.weight_decay, pv, grad);
            if (h.momentum != 0.f) {
              const float buf = h.first_step ? grad : fmaf(h.momentum, mv[j], (1.f - h.dampening) * grad);
              mv[j] = buf;
              grad = h.nesterov ? fmaf(h.momentum, buf, grad) : buf;
            }
            pv = fmaf(-h.lr, grad, pv);
          } else {
            if (h.weight_decay != 0.f) {
              if (h.kind == 2) pv *= (1.f - h.lr * h.weight_decay);
              else grad = fmaf(h.weight_decay, pv, grad);
            }
            mv[j] = fmaf(h.beta1, mv[j], (1.f - h.beta1) * grad);
            sv[j] = fmaf(h.beta2, sv[j], (1.f - h.beta2) * grad * grad);
            pv -= (h.lr / h.bias_c1) * (mv[j] / (sqrtf(sv[j]) / h.bias_c2_sqrt + h.eps));
          }
          wv[j] = pv;
        }
        *reinterpret_cast<float4*>(p.master + li[hf]) = make_float4(wv[0], wv[1], wv[2], wv[3]);
        if (has_m) *reinterpret_cast<float4*>(p.state0 + li[hf]) = make_float4(mv[0], mv[1], mv[2], mv[3]);
        if (h.kind != 0) *reinterpret_cast<float4*>(p.state1 + li[hf]) = make_float4(sv[0], sv[1], sv[2], sv[3]);
        if (p.param_bf16) {
          const __nv_bfloat162 h0 = __floats2bfloat162_rn(wv[0], wv[1]), h1 = __floats2bfloat162_rn(wv[2], wv[3]);
          const uint2 pk = make_uint2(*reinterpret_cast<const uint32_t*>(&h0), *reinterpret_cast<const uint32_t*>(&h1));
          if (p.param_mc != nullptr) {
            multimem_st_b64(reinterpret_cast<__nv_bfloat16*>(p.param_mc) + gi[hf], pk);
          } else {
#pragma unroll 1
            for (int q = 0; q < p.world; ++q) {
              int r = p.rank + q;
              if (r >= p.world) r -= p.world;
              *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p.param[r]) + gi[hf]) = pk;
            }
          }
        } else {
          const uint4 pk = make_uint4(__float_as_uint(wv[0]), __float_as_uint(wv[1]), __float_as_uint(wv[2]),
                                      __float_as_uint(wv[3]));
          if (p.param_mc != nullptr) {
            multimem_st_b128(reinterpret_cast<float*>(p.param_mc) + gi[hf], pk);
          } else {
#pragma unroll 1
            for (int q = 0; q < p.world; ++q) {
              int r = p.rank + q;
              if (r >= p.world) r -= p.world;
              *reinterpret_cast<uint4*>(reinterpret_cast<float*>(p.param[r]) + gi[hf]) = pk;
            }
          }
        }
      }
    }
  }

  // ---------------------------------------------------------------- meet #2
  __threadfence_system();
  __syncthreads();
  __shared__ uint32_t sh_last;
  if (threadIdx.x == 0) {
    const uint32_t old = atomicAdd(const_cast<uint32_t*>(my_flags + kSlotCount), 1u);
    sh_last = (old == gridDim.x - 1) ? 1u : 0u;
    if (sh_last) my_flags[kSlotCount] = 0;
  }
  __syncthreads();
  if (sh_last && go && threadIdx.x < p.world) {
    __threadfence_system();
    volatile uint32_t* theirs = p.flags[threadIdx.x] + kSlotDone + p.rank;
    *theirs = p.epoch;
    spin_until_epoch(my_flags + kSlotDone + threadIdx.x, p.epoch, p.status, 23);
  }
}

}  // namespace dpk

extern "C" int dpk_sharded_dp_step(const DpkShardedStep* ph, cudaStream_t stream) {
  using namespace dpk;
  const DpkShardedStep& p = *ph;
  if (p.world < 1 || p.world > 8 || p.rank < 0 || p.rank >= p.world || (p.slice_len & 7) || (p.slice_begin & 7))
    return cudaErrorInvalidValue;
  if (p.nseg < 0 || (p.nseg > 1 && p.segs == nullptr)) return cudaErrorInvalidValue;
  if (p.slice_len == 0) return cudaErrorInvalidValue;
  if (p.stripe_len < 0 || (p.stripe_len & 7) || (p.stripe_stride & 7) || (p.stripe_len > 0 && p.stripe_stride < p.stripe_len))
    return cudaErrorInvalidValue;     // every launch is a meeting of all ranks: no empty ranges
  if ((reinterpret_cast<uintptr_t>(p.grad_mc) & 15) || (reinterpret_cast<uintptr_t>(p.param_mc) & 15))
    return cudaErrorInvalidValue;
  if (p.noise_split & 3 || p.noise_shift & 3) return cudaErrorInvalidValue;   // one Philox counter per 4 elements
  // every block spins on flags, so all of them must be resident at once: as many per SM as fit
  void (*kernel)(DpkShardedStep) = sharded_step_kernel<0>;
  int slot = 0;
  switch (p.world) {
    case 1: kernel = sharded_step_kernel<1>; slot = 1; break;
    case 2: kernel = sharded_step_kernel<2>; slot = 2; break;
    case 4: kernel = sharded_step_kernel<4>; slot = 3; break;
    case 8: kernel = sharded_step_kernel<8>; slot = 4; break;
    default: break;
  }
  static int per_sm_cached[5] = {0, 0, 0, 0, 0};
  if (per_sm_cached[slot] == 0) {
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, kShThreads, 0) != cudaSuccess || n < 1) n = 1;
    per_sm_cached[slot] = n > 4 ? 4 : n;
  }
  // A capped launch shares the GPU with compute-bound kernels (the weight-gradient GEMMs: one 256-thread CTA per
  // SM holding ~23 K registers): blocks of 256 threads keep this kernel's registers per block low enough for one
  // block to be resident on every SM beside a GEMM CTA, which 512-thread blocks are not.
  const int threads = p.max_blocks > 0 ? 256 : kShThreads;
  int grid = num_sms() * per_sm_cached[slot];
  if (p.max_blocks > 0 && p.max_blocks < grid) grid = p.max_blocks;   // a piece beside GEMMs leaves them the SMs
  const int64_t nvec = p.slice_len >> 3;
  const int64_t need = (nvec + threads - 1) / threads;
  if (need < grid) grid = need < 1 ? 1 : (int)need;
  kernel<<<grid, threads, 0, stream>>>(p);
  return cudaGetLastError();
}
