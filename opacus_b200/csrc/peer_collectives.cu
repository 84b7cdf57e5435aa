// Small collectives over NVLink peer memory, fused with the arithmetic that follows them.
//
// norm_allreduce_clip_kernel: the per-sample squared-norm all-reduce of tensor-parallel
// ghost clipping and the clip factor in ONE single-block kernel per rank.  Every rank
// stores its partial [B] vector into "its" slot of every rank's symmetric buffer (plain
// peer stores), raises a flag at every peer, waits (bounded) for the peers' flags, then
// adds the slots in rank order -- so all ranks obtain bit-identical norms and clip
// factors, which the privacy guarantee needs (every rank must scale sample b by the same
// factor).  Parameters that are replicated over the group enter once, unreduced.
//
// The reference does this with an NCCL all-reduce per step followed by three elementwise
// kernels (opacus/grad_sample/grad_sample_module_fast_gradient_clipping_tp.py:91-115,
// opacus/grad_sample/grad_sample_module_fast_gradient_clipping.py:137-150).
//
// Pull form (p.pull != 0): the partial sums are not copied anywhere.  The ghost-norm kernels of the backward pass
// accumulate straight into this rank's own slot of its own symmetric buffer (the epilogue of the Gram kernel adds
// into that address), and this kernel, after the flag meeting, reads every rank's slot from that rank's memory with
// plain peer loads.  The all-reduce is then nothing but the operand fetch of the clip-factor computation.
//
// Slots are double-buffered by the parity of the call number: a rank can run at most one
// call ahead of a peer (it cannot pass the wait of call e+1 before every peer has raised
// flag e+1, i.e. has finished reading the slots of call e).
#include "api.h"
#include "common.cuh"
#include "host_util.h"

namespace dpk {

__global__ void __launch_bounds__(256) norm_allreduce_clip_kernel(DpkNormAllReduce p) {
  __shared__ uint32_t sh_ok;
  const int64_t half = (int64_t)p.world * p.capacity;          // floats per parity
  const int64_t my_slot = (int64_t)(p.epoch & 1u) * half + (int64_t)p.rank * p.capacity;
  if (threadIdx.x == 0) sh_ok = 1;
  // 1. publish my partial sums at every rank (my own copy included); in pull form they already sit in my own slot
  if (!p.pull) {
    for (int r = 0; r < p.world; ++r) {
      float* dst = p.slots[r] + my_slot;
      for (int i = threadIdx.x; i < p.n; i += blockDim.x) dst[i] = p.sharded ? p.sharded[i] : 0.f;
    }
  }
  __threadfence_system();
  __syncthreads();
  // 2. tell every peer, then wait for every peer
  if (threadIdx.x < p.world) {
    volatile uint32_t* theirs = p.flags[threadIdx.x] + p.flag_base + p.rank;
    *theirs = p.epoch;
    if (!spin_until_epoch(p.flags[p.rank] + p.flag_base + threadIdx.x, p.epoch, p.status, 31)) sh_ok = 0;
  }
  __syncthreads();
  if (!sh_ok) {
    // a peer never arrived: the host learns it from the status word, but kernels already queued behind this
    // one read the outputs first -- they must see "no gradient passes" (NaN), not uninitialised memory
    const float nan = __int_as_float(0x7fc00000);
    for (int i = threadIdx.x; i < p.n; i += blockDim.x) {
      if (p.total_out) p.total_out[i] = nan;
      if (p.clip_out) p.clip_out[i] = nan;
    }
    return;
  }
  __threadfence_system();
  // 3. sum in rank order, add what is replicated, form the clip factor
  const volatile float* mine = p.slots[p.rank] + (int64_t)(p.epoch & 1u) * half;
  for (int i = threadIdx.x; i < p.n; i += blockDim.x) {
    float t = 0.f;
    if (p.pull) {
      for (int r = 0; r < p.world; ++r) {
        const volatile float* theirs = p.slots[r] + (int64_t)(p.epoch & 1u) * half + (int64_t)r * p.capacity;
        t += theirs[i];
      }
    } else {
      for (int r = 0; r < p.world; ++r) t += mine[(int64_t)r * p.capacity + i];
    }
    if (p.replicated) t += p.replicated[i];
    if (p.total_out) p.total_out[i] = t;
    if (p.clip_out) p.clip_out[i] = clip_factor_of(t, p.max_norm);
  }
}

}  // namespace dpk

extern "C" int dpk_norm_allreduce_clip(const DpkNormAllReduce* p, cudaStream_t stream) {
  if (p->world < 1 || p->world > 8 || p->rank < 0 || p->rank >= p->world || p->n < 0 || p->n > p->capacity)
    return cudaErrorInvalidValue;
  if (p->n == 0) return 0;
  dpk::norm_allreduce_clip_kernel<<<1, 256, 0, stream>>>(*p);
  return cudaGetLastError();
}
