"""Symmetric (peer-visible) device buffers over NVLink.

One process per GPU; every rank allocates the same sizes in the same order and
then holds, for each buffer, the addresses of all ranks' copies mapped into its
own address space.  Allocation and handle exchange use
``torch.distributed._symmetric_memory`` (CUDA virtual memory management plus a
rendezvous through the process group's store); nothing else of that module is
used -- every access to peer memory happens inside this package's own kernels:
plain loads and stores through the peers' addresses, or ``multimem`` loads and
stores through the address of the NVLink multicast object that the rendezvous
binds all copies to when the fabric supports it (NVLS; ``mc_ptr``, 0 otherwise).
``OPACUS_B200_MULTICAST=0`` makes every buffer report no multicast address, which
keeps all kernels on plain peer accesses (jobs that test what happens when a rank
leaves should run that way).
"""
from __future__ import annotations

import os
from typing import List, Optional

import torch
import torch.distributed as dist


class SymmetricBuffer:
    """``tensor`` is this rank's copy; ``ptrs[r]`` is rank ``r``'s copy as seen from this GPU; ``mc_ptr`` is the
    multicast address that reaches all copies at once (0: none)."""

    def __init__(self, tensor: torch.Tensor, ptrs: List[int], handle=None, mc_ptr: int = 0):
        self.tensor = tensor
        self.ptrs = ptrs
        self.handle = handle
        self.mc_ptr = mc_ptr


def world_info(group=None):
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(group), dist.get_world_size(group)
    return 0, 1


def alloc(numel: int, dtype: torch.dtype, device, group=None, zero: bool = True) -> SymmetricBuffer:
    rank, world = world_info(group)
    if world == 1:
        t = torch.zeros(numel, dtype=dtype, device=device) if zero else torch.empty(numel, dtype=dtype, device=device)
        return SymmetricBuffer(t, [t.data_ptr()])
    import torch.distributed._symmetric_memory as symm_mem

    t = symm_mem.empty(numel, dtype=dtype, device=device)
    handle = symm_mem.rendezvous(t, group if group is not None else dist.group.WORLD)
    if zero:
        t.zero_()
    ptrs = [int(p) for p in handle.buffer_ptrs]
    assert ptrs[rank] == t.data_ptr(), "symmetric buffer does not start at its allocation"
    mc = 0
    if os.environ.get("OPACUS_B200_MULTICAST", "1") != "0":
        try:
            mc = int(getattr(handle, "multicast_ptr", 0) or 0)
        except Exception:
            mc = 0
    return SymmetricBuffer(t, ptrs, handle, mc)


def available(group=None) -> Optional[str]:
    """``None`` if peer-visible buffers can be used by this job, else the reason."""
    rank, world = world_info(group)
    if world == 1:
        return None
    if not torch.cuda.is_available():
        return "no CUDA device"
    try:
        import importlib

        importlib.import_module("torch.distributed._symmetric_memory")
    except Exception as e:  # pragma: no cover
        return f"symmetric memory module unavailable: {e}"
    if dist.get_backend(group) != "nccl":
        return "process group backend is not nccl"
    return None


class PeerNormReducer:
    """All-reduce of a per-sample ``[B]`` fp32 vector over the group plus the clip
    factor, as one single-block kernel per rank over peer memory
    (``csrc/peer_collectives.cu``); every rank obtains the same bits.  ``capacity``
    is the longest vector the current buffers hold; a longer one makes every rank
    allocate larger buffers (all ranks of the group see the same batch, so they
    grow in the same call).  Construction, and growth, are collective (symmetric
    allocation)."""

    def __init__(self, device, group=None, capacity: int = 8192):
        self.group = group
        self.rank, self.world = world_info(group)
        self.capacity = int(capacity)
        self.device = torch.device(device)
        self._allocate()

    def _allocate(self):
        self._slots = alloc(2 * self.world * self.capacity, torch.float32, self.device, self.group)
        self._flags = alloc(64, torch.int32, self.device, self.group)
        self._epoch = 0
        if self.world > 1:
            dist.barrier(group=self.group)  # every rank's buffers are zeroed before anyone's first kernel

    def accumulator(self, n: int) -> Optional[torch.Tensor]:
        """A zeroed ``[n]`` fp32 vector inside this rank's symmetric buffer for the partial sums of the NEXT call:
        kernels that add their per-sample norms into it (the ghost-norm epilogues) leave nothing to copy -- the
        next call, given this very tensor as ``sharded``, reads every rank's vector from that rank's memory.
        None when ``n`` exceeds the capacity (the caller then uses an ordinary tensor; the call grows the buffers)."""
        if n > self.capacity:
            return None
        half = self.world * self.capacity
        start = ((self._epoch + 1) & 1) * half + self.rank * self.capacity
        acc = self._slots.tensor[start: start + n]
        acc.zero_()
        self._handed_out = (self._epoch + 1, acc.data_ptr(), n)
        return acc

    def __call__(self, sharded: Optional[torch.Tensor], replicated: Optional[torch.Tensor], max_norm: float):
        """-> ``(total, clip)`` with ``total = sum_ranks sharded + replicated``."""
        from ..ops import _cuda

        ref = sharded if sharded is not None else replicated
        n = ref.numel()
        if n > self.capacity:
            if n > (1 << 22):
                raise ValueError(f"a batch of {n} samples is beyond what the reducer supports")
            torch.cuda.synchronize(self.device)          # kernels of earlier calls are done with the old buffers
            while self.capacity < n:
                self.capacity *= 2
            self._allocate()
        self._epoch += 1
        handed = getattr(self, "_handed_out", None)
        pull = (sharded is not None and handed is not None
                and handed == (self._epoch, sharded.data_ptr(), sharded.numel()))
        self._handed_out = None
        if self.world > 1:
            # every rank must take the same form: a rank that pulls reads the peers' own slots
            pull = self._agree(pull)
        prep = lambda t: None if t is None else t.float().contiguous()
        total, clip = _cuda.load().norm_allreduce_clip(self._slots.ptrs, self._flags.ptrs,
                                                       None if pull else prep(sharded), prep(replicated),
                                                       n, self.capacity, self.rank, 0, self._epoch, float(max_norm),
                                                       self.device, pull)
        return total, clip

    def _agree(self, pull: bool) -> bool:
        """All ranks run the same program, so they normally agree by construction; the first call checks it once
        (a cheap all-reduce) and later calls trust it unless this rank's own answer changes."""
        known = getattr(self, "_pull_agreed", None)
        if known is not None and known[0] == pull:
            return known[1]
        flag = torch.tensor([1 if pull else 0], device=self.device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
        agreed = bool(flag.item())
        self._pull_agreed = (pull, agreed)
        return agreed
