"""Gradient synchronisation shared by the data-parallel optimisers.

The portable path flattens all gradients into a few large buckets and issues
one ``all_reduce`` per bucket (instead of one per parameter).  On GPUs with
peer access the :mod:`opacus_b200.parallel` engine replaces it by a kernel that
reduces, adds noise, updates and redistributes in one launch.
"""
from typing import List

import torch
import torch.distributed as dist

_BUCKET_BYTES = 256 << 20


def all_reduce_grads(tensors: List[torch.Tensor], *, average_by: int = 1, group=None) -> None:
    """In-place SUM all-reduce of ``tensors`` (then ``/ average_by``), bucketed
    by dtype/device so that launch count does not scale with parameter count."""
    buckets = {}
    for t in tensors:
        buckets.setdefault((t.dtype, t.device), []).append(t)
    for (_dtype, _dev), group_tensors in buckets.items():
        chunk, size = [], 0
        for t in group_tensors + [None]:
            if t is not None and (size == 0 or size + t.numel() * t.element_size() <= _BUCKET_BYTES):
                chunk.append(t)
                size += t.numel() * t.element_size()
                continue
            if chunk:
                flat = torch.cat([c.reshape(-1) for c in chunk]) if len(chunk) > 1 else chunk[0].reshape(-1)
                dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
                if average_by != 1:
                    flat /= average_by
                if len(chunk) > 1:
                    ofs = 0
                    for c in chunk:
                        c.copy_(flat[ofs: ofs + c.numel()].view_as(c))
                        ofs += c.numel()
                elif flat.data_ptr() != chunk[0].data_ptr():
                    chunk[0].copy_(flat.view_as(chunk[0]))
            chunk, size = ([t], t.numel() * t.element_size()) if t is not None else ([], 0)
