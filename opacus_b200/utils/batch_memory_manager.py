"""Virtual batches: split each logical (privacy-relevant) batch into physical
chunks that fit in memory, and tell the optimizer which ``step()`` calls only
accumulate.

Behavioural parity: ``opacus/utils/batch_memory_manager.py:27-183``.
"""
import math
from typing import List

import numpy as np
from torch.utils.data import BatchSampler, DataLoader, Sampler

from .uniform_sampler import DistributedUniformWithReplacementSampler, UniformWithReplacementSampler


class BatchSplittingSampler(Sampler[List[int]]):
    """Wraps a batch sampler.  For a logical batch of ``n`` indices yields
    ``ceil(n / max_batch_size)`` nearly equal chunks and queues
    ``signal_skip_step(True)`` for all but the last (``False`` for the last, and
    for an empty logical batch, which still counts as a step)."""

    def __init__(self, *, sampler: Sampler[List[int]], max_batch_size: int, optimizer):
        self.sampler = sampler
        self.max_batch_size = max_batch_size
        self.optimizer = optimizer

    def __iter__(self):
        for logical in self.sampler:
            n = len(logical)
            if n == 0:
                self.optimizer.signal_skip_step(do_skip=False)
                yield []
                continue
            chunks = np.array_split(np.asarray(logical), math.ceil(n / self.max_batch_size))
            for k, chunk in enumerate(chunks):
                self.optimizer.signal_skip_step(do_skip=k < len(chunks) - 1)
                yield chunk.tolist()

    def __len__(self):
        if isinstance(self.sampler, BatchSampler):
            per_batch = self.sampler.batch_size
        elif isinstance(self.sampler, (UniformWithReplacementSampler, DistributedUniformWithReplacementSampler)):
            per_batch = self.sampler.sample_rate * self.sampler.num_samples
        else:
            return len(self.sampler)
        return math.ceil(len(self.sampler) * (per_batch / self.max_batch_size))


def wrap_data_loader(*, data_loader: DataLoader, max_batch_size: int, optimizer):
    from ..data_loader import _carry

    return DataLoader(
        dataset=data_loader.dataset,
        batch_sampler=BatchSplittingSampler(
            sampler=data_loader.batch_sampler, max_batch_size=max_batch_size, optimizer=optimizer),
        collate_fn=data_loader.collate_fn,
        generator=data_loader.generator,
        **_carry(data_loader),
    )


class BatchMemoryManager:
    """``with BatchMemoryManager(data_loader=dl, max_physical_batch_size=k, optimizer=opt) as dl2:``
    iterate ``dl2`` and call ``opt.step()``/``opt.zero_grad()`` after every
    physical batch; parameters change only at logical batch boundaries."""

    def __init__(self, *, data_loader: DataLoader, max_physical_batch_size: int, optimizer):
        self.data_loader = data_loader
        self.optimizer = optimizer
        self.max_physical_batch_size = max_physical_batch_size

    def __enter__(self):
        return wrap_data_loader(data_loader=self.data_loader, max_batch_size=self.max_physical_batch_size,
                                optimizer=self.optimizer)

    def __exit__(self, exc_type, exc, tb):
        return None
