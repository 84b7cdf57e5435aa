"""Poisson batch samplers: every example joins a batch independently with
probability ``sample_rate``, so batch sizes vary (and can be zero).

Behavioural parity: ``opacus/utils/uniform_sampler.py:22-175``.
"""
from typing import Iterator, List, Optional

import torch
from torch.utils.data import Sampler


def _bernoulli_indices(n: int, rate: float, generator) -> torch.Tensor:
    """Indices ``i < n`` kept by independent coin flips of probability ``rate``.  ``generator``: a ``torch.Generator``
    (or None), or this package's ``SecureGenerator``, which draws its own uniforms."""
    if getattr(generator, "gaussian_like", None) is not None:
        return (generator.rand(n) < rate).nonzero(as_tuple=False).reshape(-1)
    return (torch.rand(n, generator=generator) < rate).nonzero(as_tuple=False).reshape(-1)


class UniformWithReplacementSampler(Sampler[List[int]]):
    """Yields ``steps`` (default ``int(1/sample_rate)``) Poisson batches of
    indices into a dataset of ``num_samples`` items."""

    def __init__(self, *, num_samples: int, sample_rate: float, generator=None, steps: Optional[int] = None):
        if num_samples <= 0:
            raise ValueError(f"num_samples should be a positive integer value, but got num_samples={num_samples}")
        self.num_samples = num_samples
        self.sample_rate = sample_rate
        self.generator = generator
        self.steps = int(1 / sample_rate) if steps is None else steps

    def __len__(self):
        return self.steps

    def __iter__(self) -> Iterator[List[int]]:
        for _ in range(self.steps):
            yield _bernoulli_indices(self.num_samples, self.sample_rate, self.generator).tolist()


class DistributedUniformWithReplacementSampler(Sampler):
    """Data-parallel Poisson sampling without communication.

    Every epoch all ranks build the same permutation (seed ``shuffle_seed +
    epoch``); rank ``r`` owns ``perm[r::world]`` and Poisson-samples inside its
    slice with its own generator.  The union over ranks is a Poisson sample of
    the whole dataset.  Empty local batches are skipped, so ranks may yield a
    different number of batches.
    """

    def __init__(self, *, total_size: int, sample_rate: float, shuffle: bool = True, shuffle_seed: int = 0,
                 steps: Optional[int] = None, generator=None, num_replicas: Optional[int] = None,
                 rank: Optional[int] = None):
        """``num_replicas`` / ``rank`` default to the whole job; a 2-d layout passes the number of data-parallel
        groups and this rank's group index (with one ``generator`` state per group), so that the ranks of a
        tensor-parallel group draw the same samples."""
        if total_size <= 0:
            raise ValueError(f"total_size should be a positive integer value, but got total_size={total_size}")
        self.total_size = total_size
        self.sample_rate = sample_rate
        self.generator = generator
        self.num_replicas = torch.distributed.get_world_size() if num_replicas is None else int(num_replicas)
        self.rank = torch.distributed.get_rank() if rank is None else int(rank)
        if not 0 <= self.rank < self.num_replicas:
            raise ValueError(f"rank {self.rank} outside [0, {self.num_replicas})")
        self.epoch = 0
        self.shuffle = shuffle
        self.shuffle_seed = shuffle_seed
        base, extra = divmod(total_size, self.num_replicas)
        self.num_samples = base + (1 if self.rank < extra else 0)
        self.num_batches = int(1 / sample_rate) if steps is None else steps

    def _local_slice(self) -> torch.Tensor:
        if self.shuffle:
            g = torch.Generator()
            g.manual_seed(self.shuffle_seed + self.epoch)
            order = torch.randperm(self.total_size, generator=g)
        else:
            order = torch.arange(self.total_size)
        mine = order[self.rank:: self.num_replicas]
        assert len(mine) == self.num_samples
        return mine

    def __iter__(self):
        mine = self._local_slice()
        for _ in range(self.num_batches):
            picked = _bernoulli_indices(self.num_samples, self.sample_rate, self.generator)
            if picked.numel():
                yield mine[picked]

    def __len__(self) -> int:
        return self.num_batches

    def set_epoch(self, epoch: int) -> None:
        """Changes the permutation (and therefore each rank's slice) of the next epoch."""
        self.epoch = epoch
