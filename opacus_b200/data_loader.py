"""``DPDataLoader``: a ``DataLoader`` whose batches are Poisson samples, with a
collate wrapper that can produce a well-formed *empty* batch.

Behavioural parity: ``opacus/data_loader.py:31-420``.
"""
import copy
import logging
from typing import Any, List, Mapping, Optional, Sequence, Tuple, Type, Union

import torch
from torch.utils.data import BatchSampler, DataLoader, Dataset, IterableDataset, RandomSampler, Sampler
from torch.utils.data._utils.collate import default_collate

from .utils.uniform_sampler import DistributedUniformWithReplacementSampler, UniformWithReplacementSampler

logger = logging.getLogger(__name__)

# DataLoader constructor arguments that are carried over when a loader is rebuilt.
_CARRIED = ("num_workers", "pin_memory", "timeout", "worker_init_fn", "multiprocessing_context",
            "prefetch_factor", "persistent_workers")


def _carry(loader: DataLoader) -> dict:
    return {k: getattr(loader, k) for k in _CARRIED}


class CollateFnWithEmpty:
    """Wraps a collate function.  Non-empty sample lists go through it and the
    structure of the first result is remembered; an empty list produces the
    same structure with batch length 0 (or 1 random row with ``rand_on_empty``)."""

    def __init__(self, collator_fn, batch_first: bool = True, rand_on_empty: bool = False,
                 sample_empty_shapes: Optional[Sequence[Tuple]] = None,
                 dtypes: Optional[Sequence[Union[torch.dtype, Type]]] = None) -> None:
        self.wrapped_collator_fn = collator_fn
        self.batch_first = batch_first
        self.rand_on_empty = rand_on_empty
        self.sample_empty_shapes = sample_empty_shapes
        self.dtypes = dtypes
        self.first_batch = None

    def __call__(self, batch: List[Any]):
        if len(batch) > 0:
            out = self.wrapped_collator_fn(batch) if self.wrapped_collator_fn else batch
            if self.first_batch is None:
                self.first_batch = copy.deepcopy(out)
            return out
        if self.first_batch is not None:
            return self._make_empty_batch(self.first_batch)
        # Nothing seen yet: fall back to what the dataset's first item told us.
        if self.sample_empty_shapes is not None and self.dtypes is not None:
            logger.warning(
                "First batch is empty. We are using a list of zero-valued tensors as a batch. This may cause "
                "issues if the model expects a different batch format. To fix, use more data, increase epsilon, "
                "or increase sampling rate."
            )
            return [torch.zeros(s, dtype=d) for s, d in zip(self.sample_empty_shapes, self.dtypes)]
        logger.warning(
            "First batch is empty. We are using an empty list as a batch. This may cause issues if the model "
            "expects a different batch format. To fix, use more data, increase epsilon, or increase sampling rate."
        )
        return []

    def _make_empty_batch(self, sample):
        if torch.is_tensor(sample):
            shape = list(sample.shape)
            shape[0 if self.batch_first else 1] = 1 if self.rand_on_empty else 0
            if self.rand_on_empty:
                return torch.randint(0, 2, shape, dtype=sample.dtype, device=sample.device)
            return torch.empty(shape, dtype=sample.dtype, device=sample.device)
        if isinstance(sample, Mapping):
            return {k: self._make_empty_batch(v) for k, v in sample.items()}
        if isinstance(sample, (list, tuple)):
            return type(sample)([self._make_empty_batch(v) for v in sample])
        raise TypeError(
            f"Unsupported batch type: {type(sample).__name__}. CollateFnWithEmpty only supports batches "
            "containing torch.Tensor, dict (Mapping), list, or tuple types."
        )


def wrap_collate_with_empty(*, collate_fn, batch_first: bool = True, rand_on_empty: bool = False,
                            sample_empty_shapes=None, dtypes=None) -> CollateFnWithEmpty:
    return CollateFnWithEmpty(collate_fn, batch_first=batch_first, rand_on_empty=rand_on_empty,
                              sample_empty_shapes=sample_empty_shapes, dtypes=dtypes)


def shape_safe(x: Any) -> Tuple:
    return getattr(x, "shape", ())


def dtype_safe(x: Any):
    return getattr(x, "dtype", type(x))


class DPDataLoader(DataLoader):
    """``DataLoader`` with Poisson batch sampling at ``sample_rate``.

    ``distributed=True`` uses the rank-sliced sampler (needs an initialised
    process group).  ``drop_last`` is ignored: dropping would change the
    sampling distribution the privacy analysis assumes.
    """

    def __init__(self, dataset: Dataset, *, sample_rate: float, collate_fn=None, drop_last: bool = False,
                 generator=None, distributed: bool = False, batch_first: bool = True,
                 rand_on_empty: bool = False, num_replicas: Optional[int] = None, rank: Optional[int] = None,
                 **kwargs):
        self.sample_rate = sample_rate
        self.distributed = distributed
        if distributed:
            sampler = DistributedUniformWithReplacementSampler(
                total_size=len(dataset), sample_rate=sample_rate, generator=generator, num_replicas=num_replicas,
                rank=rank)
        else:
            sampler = UniformWithReplacementSampler(
                num_samples=len(dataset), sample_rate=sample_rate, generator=generator)
        probe = dataset[0]
        if drop_last:
            logger.warning("Ignoring drop_last as it is not compatible with DPDataLoader.")
        super().__init__(
            dataset=dataset,
            batch_sampler=sampler,
            collate_fn=wrap_collate_with_empty(
                collate_fn=default_collate if collate_fn is None else collate_fn,
                batch_first=batch_first,
                rand_on_empty=rand_on_empty,
                sample_empty_shapes=[(0, *shape_safe(x)) for x in probe],
                dtypes=[dtype_safe(x) for x in probe],
            ),
            generator=_torch_generator(generator),
            **kwargs,
        )

    @classmethod
    def from_data_loader(cls, data_loader: DataLoader, *, distributed: bool = False, generator=None,
                         batch_first: bool = True, rand_on_empty: bool = False,
                         num_replicas: Optional[int] = None, rank: Optional[int] = None):
        """Same dataset and worker settings; the batch size only enters through
        ``sample_rate = 1 / len(data_loader)``.  ``num_replicas`` / ``rank``: see
        ``DistributedUniformWithReplacementSampler``."""
        if isinstance(data_loader.dataset, IterableDataset):
            raise ValueError("Uniform sampling is not supported for IterableDataset")
        return cls(
            dataset=data_loader.dataset,
            sample_rate=1 / len(data_loader),
            collate_fn=data_loader.collate_fn,
            drop_last=data_loader.drop_last,
            generator=generator if generator else data_loader.generator,
            distributed=distributed,
            batch_first=batch_first,
            rand_on_empty=rand_on_empty,
            num_replicas=num_replicas,
            rank=rank,
            **_carry(data_loader),
        )


def _torch_generator(generator):
    """What ``DataLoader(generator=...)`` may be given: a ``torch.Generator`` or None (it seeds worker processes and
    the default sampler only; this package's ``SecureGenerator`` feeds the samplers directly)."""
    return generator if generator is None or isinstance(generator, torch.Generator) else None


def _is_supported_batch_sampler(sampler: Sampler):
    return isinstance(sampler, (BatchSampler, UniformWithReplacementSampler, DistributedUniformWithReplacementSampler))


def switch_generator(*, data_loader: DataLoader, generator):
    """Rebuild ``data_loader`` so that all of its randomness comes from ``generator``."""
    bs = data_loader.batch_sampler
    if bs is None or not _is_supported_batch_sampler(bs):
        raise ValueError(
            "Non-batch processing is not supported: Opacus always assumes one of the input dimensions to be "
            "batch dimension."
        )
    if isinstance(bs, BatchSampler):
        if not hasattr(bs.sampler, "generator"):
            raise ValueError("Target sampler doesn't have generator attribute: nothing to switch")
        if getattr(generator, "gaussian_like", None) is not None and isinstance(bs.sampler, RandomSampler):
            # torch's sampler can only draw from a torch.Generator: same sampling, drawn from the ChaCha20 stream
            from .utils.secure_rng import SecureRandomSampler

            bs.sampler = SecureRandomSampler(bs.sampler.data_source, generator, replacement=bs.sampler.replacement,
                                             num_samples=bs.sampler._num_samples)
        else:
            bs.sampler.generator = generator
    else:
        bs.generator = generator
    return DataLoader(dataset=data_loader.dataset, batch_sampler=bs, collate_fn=data_loader.collate_fn,
                      generator=_torch_generator(generator), **_carry(data_loader))
