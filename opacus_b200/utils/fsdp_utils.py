"""``FSDP2Wrapper``: prepare a model for sharded data-parallel DP training.

``engine="native"`` (default on CUDA) returns this package's
:class:`~opacus_b200.parallel.sharded.ShardedDataParallel`;
``engine="torch"`` applies ``torch.distributed.fsdp.fully_shard`` to every
submodule that has a sampler (or no trainable parameters) and then to the root,
as ``opacus/utils/fsdp_utils.py:27-61`` does.
"""
from typing import Iterable

import torch
import torch.nn as nn

from .module_utils import has_trainable_params


def has_params(module: nn.Module) -> bool:
    return any(True for _ in module.parameters(recurse=False))


def iterate_submodules(module: nn.Module) -> Iterable[nn.Module]:
    if has_params(module):
        yield module
    for child in module.children():
        yield from iterate_submodules(child)


def FSDP2Wrapper(model: nn.Module, engine: str = "auto", **kwargs) -> nn.Module:
    if engine == "auto":
        first = next(model.parameters(), None)
        engine = "native" if first is not None and first.is_cuda else "torch"
    if engine == "native":
        from ..parallel.sharded import ShardedDataParallel

        return ShardedDataParallel(model, **kwargs)

    from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard

    from ..grad_sample import GradSampleModuleFastGradientClippingFSDP as G

    known = set(G.GRAD_SAMPLERS) | set(G.NORM_SAMPLERS)
    mp_policy = kwargs.get("mp_policy", MixedPrecisionPolicy())
    high = tuple(kwargs.get("opacus_high_precision_layers", []))
    for sub in iterate_submodules(model):
        if type(sub) in known or not has_trainable_params(sub):
            if high and isinstance(sub, high):
                fully_shard(sub, mp_policy=MixedPrecisionPolicy(param_dtype=torch.get_default_dtype()))
            else:
                fully_shard(sub, mp_policy=mp_policy)
    return fully_shard(model, mp_policy=mp_policy)
