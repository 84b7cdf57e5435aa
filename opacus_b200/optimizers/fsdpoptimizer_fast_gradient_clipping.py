"""Optimizer for sharded data parallelism with ghost clipping.

With this package's :class:`~opacus_b200.parallel.sharded.ShardedDataParallel`
engine the whole tail of the step -- reduce-scatter of the clipped gradient
sums over NVLink, one Gaussian draw per owned element, scaling, the sharded
SGD/Adam(W) update and the all-gather of the updated parameters -- is a single
kernel launched from :meth:`step`.

With ``torch.distributed.fsdp.fully_shard`` models (or tensor-parallel DTensor
parameters) gradients arrive already reduce-scattered and averaged by FSDP2, so
every rank adds noise to *its shard* and, for mean reduction, divides that
noise by the world size; accumulated state lives in ``grad_state`` because
FSDP2 replaces parameter objects.

Behavioural parity: ``opacus/optimizers/fsdpoptimizer_fast_gradient_clipping.py:32-181``.
"""
from __future__ import annotations

import contextlib
import logging
from typing import Callable, Optional

import torch
from torch.optim import Optimizer

from .optimizer import _generate_noise
from .optimizer_fast_gradient_clipping import DPOptimizerFastGradientClipping

logger = logging.getLogger(__name__)
logger.disabled = True


def _implicit_replication():
    try:
        from torch.distributed.tensor.experimental import implicit_replication
    except Exception:
        try:
            from torch.distributed._tensor.experimental import implicit_replication
        except Exception:  # pragma: no cover
            return contextlib.nullcontext()
    return implicit_replication()


class FSDPOptimizerFastGradientClipping(DPOptimizerFastGradientClipping):
    _fused_ok = False

    def __init__(self, optimizer: Optimizer, *, noise_multiplier: float, max_grad_norm: float,
                 expected_batch_size: Optional[int], loss_reduction: str = "mean",
                 generator: Optional[torch.Generator] = None, secure_mode: bool = False, engine=None, **kwargs):
        super().__init__(optimizer=optimizer, noise_multiplier=noise_multiplier, max_grad_norm=max_grad_norm,
                         expected_batch_size=expected_batch_size, loss_reduction=loss_reduction,
                         generator=generator, secure_mode=secure_mode, **kwargs)
        self.rank = torch.distributed.get_rank()
        self.world_size = torch.distributed.get_world_size()
        self.engine = engine  # ShardedDataParallel, when the native path is used
        if engine is not None and hasattr(engine, "attach_optimizer"):
            engine.attach_optimizer(self)
        self.grad_state = {p: {"summed_grad": None} for p in self.params}

    def accumulate(self):
        for p in self.params:
            if p.grad is None:
                continue
            slot = self.grad_state.setdefault(p, {"summed_grad": None})
            if slot["summed_grad"] is None:
                slot["summed_grad"] = p.grad.detach().clone()
            else:
                slot["summed_grad"].add_(p.grad.detach())

    def zero_grad(self, set_to_none: bool = False):
        for p in self.params:
            if not self._is_last_step_skipped:
                self.grad_state.setdefault(p, {})["summed_grad"] = None
        if self.engine is not None and not self._is_last_step_skipped:
            self.engine.mark_grads_fresh()
        self.original_optimizer.zero_grad(set_to_none)

    def add_noise(self):
        std = self._noise_std()
        for p in self.params:
            summed = self.grad_state[p]["summed_grad"]
            noise = _generate_noise(std=std, reference=p.grad if p.grad is not None else summed,
                                    generator=self.generator, secure_mode=self.secure_mode)
            if self.loss_reduction == "mean":
                noise.div_(self.world_size)
            p.grad = (summed + noise).view_as(p)

    def pre_step(self, closure: Optional[Callable[[], float]] = None) -> Optional[float]:
        self.accumulate()
        if self._check_skip_next_step():
            self._is_last_step_skipped = True
            return False
        with _implicit_replication():
            self.add_noise()
        self.scale_grad()
        if self.step_hook:
            self.step_hook(self)
        self._is_last_step_skipped = False
        return True

    def step(self, closure: Optional[Callable[[], float]] = None):
        if self.engine is not None:
            return self.engine.optimizer_step(self, closure)
        return super().step(closure)
