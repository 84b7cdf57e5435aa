"""Data-parallel per-layer clipping.

``SimpleDistributedPerLayerOptimizer`` clips at ``step()`` like the
single-process version and then synchronises.  ``DistributedPerLayerOptimizer``
does the work inside backward: because each parameter has its own bound, its
private gradient is final as soon as its per-sample gradient exists, so a
tensor hook can emit the clipped, noised, scaled gradient straight into stock
``DistributedDataParallel``'s bucketed all-reduce, which then overlaps with the
rest of backward.

Behavioural parity: ``opacus/optimizers/ddp_perlayeroptimizer.py:29-175``.
"""
from __future__ import annotations

import math
from functools import partial
from typing import Callable, List, Optional

import torch
from torch import nn
from torch.optim import Optimizer

from .. import ops
from .ddpoptimizer import DistributedDPOptimizer
from .optimizer import DPOptimizer, _generate_noise
from .perlayeroptimizer import DPPerLayerOptimizer


def _clip_and_accumulate_parameter(p: nn.Parameter, max_grad_norm: float):
    factor = ops.clip_factor(ops.grad_sample_norm_sq(p.grad_sample), float(max_grad_norm))
    grad = ops.weighted_sum(p.grad_sample, factor)
    if p.summed_grad is not None:
        p.summed_grad += grad
    else:
        p.summed_grad = grad


class SimpleDistributedPerLayerOptimizer(DPPerLayerOptimizer, DistributedDPOptimizer):
    def __init__(self, optimizer: Optimizer, *, noise_multiplier: float, max_grad_norm: float,
                 expected_batch_size: Optional[int], loss_reduction: str = "mean", generator=None,
                 secure_mode: bool = False, **kwargs):
        self.rank = torch.distributed.get_rank()
        self.world_size = torch.distributed.get_world_size()
        super().__init__(optimizer, noise_multiplier=noise_multiplier, max_grad_norm=max_grad_norm,
                         expected_batch_size=expected_batch_size, loss_reduction=loss_reduction,
                         generator=generator, secure_mode=secure_mode)


class DistributedPerLayerOptimizer(DPOptimizer):
    """For models wrapped in stock ``torch.nn.parallel.DistributedDataParallel``."""

    _fused_ok = False

    def __init__(self, optimizer: Optimizer, *, noise_multiplier: float, max_grad_norm: List[float],
                 expected_batch_size: Optional[int], loss_reduction: str = "mean", generator=None,
                 secure_mode: bool = False, **kwargs):
        self.rank = torch.distributed.get_rank()
        self.world_size = torch.distributed.get_world_size()
        self.max_grad_norms = max_grad_norm
        overall = math.sqrt(sum(float(c) ** 2 for c in max_grad_norm))
        super().__init__(optimizer, noise_multiplier=noise_multiplier, max_grad_norm=overall,
                         expected_batch_size=expected_batch_size, loss_reduction=loss_reduction,
                         generator=generator, secure_mode=secure_mode)
        self._register_hooks()

    def _add_noise_parameter(self, p: nn.Parameter):
        noise = _generate_noise(std=self.noise_multiplier * self.max_grad_norm, reference=p.summed_grad,
                                generator=None, secure_mode=self.secure_mode)
        p.grad = p.summed_grad + noise

    @property
    def accumulated_iterations(self) -> int:
        return max(p.accumulated_iterations for p in self.params)

    def _scale_grad_parameter(self, p: nn.Parameter):
        p.accumulated_iterations = getattr(p, "accumulated_iterations", 0) + 1
        if self.loss_reduction == "mean":
            p.grad /= self.expected_batch_size * p.accumulated_iterations * self.world_size

    def clip_and_accumulate(self):
        raise NotImplementedError("Clip and accumulate is added per layer in DPDDP Per Layer.")

    def add_noise(self):
        raise NotImplementedError("Noise is added per layer in DPDDP Per Layer.")

    def pre_step(self, closure: Optional[Callable[[], float]] = None) -> Optional[float]:
        if self._check_skip_next_step():
            self._is_last_step_skipped = True
            return False
        if self.step_hook:
            self.step_hook(self)
        for p in self.params:
            p.accumulated_iterations = 0
        self._is_last_step_skipped = False
        return True

    def _ddp_per_layer_hook(self, p: nn.Parameter, max_grad_norm: float, _: torch.Tensor):
        _clip_and_accumulate_parameter(p, max_grad_norm)
        if self._check_skip_next_step(pop_next=False):
            return None
        if self.rank == 0:
            self._add_noise_parameter(p)
        else:
            p.grad = p.summed_grad
        self._scale_grad_parameter(p)
        return p.grad

    def _register_hooks(self):
        for p, bound in zip(self.params, self.max_grad_norms):
            if not p.requires_grad:
                continue
            if not hasattr(p, "ddp_hooks"):
                p.ddp_hooks = []
            p.ddp_hooks.append(p.register_hook(partial(self._ddp_per_layer_hook, p, bound)))
