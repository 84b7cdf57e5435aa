"""Data-parallel per-layer clipping.

With one clipping bound per parameter, a parameter's private gradient does not
depend on any other parameter: it is final the moment its per-sample gradient
exists.  ``DistributedPerLayerOptimizer`` uses that to finish each parameter
*inside* the backward pass -- a gradient hook replaces the gradient autograd is
about to hand to stock ``DistributedDataParallel`` by the clipped sum (plus the
single noise draw on rank 0, divided by the global batch), so DDP's bucketed
all-reduce carries private gradients and overlaps with the rest of backward.
What is left for ``step()`` is the accountant hook and the wrapped optimiser.

All bookkeeping lives in one ``_Layer`` record per parameter, owned by the
optimiser (bound, number of physical batches folded into the running sum, hook
handle); the three stages are this package's kernels (``ops.clip_factor``,
``ops.weighted_sum``) -- the same pipeline ``DPPerLayerOptimizer`` runs at
``step()`` time, applied to one parameter.

The hook needs the parameter's per-sample gradient to exist when autograd
delivers the parameter's batch gradient.  Module backward hooks run after the
layer's own backward, i.e. too late for all but the first layer, so the model is
wrapped as ``GradSampleModule(model, early_capture=True)``: per-sample gradients
are then computed when the gradient of the layer's output arrives.

``SimpleDistributedPerLayerOptimizer`` is the variant for
:class:`~opacus_b200.distributed.DifferentiallyPrivateDistributedDataParallel`:
per-layer clipping at ``step()``, then one bucketed all-reduce.

Behavioural parity: ``opacus/optimizers/ddp_perlayeroptimizer.py:29-175``.
"""
from __future__ import annotations

import math
from typing import Callable, Dict, List, Optional

import torch
from torch import nn
from torch.optim import Optimizer

from .. import ops
from .ddpoptimizer import DistributedDPOptimizer
from .optimizer import DPOptimizer, _generate_noise
from .perlayeroptimizer import DPPerLayerOptimizer


def _clip_and_accumulate_parameter(p: nn.Parameter, max_grad_norm: float) -> None:
    """Clip the per-sample gradients of ONE parameter to ``max_grad_norm`` and add their sum to ``p.summed_grad``
    (created on the parameter's device when it is None).  Module-level helper kept under the name the reference
    exports (``opacus/optimizers/ddp_perlayeroptimizer.py:29-37``); the optimiser below runs the same three stages
    from its gradient hook."""
    gs = p.grad_sample
    clipped = ops.weighted_sum(gs, ops.clip_factor(ops.grad_sample_norm_sq(gs), float(max_grad_norm))).view_as(p)
    p.summed_grad = clipped if p.summed_grad is None else p.summed_grad + clipped.to(p.summed_grad.dtype)


class SimpleDistributedPerLayerOptimizer(DPPerLayerOptimizer, DistributedDPOptimizer):
    def __init__(self, optimizer: Optimizer, *, noise_multiplier: float, max_grad_norm: float,
                 expected_batch_size: Optional[int], loss_reduction: str = "mean", generator=None,
                 secure_mode: bool = False, **kwargs):
        self.rank = torch.distributed.get_rank()
        self.world_size = torch.distributed.get_world_size()
        super().__init__(optimizer, noise_multiplier=noise_multiplier, max_grad_norm=max_grad_norm,
                         expected_batch_size=expected_batch_size, loss_reduction=loss_reduction,
                         generator=generator, secure_mode=secure_mode)


class _Layer:
    """Per-parameter state of :class:`DistributedPerLayerOptimizer`."""

    __slots__ = ("bound", "batches", "handle")

    def __init__(self, bound: float):
        self.bound = float(bound)
        self.batches = 0          # physical batches in the running sum since the last logical step
        self.handle = None


class DistributedPerLayerOptimizer(DPOptimizer):
    """For models wrapped in stock ``torch.nn.parallel.DistributedDataParallel``."""

    _fused_ok = False

    def __init__(self, optimizer: Optimizer, *, noise_multiplier: float, max_grad_norm: List[float],
                 expected_batch_size: Optional[int], loss_reduction: str = "mean", generator=None,
                 secure_mode: bool = False, **kwargs):
        self.rank = torch.distributed.get_rank()
        self.world_size = torch.distributed.get_world_size()
        self.max_grad_norms = list(max_grad_norm)
        sensitivity = math.sqrt(sum(float(c) ** 2 for c in self.max_grad_norms))
        super().__init__(optimizer, noise_multiplier=noise_multiplier, max_grad_norm=sensitivity,
                         expected_batch_size=expected_batch_size, loss_reduction=loss_reduction,
                         generator=generator, secure_mode=secure_mode)
        self._layers: Dict[nn.Parameter, _Layer] = {}
        for p, bound in zip(self.params, self.max_grad_norms):
            if p.requires_grad:
                layer = self._layers[p] = _Layer(bound)
                layer.handle = p.register_hook(self._finisher(p, layer))

    # ---- what happens to one parameter when its gradient arrives
    def _finisher(self, p: nn.Parameter, layer: _Layer):
        def on_grad(_batch_grad: torch.Tensor):
            if getattr(p, "grad_sample", None) is None:
                raise ValueError("the per-sample gradient of a parameter is not there when its gradient arrives: "
                                 "wrap the model as GradSampleModule(model, early_capture=True)")
            gs = self._get_flat_grad_sample(p)
            factor = ops.clip_factor(ops.grad_sample_norm_sq(gs), layer.bound)
            clipped = ops.weighted_sum(gs, factor)
            p.summed_grad = clipped if p.summed_grad is None else p.summed_grad.add_(clipped)
            layer.batches += 1
            if self._check_skip_next_step(pop_next=False):
                return None                       # virtual step: keep accumulating, DDP sees the plain gradient
            private = p.summed_grad
            if self.rank == 0:                    # the noise belongs to the global sum: one rank draws it
                private = private + _generate_noise(std=self._noise_std(), reference=private, generator=None,
                                                    secure_mode=self.secure_mode)
            if self.loss_reduction == "mean":
                private = private / (self.expected_batch_size * layer.batches * self.world_size)
            p.grad = private
            return private

        return on_grad

    @property
    def accumulated_iterations(self) -> int:
        return max((layer.batches for layer in self._layers.values()), default=0)

    def remove_hooks(self):
        for layer in self._layers.values():
            if layer.handle is not None:
                layer.handle.remove()
                layer.handle = None

    # ---- the staged API of the base class does not apply: the stages ran per parameter during backward
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
        for layer in self._layers.values():
            layer.batches = 0
        self._is_last_step_skipped = False
        return True
