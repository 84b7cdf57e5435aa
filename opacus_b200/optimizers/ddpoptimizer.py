"""Data-parallel ``DPOptimizer``: every rank clips its local samples, exactly
one Gaussian draw is added globally (by rank 0), gradients are summed across
ranks and averaged.

Behavioural parity: ``opacus/optimizers/ddpoptimizer.py:25-83`` (which issues
one all-reduce per parameter; here they are bucketed).
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
from torch.optim import Optimizer

from ._collectives import all_reduce_grads
from .optimizer import DPOptimizer


class DistributedDPOptimizer(DPOptimizer):
    _fused_ok = False  # the update follows a collective; the fused form is the sharded engine's step (engine=)

    def __init__(self, optimizer: Optimizer, *, noise_multiplier: float, max_grad_norm: float,
                 expected_batch_size: Optional[int], loss_reduction: str = "mean", generator=None,
                 secure_mode: bool = False, engine=None, **kwargs):
        super().__init__(optimizer, noise_multiplier=noise_multiplier, max_grad_norm=max_grad_norm,
                         expected_batch_size=expected_batch_size, loss_reduction=loss_reduction,
                         generator=generator, secure_mode=secure_mode, **kwargs)
        self.rank = torch.distributed.get_rank()
        self.world_size = torch.distributed.get_world_size()
        # With a ShardedDataParallel engine the all-reduce, the single noise draw and the update
        # run as one kernel over peer memory instead of NCCL + per-parameter kernels.
        self.engine = engine

    def add_noise(self):
        # Noise is a property of the *global* sum: draw it once.
        if self.rank == 0:
            super().add_noise()
        else:
            for p in self.params:
                p.grad = p.summed_grad.view_as(p)

    def reduce_gradients(self):
        grads = [p.grad for p in self.params if p.requires_grad]
        all_reduce_grads(grads, average_by=self.world_size if self.loss_reduction == "mean" else 1)

    def step(self, closure: Optional[Callable[[], float]] = None) -> Optional[torch.Tensor]:
        if closure is not None:
            with torch.enable_grad():
                closure()
        if self.engine is not None:
            return self._engine_step()
        if self.pre_step():
            self.reduce_gradients()
            return self.original_optimizer.step()
        return None

    def _engine_step(self):
        """Hand the clipped sums to the engine's flat gradient buffer and let its
        fused kernel do reduce + noise + update + publish."""
        if self._collect():
            for p in self.params:
                dst = getattr(p, "_dp_grad_out", None)
                if dst is None or p.summed_grad is None:
                    continue
                if p.summed_grad.data_ptr() != dst.data_ptr():
                    dst.copy_(p.summed_grad.view_as(dst))
                    p.summed_grad = dst          # later physical batches accumulate in place
                p._dp_grad_fresh = False
        return self.engine.optimizer_step(self)
