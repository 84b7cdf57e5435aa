"""Optimizer for ghost / fast gradient clipping: by the time ``step()`` runs,
``p.grad`` already holds the clipped sum ``sum_n c_n g_n`` (produced by the
single-pass engine or by the second backward pass), so this class only
accumulates it, adds noise, scales and steps.

Behavioural parity: ``opacus/optimizers/optimizer_fast_gradient_clipping.py:36-224``.
"""
from __future__ import annotations

import logging
from typing import Optional

import torch
from torch.optim import Optimizer

from .optimizer import DPOptimizer, _check_processed_flag, _generate_noise, _mark_as_processed

logger = logging.getLogger(__name__)
logger.disabled = True


class DPOptimizerFastGradientClipping(DPOptimizer):
    def __init__(self, optimizer: Optimizer, *, noise_multiplier: float, max_grad_norm: float,
                 expected_batch_size: Optional[int], loss_reduction: str = "mean", generator=None,
                 secure_mode: bool = False, **kwargs):
        super().__init__(optimizer=optimizer, noise_multiplier=noise_multiplier, max_grad_norm=max_grad_norm,
                         expected_batch_size=expected_batch_size, loss_reduction=loss_reduction,
                         generator=generator, secure_mode=secure_mode, **kwargs)

    @property
    def accumulated_iterations(self) -> int:
        """Virtual batches are the only supported form of accumulation here."""
        return 1

    def accumulate(self):
        """``summed_grad += grad``; the first time the gradient tensor itself is
        adopted (the engine hands over a fresh buffer every backward pass)."""
        for p in self.params:
            if p.grad is None:
                continue
            if p.summed_grad is None:
                p.summed_grad = p.grad.detach()
                p.grad = None
            else:
                p.summed_grad.add_(p.grad.detach())

    def zero_grad(self, set_to_none: bool = False):
        for p in self.params:
            if not self._is_last_step_skipped:
                p.summed_grad = None
        self.original_optimizer.zero_grad(set_to_none)

    def _collect(self) -> bool:
        self.accumulate()
        return True

    def _get_flat_grad_sample(self, p: torch.Tensor):
        return None

    def clip_and_accumulate(self):
        """Clipping already happened when the gradient was formed."""

    def _noise_std(self) -> float:
        # adaptive clipping spends part of the budget on the unclipped count
        sigma = getattr(self, "_adjusted_noise_multiplier", self.noise_multiplier)
        return sigma * self.max_grad_norm

    def add_noise(self):
        std = self._noise_std()
        for p in self.params:
            _check_processed_flag(p.summed_grad)
            noise = _generate_noise(std=std, reference=p.summed_grad, generator=self.generator,
                                    secure_mode=self.secure_mode)
            p.grad = (p.summed_grad + noise).view_as(p)
            _mark_as_processed(p.summed_grad)
