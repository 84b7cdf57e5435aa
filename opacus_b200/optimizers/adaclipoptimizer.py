"""Adaptive clipping (Andrew, Thakkar, McMahan, Ramaswamy 2019): the clipping
bound follows a target quantile of the per-sample gradient norms.  The fraction
of unclipped samples is released with its own Gaussian noise
(``unclipped_num_std``), and the gradient noise is increased so that the total
privacy cost equals that of ``noise_multiplier`` alone (their Theorem 1).

Behavioural parity: ``opacus/optimizers/adaclipoptimizer.py:34-191``.
"""
from __future__ import annotations

import logging
from typing import Callable, Optional

import torch
from torch.optim import Optimizer

from .optimizer import DPOptimizer, _check_processed_flag, _generate_noise, _mark_as_processed

logger = logging.getLogger(__name__)


class AdaClipDPOptimizer(DPOptimizer):
    _fused_ok = False

    def __init__(self, optimizer: Optimizer, *, noise_multiplier: float, target_unclipped_quantile: float,
                 clipbound_learning_rate: float, max_clipbound: float, min_clipbound: float,
                 unclipped_num_std: float, max_grad_norm: float, expected_batch_size: Optional[int],
                 loss_reduction: str = "mean", generator=None, secure_mode: bool = False, **kwargs):
        super().__init__(optimizer, noise_multiplier=noise_multiplier, max_grad_norm=max_grad_norm,
                         expected_batch_size=expected_batch_size, loss_reduction=loss_reduction,
                         generator=generator, secure_mode=secure_mode)
        if max_clipbound <= min_clipbound:
            raise ValueError("max_clipbound must be larger than min_clipbound.")
        if noise_multiplier >= 2 * unclipped_num_std:
            raise ValueError(
                "noise_multiplier must be smaller than 2 * unclipped_num_std. This is a requirement stemming "
                "from Theorem 1 in https://arxiv.org/pdf/1905.03871.pdf"
            )
        self.target_unclipped_quantile = target_unclipped_quantile
        self.clipbound_learning_rate = clipbound_learning_rate
        self.max_clipbound = max_clipbound
        self.min_clipbound = min_clipbound
        self.unclipped_num_std = unclipped_num_std
        self.sample_size = 0
        self.unclipped_num = 0

    def zero_grad(self, set_to_none: bool = False):
        super().zero_grad(set_to_none)
        self.sample_size = 0
        self.unclipped_num = 0

    def clip_and_accumulate(self):
        factor = self._per_sample_clip_factor()
        self.sample_size += len(factor)
        self.unclipped_num += len(factor) - (factor < 1).sum()
        for p in self.params:
            _check_processed_flag(p.grad_sample)
            self._accumulate_clipped(p, self._get_flat_grad_sample(p), factor)
            _mark_as_processed(p.grad_sample)

    def _noise_std(self) -> float:
        if self.noise_multiplier <= 0:
            return 0.0
        sigma = (self.noise_multiplier ** (-2) - (2 * self.unclipped_num_std) ** (-2)) ** (-0.5)
        return sigma * self.max_grad_norm

    def add_noise(self):
        super().add_noise()
        count = self.unclipped_num if torch.is_tensor(self.unclipped_num) else torch.tensor(self.unclipped_num)
        noise = _generate_noise(std=self.unclipped_num_std, reference=count.float(), generator=self.generator)
        self.unclipped_num = float(count) + noise

    def update_max_grad_norm(self):
        """``C <- C * exp(-lr * (unclipped_fraction - target))``, clamped."""
        frac = self.unclipped_num / self.sample_size
        self.max_grad_norm *= torch.exp(-self.clipbound_learning_rate * (frac - self.target_unclipped_quantile))
        if self.max_grad_norm > self.max_clipbound:
            self.max_grad_norm = self.max_clipbound
        elif self.max_grad_norm < self.min_clipbound:
            self.max_grad_norm = self.min_clipbound

    def pre_step(self, closure: Optional[Callable[[], float]] = None) -> Optional[float]:
        ran = super().pre_step()
        if ran:
            self.update_max_grad_norm()
        return ran
