"""Per-layer clipping: parameter ``i`` is clipped to its own bound ``C_i``; the
noise scale uses the overall sensitivity ``||(C_1, ..., C_P)||_2``
(``opacus/optimizers/perlayeroptimizer.py:26-76``)."""
from __future__ import annotations

import math
from typing import List, Optional

from torch.optim import Optimizer

from .. import ops
from .optimizer import DPOptimizer, _check_processed_flag, _mark_as_processed
from .utils import params


class DPPerLayerOptimizer(DPOptimizer):
    def __init__(self, optimizer: Optimizer, *, noise_multiplier: float, max_grad_norm: List[float],
                 expected_batch_size: Optional[int], loss_reduction: str = "mean", generator=None,
                 secure_mode: bool = False, **kwargs):
        assert len(max_grad_norm) == len(params(optimizer))
        self.max_grad_norms = max_grad_norm
        overall = math.sqrt(sum(float(c) ** 2 for c in max_grad_norm))
        super().__init__(optimizer, noise_multiplier=noise_multiplier, max_grad_norm=overall,
                         expected_batch_size=expected_batch_size, loss_reduction=loss_reduction,
                         generator=generator, secure_mode=secure_mode, **kwargs)

    def clip_and_accumulate(self):
        for p, bound in zip(self.params, self.max_grad_norms):
            _check_processed_flag(p.grad_sample)
            gs = self._get_flat_grad_sample(p)
            factor = ops.clip_factor(ops.grad_sample_norm_sq(gs), float(bound))
            self._accumulate_clipped(p, gs, factor)
            _mark_as_processed(p.grad_sample)
