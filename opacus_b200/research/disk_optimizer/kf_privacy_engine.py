"""``PrivacyEngine`` whose ``make_private(..., kalman=True, kappa=..., gamma=...)`` wraps the
optimizer in its Kalman-filtered form (``research/disk_optimizer/KFprivacy_engine.py:24-70``)."""
from __future__ import annotations

from typing import List, Union

from torch import optim

from ...optimizers import DPOptimizer
from ...privacy_engine import PrivacyEngine
from .kf_optimizer import KalmanFilterMixin, get_optimizer_class


class KF_PrivacyEngine(PrivacyEngine):
    def __init__(self, *, accountant: str = "prv", secure_mode: bool = False):
        super().__init__(accountant=accountant, secure_mode=secure_mode)

    def _prepare_optimizer(self, *, optimizer: optim.Optimizer, noise_multiplier: float,
                           max_grad_norm: Union[float, List[float]], expected_batch_size: int,
                           loss_reduction: str = "mean", distributed: bool = False, clipping: str = "flat",
                           noise_generator=None, grad_sample_mode="hooks", kalman: bool = False,
                           **kwargs) -> DPOptimizer:
        if isinstance(optimizer, DPOptimizer) and (not kalman or isinstance(optimizer, KalmanFilterMixin)):
            optimizer = optimizer.original_optimizer
        generator = self.secure_rng if self.secure_mode else noise_generator
        if not kalman:
            kwargs.pop("kappa", None)
            kwargs.pop("gamma", None)
        kwargs.pop("engine", None)
        cls = get_optimizer_class(clipping=clipping, distributed=distributed, grad_sample_mode=grad_sample_mode,
                                  kalman=kalman)
        return cls(optimizer=optimizer, noise_multiplier=noise_multiplier, max_grad_norm=max_grad_norm,
                   expected_batch_size=expected_batch_size, loss_reduction=loss_reduction, generator=generator,
                   secure_mode=self.secure_mode, **kwargs)
