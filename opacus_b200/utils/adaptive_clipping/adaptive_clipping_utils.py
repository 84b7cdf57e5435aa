"""Adaptive clipping for ghost clipping: between measuring the per-sample norms
and applying the clip factors, the bound is moved towards a target quantile of
the norms, using a noised count of unclipped samples (its noise is paid for by
a slightly larger gradient noise multiplier).

Behavioural parity: ``opacus/utils/adaptive_clipping/adaptive_clipping_utils.py:33-279``.
"""
import math
from typing import Tuple

import torch

from ...privacy_engine import PrivacyEngine
from ..fast_gradient_clipping_utils import DPLossFastGradientClipping, DPTensorFastGradientClipping


class DPTensorFastGradientAdaptiveClipping(DPTensorFastGradientClipping):
    def __init__(self, module, optimizer, loss_per_sample: torch.Tensor, loss_reduction: str = "mean",
                 target_unclipped_quantile: float = 0.5, min_clipbound: float = 1, max_clipbound: float = 1e8,
                 clipbound_learning_rate: float = 0.2, initial_noise_multiplier: float = 1.0):
        super().__init__(module, optimizer, loss_per_sample, loss_reduction)
        self.target_unclipped_quantile = target_unclipped_quantile
        self.min_clipbound = min_clipbound
        self.max_clipbound = max_clipbound
        self.clipbound_learning_rate = clipbound_learning_rate
        self.initial_clipping_norm = self.optimizer.max_grad_norm
        self.initial_noise_multiplier = initial_noise_multiplier

    def _is_distributed(self) -> bool:
        from torch.nn.parallel import DistributedDataParallel as DDP

        from ...distributed import DifferentiallyPrivateDistributedDataParallel as DPDDP

        inner = getattr(self.module, "_module", None)
        return isinstance(self.module, (DPDDP, DDP)) or isinstance(inner, (DPDDP, DDP))

    def _update_clip_and_noise(self, per_sample_norms) -> Tuple[float, float]:
        assert self.module.max_grad_norm == self.optimizer.max_grad_norm, \
            "Max grad norm does not match between optimizer and model."
        bound = self.module.max_grad_norm
        local = torch.stack([(per_sample_norms <= bound).sum().float(),
                             per_sample_norms.new_tensor(float(len(per_sample_norms)))])
        if self._is_distributed():
            torch.distributed.all_reduce(local, op=torch.distributed.ReduceOp.SUM)
        unclipped, batch = local.tolist()
        count_std = batch / 20.0
        unclipped += torch.normal(mean=0.0, std=count_std, size=(1,)).item()
        frac = unclipped / batch
        new_bound = bound * math.exp(-self.clipbound_learning_rate * (frac - self.target_unclipped_quantile))
        new_bound = min(max(new_bound, self.min_clipbound), self.max_clipbound)
        assert batch > 10 * self.initial_noise_multiplier, (
            "Batch size is too small. For adaptive clipping, please use a batch size larger than "
            "10 * noise_multiplier.")
        sigma = self.initial_noise_multiplier
        if sigma > 0:
            sigma = (sigma ** (-2) - (2.0 * count_std) ** (-2)) ** (-0.5)
        return new_bound, sigma

    def _retarget(self):
        norms = self.module.get_norm_sample()
        bound, sigma = self._update_clip_and_noise(norms)
        self.module.max_grad_norm = bound
        self.optimizer.max_grad_norm = bound
        self.optimizer._adjusted_noise_multiplier = sigma
        return norms

    def _before_finish(self):
        self._retarget()

    def _coefficients(self):
        norms = self._retarget()
        bound = self.module.max_grad_norm
        return torch.where(norms <= bound, torch.ones_like(norms), bound / norms)


class DPLossFastGradientAdaptiveClipping(DPLossFastGradientClipping):
    def __init__(self, module, optimizer, criterion, loss_reduction: str = "mean",
                 target_unclipped_quantile: float = 0.5, min_clipbound: float = 1, max_clipbound: float = 1e8,
                 clipbound_learning_rate: float = 0.2, initial_noise_multiplier: float = 1.0):
        super().__init__(module, optimizer, criterion, loss_reduction)
        self.target_unclipped_quantile = target_unclipped_quantile
        self.min_clipbound = min_clipbound
        self.max_clipbound = max_clipbound
        self.clipbound_learning_rate = clipbound_learning_rate
        self.initial_noise_multiplier = initial_noise_multiplier

    def __call__(self, *args, shape=None, **kwargs) -> DPTensorFastGradientAdaptiveClipping:
        return DPTensorFastGradientAdaptiveClipping(
            self.module, self.optimizer, self._per_sample(*args, shape=shape, **kwargs), self.loss_reduction,
            self.target_unclipped_quantile, self.min_clipbound, self.max_clipbound,
            self.clipbound_learning_rate, self.initial_noise_multiplier)


class PrivacyEngineAdaptiveClipping(PrivacyEngine):
    """``PrivacyEngine`` whose ghost-mode criterion adapts the clipping bound.
    Extra ``make_private`` kwargs: ``target_unclipped_quantile``,
    ``min_clipbound``, ``max_clipbound``, ``clipbound_learning_rate``."""

    _CRITERION_KWARGS = ("target_unclipped_quantile", "min_clipbound", "max_clipbound", "clipbound_learning_rate")

    def __init__(self, *, accountant: str = "prv", secure_mode: bool = False):
        super().__init__(accountant=accountant, secure_mode=secure_mode)

    def _prepare_criterion(self, *, module, optimizer, criterion=torch.nn.CrossEntropyLoss(),
                           loss_reduction: str = "mean", target_unclipped_quantile: float = 0.5,
                           min_clipbound: float = 1, max_clipbound: float = 1e8,
                           clipbound_learning_rate: float = 0.2, **kwargs):
        return DPLossFastGradientAdaptiveClipping(
            module, optimizer, criterion, loss_reduction=loss_reduction,
            target_unclipped_quantile=target_unclipped_quantile, min_clipbound=min_clipbound,
            max_clipbound=max_clipbound, clipbound_learning_rate=clipbound_learning_rate,
            initial_noise_multiplier=optimizer.noise_multiplier)
