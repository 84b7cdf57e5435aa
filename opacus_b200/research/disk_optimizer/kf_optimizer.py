"""DiSK -- a scalar-gain Kalman filter around any DP optimizer.

The privatised gradient ``g_t`` of step ``t`` is treated as a noisy observation
of a slowly moving true gradient.  With gain ``1 - kappa`` the filter keeps

    m_t = kappa * m_{t-1} + (1 - kappa) * g_t ,

hands ``m_t`` to the wrapped optimizer instead of ``g_t`` and remembers the
last displacement ``d_t = x_{t+1} - x_t``.  The observation itself is taken one
step ahead along that displacement: the closure is evaluated at
``x_t + gamma * d_{t-1}``.  When ``gamma`` equals ``(1 - kappa) / kappa`` one
evaluation suffices; otherwise the per-sample gradients at ``x_t`` and at the
look-ahead point are mixed as ``(1 - c) g(x_t) + c g(x_t + gamma d)`` with
``c = (1 - kappa) / (gamma kappa)`` before clipping, and because one sample then
enters with total weight ``sqrt(c^2 + (1-c)^2)`` the noise multiplier is divided
by that factor so the privacy accounting is unchanged.

``step(closure)`` needs the closure (forward + backward) because the filter
moves the parameters before the gradients are taken.

Behavioural parity: ``research/disk_optimizer/optimizers/KFoptimizer.py:31-163`` and
its seven siblings in the reference; here one mixin serves every DP optimizer.
"""
from __future__ import annotations

import math
from typing import Callable, Optional

import torch

from ...optimizers import (
    AdaClipDPOptimizer,
    DistributedDPOptimizer,
    DistributedDPOptimizerFastGradientClipping,
    DistributedPerLayerOptimizer,
    DPOptimizer,
    DPOptimizerFastGradientClipping,
    DPPerLayerOptimizer,
    SimpleDistributedPerLayerOptimizer,
)
from ...optimizers import get_optimizer_class as _plain_optimizer_class


class KalmanFilterMixin:
    """Put in front of a DP optimizer class: ``class KF_X(KalmanFilterMixin, X)``."""

    def __init__(self, optimizer, *, noise_multiplier: float, kappa: float = 0.7, gamma: float = 0.5, **kwargs):
        if not 0.0 < kappa <= 1.0:
            raise ValueError("kappa must be in (0, 1]")
        natural = (1.0 - kappa) / kappa
        if gamma == 0 or abs(gamma - natural) < 1e-3:
            gamma = natural
            self.kf_compute_grad_at_original = False
            self.scaling_factor = 1.0
        else:
            c = (1.0 - kappa) / (gamma * kappa)
            self.scaling_factor = c
            self.kf_compute_grad_at_original = True
            noise_multiplier = noise_multiplier / math.sqrt(c * c + (1.0 - c) ** 2)
        super().__init__(optimizer, noise_multiplier=noise_multiplier, **kwargs)
        self.kappa = kappa
        self.gamma = gamma

    # ---- helpers
    def _shift(self, sign: float) -> bool:
        """``x += sign * gamma * d`` for every parameter that already has a displacement."""
        moved = False
        for p in self.params:
            d = self.state[p].get("kf_d_t") if p in self.state else None
            if d is not None:
                p.data.add_(d, alpha=sign * self.gamma)
                moved = True
        return moved

    def _take_grad_samples(self):
        out = []
        for p in self.params:
            gs = getattr(p, "grad_sample", None)
            out.append(gs)
            p.grad_sample = None
        return out

    def _observe(self, closure):
        """Run the closure(s) so that ``grad_sample`` holds the (mixed) look-ahead observation."""
        if not self.kf_compute_grad_at_original:
            moved = self._shift(+1.0)
            with torch.enable_grad():
                loss = closure()
            if moved:
                self._shift(-1.0)
            return loss
        with torch.enable_grad():
            loss = closure()
        if not any("kf_d_t" in self.state[p] for p in self.params if p in self.state):
            return loss                                   # first step: nothing to look ahead along
        here = self._take_grad_samples()
        c = self.scaling_factor
        self._shift(+1.0)
        with torch.enable_grad():
            loss = closure()
        self._shift(-1.0)
        for p, g0 in zip(self.params, here):
            g1 = getattr(p, "grad_sample", None)
            if g0 is None or g1 is None:
                continue
            if isinstance(g1, list):
                g1 = g1[-1]
            if isinstance(g0, list):
                g0 = g0[-1]
            p.grad_sample = g1.mul(c).add_(g0, alpha=1.0 - c)
        return loss

    def step(self, closure: Optional[Callable[[], float]] = None) -> Optional[float]:
        if closure is None:
            raise ValueError("Kalman-filtered optimizers need step(closure): the gradient is taken at a shifted point")
        loss = self._observe(closure)
        if not self.pre_step():
            return loss
        before = {}
        for p in self.params:
            st = self.state[p]
            g = p.grad
            if "kf_m_t" not in st:
                st["kf_m_t"] = g.detach().clone()
            else:
                st["kf_m_t"].lerp_(g, weight=1.0 - self.kappa)
            p.grad = st["kf_m_t"].clone()
            before[p] = p.data.clone()
        self.original_optimizer.step()
        for p in self.params:
            # the wrapped optimizer may have (re)created its own state dict entry for p
            self.state[p]["kf_d_t"] = p.data - before[p]
        return loss


class KF_DPOptimizer(KalmanFilterMixin, DPOptimizer):
    pass


class KF_DPOptimizerFastGradientClipping(KalmanFilterMixin, DPOptimizerFastGradientClipping):
    pass


class KF_DistributedDPOptimizer(KalmanFilterMixin, DistributedDPOptimizer):
    pass


class KF_DistributedDPOptimizerFastGradientClipping(KalmanFilterMixin, DistributedDPOptimizerFastGradientClipping):
    pass


class KF_DPPerLayerOptimizer(KalmanFilterMixin, DPPerLayerOptimizer):
    pass


class KF_DistributedPerLayerOptimizer(KalmanFilterMixin, DistributedPerLayerOptimizer):
    pass


class KF_SimpleDistributedPerLayerOptimizer(KalmanFilterMixin, SimpleDistributedPerLayerOptimizer):
    pass


class KF_AdaClipDPOptimizer(KalmanFilterMixin, AdaClipDPOptimizer):
    pass


_KF = {
    DPOptimizer: KF_DPOptimizer,
    DPOptimizerFastGradientClipping: KF_DPOptimizerFastGradientClipping,
    DistributedDPOptimizer: KF_DistributedDPOptimizer,
    DistributedDPOptimizerFastGradientClipping: KF_DistributedDPOptimizerFastGradientClipping,
    DPPerLayerOptimizer: KF_DPPerLayerOptimizer,
    DistributedPerLayerOptimizer: KF_DistributedPerLayerOptimizer,
    SimpleDistributedPerLayerOptimizer: KF_SimpleDistributedPerLayerOptimizer,
    AdaClipDPOptimizer: KF_AdaClipDPOptimizer,
}


def get_optimizer_class(clipping: str, distributed: bool, grad_sample_mode: str = None, kalman: bool = False):
    """The (Kalman-filtered, if ``kalman``) optimizer class for a clipping / distribution / mode combination."""
    base = _plain_optimizer_class(clipping=clipping, distributed=distributed, grad_sample_mode=grad_sample_mode)
    if not kalman:
        return base
    if base not in _KF:
        raise ValueError(f"no Kalman-filtered variant of {base.__name__}")
    return _KF[base]
