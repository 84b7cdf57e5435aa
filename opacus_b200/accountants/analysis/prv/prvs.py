"""Privacy-loss random variable of the Poisson-subsampled Gaussian mechanism,
its truncation and its discretisation (Gopi et al. 2021, propositions B1/B4).

Behavioural parity: ``opacus/accountants/analysis/prv/prvs.py:30-198``.
"""
from dataclasses import dataclass
from typing import Tuple

import numpy as np
from scipy import integrate
from scipy.special import erfc

from ..rdp import _compute_rdp
from .domain import Domain

_SQRT2 = np.sqrt(2)


class PoissonSubsampledGaussianPRV:
    def __init__(self, sample_rate: float, noise_multiplier: float) -> None:
        self.sample_rate = sample_rate
        self.noise_multiplier = noise_multiplier

    def pdf(self, t):
        q, s = self.sample_rate, self.noise_multiplier
        with np.errstate(all="ignore"):
            u = np.exp(t) + q - 1  # positive exactly on the support t > log(1-q)
            z = np.log(u / q)
            dens = (
                s * np.exp(-(s**2) * z**2 / 2 - 1 / (8 * s**2) + 2 * t)
                / (_SQRT2 * np.sqrt(np.pi) * u * (u / q) ** 0.5)
            )
        return np.where(t > np.log(1 - q), dens, 0.0)

    def cdf(self, t):
        q, s = self.sample_rate, self.noise_multiplier
        inside = t > np.log(1 - q)
        z = np.log(np.where(inside, (np.exp(t) + q - 1) / q, 1))
        val = (
            1.0
            - q * erfc((2 * z * s**2 - 1) / (2 * _SQRT2 * s)) / 2
            - (1 - q) * erfc((2 * z * s**2 + 1) / (2 * _SQRT2 * s)) / 2
        )
        return np.where(inside, val, 0.0)

    def rdp(self, alpha: float) -> float:
        return _compute_rdp(self.sample_rate, self.noise_multiplier, alpha)


class TruncatedPrivacyRandomVariable:
    """``prv`` conditioned on ``[t_min, t_max)``; works for any object with
    ``pdf``/``cdf``."""

    def __init__(self, prv, t_min: float, t_max: float) -> None:
        self._prv = prv
        self.t_min = t_min
        self.t_max = t_max
        self._remaining_mass = prv.cdf(t_max) - prv.cdf(t_min)

    def pdf(self, t):
        inner = np.where(t < self.t_max, self._prv.pdf(t) / self._remaining_mass, 0.0)
        return np.where(t < self.t_min, 0.0, inner)

    def cdf(self, t):
        inner = np.where(
            t < self.t_max, (self._prv.cdf(t) - self._prv.cdf(self.t_min)) / self._remaining_mass, 1.0
        )
        return np.where(t < self.t_min, 0.0, inner)

    def mean(self) -> float:
        """E[t] by parts, ``[t F]_a^b - int F``, over log-spaced sub-intervals
        so that the mass concentrated near zero is resolved."""
        e_lo = int(np.log10(np.abs(self.t_min)))
        e_hi = int(np.log10(self.t_max))
        knots = np.concatenate(
            [
                [self.t_min],
                -np.logspace(start=e_lo, stop=-5, num=10),
                [0],
                np.logspace(start=-5, stop=e_hi, num=10),
                [self.t_max],
            ]
        )
        total = 0.0
        for a, b in zip(knots[:-1], knots[1:]):
            area, _ = integrate.quad(self.cdf, a, b, limit=500)
            total += b * self.cdf(b) - a * self.cdf(a) - area
        return total


@dataclass
class DiscretePRV:
    pmf: np.ndarray
    domain: Domain

    def __len__(self) -> int:
        if len(self.pmf) != self.domain.size:
            raise ValueError("pmf and domain must have the same length")
        return len(self.pmf)

    def compute_epsilon(self, delta: float, delta_error: float, eps_error: float) -> Tuple[float, float, float]:
        """(lower, estimate, upper) epsilon at ``delta`` from the tail sums
        ``d1 = P[T >= t]`` and ``d2 = E[exp(-T); T >= t]``."""
        if delta <= 0:
            return (float("inf"),) * 3
        if np.finfo(np.longdouble).eps * self.domain.size > delta - delta_error:
            raise ValueError(
                "Floating point errors will dominate for such small values of delta. "
                "Increase delta or reduce domain size."
            )
        t = self.domain.ts
        tail_p = np.cumsum(self.pmf[::-1])[::-1]
        tail_pe = np.cumsum((self.pmf * np.exp(-t))[::-1])[::-1]
        neg_delta = np.exp(t) * tail_pe - tail_p

        def solve(target):
            k = np.searchsorted(neg_delta, -target, side="left")
            if k <= 0:
                raise RuntimeError("Cannot compute epsilon")
            return np.log((tail_p[k] - target) / tail_pe[k])

        return (
            solve(delta + delta_error) - eps_error,
            solve(delta),
            solve(delta - delta_error) + eps_error,
        )

    def compute_delta_estimate(self, eps: float) -> float:
        t = self.domain.ts
        return np.where(t >= eps, self.pmf * (1.0 - np.exp(eps) * np.exp(-t)), 0.0).sum()


def discretize(prv, domain: Domain) -> DiscretePRV:
    """Bin ``prv`` on ``domain`` (cell mass from the cdf), then translate the
    grid so the discrete mean equals the continuous one."""
    centres = domain.ts
    half = domain.dt / 2
    pmf = prv.cdf(centres + half) - prv.cdf(centres - half)
    shift = prv.mean() - np.dot(domain.ts, pmf)
    if np.abs(shift) >= half:
        raise RuntimeError("Discrete mean differs significantly from continuous mean.")
    return DiscretePRV(pmf=pmf, domain=domain.shift_right(shift))
