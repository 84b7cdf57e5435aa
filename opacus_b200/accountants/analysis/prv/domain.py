"""Uniform grid on which privacy-loss random variables are discretised, and the
rule for how wide it must be (``opacus/accountants/analysis/prv/domain.py:23-114``)."""
from dataclasses import dataclass
from typing import Sequence

import numpy as np


@dataclass
class Domain:
    """``size`` equally spaced points on ``[t_min, t_max]``; ``shifts`` records
    how far the grid has been translated from its aligned position."""

    t_min: float
    t_max: float
    size: int
    shifts: float = 0.0

    def __post_init__(self):
        if not isinstance(self.size, int):
            raise TypeError("`size` must be an integer")
        if self.size % 2:
            raise ValueError("`size` must be even")

    @classmethod
    def create_aligned(cls, t_min: float, t_max: float, dt: float) -> "Domain":
        """Grid whose end points are integer multiples of ``dt`` and whose
        size is even (needed by the FFT self-composition)."""
        lo = np.floor(t_min / dt) * dt
        hi = np.ceil(t_max / dt) * dt
        n = int(np.round((hi - lo) / dt)) + 1
        if n % 2:
            n, hi = n + 1, hi + dt
        grid = cls(lo, hi, n)
        if abs(grid.dt - dt) / dt >= 1e-8:
            raise RuntimeError
        return grid

    def shift_right(self, dt: float) -> "Domain":
        return Domain(self.t_min + dt, self.t_max + dt, self.size, self.shifts + dt)

    @property
    def dt(self):
        return (self.t_max - self.t_min) / (self.size - 1)

    @property
    def ts(self):
        return np.linspace(self.t_min, self.t_max, self.size)

    def __getitem__(self, i: int) -> float:
        return self.t_min + i * self.dt


def compute_safe_domain_size(prvs, max_self_compositions: Sequence[int], eps_error: float,
                             delta_error: float) -> float:
    """Half-width ``L`` of the truncation interval (Gopi et al., remark 5.6),
    bounded through RDP tail bounds of the whole composition and of each single
    mechanism."""
    from ...rdp import RDPAccountant

    n_total = sum(max_self_compositions)
    whole = RDPAccountant()
    whole.history = [(p.noise_multiplier, p.sample_rate, n) for p, n in zip(prvs, max_self_compositions)]
    width = whole.get_epsilon(delta_error / 4)
    for p in prvs:
        single = RDPAccountant()
        single.history = [(p.noise_multiplier, p.sample_rate, 1)]
        width = max(width, single.get_epsilon(delta=delta_error / (8 * n_total)))
    return max(width, eps_error) + 3
