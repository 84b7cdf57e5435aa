"""Composition of discretised PRVs: FFT powers for repeated mechanisms, then a
pairwise convolution tree (``opacus/accountants/analysis/prv/compose.py:24-76``)."""
from typing import List

import numpy as np
from scipy.fft import irfft, rfft
from scipy.signal import convolve

from .prvs import DiscretePRV


def _compose_fourier(dprv: DiscretePRV, num_self_composition: int) -> DiscretePRV:
    """``num_self_composition``-fold self-convolution by raising the spectrum
    to that power; the circular result is rolled back so that index ``i`` keeps
    its meaning on the (shifted) grid."""
    n = len(dprv)
    if n % 2:
        raise ValueError("Can only compose evenly sized discrete PRVs")
    pmf = irfft(rfft(dprv.pmf) ** num_self_composition)
    roll = num_self_composition - 1
    if num_self_composition % 2 == 0:
        roll += len(pmf) // 2
    grid = dprv.domain.shift_right(dprv.domain.shifts * (num_self_composition - 1))
    return DiscretePRV(pmf=np.roll(pmf, roll), domain=grid)


def _compose_two(a: DiscretePRV, b: DiscretePRV) -> DiscretePRV:
    return DiscretePRV(
        pmf=convolve(a.pmf, b.pmf, mode="same"),
        domain=a.domain.shift_right(b.domain.shifts),
    )


def _compose_convolution_tree(dprvs: List[DiscretePRV]) -> DiscretePRV:
    level = list(dprvs)
    while len(level) > 1:
        nxt = [level.pop()] if len(level) % 2 else []
        nxt.extend(_compose_two(level[k], level[k + 1]) for k in range(0, len(level), 2))
        level = nxt
    return level[0]


def compose_heterogeneous(dprvs: List[DiscretePRV], num_self_compositions: List[int]) -> DiscretePRV:
    if len(dprvs) != len(num_self_compositions):
        raise ValueError("dprvs and num_self_compositions must have the same length")
    return _compose_convolution_tree(
        [_compose_fourier(d, k) for d, k in zip(dprvs, num_self_compositions)]
    )
