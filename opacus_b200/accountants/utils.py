"""Noise calibration: smallest sigma (to tolerance) that stays within a target
epsilon (``opacus/accountants/utils.py:23-78``)."""
from typing import Optional

from .registry import create_accountant

MAX_SIGMA = 1e6


def get_noise_multiplier(
    *,
    target_epsilon: float,
    target_delta: float,
    sample_rate: float,
    epochs: Optional[int] = None,
    steps: Optional[int] = None,
    accountant: str = "rdp",
    epsilon_tolerance: float = 0.01,
    **kwargs,
) -> float:
    """Bracket by doubling, then bisect.  The returned value is always the
    upper end of the bracket, so the resulting epsilon never exceeds the target."""
    if (steps is None) == (epochs is None):
        raise ValueError(
            "get_noise_multiplier takes as input EITHER a number of steps or a number of epochs"
        )
    if steps is None:
        steps = int(epochs / sample_rate)

    acct = create_accountant(mechanism=accountant)

    def eps_at(sigma: float) -> float:
        acct.history = [(sigma, sample_rate, steps)]
        return acct.get_epsilon(delta=target_delta, **kwargs)

    lo, hi = 0, 10
    eps_hi = float("inf")
    while eps_hi > target_epsilon:
        hi = 2 * hi
        eps_hi = eps_at(hi)
        if hi > MAX_SIGMA:
            raise ValueError("The privacy budget is too low.")

    while target_epsilon - eps_hi > epsilon_tolerance:
        mid = (lo + hi) / 2
        eps_mid = eps_at(mid)
        if eps_mid < target_epsilon:
            hi, eps_hi = mid, eps_mid
        else:
            lo = mid
    return hi
