"""Renyi differential privacy of the sampled Gaussian mechanism (SGM).

For sampling rate ``q``, noise ``sigma`` and order ``alpha`` the RDP is
``log(A_alpha) / (alpha - 1)`` with ``A_alpha`` from Mironov, Talwar, Zhang,
"Renyi Differential Privacy of the Sampled Gaussian Mechanism", section 3.3:
a finite binomial sum for integer orders and a two-sided convergent series with
erfc weights for fractional orders.  All sums are carried in log space.

Conversion to (epsilon, delta) uses Balle et al. 2020, Theorem 21.

Behavioural parity: ``opacus/accountants/analysis/rdp.py:60-335``.

Example
    >>> rdp = compute_rdp(q=0.01, noise_multiplier=1.1, steps=100, orders=[2.0, 8.0, 32.0])
    >>> eps, order = get_privacy_spent(orders=[2.0, 8.0, 32.0], rdp=rdp, delta=1e-5)
    >>> bool(0 < eps < 2)
    True
"""
import math
import warnings
from typing import List, Tuple, Union

import numpy as np
from scipy import special

_NEG_INF = -np.inf


def _log_add(logx: float, logy: float) -> float:
    """log(exp(logx) + exp(logy))."""
    lo, hi = (logx, logy) if logx <= logy else (logy, logx)
    if lo == _NEG_INF:
        return hi
    return hi + math.log1p(math.exp(lo - hi))


def _log_sub(logx: float, logy: float) -> float:
    """log(exp(logx) - exp(logy)); requires logx >= logy."""
    if logx < logy:
        raise ValueError("The result of subtraction must be non-negative.")
    if logy == _NEG_INF:
        return logx
    if logx == logy:
        return _NEG_INF
    try:
        return logy + math.log(math.expm1(logx - logy))
    except OverflowError:
        return logx


def _log_erfc(x: float) -> float:
    """log(erfc(x)), accurate in the far tail."""
    return math.log(2) + special.log_ndtr(-x * math.sqrt(2.0))


def _compute_log_a_for_int_alpha(q: float, sigma: float, alpha: int) -> float:
    """log A_alpha for integer alpha: binomial expansion, one logsumexp."""
    i = np.arange(alpha + 1, dtype=np.float64)
    log_binom = (
        special.gammaln(alpha + 1) - special.gammaln(i + 1) - special.gammaln(alpha - i + 1)
    )
    terms = log_binom + i * math.log(q) + (alpha - i) * math.log1p(-q) + (i * i - i) / (2.0 * sigma**2)
    return float(special.logsumexp(terms))


def _compute_log_a_for_frac_alpha(q: float, sigma: float, alpha: float) -> float:
    """log A_alpha for non-integer alpha.

    The integral is split at ``z0`` (where the two mixture components cross);
    each half is expanded in a generalised binomial series whose coefficients
    alternate in sign once ``i > alpha``.
    """
    z0 = sigma**2 * math.log(1.0 / q - 1.0) + 0.5
    two_s2 = 2.0 * sigma**2
    root2s = math.sqrt(2.0) * sigma
    log_q, log_1mq = math.log(q), math.log(1.0 - q)
    left, right = _NEG_INF, _NEG_INF
    i = 0
    while True:
        coef = special.binom(alpha, i)
        j = alpha - i
        lc = math.log(abs(coef))
        s_left = (
            lc + i * log_q + j * log_1mq + (i * i - i) / two_s2
            + math.log(0.5) + _log_erfc((i - z0) / root2s)
        )
        s_right = (
            lc + j * log_q + i * log_1mq + (j * j - j) / two_s2
            + math.log(0.5) + _log_erfc((z0 - j) / root2s)
        )
        combine = _log_add if coef > 0 else _log_sub
        left = combine(left, s_left)
        right = combine(right, s_right)
        i += 1
        if max(s_left, s_right) < -30:
            break
    return _log_add(left, right)


def _compute_log_a(q: float, sigma: float, alpha: float) -> float:
    if float(alpha).is_integer():
        return _compute_log_a_for_int_alpha(q, sigma, int(alpha))
    return _compute_log_a_for_frac_alpha(q, sigma, alpha)


def _compute_rdp(q: float, sigma: float, alpha: float) -> float:
    """RDP of one SGM step at one order (may be ``inf``)."""
    if q == 0:
        return 0
    if sigma == 0:
        return np.inf
    if q == 1.0:
        return alpha / (2 * sigma**2)
    if np.isinf(alpha):
        return np.inf
    return _compute_log_a(q, sigma, alpha) / (alpha - 1)


def compute_rdp(
    *, q: float, noise_multiplier: float, steps: int, orders: Union[List[float], float]
) -> Union[np.ndarray, float]:
    """RDP of ``steps`` compositions of the SGM at each of ``orders``."""
    if isinstance(orders, float):
        return _compute_rdp(q, noise_multiplier, orders) * steps
    return np.array([_compute_rdp(q, noise_multiplier, a) for a in orders]) * steps


def get_privacy_spent(
    *, orders: Union[List[float], float], rdp: Union[List[float], float], delta: float
) -> Tuple[float, float]:
    """Best ``(epsilon, order)`` over the supplied orders at ``delta``."""
    a = np.atleast_1d(orders).astype(np.float64) if not np.isscalar(orders) else np.atleast_1d(float(orders))
    r = np.atleast_1d(rdp)
    if len(a) != len(r):
        raise ValueError(
            f"Input lists must have the same length.\n\torders_vec = {a}\n\trdp_vec = {r}\n"
        )
    with np.errstate(divide="ignore", invalid="ignore"):
        eps = r - (np.log(delta) + np.log(a)) / (a - 1) + np.log((a - 1) / a)
    if np.isnan(eps).all():
        return np.inf, np.nan
    best = int(np.nanargmin(eps))
    if best in (0, len(eps) - 1):
        which = "smallest" if best == 0 else "largest"
        warnings.warn(
            f"Optimal order is the {which} alpha. Please consider expanding the range of alphas to get a tighter privacy bound."
        )
    return eps[best], a[best]
