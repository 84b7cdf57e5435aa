"""Gaussian differential privacy via the central limit theorem (Dong, Roth, Su;
Bu et al.).  ``mu`` summarises the composition; epsilon follows from the
(epsilon, delta) dual of mu-GDP.

Behavioural parity: ``opacus/accountants/analysis/gdp.py:28-145``.
"""
import numpy as np
from scipy import optimize
from scipy.stats import norm


def compute_mu_uniform(*, steps: int, noise_multiplier: float, sample_rate: float) -> float:
    """mu for fixed-size (uniform, without replacement) subsampling."""
    s = noise_multiplier
    inner = np.exp(s ** (-2)) * norm.cdf(1.5 / s) + 3 * norm.cdf(-0.5 / s) - 2
    return np.sqrt(2) * sample_rate * np.sqrt(steps) * np.sqrt(inner)


def compute_mu_poisson(*, steps: int, noise_multiplier: float, sample_rate: float) -> float:
    """mu for Poisson subsampling."""
    return np.sqrt(np.exp(noise_multiplier ** (-2)) - 1) * np.sqrt(steps) * sample_rate


def delta_eps_mu(*, eps: float, mu: float) -> float:
    """delta(eps) of a mu-GDP mechanism."""
    return norm.cdf(mu / 2 - eps / mu) - np.exp(eps) * norm.cdf(-mu / 2 - eps / mu)


def eps_from_mu(*, mu: float, delta: float) -> float:
    """Invert :func:`delta_eps_mu` for epsilon on the bracket [0, 500]."""
    sol = optimize.root_scalar(
        lambda e: delta_eps_mu(eps=e, mu=mu) - delta, bracket=[0, 500], method="brentq"
    )
    return sol.root


def compute_eps_uniform(*, steps: int, noise_multiplier: float, sample_rate: float, delta: float) -> float:
    mu = compute_mu_uniform(steps=steps, noise_multiplier=noise_multiplier, sample_rate=sample_rate)
    return eps_from_mu(mu=mu, delta=delta)


def compute_eps_poisson(*, steps: int, noise_multiplier: float, sample_rate: float, delta: float) -> float:
    mu = compute_mu_poisson(steps=steps, noise_multiplier=noise_multiplier, sample_rate=sample_rate)
    return eps_from_mu(mu=mu, delta=delta)
