"""Gaussian-DP (CLT) accountant (``opacus/accountants/gdp.py:21-75``)."""
import warnings

from .accountant import IAccountant
from .analysis import gdp as privacy_analysis


class GaussianAccountant(IAccountant):
    def __init__(self):
        warnings.warn(
            "GDP accounting is experimental and can underestimate privacy expenditure."
            "Proceed with caution. More details: https://arxiv.org/pdf/2106.02848.pdf"
        )
        super().__init__()

    def step(self, *, noise_multiplier: float, sample_rate: float):
        # The CLT bound is only valid for a homogeneous sequence of steps.
        if not self.history:
            self.history = [(noise_multiplier, sample_rate, 1)]
            return
        sigma, q, n = self.history[-1]
        if sigma != noise_multiplier or q != sample_rate:
            raise ValueError(
                "Noise multiplier and sample rate have to stay constant in GaussianAccountant."
            )
        self.history = [(sigma, q, n + 1)]

    def get_epsilon(self, delta: float, poisson: bool = True, **kwargs) -> float:
        sigma, q, n = self.history[-1]
        fn = privacy_analysis.compute_eps_poisson if poisson else privacy_analysis.compute_eps_uniform
        return fn(steps=n, noise_multiplier=sigma, sample_rate=q, delta=delta)

    def __len__(self):
        return len(self.history)

    @classmethod
    def mechanism(cls) -> str:
        return "gdp"
