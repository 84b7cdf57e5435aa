"""Renyi-DP accountant (``opacus/accountants/rdp.py:21-92``)."""
from typing import List, Optional, Tuple, Union

from .accountant import IAccountant, push_run
from .analysis import rdp as privacy_analysis


class RDPAccountant(IAccountant):
    # 1.1 .. 10.9 in steps of 0.1, then the integers 12 .. 63
    DEFAULT_ALPHAS = [1 + x / 10.0 for x in range(1, 100)] + list(range(12, 64))

    def __init__(self):
        super().__init__()

    def step(self, *, noise_multiplier: float, sample_rate: float):
        push_run(self.history, noise_multiplier, sample_rate)

    def get_privacy_spent(
        self, *, delta: float, alphas: Optional[List[Union[float, int]]] = None
    ) -> Tuple[float, float]:
        if not self.history:
            return 0, 0
        orders = self.DEFAULT_ALPHAS if alphas is None else alphas
        total = 0
        for sigma, q, n in self.history:
            total = total + privacy_analysis.compute_rdp(
                q=q, noise_multiplier=sigma, steps=n, orders=orders
            )
        eps, alpha = privacy_analysis.get_privacy_spent(orders=orders, rdp=total, delta=delta)
        return float(eps), float(alpha)

    def get_epsilon(self, delta: float, alphas=None, **kwargs):
        return self.get_privacy_spent(delta=delta, alphas=alphas)[0]

    def __len__(self):
        return len(self.history)

    @classmethod
    def mechanism(cls) -> str:
        return "rdp"
