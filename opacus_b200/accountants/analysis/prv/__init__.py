from .compose import compose_heterogeneous
from .domain import Domain, compute_safe_domain_size
from .prvs import (
    DiscretePRV,
    PoissonSubsampledGaussianPRV,
    TruncatedPrivacyRandomVariable,
    discretize,
)

__all__ = [
    "DiscretePRV",
    "Domain",
    "PoissonSubsampledGaussianPRV",
    "TruncatedPrivacyRandomVariable",
    "compose_heterogeneous",
    "compute_safe_domain_size",
    "discretize",
]
