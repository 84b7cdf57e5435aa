"""Privacy accountants (pure CPU numpy/scipy): RDP, Gaussian-DP and PRV."""
from .accountant import IAccountant
from .gdp import GaussianAccountant
from .prv import PRVAccountant
from .rdp import RDPAccountant
from .registry import create_accountant, register_accountant

__all__ = [
    "IAccountant",
    "GaussianAccountant",
    "RDPAccountant",
    "PRVAccountant",
    "register_accountant",
    "create_accountant",
]
