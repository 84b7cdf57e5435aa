"""Name -> accountant class table (``opacus/accountants/registry.py:23-67``)."""
from typing import Dict, Type

from .accountant import IAccountant
from .gdp import GaussianAccountant
from .prv import PRVAccountant
from .rdp import RDPAccountant

_ACCOUNTANTS: Dict[str, Type[IAccountant]] = {
    RDPAccountant.mechanism(): RDPAccountant,
    GaussianAccountant.mechanism(): GaussianAccountant,
    PRVAccountant.mechanism(): PRVAccountant,
}


def register_accountant(mechanism: str, accountant: Type[IAccountant], force: bool = False):
    """Make ``accountant`` available under ``mechanism``; refuses to overwrite
    unless ``force``."""
    if not force and mechanism in _ACCOUNTANTS:
        raise ValueError(f"Accountant for mechanism {mechanism} is already registered")
    _ACCOUNTANTS[mechanism] = accountant


def create_accountant(mechanism: str) -> IAccountant:
    try:
        cls = _ACCOUNTANTS[mechanism]
    except KeyError:
        raise ValueError(f"Unexpected accounting mechanism: {mechanism}") from None
    return cls()
