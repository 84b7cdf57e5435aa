"""Importing this package registers the built-in validators and fixers."""
from . import batch_norm, gru, instance_norm, lstm, multihead_attention, rnn  # noqa: F401  (registration)
from .module_validator import ModuleValidator
from .utils import register_module_fixer, register_module_validator

__all__ = ["ModuleValidator", "register_module_validator", "register_module_fixer"]
