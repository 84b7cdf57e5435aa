"""Decorators that fill the validator/fixer tables (``opacus/validators/utils.py:24-83``)."""
from typing import Sequence, Union

from .module_validator import ModuleValidator

DEFAULT_MODULE_VALIDATOR = ModuleValidator


def _as_list(x):
    return list(x) if isinstance(x, Sequence) else [x]


def register_module_validator(target_class_or_classes: Union[type, Sequence[type]],
                              validator_class: type = DEFAULT_MODULE_VALIDATOR):
    """``@register_module_validator(nn.Foo)`` on ``f(module) -> List[error]``."""

    def decorator(f):
        for t in _as_list(target_class_or_classes):
            validator_class.VALIDATORS[t] = f
        return f

    return decorator


def register_module_fixer(target_class_or_classes: Union[type, Sequence[type]],
                          validator_class: type = DEFAULT_MODULE_VALIDATOR):
    """``@register_module_fixer(nn.Foo)`` on ``f(module, **kwargs) -> nn.Module``."""

    def decorator(f):
        for t in _as_list(target_class_or_classes):
            validator_class.FIXERS[t] = f
        return f

    return decorator
