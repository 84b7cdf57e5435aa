"""Model checks and automatic repairs for DP training.

``VALIDATORS`` and ``FIXERS`` map a module *type* to a function; they are
filled by the decorators in :mod:`.utils`.

Behavioural parity: ``opacus/validators/module_validator.py:30-167``.
"""
import logging
from typing import List

import torch.nn as nn

from ..utils.module_utils import clone_module, get_submodule, trainable_modules
from .errors import IllegalModuleConfigurationError, UnsupportedModuleError

logger = logging.getLogger(__name__)


class ModuleValidator:
    VALIDATORS = {}
    FIXERS = {}

    @classmethod
    def validate(cls, module: nn.Module, *, strict: bool = False) -> List[UnsupportedModuleError]:
        """Collect problems of every trainable submodule; the model must also
        be in training mode.  ``strict`` raises instead of returning."""
        problems: List[UnsupportedModuleError] = []
        if not module.training:
            problems.append(IllegalModuleConfigurationError("Model needs to be in training mode"))
        for _, sub in trainable_modules(module):
            check = cls.VALIDATORS.get(type(sub))
            if check is not None:
                problems.extend(check(sub))
        if strict and problems:
            raise UnsupportedModuleError(problems)
        return problems

    @classmethod
    def is_valid(cls, module: nn.Module) -> bool:
        return not cls.validate(module, strict=False)

    @classmethod
    def fix(cls, module: nn.Module, **kwargs) -> nn.Module:
        """Return a *copy* of ``module`` in which every submodule that has a
        registered fixer is replaced by the fixer's result."""
        module = clone_module(module)
        for name in [n for n, _ in trainable_modules(module)]:
            sub = get_submodule(module, name)
            repair = cls.FIXERS.get(type(sub))
            if repair is None:
                continue
            replacement = repair(sub, **kwargs)
            replacement.to(next(sub.parameters()).device)
            module = cls._replace_sub_module(root=module, sub_module_name=name, new_sub_module=replacement)
            logger.info(f"Replaced sub_module {name} : {sub} with {replacement}")
        return module

    @classmethod
    def _replace_sub_module(cls, *, root: nn.Module, sub_module_name: str, new_sub_module: nn.Module) -> nn.Module:
        if sub_module_name == "":
            return new_sub_module
        *parents, leaf = sub_module_name.split(".")
        node = root
        for p in parents:
            node = node._modules[p]
        node._modules[leaf] = new_sub_module
        return root

    @classmethod
    def fix_and_validate(cls, module: nn.Module, **kwargs) -> nn.Module:
        fixed = cls.fix(module, **kwargs)
        cls.validate(fixed, strict=True)
        return fixed
