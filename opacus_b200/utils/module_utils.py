"""Small helpers for walking ``nn.Module`` trees.

Behavioural parity: ``opacus/utils/module_utils.py:34-165`` (without the
import-time ``logging.basicConfig`` side effect of the original).
"""
import io
import logging
from typing import Dict, Iterable, Tuple

import torch
import torch.nn as nn

logger = logging.getLogger(__name__)


def _own_params(module: nn.Module):
    return module.parameters(recurse=False)


def has_trainable_params(module: nn.Module) -> bool:
    """True if ``module`` directly owns a parameter that requires grad."""
    return any(p.requires_grad for p in _own_params(module))


def parametrized_modules(module: nn.Module) -> Iterable[Tuple[str, nn.Module]]:
    """``(name, submodule)`` for every submodule that directly owns parameters."""
    for name, m in module.named_modules():
        if any(p is not None for p in _own_params(m)):
            yield name, m


def trainable_modules(module: nn.Module) -> Iterable[Tuple[str, nn.Module]]:
    """``(name, submodule)`` for every submodule that directly owns a trainable parameter."""
    for name, m in parametrized_modules(module):
        if has_trainable_params(m):
            yield name, m


def trainable_parameters(module: nn.Module) -> Iterable[Tuple[str, nn.Parameter]]:
    for name, p in module.named_parameters():
        if p.requires_grad:
            yield name, p


def requires_grad(module: nn.Module, *, recurse: bool = False) -> bool:
    return any(p.requires_grad for p in module.parameters(recurse))


def clone_module(module: nn.Module) -> nn.Module:
    """Independent copy of ``module`` on the same device (serialisation round
    trip, so that custom ``__reduce__``/state hooks are honoured)."""
    buf = io.BytesIO()
    torch.save(module, buf)
    buf.seek(0)
    twin = torch.load(buf, weights_only=False)
    first = next(module.parameters(), None)
    return twin if first is None else twin.to(first.device)


def get_submodule(module: nn.Module, target: str) -> nn.Module:
    """Resolve a dotted path (``""`` is the module itself)."""
    node = module
    if not target:
        return node
    for atom in target.split("."):
        if not hasattr(node, atom):
            raise AttributeError(f"{node._get_name()} has no attribute `{atom}`")
        node = getattr(node, atom)
        if not isinstance(node, nn.Module):
            raise AttributeError(f"`{atom}` is not an nn.Module")
    return node


def are_state_dict_equal(sd1: Dict, sd2: Dict) -> bool:
    if len(sd1) != len(sd2):
        return False
    return all(k in sd2 and torch.allclose(v, sd2[k]) for k, v in sd1.items())
