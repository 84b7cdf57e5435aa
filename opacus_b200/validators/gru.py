"""``nn.GRU`` runs inside one fused library call, so its per-step linear maps are
not visible to the gradient engine; it is replaced by ``DPGRU`` with the same
weights (``opacus/validators/gru.py:25-50``)."""
from typing import List

import torch.nn as nn

from ..layers import DPGRU
from .errors import ShouldReplaceModuleError, UnsupportedModuleError
from .utils import register_module_fixer, register_module_validator


@register_module_validator(nn.GRU)
def validate(module: nn.GRU) -> List[UnsupportedModuleError]:
    return [
        ShouldReplaceModuleError(
            "We do not support nn.GRU because its implementation is a single fused call. DPGRU is a drop-in "
            "replacement compatible with per-sample gradients. Please run the recommended replacement!"
        )
    ]


@register_module_fixer(nn.GRU)
def fix(module: nn.GRU, **kwargs) -> DPGRU:
    twin = DPGRU(
        input_size=module.input_size, hidden_size=module.hidden_size, num_layers=module.num_layers,
        bias=module.bias, batch_first=module.batch_first, dropout=module.dropout,
        bidirectional=module.bidirectional,
    )
    twin.load_state_dict(module.state_dict())
    return twin
