"""``nn.RNN`` -> ``DPRNN`` (same reasoning as for LSTM/GRU; the reference has no
fixer for the plain Elman RNN, this one is an addition)."""
from typing import List

import torch.nn as nn

from ..layers import DPRNN
from .errors import ShouldReplaceModuleError, UnsupportedModuleError
from .utils import register_module_fixer, register_module_validator


@register_module_validator(nn.RNN)
def validate(module: nn.RNN) -> List[UnsupportedModuleError]:
    return [ShouldReplaceModuleError("nn.RNN is a single fused call; use DPRNN (ModuleValidator.fix does it).")]


@register_module_fixer(nn.RNN)
def fix(module: nn.RNN, **kwargs) -> DPRNN:
    twin = DPRNN(
        input_size=module.input_size, hidden_size=module.hidden_size, num_layers=module.num_layers,
        bias=module.bias, batch_first=module.batch_first, dropout=module.dropout,
        bidirectional=module.bidirectional, nonlinearity=module.nonlinearity,
    )
    twin.load_state_dict(module.state_dict())
    return twin
