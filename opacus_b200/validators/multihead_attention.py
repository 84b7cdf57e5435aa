"""``nn.MultiheadAttention`` packs q/k/v into one parameter used through a
functional call; ``DPMultiheadAttention`` holds them in ``nn.Linear`` children
(``opacus/validators/multihead_attention.py:25-51``)."""
from typing import List

import torch.nn as nn

from ..layers import DPMultiheadAttention
from .errors import ShouldReplaceModuleError, UnsupportedModuleError
from .utils import register_module_fixer, register_module_validator


@register_module_validator(nn.MultiheadAttention)
def validate(module: nn.MultiheadAttention) -> List[UnsupportedModuleError]:
    return [
        ShouldReplaceModuleError(
            "We do not support nn.MultiheadAttention because its projections are not nn.Linear modules. "
            "DPMultiheadAttention is a drop-in replacement compatible with per-sample gradients. "
            "Please run the recommended replacement!"
        )
    ]


@register_module_fixer(nn.MultiheadAttention)
def fix(module: nn.MultiheadAttention, **kwargs) -> DPMultiheadAttention:
    twin = DPMultiheadAttention(
        embed_dim=module.embed_dim, num_heads=module.num_heads, dropout=module.dropout,
        bias=module.in_proj_bias is not None, add_bias_kv=module.bias_k is not None,
        add_zero_attn=module.add_zero_attn, kdim=module.kdim, vdim=module.vdim,
        batch_first=module.batch_first,
    )
    twin.load_state_dict(module.state_dict())
    return twin
