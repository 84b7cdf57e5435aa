"""``SequenceBias`` adds one learned row at the end of the sequence, so its
per-sample gradient is the output gradient of that row
(``opacus/grad_sample/dp_multihead_attention.py:26-41``)."""
from typing import Dict, List

import torch
import torch.nn as nn

from ..layers.dp_multihead_attention import SequenceBias
from .utils import register_grad_sampler


@register_grad_sampler(SequenceBias)
def compute_sequence_bias_grad_sample(layer: SequenceBias, activations: List[torch.Tensor],
                                      backprops: torch.Tensor) -> Dict[nn.Parameter, torch.Tensor]:
    if not layer.bias.requires_grad:
        return {}
    return {layer.bias: backprops[:, -1]}
