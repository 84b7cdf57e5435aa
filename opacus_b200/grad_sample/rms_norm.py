"""RMSNorm (``opacus/grad_sample/rms_norm.py:27-48``)."""
from typing import Dict, List

import torch
import torch.nn as nn

from .. import ops
from ..layers.add_rms_norm import AddRMSNorm
from .utils import register_grad_sampler


@register_grad_sampler([nn.RMSNorm, AddRMSNorm])
def compute_rms_norm_grad_sample(layer: nn.RMSNorm, activations: List[torch.Tensor],
                                 backprops: torch.Tensor) -> Dict[nn.Parameter, torch.Tensor]:
    if layer.weight is None or not layer.weight.requires_grad:
        return {}
    eps = layer.eps if layer.eps is not None else torch.finfo(activations[0].dtype).eps
    gw, _ = ops.norm_affine_grad_sample(
        "rms", activations[0], backprops, eps=eps, normalized_ndim=len(layer.normalized_shape),
        want_weight=True, want_bias=False)
    return {layer.weight: gw}
