"""InstanceNorm1d/2d/3d (``opacus/grad_sample/instance_norm.py:25-56``)."""
from typing import Dict, List

import torch
import torch.nn as nn

from .. import ops
from .utils import register_grad_sampler


@register_grad_sampler([nn.InstanceNorm1d, nn.InstanceNorm2d, nn.InstanceNorm3d])
def compute_instance_norm_grad_sample(layer, activations: List[torch.Tensor],
                                      backprops: torch.Tensor) -> Dict[nn.Parameter, torch.Tensor]:
    if layer.weight is None:
        return {}
    want_w = layer.weight.requires_grad
    want_b = layer.bias is not None and layer.bias.requires_grad
    gw, gb = ops.norm_affine_grad_sample(
        "instance", activations[0], backprops, eps=layer.eps, want_weight=want_w, want_bias=want_b)
    out = {}
    if want_w:
        out[layer.weight] = gw
    if want_b:
        out[layer.bias] = gb
    return out
