"""LayerNorm: ``grad_w[n] = sum_t xhat[n,t] * g[n,t]``, ``grad_b[n] = sum_t g[n,t]``
with ``xhat`` recomputed inside the kernel (``opacus/grad_sample/layer_norm.py:27-51``)."""
from typing import Dict, List

import torch
import torch.nn as nn

from .. import ops
from .utils import register_grad_sampler


@register_grad_sampler(nn.LayerNorm)
def compute_layer_norm_grad_sample(layer: nn.LayerNorm, activations: List[torch.Tensor],
                                   backprops: torch.Tensor) -> Dict[nn.Parameter, torch.Tensor]:
    if layer.weight is None:
        return {}
    want_w = layer.weight.requires_grad
    want_b = layer.bias is not None and layer.bias.requires_grad
    gw, gb = ops.norm_affine_grad_sample(
        "layer", activations[0], backprops, eps=layer.eps, normalized_ndim=len(layer.normalized_shape),
        want_weight=want_w, want_bias=want_b)
    out = {}
    if want_w:
        out[layer.weight] = gw
    if want_b:
        out[layer.bias] = gb
    return out
