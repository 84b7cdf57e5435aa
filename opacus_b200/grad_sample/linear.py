"""Linear layer rules.

Per-sample gradient ``g^T a`` (``opacus/grad_sample/linear.py:29-51``), ghost
norm ``<a a^T, g g^T>`` (``:54-93``), and the clipped sum ``a^T diag(c) g`` that
replaces the second backward pass
(``opacus/utils/fast_gradient_clipping_utils.py:194-201``)."""
from typing import Dict, List

import torch
import torch.nn as nn

from .. import ops
from .utils import register_grad_sampler, register_norm_sampler, register_norm_sq_sampler, register_wgrad_sampler


def _wants(layer):
    w = layer.weight.requires_grad
    b = layer.bias is not None and layer.bias.requires_grad
    return w, b


@register_grad_sampler(nn.Linear)
def compute_linear_grad_sample(layer: nn.Linear, activations: List[torch.Tensor],
                               backprops: torch.Tensor) -> Dict[nn.Parameter, torch.Tensor]:
    a = activations[0]
    w, b = _wants(layer)
    out = {}
    if w:
        out[layer.weight] = ops.linear_grad_sample(a, backprops)
    if b:
        out[layer.bias] = ops.linear_bias_grad_sample(backprops)
    return out


@register_norm_sq_sampler(nn.Linear)
def compute_linear_norm_sq(layer, activations, backprops, g_scale: float = 1.0, total=None):
    """``total``: running ``[B]`` sum of squared norms; when given and the
    parameters are not shared with another layer, contributions are added to it
    directly and nothing is returned."""
    w, b = _wants(layer)
    if total is not None:
        ops.linear_norm_sq(activations[0], backprops, w, b, g_scale, total=total)
        return {}
    nw, nb = ops.linear_norm_sq(activations[0], backprops, w, b, g_scale)
    out = {}
    if w:
        out[layer.weight] = nw
    if b:
        out[layer.bias] = nb
    return out


@register_norm_sampler(nn.Linear)
def compute_linear_norm_sample(layer: nn.Linear, activations: List[torch.Tensor],
                               backprops: torch.Tensor) -> Dict[nn.Parameter, torch.Tensor]:
    return {p: v.sqrt().to(backprops.dtype) for p, v in compute_linear_norm_sq(layer, activations, backprops).items()}


@register_wgrad_sampler(nn.Linear)
def compute_linear_weighted_grad(layer, activations, backprops, coef, g_scale: float = 1.0):
    w, b = _wants(layer)
    # An engine may designate where the clipped sum of this weight has to go
    # (a slice of its flat gradient buffer); the GEMM then writes there directly.
    dst = getattr(layer.weight, "_dp_grad_out", None) if w else None
    fresh = getattr(layer.weight, "_dp_grad_fresh", True)
    gw, gb = ops.linear_weighted_grad(activations[0], backprops, coef, g_scale, want_bias=b, out=dst,
                                      accumulate=not fresh)
    if dst is not None:
        layer.weight._dp_grad_fresh = False
    out = {}
    if w:
        out[layer.weight] = gw
    if b:
        out[layer.bias] = gb
    return out
