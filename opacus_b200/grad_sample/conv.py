"""Conv1d/2d/3d rules.

Per-sample gradient: ``gs[n] = G[n] unfold(x[n])^T`` with the contraction over
output positions; groups are handled block by block (no off-diagonal blocks are
ever formed).  The clipped sum is an ordinary convolution weight gradient with
``G`` scaled per sample.

Behavioural parity: ``opacus/grad_sample/conv.py:28-119``.
"""
from typing import Dict, List, Union

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..utils.tensor_utils import unfold_nd
from .utils import register_grad_sampler, register_norm_sq_sampler, register_wgrad_sampler

_CONVS = [nn.Conv1d, nn.Conv2d, nn.Conv3d]


def _base_type(layer):
    """FSDP2 renames a wrapped ``Conv2d`` to ``FSDPConv2d(FSDPModule, Conv2d)``."""
    for cls in type(layer).__mro__:
        if cls in _CONVS:
            return cls
    return type(layer)


@register_grad_sampler(_CONVS)
def compute_conv_grad_sample(layer: Union[nn.Conv1d, nn.Conv2d, nn.Conv3d], activations: List[torch.Tensor],
                             backprops: torch.Tensor) -> Dict[nn.Parameter, torch.Tensor]:
    x = activations[0].to(backprops.dtype)
    n = x.shape[0]
    want_b = layer.bias is not None and layer.bias.requires_grad
    if n == 0:
        out = {layer.weight: torch.zeros_like(layer.weight).unsqueeze(0)}
        if want_b:
            out[layer.bias] = torch.zeros_like(layer.bias).unsqueeze(0)
        return out
    O = layer.out_channels
    ck = layer.weight[0].numel() * layer.groups
    geom = _implicit_geometry(layer, x, backprops)
    if geom is not None:
        # implicit-unfold tensor-core kernel: no unfolded copy, norm from the accumulators
        from ..ops import _cuda

        out = {}
        if layer.weight.requires_grad:
            out[layer.weight] = (_conv3d_grad_sample(layer, x, backprops, geom) if x.dim() == 5
                                 else _cuda.conv_grad_sample(x, backprops, geom))
        if want_b:
            out[layer.bias] = backprops.reshape(n, O, -1).sum(dim=2)
        return out
    if (x.is_cuda and backprops.dtype == torch.bfloat16 and layer.groups == 1 and O % 8 == 0 and ck % 8 == 0):
        # tensor-core path: both operands with the output positions (the contraction) outermost
        cols_t = unfold_nd(x, kernel_size=layer.kernel_size, padding=layer.padding, stride=layer.stride,
                           dilation=layer.dilation, positions_first=True)            # [n, L, C*k]
        g_t = backprops.reshape(n, O, -1).transpose(1, 2).contiguous()                # [n, L, O]
        out = {}
        if layer.weight.requires_grad:
            from .. import ops

            gs = ops.linear_grad_sample(cols_t, g_t)                                  # [n, O, C*k] + fused norm
            norm = getattr(gs, "_dp_norm_sq", None)
            gs = gs.view((n,) + tuple(layer.weight.shape))
            if norm is not None:
                gs._dp_norm_sq = norm
            out[layer.weight] = gs
        if want_b:
            out[layer.bias] = g_t.sum(dim=1)
        return out
    cols = unfold_nd(x, kernel_size=layer.kernel_size, padding=layer.padding, stride=layer.stride,
                     dilation=layer.dilation)                      # [n, C*k, L]
    L = cols.shape[-1]
    g = backprops.reshape(n, layer.out_channels, L)                # [n, O, L]
    out = {}
    if layer.weight.requires_grad:
        G_ = layer.groups
        k = cols.shape[1] // layer.in_channels
        cols_g = cols.reshape(n * G_, (layer.in_channels // G_) * k, L)
        g_g = g.reshape(n * G_, layer.out_channels // G_, L)
        gs = torch.bmm(g_g, cols_g.transpose(1, 2))                # [n*G, O/G, C/G*k]
        out[layer.weight] = gs.reshape((n,) + tuple(layer.weight.shape))
    if want_b:
        out[layer.bias] = g.sum(dim=2)
    return out


def _implicit_geometry(layer, x, backprops):
    """Geometry tuple when the implicit-unfold CUDA kernel covers this call, else None.  A Conv3d is covered through
    its depth-stacked 2-d form (:func:`depth_stacked_pairs`); its tuple is the plan of those 2-d problems."""
    if not x.is_cuda or backprops.dtype not in (torch.bfloat16, torch.float32):
        return None
    from ..ops import _cuda

    if _base_type(layer) is nn.Conv3d:
        if getattr(layer, "padding_mode", "zeros") != "zeros" or x.dim() != 5:
            return None
        return _cuda.conv_plan2d(layer.kernel_size[1:], layer.stride[1:], (0, 0), layer.dilation[1:], layer.groups,
                                 None, backprops.shape[-1], backprops.dtype == torch.float32)
    return _cuda.conv_geometry(layer, x, backprops)


def _explicit_pads(layer):
    """``[(low, high)]`` zero padding per spatial axis, whatever form ``layer.padding`` has."""
    pad = layer.padding
    if isinstance(pad, str):
        if pad == "valid":
            return [(0, 0)] * len(layer.kernel_size)
        tot = [d * (k - 1) for k, d in zip(layer.kernel_size, layer.dilation)]
        return [(t // 2, t - t // 2) for t in tot]
    return [(int(p), int(p)) for p in pad]


def depth_stacked_pairs(layer: nn.Conv3d, x: torch.Tensor, backprops: torch.Tensor):
    """A Conv3d weight gradient as ``kernel_depth`` Conv2d weight gradients.

    For the kernel's depth offset ``a`` the gradient slice ``grad[:, :, a]`` is
    ``sum_d conv2d_weight(x_pad[:, :, d * stride_d + a * dilation_d], backprops[:, :, d])``.  The sum over output depth
    is folded into the image: the ``D_out`` input slices are laid one under the other (each padded to a height that is
    a multiple of the stride, so that output rows of different slices never mix) and so are the output-gradient
    slices (with zero rows where a slice has fewer output rows than its pitch).  Yields
    ``(a, x2d [B, C, D_out * pitch, W_pad], g2d [B, O, rows, W_out])``; the 2-d problem has the layer's in-plane kernel,
    stride and dilation and no padding.  Values are exact (only zeros are added)."""
    kd, kh, _ = layer.kernel_size
    sd, sh, _ = layer.stride
    dd, dh, _ = layer.dilation
    pads = _explicit_pads(layer)
    xp = F.pad(x, [v for lr in reversed(pads) for v in lr]) if any(v for lr in pads for v in lr) else x
    B, C, _, Hp, Wp = xp.shape
    _, O, Do, Ho, Wo = backprops.shape
    pitch = -(-Hp // sh) * sh
    rows = pitch // sh
    g2 = F.pad(backprops, (0, 0, 0, rows - Ho)) if rows != Ho else backprops
    g2 = g2.reshape(B, O, Do * rows, Wo)
    g2 = g2[:, :, :(Do * pitch - dh * (kh - 1) - 1) // sh + 1]          # what a 2-d convolution of the stack puts out
    for a in range(kd):
        xs = xp[:, :, a * dd: a * dd + (Do - 1) * sd + 1: sd]
        if pitch != Hp:
            xs = F.pad(xs, (0, 0, 0, pitch - Hp))
        yield a, xs.reshape(B, C, Do * pitch, Wp), g2


def _conv3d_grad_sample(layer, x, backprops, plan, want_out=True):
    """Per-sample Conv3d weight gradients (and their squared norms) on the 2-d implicit-unfold kernel."""
    from ..ops import _cuda

    norm = torch.zeros(x.shape[0], dtype=torch.float32, device=x.device)
    slices = []
    for _, x2, g2 in depth_stacked_pairs(layer, x, backprops):
        if want_out:
            gs = _cuda.conv_grad_sample(x2, g2, plan)
            norm += gs._dp_norm_sq
            slices.append(gs)
        else:
            _cuda.conv_grad_sample(x2, g2, plan, want_out=False, norm_total=norm)
    if not want_out:
        return norm
    out = torch.stack(slices, dim=3)                    # [B, O, C/groups, kd, kh, kw]
    out._dp_norm_sq = norm
    return out


def _conv3d_weighted_grad(layer, x, backprops, coef, plan, g_scale):
    from ..ops import _cuda

    return torch.stack([_cuda.conv_weighted_grad(x2, g2, coef, plan, g_scale)
                        for _, x2, g2 in depth_stacked_pairs(layer, x, backprops)], dim=2)


@register_norm_sq_sampler(_CONVS)
def compute_conv_norm_sq(layer, activations, backprops, g_scale: float = 1.0, total=None):
    """Squared per-sample gradient norms of a conv layer.  On the GPU (bf16 or fp32 data, up to 8
    groups; 3-d layers through their depth-stacked 2-d form) the per-sample gradient tiles are formed in tensor
    memory and squared there, never written; otherwise the gradients are instantiated
    (``opacus/grad_sample/grad_sample_module_fast_gradient_clipping.py:226-250``)."""
    x = activations[0]
    n = x.shape[0]
    want_w = layer.weight.requires_grad
    want_b = layer.bias is not None and layer.bias.requires_grad
    out = {}
    geom = _implicit_geometry(layer, x, backprops) if n else None
    if geom is not None:
        from ..ops import _cuda

        if want_w:
            n2 = (_conv3d_grad_sample(layer, x.to(backprops.dtype), backprops, geom, want_out=False) if x.dim() == 5
                  else _cuda.conv_grad_sample(x, backprops, geom, want_out=False))
            out[layer.weight] = n2 * (g_scale * g_scale)
        if want_b:
            out[layer.bias] = (backprops.reshape(n, layer.out_channels, -1).sum(dim=2).float() * g_scale).square().sum(dim=1)
    else:
        from .. import ops

        scaled = backprops * g_scale if g_scale != 1.0 else backprops
        for p, gs in compute_conv_grad_sample(layer, activations, scaled).items():
            out[p] = ops.grad_sample_norm_sq(gs)
    if total is not None:
        for v in out.values():
            total.add_(v.to(total.dtype))
        return {}
    return out


@register_wgrad_sampler(_CONVS)
def compute_conv_weighted_grad(layer, activations, backprops, coef, g_scale: float = 1.0):
    x = activations[0]
    geom = _implicit_geometry(layer, x, backprops) if x.shape[0] else None
    if geom is not None:
        from ..ops import _cuda

        out = {}
        if layer.weight.requires_grad:
            out[layer.weight] = (_conv3d_weighted_grad(layer, x.to(backprops.dtype), backprops, coef, geom, g_scale)
                                 if x.dim() == 5 else _cuda.conv_weighted_grad(x, backprops, coef, geom, g_scale))
        if layer.bias is not None and layer.bias.requires_grad:
            per = backprops.reshape(backprops.shape[0], backprops.shape[1], -1).sum(dim=2).float()
            out[layer.bias] = (per * (coef.float() * g_scale)[:, None]).sum(dim=0)
        return out
    shape = (-1,) + (1,) * (backprops.dim() - 1)
    gw = backprops * (coef.to(backprops.dtype) * g_scale).reshape(shape)
    out = {}
    if layer.weight.requires_grad:
        pad = layer.padding
        if isinstance(pad, str):
            # explicit symmetric/asymmetric padding, then a "valid" weight gradient
            nsp = x.dim() - 2
            if pad == "same":
                pads = []
                for k_, d_ in zip(layer.kernel_size, layer.dilation):
                    tot = d_ * (k_ - 1)
                    pads.append((tot // 2, tot - tot // 2))
                x = F.pad(x, [v for lr in reversed(pads) for v in lr])
            pad = (0,) * nsp
        fn = {nn.Conv1d: torch.nn.grad.conv1d_weight, nn.Conv2d: torch.nn.grad.conv2d_weight,
              nn.Conv3d: torch.nn.grad.conv3d_weight}[_base_type(layer)]
        out[layer.weight] = fn(x.to(gw.dtype), layer.weight.shape, gw, stride=layer.stride, padding=pad,
                               dilation=layer.dilation, groups=layer.groups)
    if layer.bias is not None and layer.bias.requires_grad:
        out[layer.bias] = gw.reshape(gw.shape[0], gw.shape[1], -1).sum(dim=(0, 2))
    return out


def convolution2d_backward_as_a_convolution(layer: nn.Conv2d, activations: List[torch.Tensor],
                                            backprops: torch.Tensor) -> Dict[nn.Parameter, torch.Tensor]:
    """Alternative Conv2d rule without im2col: the per-sample weight gradient is
    itself a correlation of the input with the output gradient in which the
    roles of stride and dilation are exchanged.  Input channels become the
    batch axis and ``(sample, group)`` pairs become convolution groups, so one
    grouped ``conv2d`` yields every sample's gradient
    (``opacus/grad_sample/conv.py:122-191``)."""
    x = activations[0]
    B, C, H, W = x.shape
    O = backprops.shape[1]
    G_ = layer.groups
    xin = x.reshape(B * G_, C // G_, H, W).transpose(0, 1)             # [C/G, B*G, H, W]
    ker = backprops.reshape(B * O, 1, backprops.shape[2], backprops.shape[3])
    res = F.conv2d(xin, ker, None, stride=layer.dilation, padding=layer.padding, dilation=layer.stride,
                   groups=B * G_)                                       # [C/G, B*O, kh+, kw+]
    kh, kw = layer.weight.shape[2], layer.weight.shape[3]
    res = res[:, :, :kh, :kw].reshape(C // G_, B, O, kh, kw).permute(1, 2, 0, 3, 4)
    out = {layer.weight: res}
    if layer.bias is not None:
        out[layer.bias] = backprops.sum(dim=(-1, -2))
    return out
