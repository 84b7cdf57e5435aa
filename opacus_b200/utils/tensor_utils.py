"""Tensor helpers: per-sample norms and im2col ("unfold") for 2-d and 3-d
convolutions with stride, dilation and ``"same"``/``"valid"`` padding.

Behavioural parity: ``opacus/utils/tensor_utils.py:27-336``.  The unfolds here
build sliding windows with ``Tensor.unfold`` along each spatial axis (views) and
materialise once, so one routine serves any number of spatial axes.
"""
from typing import Iterator, List, Sequence, Tuple, Union

import torch
import torch.nn.functional as F


def calc_sample_norms(named_params: Iterator[Tuple[str, torch.Tensor]], *, flat: bool = True) -> List[torch.Tensor]:
    """Per-sample L2 norms of a set of ``[B, ...]`` tensors; ``flat`` combines
    them into one norm per sample."""
    norms = [calc_sample_norms_one_layer(t) for _, t in named_params]
    if flat:
        norms = [torch.stack(norms, dim=0).norm(2, dim=0)]
    return norms


def calc_sample_norms_one_layer(param: torch.Tensor) -> torch.Tensor:
    return param.reshape(len(param), -1).norm(2, dim=-1)


def sum_over_all_but_batch_and_last_n(tensor: torch.Tensor, n_dims: int) -> torch.Tensor:
    """Sum every axis except the first and the trailing ``n_dims``."""
    middle = tensor.dim() - n_dims - 1
    if middle == 0:
        return tensor
    return tensor.sum(dim=list(range(1, 1 + middle)))


def _tuple(v, n):
    return (v,) * n if isinstance(v, int) else tuple(v)


def _pads(padding, kernel, dilation) -> List[Tuple[int, int]]:
    """(left, right) padding per spatial axis."""
    n = len(kernel)
    if padding == "valid":
        return [(0, 0)] * n
    if padding == "same":
        out = []
        for k, d in zip(kernel, dilation):
            total = d * (k - 1)
            out.append((total // 2, total - total // 2))
        return out
    return [(p, p) for p in _tuple(padding, n)]


def unfold_nd(x: torch.Tensor, *, kernel_size: Sequence[int], padding, stride: Sequence[int],
              dilation: Sequence[int], positions_first: bool = False) -> torch.Tensor:
    """im2col for ``x`` of shape ``[B, C, *spatial]``.

    Returns ``[B, C * prod(kernel), L]`` with ``L`` the number of output
    positions; rows are ordered channel-major then kernel taps (row-major),
    the layout of ``torch.nn.functional.unfold``.  ``positions_first`` returns
    the transpose ``[B, L, C * prod(kernel)]`` (the layout the batched
    tensor-core GEMM wants: contraction index outermost) at no extra cost.
    """
    n = len(kernel_size)
    kernel_size, stride, dilation = _tuple(kernel_size, n), _tuple(stride, n), _tuple(dilation, n)
    pads = _pads(padding, kernel_size, dilation)
    flat_pad = [v for lr in reversed(pads) for v in lr]
    x = F.pad(x, flat_pad)
    B, C = x.shape[:2]
    k_total = 1
    for k in kernel_size:
        k_total *= k
    spans = [dilation[a] * (kernel_size[a] - 1) + 1 for a in range(n)]
    if any(x.shape[2 + a] < spans[a] for a in range(n)):
        return x.new_zeros(B, 0, C * k_total) if positions_first else x.new_zeros(B, C * k_total, 0)
    # Sliding windows as strided views (no copy): axis a keeps the output positions,
    # a new trailing axis holds the (dilated) window, thinned to the kernel taps.
    for a in range(n):
        x = x.unfold(2 + a, spans[a], stride[a])
    for a in range(n):
        if dilation[a] > 1:
            x = x.narrow(2 + n + a, 0, spans[a])[(slice(None),) * (2 + n + a) + (slice(None, None, dilation[a]),)]
    # [B, C, o0, o1, ..., k0, k1, ...] -> [B, C, k0, k1, ..., o0, o1, ...]; the reshape is the one copy
    if positions_first:
        order = [0] + [2 + a for a in range(n)] + [1] + [2 + n + a for a in range(n)]
        return x.permute(order).reshape(B, -1, C * k_total)
    order = [0, 1] + [2 + n + a for a in range(n)] + [2 + a for a in range(n)]
    return x.permute(order).reshape(B, C * k_total, -1)


def unfold2d(input, *, kernel_size: Tuple[int, int], padding: Union[str, Tuple[int, int]],
             stride: Tuple[int, int], dilation: Tuple[int, int]):
    """``[B, C, H, W] -> [B, C*kh*kw, H_out*W_out]``."""
    return unfold_nd(input, kernel_size=kernel_size, padding=padding, stride=stride, dilation=dilation)


def unfold3d(tensor: torch.Tensor, *, kernel_size, padding=0, stride=1, dilation=1):
    """``[B, C, D, H, W] -> [B, C*kd*kh*kw, D_out*H_out*W_out]``."""
    if tensor.dim() != 5:
        raise ValueError(f"Input tensor must be of the shape [B, C, D, H, W]. Got{tensor.shape}")
    return unfold_nd(
        tensor, kernel_size=_tuple(kernel_size, 3), padding=padding,
        stride=_tuple(stride, 3), dilation=_tuple(dilation, 3),
    )


def filter_dilated_rows(tensor: torch.Tensor, dilation: Tuple[int, ...], dilated_kernel_size: Tuple[int, ...],
                        kernel_size: Tuple[int, ...]):
    """Keep every ``dilation``-th entry along the trailing kernel axes of a
    tensor that was unfolded with a dense (dilated-extent) window."""
    rank = len(kernel_size)
    first = tensor.dim() - rank
    for a in range(rank):
        keep = torch.arange(0, dilated_kernel_size[a], dilation[a], device=tensor.device)
        tensor = tensor.index_select(first + a, keep)
    return tensor
