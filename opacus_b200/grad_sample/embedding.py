"""Embedding rules: dense per-sample gradient, ghost norm as a masked Gram
product (no sort/unique), clipped sum as a weighted scatter-add
(``opacus/grad_sample/embedding.py:25-115``,
``opacus/grad_sample/embedding_norm_sample.py:27-151``)."""
from typing import Dict, List

import torch
import torch.nn as nn

from .. import ops
from .utils import register_grad_sampler, register_norm_sampler, register_norm_sq_sampler, register_wgrad_sampler


@register_grad_sampler(nn.Embedding)
def compute_embedding_grad_sample(layer: nn.Embedding, activations, backprops) -> Dict[nn.Parameter, torch.Tensor]:
    if not layer.weight.requires_grad:
        return {}
    ids = activations[0]
    if ids.shape[0] == 0:
        return {layer.weight: torch.zeros_like(layer.weight).unsqueeze(0)}
    return {layer.weight: ops.embedding_grad_sample(ids, backprops, layer.num_embeddings)}


@register_grad_sampler(nn.EmbeddingBag)
def compute_embeddingbag_gradsampler(layer, inputs, backprops):
    """Bags are given as (flat indices, offsets); modes ``sum`` and ``mean``."""
    index, offset = inputs[0], inputs[1]
    B = offset.shape[0]
    V, D = layer.num_embeddings, layer.embedding_dim
    ends = torch.cat([offset[1:], offset.new_tensor([index.shape[0]])])
    lengths = ends - offset
    bag_of = torch.repeat_interleave(torch.arange(B, device=index.device), lengths)
    rows = backprops[bag_of]
    if layer.mode == "mean":
        rows = rows / lengths[bag_of].unsqueeze(-1).to(rows.dtype)
    elif layer.mode != "sum":
        raise NotImplementedError(f"EmbeddingBag mode {layer.mode}")
    out = torch.zeros(B * V, D, device=index.device, dtype=backprops.dtype)
    out.index_add_(0, bag_of * V + index, rows)
    return {layer.weight: out.view(B, V, D)}


@register_norm_sq_sampler(nn.Embedding)
def compute_embedding_norm_sq(layer, activations, backprops, g_scale: float = 1.0, total=None):
    if not layer.weight.requires_grad:
        return {}
    if total is not None:
        ops.embedding_norm_sq(activations[0], backprops, g_scale, total=total)
        return {}
    return {layer.weight: ops.embedding_norm_sq(activations[0], backprops, g_scale)}


@register_norm_sampler(nn.Embedding)
def compute_embedding_norm_sample(layer: nn.Embedding, activations: List[torch.Tensor],
                                  backprops: torch.Tensor) -> Dict[nn.Parameter, torch.Tensor]:
    return {p: v.sqrt().to(backprops.dtype)
            for p, v in compute_embedding_norm_sq(layer, activations, backprops).items()}


@register_wgrad_sampler(nn.Embedding)
def compute_embedding_weighted_grad(layer, activations, backprops, coef, g_scale: float = 1.0):
    if not layer.weight.requires_grad:
        return {}
    dst = getattr(layer.weight, "_dp_grad_out", None)
    fresh = getattr(layer.weight, "_dp_grad_fresh", True)
    grad = ops.embedding_weighted_grad(
        activations[0], backprops, coef, layer.num_embeddings, g_scale,
        out_dtype=layer.weight.dtype if dst is None else None, out=dst, accumulate=not fresh)
    if dst is not None:
        layer.weight._dp_grad_fresh = False
    return {layer.weight: grad}
