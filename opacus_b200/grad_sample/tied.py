"""Cross terms of the per-sample gradient norm for a parameter shared by two
layers (no counterpart in the reference, which rejects tied parameters under
ghost clipping: ``opacus/grad_sample/grad_sample_module_fast_gradient_clipping.py:172-179``).

For per-sample gradients ``g_1 = G_1^T A_1`` and ``g_2 = G_2^T A_2`` of the same
weight, ``<g_1, g_2> = <A_1 A_2^T, G_1 G_2^T>``: the same contraction as the
ghost norm with two different operand pairs.  For an embedding tied to an
output projection (``W`` used as ``E[ids]`` and as ``h W^T``) the embedding
side is a scatter of ``G_E`` rows, which turns the product into
``sum_{t,s} G_H[s, ids_t] * <A_H[s], G_E[t]>``.
"""
import torch
import torch.nn as nn

from ..layers.dp_rnn import RNNLinear
from .utils import register_cross_norm_sampler


def _bt(x):
    return x.unsqueeze(1) if x.dim() == 2 else x.reshape(x.shape[0], -1, x.shape[-1])


def _linear_linear(p, s1, s2):
    a1, g1, a2, g2 = _bt(s1.inputs[0]), _bt(s1.backprops), _bt(s2.inputs[0]), _bt(s2.backprops)
    b = min(a1.shape[0], a2.shape[0])
    if p is s1.module.weight:
        aa = torch.bmm(a1[:b].to(g1.dtype), a2[:b].to(g1.dtype).transpose(1, 2)).float()
    else:  # shared bias: the activation Gram is all ones
        aa = 1.0
    gg = torch.bmm(g1[:b], g2[:b].transpose(1, 2)).float()
    return (aa * gg).sum(dim=(1, 2)) * (s1.g_scale * s2.g_scale)


for _t1 in (nn.Linear, RNNLinear):
    for _t2 in (nn.Linear, RNNLinear):
        register_cross_norm_sampler(_t1, _t2)(_linear_linear)


@register_cross_norm_sampler(nn.Embedding, nn.Linear)
def _embedding_linear(p, s_emb, s_lin):
    ids = s_emb.inputs[0]
    B = ids.shape[0]
    ids = ids.reshape(B, -1)                                  # [B, T]
    g_e = s_emb.backprops.reshape(B, ids.shape[1], -1)        # [B, T, D]
    a_h, g_h = _bt(s_lin.inputs[0]), _bt(s_lin.backprops)     # [B, S, D], [B, S, V]
    if (g_e.is_cuda and g_e.dtype == torch.bfloat16 and a_h.shape[:2] == g_e.shape[:2] and g_h.shape[:2] == g_e.shape[:2]
            and g_e.shape[2] % 8 == 0 and g_h.dtype in (torch.bfloat16, torch.float32)):
        # one tensor-core kernel: tiles of G_E A_H^T weighted by gathered output-layer gradients, nothing materialised
        from ..ops import _cuda

        return _cuda.load().tied_cross_norm(ids.contiguous(), g_e.contiguous(), a_h.to(torch.bfloat16).contiguous(),
                                            g_h.contiguous(), float(s_emb.g_scale * s_lin.g_scale), None)
    picked = torch.gather(g_h, 2, ids[:, None, :].expand(-1, g_h.shape[1], -1))   # [B, S, T]
    inner = torch.bmm(a_h.to(g_e.dtype), g_e.transpose(1, 2))                     # [B, S, T]
    return (picked.float() * inner.float()).sum(dim=(1, 2)) * (s_emb.g_scale * s_lin.g_scale)
