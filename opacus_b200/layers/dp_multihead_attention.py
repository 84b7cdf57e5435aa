"""Multi-head attention whose projections are separate ``nn.Linear`` modules
(so per-sample gradients apply), interchangeable with ``nn.MultiheadAttention``
through its ``state_dict``.

The attention core itself is parameter free.  When the caller does not need the
attention weights it runs through ``scaled_dot_product_attention`` (a fused
flash-style kernel on GPU); otherwise the weights are formed explicitly.

Behavioural parity: ``opacus/layers/dp_multihead_attention.py:25-455``.
"""
import warnings
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F


class SequenceBias(nn.Module):
    """Appends one learned vector as an extra sequence position (the
    ``bias_k``/``bias_v`` of ``nn.MultiheadAttention``)."""

    def __init__(self, embed_dim: int, batch_first: bool = False):
        super().__init__()
        self.batch_first = batch_first
        self.bias = nn.Parameter(torch.empty(embed_dim))
        self._reset_parameters()

    def _reset_parameters(self):
        nn.init.normal_(self.bias)

    def forward(self, x):
        if self.batch_first:
            return torch.cat([x, self.bias.expand(x.shape[0], 1, -1)], dim=1)
        return torch.cat([x, self.bias.expand(1, x.shape[1], -1)], dim=0)


_FUSED_KEYS = {"in_proj_weight": "weight", "in_proj_bias": "bias"}
_SPLIT_KEYS = {"q_proj_weight": "qlinear.weight", "k_proj_weight": "klinear.weight", "v_proj_weight": "vlinear.weight"}


class DPMultiheadAttention(nn.Module):
    def __init__(self, embed_dim, num_heads, dropout=0.0, bias=True, add_bias_kv=False, add_zero_attn=False,
                 kdim=None, vdim=None, batch_first=False, device=None, dtype=None):
        super().__init__()
        fk = {"device": device, "dtype": dtype}
        self.embed_dim = embed_dim
        self.kdim = embed_dim if kdim is None else kdim
        self.vdim = embed_dim if vdim is None else vdim
        self._qkv_same_embed_dim = False
        self.num_heads = num_heads
        self.batch_first = batch_first
        self.head_dim = embed_dim // num_heads
        assert self.head_dim * num_heads == embed_dim, "embed_dim must be divisible by num_heads"

        self.qlinear = nn.Linear(embed_dim, embed_dim, bias=bias, **fk)
        self.klinear = nn.Linear(self.kdim, embed_dim, bias=bias, **fk)
        self.vlinear = nn.Linear(self.vdim, embed_dim, bias=bias, **fk)
        self.out_proj = nn.Linear(embed_dim, embed_dim, bias=bias, **fk)

        self.add_bias_kv = add_bias_kv
        if add_bias_kv:
            # same layout as the module's inputs, so that per-sample gradient
            # capture sees the batch on the axis it expects
            self.seq_bias_k = SequenceBias(embed_dim, batch_first=batch_first)
            self.seq_bias_v = SequenceBias(embed_dim, batch_first=batch_first)
        self.add_zero_attn = add_zero_attn
        self.dropout = nn.Dropout(dropout)
        # attributes probed by nn.TransformerEncoderLayer's fast-path check
        self.in_proj_weight = None
        self.in_proj_bias = None

        self._register_state_dict_hook(_to_torch_layout)
        self._register_load_state_dict_pre_hook(_from_torch_layout, with_module=True)

    # ------------------------------------------------------------------ forward
    def forward(self, query, key, value, key_padding_mask=None, need_weights=True, attn_mask=None, is_causal=False):
        assert query.dim() == 3, "The query must have a dimension of 3."
        assert not is_causal, "We currently do not support causal mask. Will fix it in the future."
        if self.batch_first:
            B, Tq, E = query.shape
        else:
            Tq, B, E = query.shape
        if E != self.embed_dim:
            raise ValueError(f"query has as size of {E} while the embedding size is {self.embed_dim}")
        H, D = self.num_heads, self.head_dim

        q = self.qlinear(query)
        k = self.klinear(key)
        v = self.vlinear(value)
        if self.add_bias_kv:
            k, v = self.seq_bias_k(k), self.seq_bias_v(v)
        if self.batch_first:  # work time-major like nn.MultiheadAttention
            q, k, v = (t.transpose(0, 1) for t in (q, k, v))

        if attn_mask is not None:
            if attn_mask.dtype not in (torch.float32, torch.float64, torch.uint8, torch.bool):
                raise ValueError(
                    f"Only float, byte, and bool types are supported for attn_mask, not {attn_mask.dtype}."
                )
            if attn_mask.dtype == torch.uint8:
                warnings.warn("Byte tensor for attn_mask in nn.MultiheadAttention is deprecated.Use bool tensor instead.")
                attn_mask = attn_mask.to(torch.bool)
            Tk_in = k.shape[0] - (1 if self.add_bias_kv else 0)
            if attn_mask.dim() == 2:
                if tuple(attn_mask.shape) != (Tq, Tk_in):
                    raise ValueError("The size of the 2D attn_mask is not correct.")
                attn_mask = attn_mask.unsqueeze(0)
            elif attn_mask.dim() == 3:
                if tuple(attn_mask.shape) != (B * H, Tq, Tk_in):
                    raise ValueError("The size of the 3D attn_mask is not correct.")
            else:
                raise ValueError(f"attn_mask's dimension {attn_mask.dim()} is not supported")
        if key_padding_mask is not None and key_padding_mask.dtype == torch.uint8:
            warnings.warn("Byte tensor for key_padding_mask in nn.MultiheadAttentionis deprecated. Use bool tensor instead.")
            key_padding_mask = key_padding_mask.to(torch.bool)

        def _grow_masks():
            nonlocal attn_mask, key_padding_mask
            if attn_mask is not None:
                attn_mask = F.pad(attn_mask, (0, 1))
            if key_padding_mask is not None:
                key_padding_mask = F.pad(key_padding_mask, (0, 1))

        if self.add_bias_kv:
            _grow_masks()
        if self.add_zero_attn:
            k = torch.cat([k, k.new_zeros(1, *k.shape[1:])], dim=0)
            v = torch.cat([v, v.new_zeros(1, *v.shape[1:])], dim=0)
            _grow_masks()

        Tk = k.shape[0]
        # [T, B, E] -> [B, H, T, D]
        q = q.reshape(Tq, B, H, D).permute(1, 2, 0, 3)
        k = k.reshape(Tk, B, H, D).permute(1, 2, 0, 3)
        v = v.reshape(Tk, B, H, D).permute(1, 2, 0, 3)

        if key_padding_mask is not None:
            assert key_padding_mask.shape == (B, Tk)

        # One additive/boolean mask broadcastable to [B, H, Tq, Tk].
        mask: Optional[torch.Tensor] = None
        if attn_mask is not None:
            mask = attn_mask.reshape(1, 1, Tq, Tk) if attn_mask.shape[0] == 1 else attn_mask.reshape(B, H, Tq, Tk)
            if mask.dtype == torch.bool:
                mask = torch.zeros_like(mask, dtype=q.dtype).masked_fill(mask, float("-inf"))
        if key_padding_mask is not None:
            pad = torch.zeros(B, 1, 1, Tk, dtype=q.dtype, device=q.device).masked_fill(
                key_padding_mask[:, None, None, :], float("-inf")
            )
            mask = pad if mask is None else mask + pad

        if need_weights:
            scores = torch.matmul(q * (float(D) ** -0.5), k.transpose(-1, -2))
            if mask is not None:
                scores = scores + mask
            probs = self.dropout(F.softmax(scores, dim=-1))
            ctx = torch.matmul(probs, v)
            weights = probs.sum(dim=1) / H
        else:
            p_drop = self.dropout.p if self.training else 0.0
            ctx = F.scaled_dot_product_attention(q, k, v, attn_mask=mask, dropout_p=p_drop)
            weights = None

        ctx = ctx.permute(2, 0, 1, 3).reshape(Tq, B, E)  # [Tq, B, E]
        if self.batch_first:
            ctx = ctx.transpose(0, 1)
        return self.out_proj(ctx), weights


def _to_torch_layout(module: DPMultiheadAttention, sd, prefix, local_metadata):
    """state_dict hook: rewrite our keys into ``nn.MultiheadAttention``'s."""

    def take(name):
        return sd.pop(prefix + name, None)

    qw, kw, vw = take("qlinear.weight"), take("klinear.weight"), take("vlinear.weight")
    qb, kb, vb = take("qlinear.bias"), take("klinear.bias"), take("vlinear.bias")
    ow, ob = take("out_proj.weight"), take("out_proj.bias")
    bk, bv = take("seq_bias_k.bias"), take("seq_bias_v.bias")
    if module.kdim == module.embed_dim and module.vdim == module.embed_dim:
        sd[prefix + "in_proj_weight"] = torch.cat((qw, kw, vw), dim=0)
    else:
        sd[prefix + "q_proj_weight"], sd[prefix + "k_proj_weight"], sd[prefix + "v_proj_weight"] = qw, kw, vw
    if qb is not None and kb is not None and vb is not None:
        sd[prefix + "in_proj_bias"] = torch.cat((qb, kb, vb), dim=0)
    if bk is not None:
        sd[prefix + "bias_k"] = bk[None, None, :]
        sd[prefix + "bias_v"] = bv[None, None, :]
    sd[prefix + "out_proj.weight"] = ow
    if ob is not None:
        sd[prefix + "out_proj.bias"] = ob
    return sd


def _from_torch_layout(module, sd, prefix, local_metadata, strict, missing, unexpected, errors):
    """load_state_dict pre-hook: accept ``nn.MultiheadAttention`` keys."""
    for fused, part in _FUSED_KEYS.items():
        t = sd.pop(prefix + fused, None)
        if t is not None:
            for name, piece in zip(("qlinear", "klinear", "vlinear"), t.chunk(3, dim=0)):
                sd[f"{prefix}{name}.{part}"] = piece
    for src, dst in _SPLIT_KEYS.items():
        t = sd.pop(prefix + src, None)
        if t is not None:
            sd[prefix + dst] = t
    for src, dst in (("bias_k", "seq_bias_k.bias"), ("bias_v", "seq_bias_v.bias")):
        t = sd.pop(prefix + src, None)
        if t is not None:
            sd[prefix + dst] = t.reshape(-1)
