"""Llama-3 style decoder (RMSNorm, rotary embeddings, grouped-query attention,
SwiGLU) written so that DP training applies directly: every parameter lives in
an ``nn.Linear``, ``nn.Embedding`` or an RMSNorm, and there are no buffers
(the rotary angles are evaluated on the fly).  On CUDA the rotary embedding,
the SwiGLU gate and every residual addition together with the RMSNorm that
follows it run as fused kernels of this package (``csrc/rope.cu``,
``csrc/swiglu.cu``, ``csrc/rmsnorm.cu``); on CPU as plain PyTorch.  Parameter
names and shapes are those of a decoder built from ``nn.RMSNorm``, so state
dicts interchange with the plain definition the benchmarks give the reference
library (``baseline/llama_plain.py``).
"""
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..layers.add_rms_norm import AddRMSNorm


@dataclass
class LlamaConfig:
    vocab_size: int = 128256
    d_model: int = 2048
    n_layers: int = 16
    n_heads: int = 32
    n_kv_heads: int = 8
    ffn_dim: int = 8192
    rope_theta: float = 500000.0
    norm_eps: float = 1e-5
    tie_embeddings: bool = True


def llama_1b_config(**kw) -> LlamaConfig:
    """Llama-3.2-1B shape."""
    return LlamaConfig(**kw)


def llama_8b_config(**kw) -> LlamaConfig:
    """Llama-3-8B shape."""
    base = dict(d_model=4096, n_layers=32, n_heads=32, n_kv_heads=8, ffn_dim=14336, tie_embeddings=False)
    base.update(kw)
    return LlamaConfig(**base)


def _rope_tables(T: int, head_dim: int, theta: float, device, dtype):
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=device, dtype=torch.float32) / head_dim))
    ang = torch.outer(torch.arange(T, device=device, dtype=torch.float32), inv)      # [T, hd/2]
    return ang.cos().to(dtype), ang.sin().to(dtype)


def _apply_rope(x, cos, sin):
    # x: [B, H, T, hd]; rotate pairs (first half, second half)
    h = x.shape[-1] // 2
    x1, x2 = x[..., :h], x[..., h:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)


class _FusedRope(torch.autograd.Function):
    """Rotary embedding of a token-major ``[B, T, H, hd]`` tensor in one kernel each way (``csrc/rope.cu``)."""

    @staticmethod
    def forward(ctx, x, theta):
        from ..ops import _cuda

        ctx.theta = float(theta)
        return _cuda.load().rope(x.contiguous(), ctx.theta, False, False, 1.0)

    @staticmethod
    def backward(ctx, g):
        from ..ops import _cuda

        C = _cuda.load()
        if g.is_contiguous():
            return C.rope(g, ctx.theta, False, False, -1.0), None
        gh = g.transpose(1, 2)                 # attention may hand the gradient back head-major
        if gh.is_contiguous():
            return C.rope(gh, ctx.theta, True, False, -1.0), None
        return C.rope(g.contiguous(), ctx.theta, False, False, -1.0), None


class _FusedSwiGLU(torch.autograd.Function):
    """``silu(gate) * up`` and its gradient as one kernel each (``csrc/swiglu.cu``)."""

    @staticmethod
    def forward(ctx, gate, up):
        from ..ops import _cuda

        gate, up = gate.contiguous(), up.contiguous()
        ctx.save_for_backward(gate, up)
        return _cuda.load().swiglu_forward(gate, up)

    @staticmethod
    def backward(ctx, dh):
        from ..ops import _cuda

        gate, up = ctx.saved_tensors
        dg, du = _cuda.load().swiglu_backward(gate, up, dh.contiguous())
        return dg, du


_KERNEL_DTYPES = (torch.bfloat16, torch.float16, torch.float32)


def rope(x, theta: float):
    """Rotary embedding of ``x [B, T, H, hd]`` (token-major in, token-major out)."""
    if x.is_cuda and x.dtype in _KERNEL_DTYPES and x.shape[-1] % 16 == 0:
        return _FusedRope.apply(x, theta)
    cos, sin = _rope_tables(x.shape[1], x.shape[-1], theta, x.device, x.dtype)
    return _apply_rope(x.transpose(1, 2), cos, sin).transpose(1, 2)


def swiglu(gate, up):
    if gate.is_cuda and gate.dtype in _KERNEL_DTYPES and gate.dtype == up.dtype and gate.numel() % 8 == 0:
        return _FusedSwiGLU.apply(gate, up)
    return F.silu(gate) * up


class Attention(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.n_heads, self.n_kv = cfg.n_heads, cfg.n_kv_heads
        self.hd = cfg.d_model // cfg.n_heads
        self.theta = cfg.rope_theta
        self.q_proj = nn.Linear(cfg.d_model, cfg.n_heads * self.hd, bias=False)
        self.k_proj = nn.Linear(cfg.d_model, cfg.n_kv_heads * self.hd, bias=False)
        self.v_proj = nn.Linear(cfg.d_model, cfg.n_kv_heads * self.hd, bias=False)
        self.o_proj = nn.Linear(cfg.n_heads * self.hd, cfg.d_model, bias=False)
        self.sp_gather = None     # set by parallelize_llama(sequence_parallel=True): [B / world, T, D] -> [B, T, D]

    def forward(self, x):
        if self.sp_gather is not None:
            x = self.sp_gather(x)
        q_lin = self.q_proj(x)
        if isinstance(q_lin, tuple):        # sequence parallel: the projection gathered its input, siblings reuse it
            q_lin, x = q_lin
        B, T, _ = x.shape
        # everything stays token-major in memory; attention gets [B, H, T, hd] *views*, so neither the
        # inputs nor the output of attention are ever transposed by a copy
        q = rope(q_lin.view(B, T, self.n_heads, self.hd), self.theta).transpose(1, 2)
        k = rope(self.k_proj(x).view(B, T, self.n_kv, self.hd), self.theta).transpose(1, 2)
        v = self.v_proj(x).view(B, T, self.n_kv, self.hd).transpose(1, 2)
        y = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=self.n_kv != self.n_heads)
        return self.o_proj(y.transpose(1, 2).reshape(B, T, self.n_heads * self.hd))


class MLP(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.gate_proj = nn.Linear(cfg.d_model, cfg.ffn_dim, bias=False)
        self.up_proj = nn.Linear(cfg.d_model, cfg.ffn_dim, bias=False)
        self.down_proj = nn.Linear(cfg.ffn_dim, cfg.d_model, bias=False)
        self.sp_gather = None

    def forward(self, x):
        if self.sp_gather is not None:
            x = self.sp_gather(x)
        gate = self.gate_proj(x)
        if isinstance(gate, tuple):         # sequence parallel: see Attention.forward
            gate, x = gate
        return self.down_proj(swiglu(gate, self.up_proj(x)))


class Block(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.input_layernorm = AddRMSNorm(cfg.d_model, eps=cfg.norm_eps)
        self.self_attn = Attention(cfg)
        self.post_attention_layernorm = AddRMSNorm(cfg.d_model, eps=cfg.norm_eps)
        self.mlp = MLP(cfg)

    def forward(self, h, delta=None):
        """``h`` is the residual stream without the previous block's MLP output ``delta``; every residual
        addition happens inside the norm that follows it.  Returns the pair for the next block."""
        x, h = self.input_layernorm(h, delta)
        x, h = self.post_attention_layernorm(h, self.self_attn(x))
        return h, self.mlp(x)


class Llama(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.cfg = cfg
        self.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.d_model)
        self.layers = nn.ModuleList(Block(cfg) for _ in range(cfg.n_layers))
        self.norm = AddRMSNorm(cfg.d_model, eps=cfg.norm_eps)
        self.lm_head = nn.Linear(cfg.d_model, cfg.vocab_size, bias=False)
        self.sp_slice = None      # set by parallelize_llama(sequence_parallel=True): this rank's samples
        self.apply(self._init)
        if cfg.tie_embeddings:
            self.lm_head.weight = self.embed_tokens.weight

    @staticmethod
    def _init(m):
        if isinstance(m, (nn.Linear, nn.Embedding)):
            nn.init.normal_(m.weight, std=0.02)

    def forward(self, ids):
        if self.sp_slice is not None:
            ids = self.sp_slice(ids)
        h, delta = self.embed_tokens(ids), None
        for blk in self.layers:
            h, delta = blk(h, delta)
        return self.lm_head(self.norm(h, delta)[0])

    def num_parameters(self) -> int:
        return sum(p.numel() for p in self.parameters())
