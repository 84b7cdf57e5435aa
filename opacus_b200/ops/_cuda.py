"""CUDA side of :mod:`opacus_b200.ops`: shape/dtype preparation around the
kernels bound in ``opacus_b200._C`` (sources in ``opacus_b200/csrc``).

The tensor-core kernels take bf16 operands and accumulate in fp32.  fp32 models
use the same kernels through a three-plane split of each operand
(``split3_rows``: ``v = hi + lo`` with both parts bf16; the planes
``(hi, hi, lo)`` of one operand are contracted against ``(hi, lo, hi)`` of the
other, stacked along the contraction axis), which reproduces the fp32 product up
to a relative 2^-16 -- tighter than a tf32 product (2^-10) at three bf16
products' cost.  The bandwidth-bound kernels are dtype generic.
"""
from __future__ import annotations

import math
import os
from typing import Dict, Optional

import numpy as np
import torch

from . import _ref

_C = None
_USE_PAIR_GEMM = os.environ.get("OPACUS_B200_PAIR_GEMM", "0") == "1"
_scratch: Dict[tuple, torch.Tensor] = {}


def load():
    """Import the native module; a GPU machine without it is an error."""
    global _C
    if _C is not None:
        return _C
    try:
        from .. import _C as mod
    except ImportError as e:
        raise RuntimeError(
            "opacus_b200: the native extension is not built. Run `python -m opacus_b200.build` "
            "(needs nvcc; compiles for sm_100a) before using CUDA tensors."
        ) from e
    _C = _Native(mod)
    return _C


class _Native:
    """The native module with one translation: the RuntimeError by which a call reports that an earlier kernel
    gave up on a bounded wait becomes :class:`CommTimeoutError`."""

    def __init__(self, mod):
        self._mod = mod

    def __getattr__(self, name):
        fn = getattr(self._mod, name)
        if not callable(fn):
            return fn

        def call(*args, **kwargs):
            try:
                return fn(*args, **kwargs)
            except RuntimeError as e:
                if "gave up on a bounded wait" in str(e):
                    from ..utils.errors import CommTimeoutError

                    raise CommTimeoutError(str(e).split("\n")[0]) from None
                raise

        call.__name__ = name
        self.__dict__[name] = call
        return call


def set_debug(on: bool = True):
    """Debug mode (also ``OPACUS_B200_DEBUG=1`` in the environment): every buffer handed to a kernel as an output
    starts filled with NaN, so an element that a kernel fails to write shows in the result."""
    load().set_debug(bool(on))


def _out(*shape, dtype, device):
    """Uninitialised output buffer for a kernel; NaN-filled in debug mode."""
    if len(shape) == 1 and isinstance(shape[0], (tuple, list)):
        shape = tuple(shape[0])
    if load().get_debug():
        return torch.full(shape, float("nan"), dtype=dtype, device=device)
    return torch.empty(shape, dtype=dtype, device=device)


def check_status(device=None):
    dev = torch.cuda.current_device() if device is None else torch.device(device).index
    load().check_status(dev or 0)


def _bt(x: torch.Tensor) -> torch.Tensor:
    if x.dim() == 2:
        return x.unsqueeze(1)
    return x.reshape(x.shape[0], -1, x.shape[-1])


def _scratch_for(device, floats: int) -> torch.Tensor:
    """Work space of the ghost-norm kernel, one buffer per (device, stream): calls on different streams never
    share it, and a buffer is only ever replaced from the stream that uses it (allocated while that stream is
    current, so the caching allocator orders its reuse after the kernels already queued there)."""
    key = (device, torch._C._cuda_getCurrentRawStream(device.index if device.index is not None
                                                      else torch.cuda.current_device()))
    buf = _scratch.get(key)
    if buf is None or buf.numel() < floats:
        buf = torch.empty(max(floats, 1 << 16), dtype=torch.float32, device=device)
        _scratch[key] = buf
    return buf


def _bf16(x: torch.Tensor) -> torch.Tensor:
    """bf16, contiguous (conversion through the row-scaling kernel when needed)."""
    if x.dtype == torch.bfloat16:
        return x.contiguous()
    if x.dtype == torch.float32 and x.shape[-1] % 8 == 0:
        x2 = x.contiguous().reshape(-1, x.shape[-1])
        return load().scale_rows(x2, None, 1, 1.0).view(x.shape)
    return x.to(torch.bfloat16).contiguous()


def _tensor_core_ok(*ts) -> bool:
    """bf16 (or fp16-free) operands whose rows are 16-byte multiples."""
    return all(t.dtype == torch.bfloat16 and t.shape[-1] % 8 == 0 for t in ts)


def _split_pair(g3, a3, c=None, g_scale: float = 1.0):
    """fp32 ``[B, T, d]`` operands of a product contracted over T -> bf16 ``[B, 3T, d]`` planes, left and right
    form (the clip factors ``c`` and ``g_scale`` go onto the left one)."""
    C = load()
    B, T = g3.shape[0], g3.shape[1]
    gl = C.split3_rows(g3.float().reshape(B * T, g3.shape[-1]).contiguous(), c, T, float(g_scale), False)
    ar = C.split3_rows(a3.float().reshape(B * T, a3.shape[-1]).contiguous(), None, T, 1.0, True)
    return gl, ar


def _split_lr(t3):
    """fp32 ``[B, T, d]`` -> (bf16 ``[B, 2 * Tp, 3d]``, Tp): rows ``[0, T)`` hold the planes (hi, hi, lo) side by
    side, rows ``[Tp, Tp + T)`` the planes (hi, lo, hi), everything else zero (Tp = T rounded up to 128).  The Gram
    kernel multiplies the first block by the transposed second one: ``hi hi^T + hi lo^T + lo hi^T``."""
    B, T, d = t3.shape
    Tp = (T + 127) // 128 * 128
    x = t3.float()
    hi = x.bfloat16()
    lo = (x - hi.float()).bfloat16()
    buf = torch.zeros(B, 2 * Tp, 3 * d, dtype=torch.bfloat16, device=t3.device)
    buf[:, :T, :d], buf[:, :T, d:2 * d], buf[:, :T, 2 * d:] = hi, hi, lo
    buf[:, Tp:Tp + T, :d], buf[:, Tp:Tp + T, d:2 * d], buf[:, Tp:Tp + T, 2 * d:] = hi, lo, hi
    return buf, Tp


# ----------------------------------------------------------------------- Linear
def linear_grad_sample(a, g):
    """``[B, d_out, d_in]`` per-sample gradients (dtype of ``g``) by the batched
    tensor-core kernel; the squared Frobenius norm of every sample's gradient is
    produced in the same pass (fp32, before rounding) and travels with the
    result as ``._dp_norm_sq`` so that clipping does not have to re-read it."""
    a3, g3 = _bt(a), _bt(g)
    B, T, d_in = a3.shape
    d_out = g3.shape[-1]
    if d_in % 8 or d_out % 8 or g3.dtype not in (torch.bfloat16, torch.float32):
        return _ref.linear_grad_sample(a, g)
    C = load()
    n2 = torch.zeros(B, dtype=torch.float32, device=g.device)
    if g3.dtype == torch.float32:
        gl, ar = _split_pair(g3, a3)
        out = _out(B, d_out, d_in, dtype=torch.float32, device=g.device)
        C.wgrad_tn_ex(gl, ar, out, 0.0, n2, 0, 0, 0)
    else:
        out = _out(B, d_out, d_in, dtype=torch.bfloat16, device=g.device)
        C.wgrad_tn_ex(g3.contiguous(), _bf16(a3), out, 0.0, n2, 0, 0, 0)
    out._dp_norm_sq = n2
    return out


def linear_norm_sq(a, g, want_weight=True, want_bias=False, g_scale: float = 1.0, total=None):
    """``total`` (fp32 ``[B]``): add both norms into it in place and return ``(None, None)``."""
    a3, g3 = _bt(a), _bt(g)
    B, T, d_in = a3.shape
    d_out = g3.shape[-1]
    s2 = float(g_scale) ** 2
    C = load()
    acc = total is not None

    def outs():
        if acc:
            return (total if want_weight else None), (total if want_bias else None)
        return (_out(B, dtype=torch.float32, device=g.device) if want_weight else None,
                _out(B, dtype=torch.float32, device=g.device) if want_bias else None)

    def done(w, b):
        return (None, None) if acc else (w, b)

    if T == 1:
        dt = g3.dtype
        a2 = a3.reshape(B, d_in).to(dt).contiguous()
        g2 = g3.reshape(B, d_out).contiguous()
        w, b = outs()
        C.outer_norm_sq(a2 if want_weight else None, g2, s2, w, b, acc)
        return done(w, b)
    tensor_core = g3.dtype == torch.bfloat16 and d_in % 8 == 0 and d_out % 8 == 0
    gram_cheaper = T * (d_in + d_out) <= 2 * d_in * d_out  # symmetric tiles halve the Gram cost
    if tensor_core and (gram_cheaper or not want_weight):
        gb = g3.contiguous()
        ab = _bf16(a3) if want_weight else None
        w, b = outs()
        scratch = _scratch_for(g.device, C.gram_pair_scratch_floats(B, T))
        C.gram_pair_norm(ab, None, gb, s2, scratch, w, b, acc)
        return done(w, b)
    if tensor_core:
        # wide layer, short sequence: form each sample's gradient tile by tile in TMEM and only keep its norm
        gb = g3.contiguous()
        n2 = torch.zeros(B, dtype=torch.float32, device=g.device)
        C.wgrad_tn_ex(gb, _bf16(a3), None, 0.0, n2, 0, 0, 0)
        w = n2 * s2 if s2 != 1.0 else n2
        b = None
        if want_bias:
            b = _out(B, dtype=torch.float32, device=g.device)
            scratch = _scratch_for(g.device, C.gram_pair_scratch_floats(B, T))
            C.gram_pair_norm(None, None, gb, s2, scratch, None, b, False)
        if acc:
            total.add_(w)
            if b is not None:
                total.add_(b)
            return None, None
        return w, b
    if g3.dtype == torch.float32 and d_in % 8 == 0 and d_out % 8 == 0:
        # fp32 model: each sample's gradient is formed tile by tile in TMEM from the split operands, only its norm is kept
        w = b = None
        if want_weight:
            gl, ar = _split_pair(g3, a3)
            n2 = torch.zeros(B, dtype=torch.float32, device=g.device)
            C.wgrad_tn_ex(gl, ar, None, 0.0, n2, 0, 0, 0)
            w = n2 * s2 if s2 != 1.0 else n2
        if want_bias:
            b = g3.sum(dim=1).square().sum(dim=1) * s2
        if acc:
            for t in (w, b):
                if t is not None:
                    total.add_(t)
            return None, None
        return w, b
    w, b = _ref.linear_norm_sq(a, g, want_weight, want_bias, g_scale)
    if acc:
        for t in (w, b):
            if t is not None:
                total.add_(t)
        return None, None
    return w, b


def linear_weighted_grad(a, g, c, g_scale: float = 1.0, want_bias: bool = False, out=None, accumulate=False):
    """``out`` (fp32 ``[d_out, d_in]``, contiguous) receives the result in place:
    overwritten, or added to when ``accumulate``."""
    a3, g3 = _bt(a), _bt(g)
    B, T, d_in = a3.shape
    d_out = g3.shape[-1]
    if d_in % 8 or d_out % 8 or g3.dtype not in (torch.bfloat16, torch.float32):
        w, b = _ref.linear_weighted_grad(a, g, c, g_scale, want_bias)
        if out is not None:
            out.add_(w) if accumulate else out.copy_(w)
            w = out
        return w, b
    C = load()
    c = c.float().contiguous()
    a2 = a3.reshape(B * T, d_in)
    g2 = g3.reshape(B * T, d_out)
    if g3.dtype == torch.float32:
        gl, ar = _split_pair(g3, a3, c, g_scale)
        g_op, a_op = gl.view(3 * B * T, d_out), ar.view(3 * B * T, d_in)
    # the clip factors go onto the narrower operand (fewer bytes to rewrite)
    elif d_in <= d_out and a2.dtype in (torch.float32, torch.bfloat16):
        a_op = C.scale_rows(a2.contiguous(), c, T, float(g_scale))
        g_op = g2.contiguous()
    else:
        g_op = C.scale_rows(g2.contiguous(), c, T, float(g_scale))
        a_op = _bf16(a2)
    if out is None or out.dtype != torch.float32 or not out.is_contiguous():
        target = _out(d_out, d_in, dtype=torch.float32, device=g.device)
        C.wgrad_tn(g_op, a_op, target, 0.0)
        if out is not None:
            out.add_(target) if accumulate else out.copy_(target)
        else:
            out = target
    elif _USE_PAIR_GEMM and d_out >= 256 and d_in >= 256:
        # the same product on pairs of SMs (cta_group::2): faster in isolation, no different inside a training step
        # (two GEMM streams already fill each other's partial waves), hence opt-in
        tiles = -(-d_out // 256) * -(-d_in // 256)
        C.wgrad2_tn(g_op, a_op, out, 1.0 if accumulate else 0.0, 1 if tiles >= 64 else min(4, 74 // tiles))
    else:
        C.wgrad_tn(g_op, a_op, out, 1.0 if accumulate else 0.0)
    bias = None
    if want_bias:
        per_sample = g3.float().sum(dim=1)                       # [B, d_out]
        bias = C.weighted_sum(per_sample.contiguous(), c * float(g_scale))
    return out, bias


# -------------------------------------------------------------------- Embedding
def embedding_norm_sq(ids, g, g_scale: float = 1.0, padding_idx: Optional[int] = None, total=None):
    B = ids.shape[0]
    ids2 = ids.reshape(B, -1)
    T = ids2.shape[1]
    g3 = g.reshape(B, T, -1)
    if padding_idx is not None or g3.dtype not in (torch.bfloat16, torch.float32) or g3.shape[-1] % 8:
        w = _ref.embedding_norm_sq(ids, g, g_scale, padding_idx)
        if total is not None:
            total.add_(w)
            return None
        return w
    C = load()
    w = total if total is not None else _out(B, dtype=torch.float32, device=g.device)
    scratch = _scratch_for(g.device, C.gram_pair_scratch_floats(B, T))
    if g3.dtype == torch.float32:
        # fp32 gradients: the same mask-Gram kernel on the three-plane split (left rows x right rows)
        both, Tp = _split_lr(g3)
        C.gram_pair_norm(None, ids2.contiguous().long(), both, float(g_scale) ** 2, scratch, w, None,
                         total is not None, Tp, T)
        return None if total is not None else w
    C.gram_pair_norm(None, ids2.contiguous().long(), g3.contiguous(), float(g_scale) ** 2, scratch, w, None,
                     total is not None)
    return None if total is not None else w


def embedding_weighted_grad(ids, g, c, num_embeddings, g_scale: float = 1.0, padding_idx=None, out_dtype=None,
                            out=None, accumulate=False):
    B = ids.shape[0]
    D = g.shape[-1]
    T = ids.numel() // B
    if out is not None and out.dtype == torch.float32 and out.is_contiguous():
        if not accumulate:
            out.zero_()
        load().embedding_scatter(ids.reshape(-1).contiguous().long(), g.reshape(-1, D).contiguous(),
                                 c.float().contiguous(), T, -1 if padding_idx is None else int(padding_idx),
                                 float(g_scale), out)
        return out
    out = torch.zeros(num_embeddings, D, dtype=torch.float32, device=g.device)
    load().embedding_scatter(ids.reshape(-1).contiguous().long(), g.reshape(-1, D).contiguous(),
                             c.float().contiguous(), T, -1 if padding_idx is None else int(padding_idx),
                             float(g_scale), out)
    return out if out_dtype in (None, torch.float32) else out.to(out_dtype)


# ----------------------------------------------------------- normalisation layers
def supports_norm(kind, x, normalized_ndim) -> bool:
    if kind in ("layer", "rms"):
        return normalized_ndim == 1 and x.dim() >= 2
    return x.dim() >= 2


def norm_affine_grad_sample(kind, x, g, eps, normalized_ndim, num_groups, want_weight, want_bias):
    C = load()
    if x.dtype != g.dtype:
        wide = torch.promote_types(x.dtype, g.dtype)
        x, g = x.to(wide), g.to(wide)
    x, g = x.contiguous(), g.contiguous()
    if kind in ("layer", "rms"):
        d = x.shape[-1]
        if want_weight:
            # one launch: statistics, per-sample gradients and their squared norms (kept on the results as
            # ``_dp_norm_sq`` so that clipping does not read them again)
            res = C.norm_lastdim_psg(0 if kind == "layer" else 1, x, g, d, float(eps),
                                     bool(want_bias) and kind == "layer")
            if res:
                gw, gb, n2w, n2b = res
                gw._dp_norm_sq = n2w
                if want_bias and kind == "layer":
                    gb._dp_norm_sq = n2b
                    return gw, gb
                return gw, None
        gw, gb = C.norm_lastdim_grad(0 if kind == "layer" else 1, x, g, d, float(eps), bool(want_weight),
                                     bool(want_bias) and kind == "layer")
    else:
        groups = x.shape[1] if kind == "instance" else int(num_groups)
        gw, gb = C.norm_channel_grad(x, g, groups, float(eps), bool(want_weight), bool(want_bias))
    # fp32 results are kept: these per-sample gradients are tiny and feed the norm
    return (gw if want_weight else None), (gb if (want_bias and gb is not None and gb.numel()) else None)


# --------------------------------------------------------------- clipping pieces
def clip_factor(norm_sq, max_grad_norm: float):
    return load().clip_factor(norm_sq.contiguous(), float(max_grad_norm))


def grad_sample_norm_sq(gs):
    cached = getattr(gs, "_dp_norm_sq", None)
    if cached is not None and cached.shape[0] == gs.shape[0]:
        return cached
    return load().row_norm_sq(gs.contiguous())


def _dense_order(t):
    """Axis order (sample axis first) in which ``t`` is laid out densely, or None."""
    if t.is_contiguous():
        return None
    order = [0] + sorted(range(1, t.dim()), key=lambda d: -t.stride(d))
    return order if t.permute(order).is_contiguous() else None


def weighted_sum(gs, c, out=None):
    """``out``: optional fp32 contiguous destination with the shape of one sample's gradient (overwritten)."""
    if out is not None and gs.is_contiguous() and out.dtype == torch.float32 and out.is_contiguous():
        load().weighted_sum(gs, c.float().contiguous(), out.view(-1))
        return out
    if out is not None:
        out.copy_(weighted_sum(gs, c).view(out.shape))
        return out
    order = _dense_order(gs)
    if order is not None:
        # a permuted view of a dense buffer (e.g. the channels-last conv gradient): sum in storage
        # order, then hand back the result in the logical axis order
        phys = gs.permute(order)
        out = load().weighted_sum(phys, c.float().contiguous()).view(phys.shape[1:])
        inv = [0] * (gs.dim() - 1)
        for pos, d in enumerate(order[1:]):
            inv[d - 1] = pos
        return out.permute(inv).contiguous().to(gs.dtype)
    out = load().weighted_sum(gs.contiguous(), c.float().contiguous())
    return out.view(gs.shape[1:]).to(gs.dtype)


# ------------------------------------------------------------------- convolution (implicit unfold)
_MAX_GROUP_CALLS = 8


def conv_geometry(layer, x, backprops):
    """A plan ``(kh, kw, sh, sw, ph, pw, dh, dw, groups, prepad, fp32)`` when the implicit-unfold kernel covers this
    Conv1d / Conv2d call, else None.  Covered: bf16 and fp32 data (fp32 as three bf16 passes over split operands),
    any channel counts (padded with zero channels to multiples of 8), up to 8 groups (one call per group; more,
    e.g. depthwise, stay on the batched-GEMM path), zero padding including ``"same"`` with an odd total (the input is
    padded explicitly first).  A Conv3d reaches the kernel as one 2-d problem per kernel-depth offset
    (``grad_sample/conv.py``: ``depth_stacked_pairs``).  Not covered: non-zero padding modes, strides above 8."""
    nsp = x.dim() - 2
    if nsp not in (1, 2) or backprops.dtype not in (torch.bfloat16, torch.float32) or not x.is_cuda:
        return None
    if getattr(layer, "padding_mode", "zeros") != "zeros" or layer.groups > _MAX_GROUP_CALLS:
        return None
    pad = layer.padding
    prepad = None
    if isinstance(pad, str):
        if pad == "valid":
            pad = (0,) * nsp
        else:
            tot = [d * (k - 1) for k, d in zip(layer.kernel_size, layer.dilation)]
            if any(t % 2 for t in tot):
                # F.pad order: last axis first, (left, right) per axis; the extra element goes to the right
                prepad = [v for t in reversed(tot) for v in (t // 2, t - t // 2)]
                pad = (0,) * nsp
            else:
                pad = tuple(t // 2 for t in tot)
    k, s, d = tuple(layer.kernel_size), tuple(layer.stride), tuple(layer.dilation)
    if nsp == 1:
        k, s, pad, d = (1,) + k, (1,) + s, (0,) + tuple(pad), (1,) + d
    return conv_plan2d(k, s, pad, d, layer.groups, prepad, backprops.shape[-1], backprops.dtype == torch.float32)


def conv_plan2d(k, s, pad, d, groups, prepad, out_width, fp32):
    """The plan tuple of a 2-d problem given as numbers, or None when the kernel's pixel boxes cannot cover the strides."""
    bw = 1
    while bw < out_width and bw < 64:
        bw *= 2
    if max(s) > 8 or bw * s[1] > 256 or (64 // bw) * s[0] > 256 or groups > _MAX_GROUP_CALLS:
        return None
    return (int(k[0]), int(k[1]), int(s[0]), int(s[1]), int(pad[0]), int(pad[1]), int(d[0]), int(d[1]), int(groups),
            prepad, bool(fp32))


def _nhwc(t):
    """[B, C, H, W] (or [B, C, W]) -> contiguous [B, H, W, C]; free for channels-last tensors."""
    if t.dim() == 3:
        return t.transpose(1, 2).contiguous().unsqueeze(1)
    return t.permute(0, 2, 3, 1).contiguous()


def _pad8(t):
    """Zero channels up to a multiple of 8 on the last axis (TMA rows are 16-byte multiples)."""
    extra = -t.shape[-1] % 8
    return torch.nn.functional.pad(t, (0, extra)) if extra else t


def _conv_passes(xh, gh, fp32):
    """Operand pairs whose products add up to the convolution gradient: one bf16 pair, or for fp32 data the three
    pairs (hi, hi), (hi, lo), (lo, hi) of the split operands."""
    if not fp32:
        return [(xh.to(torch.bfloat16), gh.to(torch.bfloat16))]
    xf, gf = xh.float(), gh.float()
    x_hi, g_hi = xf.bfloat16(), gf.bfloat16()
    x_lo, g_lo = (xf - x_hi.float()).bfloat16(), (gf - g_hi.float()).bfloat16()
    return [(x_hi, g_hi), (x_lo, g_hi), (x_hi, g_lo)]


def _conv_groups(x, backprops, plan):
    """Channels-last operands of every group, channels padded to multiples of 8: [(xh, gh, C_g, O_g)]."""
    groups, prepad = plan[8], plan[9]
    if prepad is not None:
        x = torch.nn.functional.pad(x, prepad)
    xh, gh = _nhwc(x), _nhwc(backprops)
    cg, og = xh.shape[3] // groups, gh.shape[3] // groups
    out = []
    for i in range(groups):
        xs = xh if groups == 1 else xh[..., i * cg:(i + 1) * cg]
        gs = gh if groups == 1 else gh[..., i * og:(i + 1) * og]
        out.append((_pad8(xs).contiguous(), _pad8(gs).contiguous(), cg, og))
    return out


def conv_grad_sample(x, backprops, plan, want_out=True, norm_total=None):
    """Per-sample conv weight gradients ``[B, O, C/groups, kh, kw]`` (a permuted view of the kernel's
    channels-last output, ``_dp_norm_sq`` attached) and/or their squared norms added into ``norm_total``."""
    geom, fp32 = list(plan[:8]), plan[10]
    kh, kw = geom[0], geom[1]
    B = x.shape[0]
    C = load()
    norm = norm_total if norm_total is not None else torch.zeros(B, dtype=torch.float32, device=x.device)
    simple = not fp32
    pieces = []
    for xh, gh, cg, og in _conv_groups(x, backprops, plan):
        Op, Cp = gh.shape[3], xh.shape[3]
        passes = _conv_passes(xh, gh, fp32)
        if simple:
            out = _out((B, Op, kh, kw, Cp), dtype=torch.bfloat16, device=x.device) if want_out else None
            C.conv_psg(passes[0][0], passes[0][1], geom, False, out, 0.0, norm)
        else:
            # the norm of a sum of three products needs the sum: the gradients are formed in fp32, then squared
            out = _out((B, Op, kh, kw, Cp), dtype=torch.float32, device=x.device)
            for i, (xs, gs) in enumerate(passes):
                C.conv_psg(xs, gs, geom, False, out, 0.0 if i == 0 else 1.0, None)
            norm.add_(C.row_norm_sq(out))
        if out is not None and want_out:
            pieces.append(out[:, :og, :, :, :cg])
    if not want_out:
        return norm
    out = pieces[0] if len(pieces) == 1 else torch.cat(pieces, dim=1)
    gs = out.permute(0, 1, 4, 2, 3)
    if x.dim() == 3:
        gs = gs.squeeze(3)
    if norm_total is None:
        gs._dp_norm_sq = norm
    return gs


def conv_weighted_grad(x, backprops, coef, plan, g_scale=1.0):
    """``sum_b coef_b * grad_b`` of a conv weight as one implicit GEMM over all samples' pixels (per group);
    fp32 ``[O, C/groups, kh, kw]``."""
    geom, fp32 = list(plan[:8]), plan[10]
    C = load()
    B = x.shape[0]
    shape = (-1,) + (1,) * (backprops.dim() - 1)
    scaled = backprops * (coef.to(backprops.dtype) * g_scale).reshape(shape) if fp32 else None
    pieces = []
    for xh, gh, cg, og in _conv_groups(x, backprops if scaled is None else scaled, plan):
        _, OH, OW, Op = gh.shape
        Cp = xh.shape[3]
        out = _out((Op, geom[0], geom[1], Cp), dtype=torch.float32, device=x.device)
        if fp32:
            for i, (xs, gs) in enumerate(_conv_passes(xh, gh, True)):
                C.conv_psg(xs, gs, geom, True, out, 0.0 if i == 0 else 1.0, None)
        else:
            gsc = C.scale_rows(gh.to(torch.bfloat16).view(B * OH * OW, Op), coef.float().contiguous(), OH * OW,
                               float(g_scale)).view(gh.shape)
            C.conv_psg(xh.to(torch.bfloat16), gsc, geom, True, out, 0.0, None)
        pieces.append(out[:og, :, :, :cg])
    out = pieces[0] if len(pieces) == 1 else torch.cat(pieces, dim=0)
    w = out.permute(0, 3, 1, 2).contiguous()
    return w.squeeze(2) if x.dim() == 3 else w


# ------------------------------------------------------------------- fused step
_ENTRY = np.dtype([("param", "<u8"), ("grad", "<u8"), ("state0", "<u8"), ("state1", "<u8"), ("master", "<u8"),
                   ("numel", "<i8"), ("rng_offset", "<i8"), ("param_bf16", "<i4"), ("pad", "<i4")])
_CHUNK = 4096
_DOMAIN = 0x6F70616375736232  # separates this generator's streams from torch's own use of (seed, offset)


def _rng_state(generator, device, n_elems: int):
    gen = generator if generator is not None else torch.cuda.default_generators[device.index]
    seed = int(gen.initial_seed())
    offset = int(gen.get_offset())
    gen.set_offset(offset + 4 * ((n_elems + 3) // 4 + 1))
    seed = (seed ^ _DOMAIN) & 0x7FFFFFFFFFFFFFFF
    return seed, offset


def fused_dp_step(kind, inner, group, ps, *, noise_std: float, inv_scale: float, generator=None):
    """p.summed_grad <- (summed_grad + N(0, std^2)) * inv_scale, then the SGD / Adam / AdamW update of ``p``
    and its state, for every tensor in ``ps``: one launch for all tensors that are at the same point of their
    history (same Adam step count / same "momentum buffer exists"), which is all of them unless parameters
    were added to the optimiser later."""
    state = inner.state
    if kind == "sgd":
        has_momentum = float(group.get("momentum", 0.0)) != 0.0
        key = (lambda p: state[p].get("momentum_buffer") is None if p in state else True) if has_momentum \
            else (lambda p: False)
    else:
        key = lambda p: float(state[p]["step"]) if p in state and len(state[p]) else 0.0
    parts = {}
    for p in ps:
        parts.setdefault(key(p), []).append(p)
    for where, part in parts.items():
        _fused_dp_step_uniform(kind, inner, group, part, where, noise_std, inv_scale, generator)


_table_cache: Dict[tuple, tuple] = {}


def _fused_dp_step_uniform(kind, inner, group, ps, where, noise_std, inv_scale, generator):
    C = load()
    assert C.tensor_entry_size() == _ENTRY.itemsize
    dev = ps[0].device
    state = inner.state
    hyper = dict(lr=float(group["lr"]), momentum=0.0, dampening=0.0, weight_decay=float(group.get("weight_decay", 0.0)),
                 beta1=0.0, beta2=0.0, eps=0.0, bias_c1=1.0, bias_c2_sqrt=1.0)
    first_step = False
    nesterov = False
    if kind == "sgd":
        hyper["momentum"] = float(group.get("momentum", 0.0))
        hyper["dampening"] = float(group.get("dampening", 0.0))
        nesterov = bool(group.get("nesterov", False))
        if hyper["momentum"] != 0.0:
            first_step = bool(where)
            for p in ps:
                st = state[p]
                if st.get("momentum_buffer") is None:
                    st["momentum_buffer"] = torch.zeros_like(p, dtype=torch.float32, memory_format=torch.preserve_format)
        kcode = 0
    else:
        beta1, beta2 = group["betas"]
        for p in ps:
            st = state[p]
            if len(st) == 0:
                st["step"] = torch.tensor(0.0, dtype=torch.float32)
                st["exp_avg"] = torch.zeros_like(p, dtype=torch.float32, memory_format=torch.preserve_format)
                st["exp_avg_sq"] = torch.zeros_like(p, dtype=torch.float32, memory_format=torch.preserve_format)
        t = float(where) + 1.0
        for p in ps:
            state[p]["step"] += 1
        hyper.update(beta1=float(beta1), beta2=float(beta2), eps=float(group["eps"]),
                     bias_c1=1.0 - float(beta1) ** t, bias_c2_sqrt=math.sqrt(1.0 - float(beta2) ** t))
        kcode = 2 if kind == "adamw" else 1

    for p in ps:
        g = p.summed_grad
        if g.dtype != torch.float32 or not g.is_contiguous():
            p.summed_grad = g.float().contiguous()
    # the table of addresses is rebuilt and uploaded only when an address changed (summed_grad is reallocated
    # by every backward pass in hooks mode, but lives in fixed storage under the engines)
    if kind == "sgd":
        st_ptrs = tuple(0 if state[p].get("momentum_buffer") is None else state[p]["momentum_buffer"].data_ptr()
                        for p in ps) if hyper["momentum"] != 0.0 else ()
    else:
        st_ptrs = tuple((state[p]["exp_avg"].data_ptr(), state[p]["exp_avg_sq"].data_ptr()) for p in ps)
    sig = tuple((p.data_ptr(), p.summed_grad.data_ptr(), p.numel()) for p in ps) + (st_ptrs, kind, dev)
    slot = (id(inner), id(group), len(ps), ps[0].data_ptr())
    cached = _table_cache.get(slot)
    if cached is not None and cached[0] == sig:
        _, table_t, prefix_t, n_chunks, rng_ofs = cached
    else:
        table = np.zeros(len(ps), dtype=_ENTRY)
        prefix = np.zeros(len(ps) + 1, dtype=np.int64)
        rng_ofs = 0
        for i, p in enumerate(ps):
            st = state[p] if p in state else {}
            e = table[i]
            e["param"] = p.data_ptr()
            e["grad"] = p.summed_grad.data_ptr()
            if kind == "sgd":
                buf = st.get("momentum_buffer")
                e["state0"] = buf.data_ptr() if buf is not None else 0
            else:
                e["state0"] = st["exp_avg"].data_ptr()
                e["state1"] = st["exp_avg_sq"].data_ptr()
            e["numel"] = p.numel()
            e["rng_offset"] = rng_ofs
            e["param_bf16"] = 1 if p.dtype == torch.bfloat16 else 0
            rng_ofs += 4 * ((p.numel() + 3) // 4)
            prefix[i + 1] = prefix[i] + (p.numel() + _CHUNK - 1) // _CHUNK
        table_t = torch.from_numpy(table.view(np.uint8)).to(dev, non_blocking=True)
        prefix_t = torch.from_numpy(prefix).to(dev, non_blocking=True)
        n_chunks = int(prefix[-1])
        if len(_table_cache) > 64:
            _table_cache.clear()
        _table_cache[slot] = (sig, table_t, prefix_t, n_chunks, rng_ofs)
    seed, offset = _rng_state(generator, dev, rng_ofs)
    C.fused_dp_step(table_t, prefix_t, len(ps), n_chunks, kcode, nesterov, first_step,
                    hyper["lr"], hyper["momentum"], hyper["dampening"], hyper["weight_decay"], hyper["beta1"],
                    hyper["beta2"], hyper["eps"], hyper["bias_c1"], hyper["bias_c2_sqrt"], float(noise_std),
                    float(inv_scale), seed, offset)


def philox_normal(n: int, seed: int, offset: int, std: float, device) -> torch.Tensor:
    return load().philox_normal(int(n), int(seed), int(offset), float(std), torch.device(device))
