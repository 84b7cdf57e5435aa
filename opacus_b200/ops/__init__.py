"""Per-sample operations.

Every function here takes torch tensors.  CUDA tensors are served by the
hand-written sm_100a kernels in ``opacus_b200/csrc`` (bound in :mod:`._cuda`);
a missing or stale extension on a machine with a GPU is an error, never a
silent fallback.  CPU tensors are served by the plain-PyTorch statements in
:mod:`._ref`, which are also the test oracle.
"""
from typing import Optional

import torch

from . import _ref

_kernels = None


def _k():
    """The CUDA binding module, loaded on first use."""
    global _kernels
    if _kernels is None:
        import importlib

        mod = importlib.import_module(__name__ + "._cuda")
        mod.load()
        _kernels = mod
    return _kernels


def _on_gpu(*ts) -> bool:
    return any(t is not None and t.is_cuda for t in ts)


def _kernel_dtype(t: torch.Tensor) -> bool:
    return t.dtype in (torch.bfloat16, torch.float16, torch.float32)


# ----------------------------------------------------------------------- Linear
def linear_grad_sample(a, g):
    if _on_gpu(a, g) and _kernel_dtype(g) and g.shape[0] > 0:
        return _k().linear_grad_sample(a, g)
    return _ref.linear_grad_sample(a, g)


def linear_bias_grad_sample(g):
    return _ref.linear_bias_grad_sample(g)


def linear_norm_sq(a, g, want_weight=True, want_bias=False, g_scale: float = 1.0, total=None):
    """``total``: optional fp32 ``[B]`` running sum; when given, the norms are
    added into it in place (inside the kernel on CUDA) and ``(None, None)`` is returned."""
    if _on_gpu(a, g) and _kernel_dtype(g) and g.shape[0] > 0:
        return _k().linear_norm_sq(a, g, want_weight, want_bias, g_scale, total=total)
    w, b = _ref.linear_norm_sq(a, g, want_weight, want_bias, g_scale)
    if total is not None:
        for t in (w, b):
            if t is not None:
                total.add_(t.to(total.dtype))
        return None, None
    return w, b


def linear_weighted_grad(a, g, c, g_scale: float = 1.0, want_bias: bool = False, out=None, accumulate=False):
    """``out``: optional fp32 destination written in place (added to when ``accumulate``)."""
    if _on_gpu(a, g) and _kernel_dtype(g) and g.shape[0] > 0:
        return _k().linear_weighted_grad(a, g, c, g_scale, want_bias, out=out, accumulate=accumulate)
    w, b = _ref.linear_weighted_grad(a, g, c, g_scale, want_bias)
    if out is not None:
        out.add_(w.to(out.dtype)) if accumulate else out.copy_(w)
        w = out
    return w, b


# -------------------------------------------------------------------- Embedding
def embedding_grad_sample(ids, g, num_embeddings, lazy: bool = True):
    """Per-sample gradient ``[B, V, D]``: by default in compact form (see :mod:`.lazy`), which the norm and
    weighted-sum operations below consume directly and every other use turns into the dense tensor."""
    if lazy and ids.shape[0] > 0:
        from .lazy import LazyEmbeddingGradSample

        return LazyEmbeddingGradSample(ids, g, num_embeddings)
    return _ref.embedding_grad_sample(ids, g, num_embeddings)


def embedding_norm_sq(ids, g, g_scale: float = 1.0, padding_idx: Optional[int] = None, total=None):
    if _on_gpu(g) and _kernel_dtype(g) and g.shape[0] > 0:
        return _k().embedding_norm_sq(ids, g, g_scale, padding_idx, total=total)
    w = _ref.embedding_norm_sq(ids, g, g_scale, padding_idx)
    if total is not None:
        total.add_(w.to(total.dtype))
        return None
    return w


def embedding_weighted_grad(ids, g, c, num_embeddings, g_scale: float = 1.0, padding_idx=None, out_dtype=None,
                            out=None, accumulate=False):
    if _on_gpu(g) and _kernel_dtype(g) and g.shape[0] > 0:
        return _k().embedding_weighted_grad(ids, g, c, num_embeddings, g_scale, padding_idx, out_dtype,
                                            out=out, accumulate=accumulate)
    w = _ref.embedding_weighted_grad(ids, g, c, num_embeddings, g_scale, padding_idx, out_dtype)
    if out is not None:
        out.add_(w.to(out.dtype)) if accumulate else out.copy_(w)
        w = out
    return w


# ----------------------------------------------------------- normalisation layers
def affine_grad_sample(xhat, g, keep_last=0, channel_dim=False, want_weight=True, want_bias=True):
    return _ref.affine_grad_sample(xhat, g, keep_last, channel_dim, want_weight, want_bias)


def norm_affine_grad_sample(kind, x, g, *, eps, normalized_ndim=1, num_groups=1, want_weight=True, want_bias=True):
    """Per-sample affine-parameter gradients of a normalisation layer from its
    *input* ``x``: the normalised activation is recomputed inside the kernel, in
    one pass over ``x`` and ``g``.  ``kind`` is ``"layer"``, ``"rms"``,
    ``"group"`` or ``"instance"``."""
    if _on_gpu(x, g) and _kernel_dtype(g) and g.shape[0] > 0:
        if kind in ("layer", "rms") and normalized_ndim > 1 and x.dim() > normalized_ndim:
            # normalising over the last k axes = normalising over one flattened axis
            lead = x.shape[: x.dim() - normalized_ndim]
            tail = x.shape[x.dim() - normalized_ndim:]
            if len(lead) == 1:
                lead = (lead[0], 1)
            xf, gf = x.reshape(*lead, -1), g.reshape(*lead, -1)
            gw, gb = _k().norm_affine_grad_sample(kind, xf, gf, eps, 1, num_groups, want_weight, want_bias)
            shape = (x.shape[0],) + tuple(tail)
            return (gw.reshape(shape) if gw is not None else None), (gb.reshape(shape) if gb is not None else None)
        if _k().supports_norm(kind, x, normalized_ndim):
            return _k().norm_affine_grad_sample(kind, x, g, eps, normalized_ndim, num_groups, want_weight, want_bias)
    import torch.nn.functional as F

    if kind == "layer":
        xhat = F.layer_norm(x, x.shape[x.dim() - normalized_ndim:], eps=eps)
        return _ref.affine_grad_sample(xhat, g, keep_last=normalized_ndim, want_weight=want_weight, want_bias=want_bias)
    if kind == "rms":
        xhat = F.rms_norm(x, x.shape[x.dim() - normalized_ndim:], eps=eps)
        return _ref.affine_grad_sample(xhat, g, keep_last=normalized_ndim, want_weight=want_weight, want_bias=False)
    if kind == "group":
        xhat = F.group_norm(x, num_groups, eps=eps)
    elif kind == "instance":
        xhat = F.instance_norm(x, eps=eps)
    else:
        raise ValueError(kind)
    return _ref.affine_grad_sample(xhat, g, channel_dim=True, want_weight=want_weight, want_bias=want_bias)


# --------------------------------------------------------------- clipping pieces
def clip_factor(norm_sq, max_grad_norm: float):
    if _on_gpu(norm_sq) and norm_sq.dtype == torch.float32 and norm_sq.numel() > 0:
        return _k().clip_factor(norm_sq, max_grad_norm)
    return _ref.clip_factor(norm_sq, max_grad_norm)


def _compact(gs):
    from .lazy import LazyEmbeddingGradSample

    return isinstance(gs, LazyEmbeddingGradSample) and not gs.is_materialized


def grad_sample_norm_sq(gs):
    if _compact(gs):
        return embedding_norm_sq(gs._ids, gs._g)
    if _on_gpu(gs) and _kernel_dtype(gs) and gs.shape[0] > 0:
        return _k().grad_sample_norm_sq(gs)
    return _ref.grad_sample_norm_sq(gs)


def weighted_sum(gs, c, out=None):
    """``sum_n c[n] gs[n]``; ``out`` (optional, shape of one sample's gradient) is overwritten with it."""
    if _compact(gs):
        res = embedding_weighted_grad(gs._ids, gs._g, c.float(), gs._num_embeddings, out_dtype=gs.dtype)
        if out is not None:
            out.copy_(res.view(out.shape))
            return out
        return res
    if _on_gpu(gs) and _kernel_dtype(gs) and gs.shape[0] > 0:
        return _k().weighted_sum(gs, c, out=out)
    res = _ref.weighted_sum(gs, c)
    if out is not None:
        out.copy_(res.view(out.shape))
        return out
    return res


gaussian_like = _ref.gaussian_like
