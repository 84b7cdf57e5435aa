"""Plain-PyTorch statements of every per-sample operation.

They run on any device and dtype, are the path taken for CPU tensors, and are
the oracle the CUDA kernels are tested against.  Shapes: ``B`` samples, ``T``
positions per sample (any number of middle axes, flattened), ``a`` activations
``[B, T, d_in]``, ``g`` output gradients ``[B, T, d_out]``.
"""
import math
from typing import Optional, Tuple

import torch


def _bt(x: torch.Tensor) -> torch.Tensor:
    """View as ``[B, T, d]`` (``T = 1`` for 2-d input)."""
    if x.dim() == 2:
        return x.unsqueeze(1)
    if x.shape[0] == 0:
        return x.new_zeros(0, 1, x.shape[-1])
    return x.reshape(x.shape[0], -1, x.shape[-1])


# ----------------------------------------------------------------------- Linear
def linear_grad_sample(a: torch.Tensor, g: torch.Tensor) -> torch.Tensor:
    """Per-sample weight gradient ``gs[n] = g[n]^T a[n]`` -> ``[B, d_out, d_in]``."""
    return torch.bmm(_bt(g).transpose(1, 2), _bt(a).to(g.dtype))


def linear_bias_grad_sample(g: torch.Tensor) -> torch.Tensor:
    """``[B, d_out]``: sum of ``g`` over positions."""
    return _bt(g).sum(dim=1)


def linear_norm_sq(a: torch.Tensor, g: torch.Tensor, want_weight: bool = True, want_bias: bool = False,
                   g_scale: float = 1.0) -> Tuple[Optional[torch.Tensor], Optional[torch.Tensor]]:
    """Squared Frobenius norm of each per-sample weight (and bias) gradient
    without forming the gradients where that is cheaper.

    ``||g^T a||_F^2 = <a a^T, g g^T>`` costs ``2 T^2 (d_in + d_out)`` against
    ``2 T d_in d_out`` for the direct product; the cheaper one is used.
    Accumulation is in fp32 (fp64 for fp64 input).
    """
    a3, g3 = _bt(a), _bt(g)
    acc = torch.float64 if g3.dtype == torch.float64 else torch.float32
    B, T, d_in = a3.shape
    d_out = g3.shape[-1]
    w = b = None
    s2 = float(g_scale) ** 2
    if want_weight:
        if T == 1:
            w = a3.to(acc).pow(2).sum(dim=(1, 2)) * g3.to(acc).pow(2).sum(dim=(1, 2))
        elif T * (d_in + d_out) <= d_in * d_out:
            aa = torch.bmm(a3, a3.transpose(1, 2)).to(acc)
            gg = torch.bmm(g3, g3.transpose(1, 2)).to(acc)
            w = (aa * gg).sum(dim=(1, 2)).clamp_(min=0)
        else:
            w = torch.bmm(g3.transpose(1, 2), a3.to(g3.dtype)).to(acc).pow(2).sum(dim=(1, 2))
        w = w * s2
    if want_bias:
        b = g3.to(acc).sum(dim=1).pow(2).sum(dim=1) * s2
    return w, b


def linear_weighted_grad(a: torch.Tensor, g: torch.Tensor, c: torch.Tensor, g_scale: float = 1.0,
                         want_bias: bool = False):
    """``sum_n c[n] g[n]^T a[n]`` (``[d_out, d_in]``) and optionally the same
    for the bias: one GEMM with contraction length ``B*T``."""
    a3, g3 = _bt(a), _bt(g)
    gw = g3 * (c.to(g3.dtype) * g_scale)[:, None, None]
    w = gw.reshape(-1, gw.shape[-1]).t() @ a3.reshape(-1, a3.shape[-1]).to(gw.dtype)
    b = gw.sum(dim=(0, 1)) if want_bias else None
    return w, b


# -------------------------------------------------------------------- Embedding
def embedding_grad_sample(ids: torch.Tensor, g: torch.Tensor, num_embeddings: int) -> torch.Tensor:
    """Dense per-sample gradient ``[B, V, D]`` (scatter-add of ``g`` rows)."""
    B = ids.shape[0]
    D = g.shape[-1]
    out = torch.zeros(B, num_embeddings, D, dtype=g.dtype, device=g.device)
    if B:
        idx = ids.reshape(B, -1, 1).expand(-1, -1, D)
        out.scatter_add_(1, idx, g.reshape(B, -1, D))
    return out


def embedding_norm_sq(ids: torch.Tensor, g: torch.Tensor, g_scale: float = 1.0,
                      padding_idx: Optional[int] = None) -> torch.Tensor:
    """``sum_v || sum_{t: id_t = v} g_t ||^2`` per sample, computed as
    ``<[id_t == id_s], g g^T>`` -- no sort, no unique, no host sync."""
    B = ids.shape[0]
    ids2 = ids.reshape(B, -1)
    g3 = g.reshape(B, ids2.shape[1], -1)
    acc = torch.float64 if g3.dtype == torch.float64 else torch.float32
    gg = torch.bmm(g3, g3.transpose(1, 2)).to(acc)
    same = ids2[:, :, None] == ids2[:, None, :]
    if padding_idx is not None:
        keep = ids2 != padding_idx
        same = same & keep[:, :, None] & keep[:, None, :]
    return (gg * same).sum(dim=(1, 2)).clamp_(min=0) * float(g_scale) ** 2


def embedding_weighted_grad(ids: torch.Tensor, g: torch.Tensor, c: torch.Tensor, num_embeddings: int,
                            g_scale: float = 1.0, padding_idx: Optional[int] = None,
                            out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """``sum_n c[n] * scatter(ids[n], g[n])`` -> ``[V, D]``."""
    B = ids.shape[0]
    D = g.shape[-1]
    dt = out_dtype or g.dtype
    out = torch.zeros(num_embeddings, D, dtype=dt, device=g.device)
    if B == 0:
        return out
    gw = (g.reshape(B, -1, D) * (c.to(g.dtype) * g_scale)[:, None, None]).reshape(-1, D).to(dt)
    flat = ids.reshape(-1)
    if padding_idx is not None:
        gw = gw * (flat != padding_idx).unsqueeze(-1).to(dt)
    out.index_add_(0, flat, gw)
    return out


# ----------------------------------------------------------- normalisation layers
def affine_grad_sample(xhat: torch.Tensor, g: torch.Tensor, keep_last: int = 0, channel_dim: bool = False,
                       want_weight: bool = True, want_bias: bool = True):
    """Per-sample gradients of an elementwise affine ``y = xhat * w + b``.

    ``channel_dim=True``: parameters are per channel (axis 1), reduce all later
    axes (GroupNorm, InstanceNorm).  Otherwise parameters have the shape of the
    last ``keep_last`` axes and every axis between batch and those is reduced
    (LayerNorm, RMSNorm).
    """
    def red(t):
        if channel_dim:
            return t.sum(dim=list(range(2, t.dim()))) if t.dim() > 2 else t
        mid = t.dim() - keep_last - 1
        return t if mid == 0 else t.sum(dim=list(range(1, 1 + mid)))

    w = red(xhat * g) if want_weight else None
    b = red(g) if want_bias else None
    return w, b


# --------------------------------------------------------------- clipping pieces
def clip_factor(norm_sq: torch.Tensor, max_grad_norm: float) -> torch.Tensor:
    """``min(1, C / (sqrt(norm_sq) + 1e-6))``."""
    return (max_grad_norm / (norm_sq.clamp(min=0).sqrt() + 1e-6)).clamp(max=1.0)


def grad_sample_norm_sq(gs: torch.Tensor) -> torch.Tensor:
    acc = torch.float64 if gs.dtype == torch.float64 else torch.float32
    if gs.shape[0] == 0:
        return torch.zeros(0, dtype=acc, device=gs.device)
    # no temporary of the size of gs
    return torch.linalg.vector_norm(gs.reshape(gs.shape[0], -1), dim=1, dtype=acc).square()


def weighted_sum(gs: torch.Tensor, c: torch.Tensor) -> torch.Tensor:
    """``sum_n c[n] gs[n]``."""
    if gs.shape[0] == 0:
        return torch.zeros(gs.shape[1:], dtype=gs.dtype, device=gs.device)
    return torch.einsum("i,i...", c.to(gs.dtype), gs)


# ------------------------------------------------------------- noise + optimiser
def gaussian_like(ref: torch.Tensor, std: float, generator=None, secure_mode: bool = False) -> torch.Tensor:
    """``N(0, std^2)`` with the shape/device/dtype of ``ref``.  ``secure_mode``
    sums four draws (after discarding one) and halves, which removes the
    floating-point artefacts a single draw exposes (Mironov 2012)."""
    if std == 0:
        return torch.zeros_like(ref)
    if getattr(generator, "gaussian_like", None) is not None:
        # this package's ChaCha20 generator (utils/secure_rng.py): it implements the draw rule itself, on either device
        return generator.gaussian_like(ref, std, draws=4 if secure_mode else 1)
    if not secure_mode:
        return torch.normal(mean=0, std=std, size=ref.shape, device=ref.device, dtype=ref.dtype, generator=generator)
    torch.normal(mean=0, std=std, size=(1, 1), device=ref.device, generator=generator)
    total = torch.zeros_like(ref)
    for _ in range(4):
        total += torch.normal(mean=0, std=std, size=ref.shape, device=ref.device, generator=generator).to(ref.dtype)
    return total / 2


def dp_sgd_step(param, summed_grad, momentum_buf, *, noise_std, inv_scale, lr, momentum=0.0, dampening=0.0,
                weight_decay=0.0, nesterov=False, first_step=False, generator=None):
    """param <- SGD(param, (summed_grad + N(0, noise_std^2)) * inv_scale).  In place."""
    grad = (summed_grad + gaussian_like(summed_grad, noise_std, generator)).to(param.dtype) * inv_scale
    if weight_decay:
        grad = grad.add(param, alpha=weight_decay)
    if momentum:
        if first_step:
            momentum_buf.copy_(grad)
        else:
            momentum_buf.mul_(momentum).add_(grad, alpha=1 - dampening)
        grad = grad.add(momentum_buf, alpha=momentum) if nesterov else momentum_buf
    param.add_(grad, alpha=-lr)


def dp_adam_step(param, summed_grad, exp_avg, exp_avg_sq, *, step, noise_std, inv_scale, lr, beta1, beta2, eps,
                 weight_decay=0.0, decoupled=True, generator=None):
    """Adam / AdamW on ``(summed_grad + noise) * inv_scale``.  In place."""
    grad = (summed_grad + gaussian_like(summed_grad, noise_std, generator)).to(exp_avg.dtype) * inv_scale
    p32 = param.to(exp_avg.dtype)
    if weight_decay:
        if decoupled:
            p32 = p32 * (1 - lr * weight_decay)
        else:
            grad = grad.add(p32, alpha=weight_decay)
    exp_avg.mul_(beta1).add_(grad, alpha=1 - beta1)
    exp_avg_sq.mul_(beta2).addcmul_(grad, grad, value=1 - beta2)
    bc1 = 1 - beta1 ** step
    bc2 = 1 - beta2 ** step
    denom = (exp_avg_sq.sqrt() / math.sqrt(bc2)).add_(eps)
    p32 = p32.addcdiv(exp_avg, denom, value=-lr / bc1)
    param.copy_(p32)
