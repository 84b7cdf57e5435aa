"""RMSNorm fused with the residual addition in front of it.

A pre-norm decoder block computes ``h = h + branch`` and at once ``y = rms_norm(h) * w``.  As two
statements that is five passes over ``[rows, D]`` each way; ``AddRMSNorm`` does both in one kernel each
way (``csrc/rmsnorm.cu``): the forward pass reads the two summands and writes ``h`` and ``y``; the backward
pass reads ``dy``, the gradient that reaches ``h`` through the residual path, and ``h``, and writes the one
gradient both summands receive.

The parameter is the ``weight`` of ``nn.RMSNorm`` (same name, same shape), so state dicts interchange, and
the per-sample gradient rule is the RMSNorm rule (``opacus/grad_sample/rms_norm.py:27-48``) applied to the
sum ``h``, which the hooks read from the module's second output (``dp_activation_output``).
"""
from typing import Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

_KERNEL_DTYPES = (torch.bfloat16, torch.float16, torch.float32)


def _weight_grad(dy, h, rstd):
    D = h.shape[-1]
    return (dy.reshape(-1, D).float() * h.reshape(-1, D).float() * rstd[:, None]).sum(0)


class _NormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps):
        from ..ops import _cuda

        x = x.contiguous()
        y, _, rstd = _cuda.load().add_rmsnorm_forward(x, None, w, eps)
        ctx.save_for_backward(x, rstd, w)
        return y

    @staticmethod
    def backward(ctx, dy):
        from ..ops import _cuda

        x, rstd, w = ctx.saved_tensors
        dy = dy.contiguous()
        dx = _cuda.load().add_rmsnorm_backward(dy, None, x, rstd, w) if ctx.needs_input_grad[0] else None
        dw = _weight_grad(dy, x, rstd).to(w.dtype) if ctx.needs_input_grad[1] else None
        return dx, dw, None


class _AddNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, delta, w, eps):
        from ..ops import _cuda

        y, h, rstd = _cuda.load().add_rmsnorm_forward(x.contiguous(), delta.contiguous(), w, eps)
        ctx.save_for_backward(h, rstd, w)
        return y, h

    @staticmethod
    def backward(ctx, dy, dres):
        from ..ops import _cuda

        h, rstd, w = ctx.saved_tensors
        if dy is None:
            return dres, dres, None, None
        dy = dy.contiguous()
        dres = dres.contiguous() if dres is not None else None
        dh = _cuda.load().add_rmsnorm_backward(dy, dres, h, rstd, w)
        dw = _weight_grad(dy, h, rstd).to(w.dtype) if ctx.needs_input_grad[2] else None
        return dh, dh, dw, None


class AddRMSNorm(nn.RMSNorm):
    """``forward(x, delta=None) -> (rms_norm(x + delta) * weight, x + delta)``."""

    dp_activation_output = 1      # the DP hooks take the sum (second output) as the activation of ``weight``

    def forward(self, x: torch.Tensor, delta: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        eps = self.eps if self.eps is not None else torch.finfo(x.dtype).eps
        D = x.shape[-1]
        fused = (x.is_cuda and x.dtype in _KERNEL_DTYPES and self.weight is not None and self.weight.dtype == x.dtype
                 and len(self.normalized_shape) == 1 and D % 8 == 0 and D <= 8192
                 and x.data_ptr() % 16 == 0
                 and (delta is None or (delta.shape == x.shape and delta.dtype == x.dtype
                                        and delta.data_ptr() % 16 == 0)))
        if fused:
            if delta is None:
                h, y = x, _NormFn.apply(x, self.weight, eps)
            else:
                y, h = _AddNormFn.apply(x, delta, self.weight, eps)
        else:
            h = x if delta is None else x + delta
            y = F.rms_norm(h, self.normalized_shape, self.weight, eps)
        return y, h
