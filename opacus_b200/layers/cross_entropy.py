"""Cross entropy over a large vocabulary straight from 16-bit logits.

``FusedCrossEntropyLoss`` is a drop-in criterion for ``[N, V]`` logits and
``[N]`` targets: on the GPU one kernel reads the logits once and produces the
per-token losses (online softmax), one kernel produces the gradient in the
logits' own precision -- no fp32 copy of the ``[N, V]`` matrix is ever made.
It exposes ``reduction`` and ``ignore_index`` the way
``DPLossFastGradientClipping`` expects from a criterion
(``opacus/utils/fast_gradient_clipping_utils.py:224-262``).  CPU tensors take
``torch.nn.functional.cross_entropy`` in fp32.
"""
import torch
import torch.nn as nn
import torch.nn.functional as F


class _FusedCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, target, ignore_index):
        from ..ops import _cuda

        logits = logits.contiguous()
        target = target.contiguous()
        loss, lse = _cuda.load().cross_entropy_forward(logits, target, int(ignore_index))
        ctx.save_for_backward(logits, target, lse)
        ctx.ignore_index = int(ignore_index)
        return loss

    @staticmethod
    def backward(ctx, g):
        from ..ops import _cuda

        logits, target, lse = ctx.saved_tensors
        dx = _cuda.load().cross_entropy_backward(logits, target, lse, g.float().contiguous(), ctx.ignore_index)
        return dx, None, None


def fused_cross_entropy(logits: torch.Tensor, target: torch.Tensor, ignore_index: int = -100) -> torch.Tensor:
    """Per-token losses ``[N]`` (fp32) for ``logits [N, V]``, ``target [N]``."""
    if logits.is_cuda and logits.dim() == 2 and logits.dtype in (torch.float32, torch.bfloat16, torch.float16):
        return _FusedCE.apply(logits, target, ignore_index)
    return F.cross_entropy(logits.float(), target, ignore_index=ignore_index, reduction="none")


class FusedCrossEntropyLoss(nn.Module):
    def __init__(self, reduction: str = "mean", ignore_index: int = -100):
        super().__init__()
        if reduction not in ("none", "mean", "sum"):
            raise ValueError(f"unknown reduction {reduction!r}")
        self.reduction = reduction
        self.ignore_index = ignore_index

    def forward(self, logits: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
        loss = fused_cross_entropy(logits, target, self.ignore_index)
        if self.reduction == "none":
            return loss
        if self.reduction == "sum":
            return loss.sum()
        return loss.sum() / (target != self.ignore_index).sum().clamp(min=1)
