"""Loss-side half of ghost clipping.

``DPLossFastGradientClipping`` wraps a criterion so that it returns per-sample
losses packaged in a ``DPTensorFastGradientClipping``; calling ``.backward()``
on that object leaves ``sum_n c_n grad(loss_n)`` in ``param.grad``.

With a single-pass module that takes one backward pass followed by
``module.finish_single_pass()``; otherwise the classic two passes
(norms, then the re-weighted loss with hooks disabled) are run.

Behavioural parity: ``opacus/utils/fast_gradient_clipping_utils.py:26-276``.
"""
import torch

from .tracing import phase


class DPTensorFastGradientClipping:
    """Per-sample losses with scalar-tensor manners (``item``, ``detach``,
    arithmetic) and a privacy-aware ``backward``."""

    def __init__(self, module, optimizer, loss_per_sample: torch.Tensor, loss_reduction: str = "mean"):
        self.module = module
        self.optimizer = optimizer
        self.loss_per_sample = loss_per_sample
        self.loss_reduction = loss_reduction

    # ---- tensor-like surface
    def _like(self, per_sample):
        return DPTensorFastGradientClipping(self.module, self.optimizer, per_sample, self.loss_reduction)

    def _reduced(self):
        if self.loss_reduction == "mean":
            return torch.mean(self.loss_per_sample, dim=0)
        if self.loss_reduction == "sum":
            return torch.sum(self.loss_per_sample, dim=0)
        raise ValueError(
            f"loss_reduction = {self.loss_reduction}. Only 'sum' and 'mean' losses are supported")

    def item(self):
        return self.detach().item()

    def detach(self):
        return self._reduced().detach()

    def _other(self, other, verb):
        if isinstance(other, DPTensorFastGradientClipping):
            if other.loss_reduction != self.loss_reduction:
                raise ValueError(
                    f"Cannot {verb} losses with different reductions: {self.loss_reduction} vs {other.loss_reduction}")
            return other.loss_per_sample
        return other

    def __truediv__(self, other):
        return self._like(self.loss_per_sample / other)

    def __mul__(self, other):
        return self._like(self.loss_per_sample * other)

    __rmul__ = __mul__

    def __add__(self, other):
        return self._like(self.loss_per_sample + self._other(other, "add"))

    __radd__ = __add__

    def __sub__(self, other):
        return self._like(self.loss_per_sample - self._other(other, "subtract"))

    def __rsub__(self, other):
        return self._like(other - self.loss_per_sample)

    def __neg__(self):
        return self._like(-self.loss_per_sample)

    def __repr__(self):
        return f"DPTensorFastGradientClipping(loss_reduction={self.loss_reduction}, shape={self.loss_per_sample.shape})"

    def __str__(self):
        return f"DPTensorFastGradientClipping({self.item():.4f})"

    # ---- the point of the class
    def _coefficients(self):
        return self.module.get_clipping_coef()

    def backward(self):
        reduced = self._reduced()
        if getattr(self.module, "single_pass", False):
            self.optimizer.zero_grad()
            with phase("dp/backward"):
                reduced.backward()
            self._before_finish()
            self.module.finish_single_pass()
            return
        reduced.backward(retain_graph=True)
        self.optimizer.zero_grad()
        coeff = self._coefficients()
        second = torch.sum(coeff.to(self.loss_per_sample.device) * self.loss_per_sample)
        self.module.disable_hooks()
        try:
            second.backward()
        finally:
            self.module.enable_hooks()

    def _before_finish(self):
        """Hook for subclasses that adjust the bound between norms and clipping."""


class DPLossFastGradientClipping:
    def __init__(self, module, optimizer, criterion, loss_reduction: str = "mean"):
        assert loss_reduction in ("mean", "sum"), "loss_reduction should be either 'mean' or 'sum'"
        if not hasattr(criterion, "reduction"):
            criterion.reduction = module.loss_reduction
        assert loss_reduction == criterion.reduction == module.loss_reduction == optimizer.loss_reduction, (
            "loss_reduction should be the same across GradSampleModule, Optimizer, Criterion, and loss_reduction")
        self.optimizer = optimizer
        self.module = module
        self.criterion = criterion
        self.loss_reduction = loss_reduction

    def _per_sample(self, *args, shape=None, **kwargs) -> torch.Tensor:
        """Un-reduced criterion output; with ``shape=(B, T, ...)`` a flat
        ``[B*T]`` token loss is folded to one value per sequence (mean respects
        the criterion's ``ignore_index``)."""
        saved = self.criterion.reduction
        self.criterion.reduction = "none"
        try:
            loss = self.criterion(*args, **kwargs)
        finally:
            self.criterion.reduction = saved
        if shape is None or loss.shape[0] != shape[0] * shape[1]:
            return loss
        loss = loss.view(shape[0], shape[1])
        if self.loss_reduction == "sum":
            return loss.sum(dim=1)
        if self.loss_reduction != "mean":
            raise ValueError(
                f"loss_reduction = {self.loss_reduction}. Only 'sum' and 'mean' losses are supported")
        ignore = getattr(self.criterion, "ignore_index", None)
        if ignore is not None and (len(args) >= 2 or "target" in kwargs):
            targets = kwargs["target"] if "target" in kwargs else args[1]
            valid = (targets.view(shape[0], shape[1]) != ignore).sum(dim=1).clamp(min=1)
            return loss.sum(dim=1) / valid
        return loss.mean(dim=1)

    def __call__(self, *args, shape=None, **kwargs) -> DPTensorFastGradientClipping:
        return DPTensorFastGradientClipping(
            self.module, self.optimizer, self._per_sample(*args, shape=shape, **kwargs), self.loss_reduction)
