""""no_op" mode: only the parameter attributes are managed; the caller fills
``p.grad_sample`` (e.g. with a whole-model ``vmap(grad(.))``)
(``opacus/grad_sample/gsm_no_op.py:24-75``)."""
import torch
import torch.nn as nn

from .gsm_base import AbstractGradSampleHooks, AbstractGradSampleModule


class GradSampleHooksNoOp(AbstractGradSampleHooks):
    def __init__(self, m: nn.Module, *, batch_first=True, loss_reduction="mean"):
        if not batch_first:
            raise NotImplementedError
        super().__init__(m, batch_first=batch_first, loss_reduction=loss_reduction)

    def remove_hooks(self) -> None:
        pass


class GradSampleModuleNoOp(GradSampleHooksNoOp, AbstractGradSampleModule):
    def __init__(self, m: nn.Module, *, batch_first=True, loss_reduction="mean"):
        nn.Module.__init__(self)
        GradSampleHooksNoOp.__init__(self, m, batch_first=batch_first, loss_reduction=loss_reduction)
        self.grad_accumulation_hook = None

    def forward(self, x: torch.Tensor, *args, **kwargs):
        return self._module.forward(x, *args, **kwargs)
