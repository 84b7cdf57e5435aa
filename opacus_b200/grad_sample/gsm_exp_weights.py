""""ew" mode: per-sample gradients through PyTorch's ExpandedWeights
(``opacus/grad_sample/gsm_exp_weights.py:21-55``)."""
import torch
import torch.nn as nn

from .gsm_base import AbstractGradSampleModule


class GradSampleModuleExpandedWeights(AbstractGradSampleModule):
    def __init__(self, m: nn.Module, *, batch_first=True, loss_reduction="mean"):
        if not batch_first:
            raise NotImplementedError
        super().__init__(m, batch_first=batch_first, loss_reduction=loss_reduction)

    def forward(self, x: torch.Tensor, *args, **kwargs):
        from torch.nn.utils._per_sample_grad import call_for_per_sample_grads

        run = call_for_per_sample_grads(module=self._module, batch_size=x.shape[0],
                                        loss_reduction=self.loss_reduction)
        return run(x, *args, **kwargs)

    def remove_hooks(self) -> None:
        pass
