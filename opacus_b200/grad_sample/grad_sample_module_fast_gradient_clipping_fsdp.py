"""Ghost clipping for sharded data-parallel training ("ghost_fsdp").

Two kinds of model are accepted:

* a model prepared by this package's sharded engine
  (:class:`opacus_b200.parallel.sharded.ShardedDataParallel`): parameters stay
  whole on every GPU in compute precision while master weights and optimiser
  state are sharded; the single-pass ghost path runs unchanged and the optimiser
  performs the reduce-scatter, noise, update and all-gather in one fused kernel;
* a model wrapped with ``torch.distributed.fsdp.fully_shard``: parameter
  *objects* are swapped by FSDP2 between sharded and gathered forms, so no state
  can live on them.  The classic two-pass protocol is used and per-call state is
  kept on the **module** (``module.norm_sample``, ``module._forward_counter``).

Samplers only read activations, output gradients and layer hyper-parameters,
never the weights, so parameter sharding is irrelevant to them.

Behavioural parity: ``opacus/grad_sample/grad_sample_module_fast_gradient_clipping_fsdp.py:36-261``.
"""
from __future__ import annotations

import logging
from typing import List

import torch
import torch.nn as nn

from .. import ops
from ..utils.module_utils import requires_grad, trainable_parameters
from .functorch import ft_compute_per_sample_gradient
from .grad_sample_module import captured_inputs
from .grad_sample_module_fast_gradient_clipping import GradSampleHooksFastGradientClipping
from .gsm_base import AbstractGradSampleModule

logger = logging.getLogger(__name__)
logger.disabled = True


def _is_torch_fsdp(module: nn.Module) -> bool:
    try:
        from torch.distributed.fsdp import FSDPModule
    except Exception:  # pragma: no cover - torch built without distributed
        return False
    return any(isinstance(m, FSDPModule) for m in module.modules())


class GradSampleHooksFastGradientClippingFSDP(GradSampleHooksFastGradientClipping):
    def __init__(self, m: nn.Module, *, batch_first: bool = True, loss_reduction="mean", strict: bool = True,
                 max_grad_norm=1, single_pass=None):
        self._torch_fsdp = _is_torch_fsdp(m)
        if single_pass is None:
            single_pass = not self._torch_fsdp
        if single_pass and self._torch_fsdp:
            raise ValueError("single_pass ghost clipping cannot drive a torch fully_shard model; use the "
                             "ShardedDataParallel engine or single_pass=False")
        super().__init__(m, batch_first=batch_first, loss_reduction=loss_reduction, strict=strict,
                         force_functorch=False, max_grad_norm=max_grad_norm, use_ghost_clipping=True,
                         single_pass=single_pass)
        if getattr(m, "_row_layers", None):
            # row-sharded layers are stepped one after the other through one set of flag words: one stream
            self.overlap_clipped_sums = False

    def _get_module_type(self, module: nn.Module):
        """``fully_shard`` turns ``Linear`` into ``FSDPLinear(FSDPModule, Linear)``."""
        t = type(module)
        if self._torch_fsdp:
            from torch.distributed.fsdp import FSDPModule

            if isinstance(module, FSDPModule):
                return t.__bases__[1]
        return t

    def get_norm_sample(self) -> torch.Tensor:
        if self.single_pass:
            return super().get_norm_sample()
        pieces = [n for sub in self.iterate_submodules(self._module) for n in getattr(sub, "norm_sample", [])]
        norm = torch.stack(pieces, dim=0).norm(2, dim=0)
        self.per_sample_gradient_norms = norm
        return norm

    def capture_activations_hook(self, module: nn.Module, forward_input: List[torch.Tensor], _forward_output):
        if not self.hooks_enabled or not module.training or not torch.is_grad_enabled() or not requires_grad(module):
            return
        if not hasattr(module, "activations"):
            module.activations = []
        module.activations.append(captured_inputs(module, forward_input, _forward_output))
        module._forward_counter = getattr(module, "_forward_counter", 0) + 1
        if self.use_ghost_clipping and module._forward_counter > 1:
            raise NotImplementedError("Parameter tying is not supported with FSDP")

    def capture_backprops_hook(self, module: nn.Module, _forward_input, forward_output, loss_reduction: str,
                               batch_first: bool):
        if not self.hooks_enabled:
            return
        backprops = forward_output[0].detach()
        activations, backprops = self.rearrange_grad_samples(
            module=module, backprops=backprops, loss_reduction=loss_reduction, batch_first=batch_first)
        activations = [t.to_local() if hasattr(t, "to_local") else t for t in activations]
        mtype = self._get_module_type(module)
        module._forward_counter -= 1
        if self.use_ghost_clipping and mtype in self.NORM_SAMPLERS:
            norms = [v for p, v in self.NORM_SAMPLERS[mtype](module, activations, backprops).items()
                     if p.requires_grad]
        else:
            sampler = self.GRAD_SAMPLERS[mtype] if mtype in self.GRAD_SAMPLERS else ft_compute_per_sample_gradient
            norms = [ops.grad_sample_norm_sq(gs).sqrt().to(gs.dtype)
                     for gs in sampler(module, activations, backprops).values()]
        module.norm_sample = norms
        if len(module.activations) == 0 and hasattr(module, "max_batch_len"):
            del module.max_batch_len


class GradSampleModuleFastGradientClippingFSDP(GradSampleHooksFastGradientClippingFSDP, AbstractGradSampleModule):
    def __init__(self, m: nn.Module, *, batch_first: bool = True, loss_reduction="mean", strict: bool = True,
                 force_functorch=False, max_grad_norm=1, use_ghost_clipping: bool = True, single_pass=None):
        nn.Module.__init__(self)
        GradSampleHooksFastGradientClippingFSDP.__init__(
            self, m, batch_first=batch_first, loss_reduction=loss_reduction, strict=strict,
            max_grad_norm=max_grad_norm, single_pass=single_pass)
        self.grad_accumulation_hook = None
