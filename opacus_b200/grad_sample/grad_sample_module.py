"""Hook-driven per-sample gradient engine ("hooks" and "functorch" modes).

A forward hook stores the (detached) inputs of every layer that directly owns
trainable parameters; a backward hook receives the gradient w.r.t. the layer's
output and calls that layer type's *sampler* ``(layer, activations, backprops)
-> {param: per_sample_grad}``.  Results are summed into
``param._current_grad_sample`` (a layer may run several times per forward pass:
recurrent steps, tied weights) and become ``param.grad_sample`` once every
forward use has been matched by a backward call.  ``grad_sample`` turns into a
list when several batches are accumulated without ``zero_grad``.

Repeated calls of a recurrent cell's linear map are not turned into ``T``
rank-one updates: their ``(activation, backprop)`` pairs are queued and
contracted once, as a single GEMM with ``K = T`` (see ``_STACKED_TYPES``).

Behavioural parity: ``opacus/grad_sample/grad_sample_module.py:43-573``.
"""
from __future__ import annotations

import logging
import warnings
from functools import partial
from typing import Iterable, List, Tuple

import torch
import torch.nn as nn

from ..layers.dp_rnn import DPGRU, DPLSTM, DPRNN, RNNLinear
from ..utils.module_utils import has_trainable_params, requires_grad, trainable_modules, trainable_parameters
from .functorch import ft_compute_per_sample_gradient, prepare_layer
from .gsm_base import AbstractGradSampleHooks, AbstractGradSampleModule

logger = logging.getLogger(__name__)
logger.disabled = True

_RNN_CONTAINERS = (DPRNN, DPLSTM, DPGRU)
# Layer types whose repeated calls inside one forward pass are time steps over
# the same samples and may be stacked along a new position axis.
_STACKED_TYPES = (RNNLinear,)


def create_or_accumulate_grad_sample(*, param: torch.Tensor, grad_sample: torch.Tensor, max_batch_len: int) -> None:
    """Add ``grad_sample`` (possibly shorter than ``max_batch_len`` rows, e.g. a
    late step of a packed sequence) into ``param._current_grad_sample``."""
    if not param.requires_grad:
        return
    n = grad_sample.shape[0]
    cur = getattr(param, "_current_grad_sample", None)
    if cur is None:
        if n == max_batch_len:
            # adopted as is (possibly a view of a tensor the sampler made); copied only if
            # a second contribution has to be added in place
            param._current_grad_sample = grad_sample
            return
        cur = torch.zeros((max_batch_len,) + tuple(grad_sample.shape[1:]), device=grad_sample.device,
                          dtype=grad_sample.dtype)
        cur._dp_owned = True
        param._current_grad_sample = cur
    elif not getattr(cur, "_dp_owned", False):
        cur = cur.clone()
        cur._dp_owned = True
        param._current_grad_sample = cur
    if hasattr(cur, "_dp_norm_sq"):
        del cur._dp_norm_sq          # a norm computed for the first contribution no longer holds
    cur[:n] += grad_sample


def promote_current_grad_sample(p: nn.Parameter) -> None:
    """Move the finished ``_current_grad_sample`` to ``grad_sample``."""
    if not p.requires_grad:
        return
    done = p._current_grad_sample
    if p.grad_sample is None:
        p.grad_sample = done
    elif isinstance(p.grad_sample, list):
        p.grad_sample.append(done)
    else:
        p.grad_sample = [p.grad_sample, done]
    del p._current_grad_sample


def _pad_rows(t: torch.Tensor, n: int) -> torch.Tensor:
    if t.shape[0] == n:
        return t
    return torch.cat([t, t.new_zeros((n - t.shape[0],) + tuple(t.shape[1:]))], dim=0)


class _OutputTap(torch.autograd.Function):
    """Identity on a layer's output whose backward hands the output gradient to
    the controller.  ``anchor`` is a dummy that requires grad so that the tap is
    part of the graph even when nothing upstream requires grad (first layer)."""

    @staticmethod
    def forward(ctx, out, anchor, controller, module):
        ctx.controller = controller
        ctx.module = module
        return out.view_as(out)

    @staticmethod
    def backward(ctx, grad_out):
        ctx.controller._on_output_grad(ctx.module, grad_out)
        return grad_out, None, None, None


def captured_inputs(module, inputs, output):
    """What a forward hook keeps for the per-sample rules: the detached inputs.  A module whose parameters
    act on a tensor it computes itself and also returns (a fused residual add) names that output by
    ``dp_activation_output``; it then stands in for the first input."""
    kept = [t.detach() if isinstance(t, torch.Tensor) else t for t in inputs]
    index = getattr(module, "dp_activation_output", None)
    if index is not None and isinstance(output, (tuple, list)):
        kept[0] = output[index].detach()
    return kept


class GradSampleHooks(AbstractGradSampleHooks):
    GRAD_SAMPLERS = {}

    def __init__(self, m: nn.Module, *, batch_first=True, loss_reduction="mean", strict: bool = True,
                 force_functorch=False, skip_param_grads: bool = False, early_capture: bool = False):
        # early_capture: per-sample gradients are computed when the gradient of a layer's OUTPUT arrives (a tap on
        # the output) instead of after the layer's own backward; parameters stay attached, so autograd still forms
        # their batch gradient -- afterwards.  Gradient hooks on parameters (per-layer clipping inside stock
        # DistributedDataParallel) then always find ``grad_sample`` in place.
        self.early_capture = early_capture
        # skip_param_grads: layers run with detached parameters, so autograd never computes the (non-private)
        # batch gradient of the weights -- a whole GEMM per layer that DP-SGD throws away.  ``p.grad`` then
        # stays None until the DP optimizer writes the private gradient.  Off by default (reference behaviour).
        self.skip_param_grads = skip_param_grads
        self._hook_args = dict(loss_reduction=loss_reduction, batch_first=batch_first)
        self._anchor = None
        super().__init__(m, batch_first=batch_first, loss_reduction=loss_reduction)
        errors = self.validate(module=m, strict=strict)
        if errors and not strict:
            logger.info(f"Validation found the following errors: {errors}.Using non-strict mode, continuing")
        self.hooks_enabled = False
        self.grad_accumulation_allowed = True
        self.force_functorch = force_functorch
        self.add_hooks(loss_reduction=loss_reduction, batch_first=batch_first, force_functorch=force_functorch)

    # ------------------------------------------------------------ instrumentation
    def iterate_submodules(self, module: nn.Module) -> Iterable[nn.Module]:
        """Modules to instrument: those owning trainable parameters directly.
        A module without a dedicated sampler is handled as one unit through
        functorch, so its children are not visited; the recurrent containers
        are transparent (their cells' linears are the units)."""
        own = has_trainable_params(module)
        if own:
            yield module
            if self._get_module_type(module) not in self.GRAD_SAMPLERS and type(module) not in _RNN_CONTAINERS:
                return
        for child in module.children():
            yield from self.iterate_submodules(child)

    def _get_module_type(self, module: nn.Module):
        return type(module)

    def _has_rule(self, module) -> bool:
        return not self.force_functorch and self._get_module_type(module) in self.GRAD_SAMPLERS

    def add_hooks(self, *, loss_reduction: str = "mean", batch_first: bool = True,
                  force_functorch: bool = False) -> None:
        if hasattr(self._module, "autograd_grad_sample_hooks"):
            raise ValueError("Trying to add hooks twice to the same model")
        handles = []
        self._module.autograd_grad_sample_hooks = handles
        self.autograd_grad_sample_hooks = handles
        for sub in self.iterate_submodules(self._module):
            if type(sub) in _RNN_CONTAINERS:
                continue
            if force_functorch or self._get_module_type(sub) not in self.GRAD_SAMPLERS:
                prepare_layer(sub, batch_first=batch_first)
            if self.skip_param_grads:
                handles.append(sub.register_forward_pre_hook(self._detach_params_pre_hook))
                handles.append(sub.register_forward_hook(self._tap_forward_hook, always_call=True))
                continue
            if self.early_capture:
                handles.append(sub.register_forward_hook(self._early_tap_forward_hook))
                continue
            handles.append(sub.register_forward_hook(self.capture_activations_hook))
            handles.append(sub.register_full_backward_hook(
                partial(self.capture_backprops_hook, loss_reduction=loss_reduction, batch_first=batch_first)))
        self.enable_hooks()

    # ---- skip_param_grads: detached parameters in forward, a tap on the output instead of a backward hook
    def _capturing(self, module) -> bool:
        return self.hooks_enabled and module.training and torch.is_grad_enabled() and requires_grad(module)

    def _detach_params_pre_hook(self, module, _inputs):
        if not self._capturing(module):
            return
        saved = []
        for sub in module.modules():
            for name, p in sub._parameters.items():
                if p is not None and p.requires_grad:
                    saved.append((sub, name, p))
                    sub._parameters[name] = p.detach()
        module.__dict__["_dp_saved_params"] = saved

    def _tap_forward_hook(self, module, inputs, output):
        saved = module.__dict__.pop("_dp_saved_params", None)
        if saved is None:
            return None
        for sub, name, p in saved:
            sub._parameters[name] = p
        if output is None:
            return None
        self.capture_activations_hook(module, inputs, output)
        first = output[0] if isinstance(output, (tuple, list)) else output
        if self._anchor is None or self._anchor.device != first.device:
            self._anchor = torch.zeros((), device=first.device, requires_grad=True)
        tapped = _OutputTap.apply(first, self._anchor, self, module)
        if isinstance(output, tuple):
            return (tapped,) + tuple(output[1:])
        if isinstance(output, list):
            return [tapped] + list(output[1:])
        return tapped

    def _early_tap_forward_hook(self, module, inputs, output):
        if not self._capturing(module) or output is None:
            return None
        self.capture_activations_hook(module, inputs, output)
        first = output[0] if isinstance(output, (tuple, list)) else output
        if self._anchor is None or self._anchor.device != first.device:
            self._anchor = torch.zeros((), device=first.device, requires_grad=True)
        tapped = _OutputTap.apply(first, self._anchor, self, module)
        if isinstance(output, tuple):
            return (tapped,) + tuple(output[1:])
        if isinstance(output, list):
            return [tapped] + list(output[1:])
        return tapped

    def _on_output_grad(self, module, grad_out):
        self.capture_backprops_hook(module, None, (grad_out,), **self._hook_args)

    def remove_hooks(self) -> None:
        self.disable_hooks()
        for p in self._module.parameters():
            if hasattr(p, "ddp_hooks"):
                while p.ddp_hooks:
                    p.ddp_hooks.pop().remove()
                delattr(p, "ddp_hooks")
        if hasattr(self, "autograd_grad_sample_hooks"):
            while self.autograd_grad_sample_hooks:
                self.autograd_grad_sample_hooks.pop().remove()
            delattr(self, "autograd_grad_sample_hooks")
            if hasattr(self._module, "autograd_grad_sample_hooks"):
                delattr(self._module, "autograd_grad_sample_hooks")
        for _, sub in trainable_modules(self._module):
            for attr in ("ft_compute_sample_grad", "activations", "max_batch_len", "_stacked_calls"):
                if attr in sub.__dict__:
                    delattr(sub, attr)

    def disable_hooks(self) -> None:
        """Switch capture off without touching the autograd graph (removing
        hooks from a graph that is already built is not reliable)."""
        self.hooks_enabled = False

    def enable_hooks(self) -> None:
        self.hooks_enabled = True

    # -------------------------------------------------------------------- hooks
    def capture_activations_hook(self, module: nn.Module, forward_input: List[torch.Tensor],
                                 _forward_output: torch.Tensor):
        if not self.hooks_enabled or not module.training or not torch.is_grad_enabled() or not requires_grad(module):
            return
        if not hasattr(module, "activations"):
            module.activations = []
        module.activations.append(captured_inputs(module, forward_input, _forward_output))
        for _, p in trainable_parameters(module):
            p._forward_counter += 1

    def capture_backprops_hook(self, module: nn.Module, _forward_input, forward_output, loss_reduction: str,
                               batch_first: bool):
        if not self.hooks_enabled:
            return
        backprops = forward_output[0].detach()
        activations, backprops = self.rearrange_grad_samples(
            module=module, backprops=backprops, loss_reduction=loss_reduction, batch_first=batch_first)
        own = module.__dict__.pop("_dp_activation", None)       # see _prepare_site of the ghost controller
        if own is not None:
            activations = [own.detach()] + list(activations[1:])

        if isinstance(module, _STACKED_TYPES) and self._has_rule(module):
            ready = self._queue_stacked_call(module, activations, backprops)
            if ready is None:
                return
            activations, backprops, uses = ready
        else:
            uses = 1

        sampler = self.GRAD_SAMPLERS[self._get_module_type(module)] if self._has_rule(module) \
            else ft_compute_per_sample_gradient
        for param, gs in sampler(module, activations, backprops).items():
            create_or_accumulate_grad_sample(param=param, grad_sample=gs, max_batch_len=module.max_batch_len)

        self._finish_backward_call(module, uses)

    def _queue_stacked_call(self, module, activations, backprops):
        """Defer one time step of a stacked layer type.  Returns ``None`` until
        the last pending call, then ``([A], G, n_calls)`` with ``A``/``G``
        stacked to ``[B, T, d]`` (short steps of packed sequences zero padded)."""
        a = activations[0]
        pending = module.__dict__.setdefault("_stacked_calls", [])
        if a.dim() != 2:  # already a whole sequence: nothing to stack
            if not pending:
                return activations, backprops, 1
        pending.append((a, backprops))
        if len(module.activations) > 0:
            return None
        del module._stacked_calls
        n = module.max_batch_len
        seq_a, seq_g, flat = [], [], []
        for a_t, g_t in pending:
            if a_t.dim() == 2:
                seq_a.append(_pad_rows(a_t, n))
                seq_g.append(_pad_rows(g_t, n))
            else:
                flat.append((a_t, g_t))
        A = torch.stack(seq_a, dim=1)
        G = torch.stack(seq_g, dim=1)
        for a_t, g_t in flat:
            A = torch.cat([A, _pad_rows(a_t, n)], dim=1)
            G = torch.cat([G, _pad_rows(g_t, n)], dim=1)
        return [A], G, len(pending)

    def _finish_backward_call(self, module, uses: int = 1):
        for _, p in trainable_parameters(module):
            p._forward_counter -= uses
            if p._forward_counter == 0:
                promote_current_grad_sample(p)
            if not self.grad_accumulation_allowed and isinstance(p.grad_sample, list) and len(p.grad_sample) > 1:
                raise ValueError(
                    "Poisson sampling is not compatible with grad accumulation. You need to call "
                    "optimizer.step() after every forward/backward pass or consider using BatchMemoryManager"
                )
        if len(module.activations) == 0 and hasattr(module, "max_batch_len"):
            del module.max_batch_len

    def rearrange_grad_samples(self, *, module: nn.Module, backprops: torch.Tensor, loss_reduction: str,
                               batch_first: bool) -> Tuple[List[torch.Tensor], torch.Tensor]:
        """Pop the matching activations, undo the ``1/B`` of a mean-reduced
        loss, and move the batch axis to the front."""
        if not hasattr(module, "activations"):
            raise ValueError(f"No activations detected for {type(module)}, run forward after add_hooks(model)")
        batch_dim = 0 if batch_first or type(module) is RNNLinear else 1
        if not hasattr(module, "max_batch_len"):
            module.max_batch_len = _get_batch_size(module=module, batch_dim=batch_dim)
        activations = module.activations.pop()
        if loss_reduction == "mean":
            backprops = backprops * module.max_batch_len
        elif loss_reduction != "sum":
            raise ValueError(f"loss_reduction = {loss_reduction}. Only 'sum' and 'mean' losses are supported")
        if batch_dim != 0:
            activations = [t.transpose(0, batch_dim) if isinstance(t, torch.Tensor) else t for t in activations]
            backprops = backprops.transpose(0, batch_dim)
        return activations, backprops

    # -------------------------------------------------------------- validation
    @classmethod
    def is_supported(cls, module: nn.Module) -> bool:
        warnings.warn(
            "GradSampleModule.is_supported is deprecated, as all layers can now be used with functorch.",
            DeprecationWarning,
        )
        return True

    @classmethod
    def validate(cls, module: nn.Module, *, strict: bool = False) -> List[NotImplementedError]:
        """Trainable layers that own buffers (running statistics and the like)
        mix information across samples and are rejected."""
        errors = [
            NotImplementedError(
                f"Model contains a trainable layer with buffers"
                f"that Opacus doesn't currently support({name}:{m}). "
            )
            for name, m in trainable_modules(module)
            if any(True for _ in m.buffers())
        ]
        if strict and errors:
            raise NotImplementedError(errors)
        return errors

    def forbid_grad_accumulation(self):
        self.grad_accumulation_allowed = False

    def allow_grad_accumulation(self):
        self.grad_accumulation_allowed = True


class GradSampleModule(GradSampleHooks, AbstractGradSampleModule):
    """``nn.Module`` wrapper flavour: ``GradSampleModule(model)(x)``."""

    def __init__(self, m: nn.Module, *, batch_first=True, loss_reduction="mean", strict: bool = True,
                 force_functorch=False, skip_param_grads: bool = False, early_capture: bool = False):
        nn.Module.__init__(self)
        GradSampleHooks.__init__(self, m, batch_first=batch_first, loss_reduction=loss_reduction, strict=strict,
                                 force_functorch=force_functorch, skip_param_grads=skip_param_grads,
                                 early_capture=early_capture)
        self.grad_accumulation_hook = None

    def forward(self, *args, **kwargs):
        return self._module(*args, **kwargs)


def _get_batch_size(*, module: nn.Module, batch_dim: int) -> int:
    """Largest batch length among the pending forward calls of ``module``
    (they differ across time steps of a packed sequence)."""
    best = 0
    for acts in module.activations:
        tensors = [t for t in acts if isinstance(t, torch.Tensor)]       # optional inputs may be None
        best = max(best, tensors[-1].shape[batch_dim])
    return best
