"""Sampler registries and the mode -> class factory.

Public decorators (``opacus/grad_sample/utils.py:37-183``):
``register_grad_sampler`` for ``(layer, activations, backprops) -> {param: [B, *param.shape]}``
and ``register_norm_sampler`` for ``(...) -> {param: [B] norms}``.

Additional decorators for the single-pass ghost path:
``register_norm_sq_sampler`` for ``(layer, activations, backprops, g_scale) -> {param: [B] squared norms}``
and ``register_wgrad_sampler`` for ``(layer, activations, backprops, coef, g_scale) -> {param: clipped grad sum}``,
where ``g_scale`` multiplies ``backprops`` (the batch size for mean-reduced losses) and is applied inside the kernels.
"""
from typing import Sequence, Type, Union

import torch.nn as nn

from .grad_sample_module import GradSampleHooks, GradSampleModule
from .grad_sample_module_fast_gradient_clipping import (
    GradSampleHooksFastGradientClipping,
    GradSampleModuleFastGradientClipping,
)
from .gsm_base import AbstractGradSampleModule
from .gsm_exp_weights import GradSampleModuleExpandedWeights
from .gsm_no_op import GradSampleHooksNoOp, GradSampleModuleNoOp


def _each(target):
    return target if isinstance(target, Sequence) else [target]


def register_grad_sampler(target_class_or_classes: Union[Type[nn.Module], Sequence[Type[nn.Module]]]):
    def decorator(f):
        for t in _each(target_class_or_classes):
            GradSampleHooks.GRAD_SAMPLERS[t] = f
            GradSampleHooksFastGradientClipping.GRAD_SAMPLERS[t] = f
        return f

    return decorator


def register_norm_sampler(target_class_or_classes: Union[Type[nn.Module], Sequence[Type[nn.Module]]]):
    def decorator(f):
        for t in _each(target_class_or_classes):
            GradSampleHooksFastGradientClipping.NORM_SAMPLERS[t] = f
        return f

    return decorator


def register_norm_sq_sampler(target_class_or_classes):
    def decorator(f):
        for t in _each(target_class_or_classes):
            GradSampleHooksFastGradientClipping.NORM_SQ_SAMPLERS[t] = f
        return f

    return decorator


def register_wgrad_sampler(target_class_or_classes):
    def decorator(f):
        for t in _each(target_class_or_classes):
            GradSampleHooksFastGradientClipping.WGRAD_SAMPLERS[t] = f
        return f

    return decorator


def register_cross_norm_sampler(type_a, type_b):
    """``f(param, site_a, site_b) -> [B]`` inner products ``<g_a, g_b>`` between
    the per-sample gradients two layer calls contribute to one shared parameter."""

    def decorator(f):
        GradSampleHooksFastGradientClipping.CROSS_NORM_SAMPLERS[(type_a, type_b)] = f
        return f

    return decorator


def prepare_module(model: nn.Module, grad_sample_mode: str, wrap_model: bool = True, *args, **kwargs):
    """Instrument ``model`` for ``grad_sample_mode``; returns the wrapper module
    (``wrap_model=True``) or the in-place controller."""
    if grad_sample_mode == "functorch":
        kwargs["force_functorch"] = True
    cls = get_gsm_class(grad_sample_mode) if wrap_model else get_hooks_class(grad_sample_mode)
    return cls(model, *args, **kwargs)


def wrap_model(model: nn.Module, grad_sample_mode: str, wrap_model: bool = True, *args, **kwargs):
    return prepare_module(model, grad_sample_mode, wrap_model, *args, **kwargs)


def get_gsm_class(grad_sample_mode: str) -> Type[AbstractGradSampleModule]:
    from .grad_sample_module_fast_gradient_clipping_fsdp import GradSampleModuleFastGradientClippingFSDP
    from .grad_sample_module_fast_gradient_clipping_tp import GradSampleModuleFastGradientClippingTP

    table = {
        "hooks": GradSampleModule,
        "functorch": GradSampleModule,
        "ew": GradSampleModuleExpandedWeights,
        "ghost": GradSampleModuleFastGradientClipping,
        "ghost_fsdp": GradSampleModuleFastGradientClippingFSDP,
        "ghost_tp": GradSampleModuleFastGradientClippingTP,
        "no_op": GradSampleModuleNoOp,
    }
    if grad_sample_mode not in table:
        raise ValueError(f"Unexpected grad_sample_mode: {grad_sample_mode}. Allowed values: {', '.join(table)}")
    return table[grad_sample_mode]


def get_hooks_class(grad_sample_mode: str):
    from .grad_sample_module_fast_gradient_clipping_fsdp import GradSampleHooksFastGradientClippingFSDP
    from .grad_sample_module_fast_gradient_clipping_tp import GradSampleHooksFastGradientClippingTP

    table = {
        "hooks": GradSampleHooks,
        "functorch": GradSampleHooks,
        "ghost": GradSampleHooksFastGradientClipping,
        "ghost_fsdp": GradSampleHooksFastGradientClippingFSDP,
        "ghost_tp": GradSampleHooksFastGradientClippingTP,
        "no_op": GradSampleHooksNoOp,
    }
    if grad_sample_mode not in table:
        raise ValueError(
            f"Unexpected grad_sample_mode: {grad_sample_mode}. Hooks-based approach supports: {', '.join(table)}")
    return table[grad_sample_mode]
