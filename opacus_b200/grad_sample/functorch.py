"""Generic per-sample gradients for layers without a dedicated rule:
``vmap(grad(.))`` of ``<layer(a), g>`` over the batch axis.

Behavioural parity: ``opacus/grad_sample/functorch.py:25-129``.
"""
import copy
from contextlib import nullcontext

import torch
import torch.nn as nn
from torch.func import functional_call, grad, vmap


def make_functional(mod: nn.Module, disable_autograd_tracking: bool = False):
    """``(fn, params)`` with ``fn(params, *args)`` a stateless call of ``mod``."""
    names = [n for n, _ in mod.named_parameters()]
    values = tuple(p for _, p in mod.named_parameters())
    skeleton = copy.deepcopy(mod).to("meta")
    if hasattr(skeleton, "allow_grad_accumulation"):
        skeleton.allow_grad_accumulation()

    def fn(new_values, *args, **kwargs):
        return functional_call(skeleton, dict(zip(names, new_values)), args, kwargs)

    if disable_autograd_tracking:
        values = tuple(v.detach() for v in values)
    return fn, values


def prepare_layer(layer, batch_first=True):
    """Attach ``layer.ft_compute_sample_grad(params, a, g)``."""
    from ..layers.dp_rnn import RNNLinear

    if any(True for _ in layer.buffers()):
        raise NotImplementedError("This layer has buffers and is not supported by Opacus")
    if type(layer) is nn.EmbeddingBag:
        raise NotImplementedError("Functorch does not support EmbeddingBag yet")

    fn, _ = make_functional(layer)
    batch_axis = 0 if (batch_first or type(layer) is RNNLinear) else 1

    def sample_objective(params, a, g):
        a1, g1 = a.unsqueeze(batch_axis), g.unsqueeze(batch_axis)
        mixed = a.dtype != params[0].dtype
        ctx = torch.amp.autocast(device_type=a.device.type, dtype=a.dtype) if mixed else nullcontext()
        with ctx:
            return (fn(params, a1) * g1).sum()

    layer.ft_compute_sample_grad = vmap(grad(sample_objective), in_dims=(None, 0, 0))


def ft_compute_per_sample_gradient(layer, activations, backprops):
    params = list(layer.parameters(recurse=True))
    if not hasattr(layer, "ft_compute_sample_grad"):
        prepare_layer(layer)
    a = activations[0]
    if a.is_floating_point() and a.dtype != backprops.dtype:
        a = a.to(backprops.dtype)
    grads = layer.ft_compute_sample_grad(params, a, backprops)
    return dict(zip(params, grads))
