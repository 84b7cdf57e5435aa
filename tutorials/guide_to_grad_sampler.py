# %% [markdown]
# # Guide to per-sample gradients and custom layers
#
# DP-SGD clips the gradient of every *sample* before summing.  Autograd only gives the sum, so this package computes
# per-sample gradients itself, layer by layer, from two tensors that the forward and backward passes already produce:
# the layer's input `a` (activations) and the gradient of the loss with respect to the layer's output `g` (backprops).
#
# This guide shows
#
# 1. what `GradSampleModule` attaches to the parameters,
# 2. how a layer type without a built-in rule is handled (functorch) and how to register a rule of your own,
# 3. the two extra rules of ghost clipping (norm only, and clipped sum directly),
# 4. how to test a rule against the micro-batch oracle.
#
#     python tutorials/guide_to_grad_sampler.py
#
# Counterpart in the reference: `tutorials/guide_to_grad_sampler.ipynb`.

# %%
import os
import sys

import torch
import torch.nn as nn

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from opacus_b200.grad_sample import GradSampleModule, register_grad_sampler  # noqa: E402
from opacus_b200.grad_sample.utils import register_norm_sq_sampler, register_wgrad_sampler  # noqa: E402
from opacus_b200.utils.per_sample_gradients_utils import check_per_sample_gradients_are_correct  # noqa: E402

torch.manual_seed(0)

# %% [markdown]
# ## 1. What the wrapper does
# After `backward()`, every trainable parameter `p` of a wrapped model has `p.grad_sample` of shape `[batch, *p.shape]`.
# For a `Linear` layer with input `a [B, T, d_in]` and output gradient `g [B, T, d_out]` the rule is
# `grad_sample[b] = g[b]^T a[b]`: one small matrix product per sample (on a B200 one tensor-core kernel for the whole
# batch, with the squared norm of every sample's gradient computed in the same pass).

# %%
model = GradSampleModule(nn.Sequential(nn.Linear(8, 16), nn.Tanh(), nn.Linear(16, 3)))
x, y = torch.randn(5, 8), torch.randint(0, 3, (5,))
nn.functional.cross_entropy(model(x), y).backward()
for name, p in model.named_parameters():
    print(f"{name:28s} grad {tuple(p.grad.shape)}  grad_sample {tuple(p.grad_sample.shape)}")
first = model._module[0].weight
# the ordinary gradient of a mean-reduced loss is the mean of the per-sample gradients
assert torch.allclose(first.grad, first.grad_sample.mean(dim=0), atol=1e-6)

# %% [markdown]
# ## 2. A layer of your own
# `ScaleShift` multiplies every feature by a learned scale and adds a learned shift.  Without a registered rule the
# wrapper falls back to `torch.func` (functorch): correct for any layer whose forward is a pure function of its
# parameters and input, but slower than a closed form.


# %%
class ScaleShift(nn.Module):
    def __init__(self, features):
        super().__init__()
        self.scale = nn.Parameter(torch.ones(features))
        self.shift = nn.Parameter(torch.zeros(features))

    def forward(self, x):                      # x: [B, ..., features]
        return x * self.scale + self.shift


net = nn.Sequential(nn.Linear(8, 16), ScaleShift(16), nn.ReLU(), nn.Linear(16, 3))
via_functorch = GradSampleModule(net)
nn.functional.cross_entropy(via_functorch(x), y).backward()
fallback = via_functorch._module[1].scale.grad_sample.clone()
via_functorch.remove_hooks()

# %% [markdown]
# The closed form: `d loss / d scale[b] = sum over positions of g * a`, `d loss / d shift[b] = sum of g`.  A rule receives
# the layer, the list of its inputs and the output gradient, and returns `{parameter: [B, *parameter.shape]}`.


# %%
@register_grad_sampler(ScaleShift)
def scale_shift_grad_sample(layer, activations, backprops):
    a = activations[0]
    reduce = tuple(range(1, a.dim() - 1))          # every axis between batch and features
    out = {}
    if layer.scale.requires_grad:
        out[layer.scale] = (backprops * a).sum(dim=reduce) if reduce else backprops * a
    if layer.shift.requires_grad:
        out[layer.shift] = backprops.sum(dim=reduce) if reduce else backprops
    return out


for p in net.parameters():
    p.grad = None
with_rule = GradSampleModule(net)
nn.functional.cross_entropy(with_rule(x), y).backward()
assert torch.allclose(with_rule._module[1].scale.grad_sample, fallback, atol=1e-6)
print("closed-form rule agrees with the functorch fallback")
with_rule.remove_hooks()

# %% [markdown]
# ## 3. Ghost clipping rules
# Ghost clipping (`grad_sample_mode="ghost"`) never stores `[B, *p.shape]`.  It needs, per layer,
#
# * the squared norm of every sample's gradient, and
# * the clipped sum `sum_b c_b * grad_b` for given per-sample factors `c`.
#
# Without dedicated rules both are derived from the per-sample-gradient rule (which materialises the gradients of that one
# layer).  For layers with large parameters it pays to register direct forms.  For `ScaleShift` on 2-d input they are
# simple:


# %%
@register_norm_sq_sampler(ScaleShift)
def scale_shift_norm_sq(layer, activations, backprops, g_scale=1.0, total=None):
    gs = scale_shift_grad_sample(layer, activations, backprops * g_scale)
    out = {p: v.flatten(1).square().sum(dim=1) for p, v in gs.items()}
    if total is not None:                      # the caller may hand in a running [B] total to add to
        for v in out.values():
            total.add_(v)
        return {}
    return out


@register_wgrad_sampler(ScaleShift)
def scale_shift_weighted_grad(layer, activations, backprops, coef, g_scale=1.0):
    shape = (-1,) + (1,) * (backprops.dim() - 1)
    weighted = backprops * (coef * g_scale).reshape(shape)
    a = activations[0]
    every = tuple(range(a.dim() - 1))
    return {layer.scale: (weighted * a).sum(dim=every), layer.shift: weighted.sum(dim=every)}


from opacus_b200 import PrivacyEngine  # noqa: E402
from torch.utils.data import DataLoader, TensorDataset  # noqa: E402

data = TensorDataset(torch.randn(64, 8), torch.randint(0, 3, (64,)))
for p in net.parameters():
    p.grad = None
engine = PrivacyEngine()
ghost, opt, criterion, loader = engine.make_private(
    module=net, optimizer=torch.optim.SGD(net.parameters(), lr=0.1), data_loader=DataLoader(data, batch_size=16),
    criterion=nn.CrossEntropyLoss(), noise_multiplier=0.0, max_grad_norm=0.5, grad_sample_mode="ghost",
    poisson_sampling=False)
xb, yb = next(iter(loader))
opt.zero_grad()
criterion(ghost(xb), yb).backward()
# with noise 0 the result must equal "clip each per-sample gradient to 0.5, then sum"
oracle = GradSampleModule(nn.Sequential(nn.Linear(8, 16), ScaleShift(16), nn.ReLU(), nn.Linear(16, 3)))
oracle._module.load_state_dict(net.state_dict())
nn.functional.cross_entropy(oracle(xb), yb, reduction="sum").backward()
norms = torch.stack([p.grad_sample.flatten(1).norm(dim=1) for p in oracle.parameters()]).norm(dim=0)
factor = (0.5 / (norms + 1e-6)).clamp(max=1.0)
for (name, p), q in zip(net.named_parameters(), oracle.parameters()):
    want = (q.grad_sample * factor.reshape((-1,) + (1,) * (q.dim()))).sum(dim=0)
    assert torch.allclose(p.grad, want, atol=1e-5), name
print("ghost clipping with the custom rules equals clip-then-sum of per-sample gradients")

# %% [markdown]
# ## 4. Testing a rule
# `check_per_sample_gradients_are_correct` runs the model once per sample (the definition of a per-sample gradient) and
# compares with what the wrapper produced, for both loss reductions.  Use it in the unit test of every rule you write.

# %%
check_per_sample_gradients_are_correct(torch.randn(6, 8), nn.Sequential(nn.Linear(8, 16), ScaleShift(16)))
check_per_sample_gradients_are_correct(torch.randn(6, 5, 8), nn.Sequential(nn.Linear(8, 16), ScaleShift(16)))
print("per-sample gradients match the micro-batch oracle")
