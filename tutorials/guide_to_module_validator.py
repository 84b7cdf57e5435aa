# %% [markdown]
# # Guide to the module validator and fixer
#
# Some layers are incompatible with per-sample clipping in principle, others only in the form PyTorch ships them:
#
# | layer | problem | what `ModuleValidator.fix` does |
# |---|---|---|
# | `BatchNorm*` | normalises a sample with its batch-mates' statistics: a sample's gradient depends on other people's data | replaces it by `GroupNorm` (or `InstanceNorm` with `replace_bn_with_in=True`) |
# | `InstanceNorm*` with `track_running_stats=True` | running statistics mix samples over time | turns tracking off |
# | `nn.LSTM`, `nn.GRU`, `nn.RNN` | fused kernels, no access to per-step activations | `DPLSTM`, `DPGRU`, `DPRNN` with the weights copied |
# | `nn.MultiheadAttention` | packed projection used inside a fused call | `DPMultiheadAttention` with the weights copied |
#
# `PrivacyEngine.make_private` validates the model and refuses to continue if problems remain, so running the validator
# yourself first gives the clearer message.
#
#     python tutorials/guide_to_module_validator.py
#
# Counterpart in the reference: `tutorials/guide_to_module_validator.ipynb`.

# %%
import os
import sys

import torch
import torch.nn as nn

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from opacus_b200 import PrivacyEngine  # noqa: E402
from opacus_b200.validators import ModuleValidator, register_module_fixer, register_module_validator  # noqa: E402
from opacus_b200.validators.errors import ShouldReplaceModuleError, UnsupportedModuleError  # noqa: E402


# %% [markdown]
# ## Validate
# `validate` returns a list of problems (or raises them all at once with `strict=True`); `is_valid` is the boolean form.


# %%
class Tagger(nn.Module):
    def __init__(self):
        super().__init__()
        self.stem = nn.Sequential(nn.Conv1d(4, 16, 3, padding=1), nn.BatchNorm1d(16), nn.ReLU())
        self.rnn = nn.LSTM(16, 32, batch_first=True)
        self.attn = nn.MultiheadAttention(32, 4, batch_first=True)
        self.head = nn.Linear(32, 5)

    def forward(self, x):                       # x: [B, 4, T]
        h, _ = self.rnn(self.stem(x).transpose(1, 2))
        return self.head(self.attn(h, h, h, need_weights=False)[0])


model = Tagger()
for problem in ModuleValidator.validate(model, strict=False):
    print(f"- {type(problem).__name__}: {str(problem)[:110]}...")
print("valid:", ModuleValidator.is_valid(model))
try:
    ModuleValidator.validate(model, strict=True)
except UnsupportedModuleError as err:
    print("strict validation raises", type(err).__name__)

# %% [markdown]
# ## Fix
# `fix` returns a repaired *copy*.  Replaced recurrent and attention layers keep their weights, so the outputs are the
# same; a BatchNorm -> GroupNorm swap changes the function (statistics are now per sample) and starts from fresh affine
# parameters.  Create the optimizer afterwards: the copy has new parameter objects.

# %%
fixed = ModuleValidator.fix(model)
print("after fix:", [type(m).__name__ for m in (fixed.stem[1], fixed.rnn, fixed.attn)], "valid:", ModuleValidator.is_valid(fixed))
x = torch.randn(3, 4, 10)
model.eval(), fixed.eval()
with torch.no_grad():
    h_old, _ = model.rnn(torch.randn(3, 10, 16, generator=torch.Generator().manual_seed(1)))
    h_new, _ = fixed.rnn(torch.randn(3, 10, 16, generator=torch.Generator().manual_seed(1)))
print("LSTM outputs equal after the swap:", torch.allclose(h_old, h_new, atol=1e-6))
model.train(), fixed.train()
grouped = ModuleValidator.fix(model, num_groups=4)
print("GroupNorm groups: default", fixed.stem[1].num_groups, "| requested", grouped.stem[1].num_groups)

# %% [markdown]
# ## The engine validates too

# %%
try:
    PrivacyEngine().make_private(module=model, optimizer=torch.optim.SGD(model.parameters(), lr=0.1),
                                 data_loader=torch.utils.data.DataLoader(torch.utils.data.TensorDataset(torch.zeros(8, 4, 10)), batch_size=4),
                                 noise_multiplier=1.0, max_grad_norm=1.0)
except UnsupportedModuleError as err:
    print("make_private refuses the unfixed model:", type(err).__name__)

# %% [markdown]
# ## Rules for your own layers
# A validator is a function `module -> list of errors`, a fixer a function `module, **kwargs -> replacement`; both are
# registered per type.  Example: a layer that normalises by the batch maximum (which couples samples) and its per-sample
# replacement.


# %%
class BatchMaxScale(nn.Module):
    def __init__(self):
        super().__init__()
        self.gain = nn.Parameter(torch.ones(1))

    def forward(self, x):
        return self.gain * x / x.abs().max().clamp_min(1e-6)


class SampleMaxScale(nn.Module):
    def __init__(self):
        super().__init__()
        self.gain = nn.Parameter(torch.ones(1))

    def forward(self, x):
        peak = x.flatten(1).abs().max(dim=1).values.clamp_min(1e-6)
        return self.gain * x / peak.reshape((-1,) + (1,) * (x.dim() - 1))


@register_module_validator(BatchMaxScale)
def _validate_batch_max(module):
    return [ShouldReplaceModuleError("BatchMaxScale divides by a statistic of the whole batch; use SampleMaxScale")]


@register_module_fixer(BatchMaxScale)
def _fix_batch_max(module, **kwargs):
    new = SampleMaxScale()
    new.gain.data.copy_(module.gain.data)
    return new


# the tables are consulted for every submodule that owns trainable parameters (a layer without parameters has no
# per-sample gradient to get wrong, so it is not looked at)
custom = nn.Sequential(nn.Linear(6, 6), BatchMaxScale(), nn.Linear(6, 2))
print("custom model valid:", ModuleValidator.is_valid(custom))
print("after fix:", ModuleValidator.fix(custom))
