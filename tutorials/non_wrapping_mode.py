# %% [markdown]
# # Non-wrapping mode: private training without changing the model's type
#
# By default `make_private` returns the model wrapped in a `GradSampleModule`.  The wrapper forwards calls and attribute
# look-ups, but it *is* another object: `isinstance(model, MyModel)` is false, state-dict keys gain a `_module.` prefix
# when saved through the wrapper, and code that walks the module tree sees one more level.
#
# With `wrap_model=False` the model is instrumented in place: hooks are registered on its layers and `make_private`
# returns a small controller object (`GradSampleHooks`) instead of a module.  The model you hold is still your model.
#
#     python tutorials/non_wrapping_mode.py
#
# Counterpart in the reference: `tutorials/non_wrapping_mode.ipynb`.

# %%
import os
import sys
import warnings

import torch
import torch.nn as nn
from torch.utils.data import DataLoader, TensorDataset

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from opacus_b200 import PrivacyEngine  # noqa: E402

warnings.filterwarnings("ignore")
torch.manual_seed(0)


class Classifier(nn.Module):
    def __init__(self):
        super().__init__()
        self.body = nn.Sequential(nn.Linear(20, 64), nn.ReLU(), nn.Linear(64, 64), nn.ReLU())
        self.head = nn.Linear(64, 3)

    def forward(self, x):
        return self.head(self.body(x))

    def predict(self, x):                           # a method of your own: still there after make_private
        with torch.no_grad():
            return self(x).argmax(dim=1)


prototypes = torch.randn(3, 20)
labels = torch.randint(0, 3, (1024,))
data = TensorDataset(prototypes[labels] + 0.8 * torch.randn(1024, 20), labels)

# %% [markdown]
# ## Wrapping mode, for comparison

# %%
model = Classifier()
wrapped, _, _ = PrivacyEngine().make_private(
    module=model, optimizer=torch.optim.SGD(model.parameters(), lr=0.1), data_loader=DataLoader(data, batch_size=128),
    noise_multiplier=1.0, max_grad_norm=1.0)
print("wrapping:     type", type(wrapped).__name__, "| isinstance(Classifier):", isinstance(wrapped, Classifier),
      "| first state-dict key:", next(iter(wrapped.state_dict())))

# %% [markdown]
# ## Non-wrapping mode
# The first return value is now the hook controller.  Keep it if you want to switch the hooks off and on
# (`disable_hooks()` / `enable_hooks()`, e.g. around an evaluation that calls `backward`) or to take them off for good
# (`remove_hooks()`); training itself only needs the model and the optimizer.

# %%
model = Classifier()
optimizer = torch.optim.SGD(model.parameters(), lr=0.2)
engine = PrivacyEngine()
hooks, optimizer, loader = engine.make_private(
    module=model, optimizer=optimizer, data_loader=DataLoader(data, batch_size=128), noise_multiplier=1.0,
    max_grad_norm=1.0, wrap_model=False)
print("non-wrapping: type", type(model).__name__, "| controller:", type(hooks).__name__,
      "| first state-dict key:", next(iter(model.state_dict())))

criterion = nn.CrossEntropyLoss()
for epoch in range(3):
    for x, y in loader:
        optimizer.zero_grad()
        criterion(model(x), y).backward()           # per-sample gradients appear on model's parameters
        optimizer.step()
x_all, y_all = data.tensors
print(f"accuracy {float((model.predict(x_all) == y_all).float().mean()):.3f}, eps = {engine.get_epsilon(1e-5):.2f}")

# %% [markdown]
# ## Taking the instrumentation off
# After `remove_hooks()` the model is an ordinary module again: no per-sample gradients are computed, and the
# `grad_sample` attributes left on the parameters can be dropped.

# %%
hooks.remove_hooks()
for p in model.parameters():
    p.grad_sample = None
criterion(model(x_all[:8]), y_all[:8]).backward()
print("after remove_hooks: grad_sample is", model.head.weight.grad_sample, "| ordinary grad", tuple(model.head.weight.grad.shape))

# %% [markdown]
# ## When to use which
# * Wrapping (default): nothing to keep track of; the wrapper's `state_dict()` and `load_state_dict()` round-trip with each
#   other, and checkpoints of `PrivacyEngine.save_checkpoint` use them.
# * Non-wrapping: when other code depends on the model's class (custom methods, `isinstance` checks, frameworks that
#   walk `named_modules()`), or when checkpoints must load into the bare model without renaming keys.
# * Both work with every hook-based mode (`hooks`, `functorch`, `ghost`, `ghost_fsdp`, `ghost_tp`, `no_op`); expanded
#   weights (`ew`) exist only as a wrapper.  With ghost clipping `make_private(..., wrap_model=False)` returns
#   `(controller, optimizer, criterion, loader)` and the loss wrapper talks to the controller.
