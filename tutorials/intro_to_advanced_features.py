# %% [markdown]
# # Advanced features
#
# Everything beyond the basic `make_private` loop, each in a few lines:
#
# 1. per-layer clipping, 2. adaptive clipping, 3. noise and clipping-norm schedulers, 4. choosing an accountant and
# writing one, 5. step hooks and clipping statistics, 6. secure random numbers and custom generators, 7. checkpoints,
# 8. virtual steps without the batch memory manager.
#
#     python tutorials/intro_to_advanced_features.py
#
# Counterpart in the reference: `tutorials/intro_to_advanced_features.ipynb`.

# %%
import io
import os
import sys
import warnings

import torch
import torch.nn as nn
from torch.utils.data import DataLoader, TensorDataset

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from opacus_b200 import PrivacyEngine  # noqa: E402
from opacus_b200.accountants import IAccountant  # noqa: E402
from opacus_b200.accountants.registry import register_accountant  # noqa: E402
from opacus_b200.schedulers import ExponentialNoise, StepGradClip  # noqa: E402

warnings.filterwarnings("ignore")
torch.manual_seed(0)
DATA = TensorDataset(torch.randn(512, 20), torch.randint(0, 4, (512,)))


def fresh(batch_size=64):
    model = nn.Sequential(nn.Linear(20, 32), nn.ReLU(), nn.Linear(32, 4))
    return model, torch.optim.SGD(model.parameters(), lr=0.1), DataLoader(DATA, batch_size=batch_size)


def steps_accounted(engine):
    return sum(count for _, _, count in engine.accountant.history)      # (noise multiplier, sample rate, steps) runs


def run(model, optimizer, loader, steps=None, criterion=None):
    criterion = criterion or nn.CrossEntropyLoss()
    for i, (x, y) in enumerate(loader):
        if steps is not None and i >= steps:
            break
        optimizer.zero_grad()
        criterion(model(x), y).backward()
        optimizer.step()


# %% [markdown]
# ## 1. Per-layer clipping
# Flat clipping bounds the norm of the whole per-sample gradient.  `clipping="per_layer"` takes one bound per parameter
# tensor and clips each separately; the overall sensitivity is the Euclidean norm of the list.  It lets a layer be
# clipped (and, under DDP, reduced) as soon as its gradient exists.

# %%
model, optimizer, loader = fresh()
n_tensors = len(list(model.parameters()))
engine = PrivacyEngine()
model, optimizer, loader = engine.make_private(
    module=model, optimizer=optimizer, data_loader=loader, noise_multiplier=1.0,
    max_grad_norm=[1.0 / n_tensors ** 0.5] * n_tensors, clipping="per_layer")
run(model, optimizer, loader)
print(f"1. per-layer clipping: {type(optimizer).__name__}, eps = {engine.get_epsilon(1e-5):.2f}")

# %% [markdown]
# ## 2. Adaptive clipping
# `clipping="adaptive"` moves the clipping norm towards a target quantile of the per-sample norms (here: 70 % of the
# samples unclipped), privately: the fraction of unclipped samples is itself released with noise (`unclipped_num_std`),
# which the accountant is charged for through a slightly larger effective noise multiplier.

# %%
model, optimizer, loader = fresh()
engine = PrivacyEngine()
model, optimizer, loader = engine.make_private(
    module=model, optimizer=optimizer, data_loader=loader, noise_multiplier=1.0, max_grad_norm=5.0, clipping="adaptive",
    target_unclipped_quantile=0.7, clipbound_learning_rate=0.3, max_clipbound=10.0, min_clipbound=0.05,
    unclipped_num_std=3.0)
run(model, optimizer, loader)
print(f"2. adaptive clipping: bound moved from 5.0 to {float(optimizer.max_grad_norm):.2f}")

# %% [markdown]
# ## 3. Schedulers
# Like learning-rate schedulers, but for `optimizer.noise_multiplier` and `optimizer.max_grad_norm`.  The accountant
# records the noise multiplier of every step, so a schedule is accounted for exactly.

# %%
model, optimizer, loader = fresh()
engine = PrivacyEngine()
model, optimizer, loader = engine.make_private(module=model, optimizer=optimizer, data_loader=loader,
                                                noise_multiplier=1.5, max_grad_norm=1.0)
noise_schedule = ExponentialNoise(optimizer, gamma=0.9)
clip_schedule = StepGradClip(optimizer, step_size=2, gamma=0.5)
for epoch in range(4):
    run(model, optimizer, loader)
    noise_schedule.step()
    clip_schedule.step()
print(f"3. after 4 epochs: noise multiplier {optimizer.noise_multiplier:.3f}, clipping norm {optimizer.max_grad_norm:.3f}, "
      f"eps = {engine.get_epsilon(1e-5):.2f}")

# %% [markdown]
# ## 4. Accountants
# `accountant="rdp"` (Renyi DP; the default, fast), `"prv"` (numerical composition of privacy-loss random variables;
# tighter, needs more memory) and `"gdp"` (Gaussian DP central-limit approximation; not an upper bound).  An accountant
# of your own implements `step`, `get_epsilon`, `__len__` and `mechanism`, and is registered under a name.

# %%
for name in ("rdp", "prv", "gdp"):
    model, optimizer, loader = fresh()
    engine = PrivacyEngine(accountant=name)
    model, optimizer, loader = engine.make_private(module=model, optimizer=optimizer, data_loader=loader,
                                                    noise_multiplier=1.0, max_grad_norm=1.0)
    for _ in range(3):
        run(model, optimizer, loader)
    print(f"4. {name}: eps(1e-5) = {engine.get_epsilon(1e-5):.3f} after {steps_accounted(engine)} steps")


class StepCounter(IAccountant):
    """Not a privacy analysis: it only shows the interface (it reports the number of steps as 'epsilon')."""

    def __init__(self):
        super().__init__()

    def step(self, *, noise_multiplier: float, sample_rate: float):
        self.history.append((noise_multiplier, sample_rate, 1))

    def get_epsilon(self, delta: float, **kwargs) -> float:
        return float(len(self.history))

    def __len__(self):
        return len(self.history)

    @classmethod
    def mechanism(cls) -> str:
        return "step_counter"


register_accountant("step_counter", StepCounter, force=True)
model, optimizer, loader = fresh()
engine = PrivacyEngine(accountant="step_counter")
model, optimizer, loader = engine.make_private(module=model, optimizer=optimizer, data_loader=loader,
                                                noise_multiplier=1.0, max_grad_norm=1.0)
run(model, optimizer, loader)
print(f"4. custom accountant saw {engine.get_epsilon(1e-5):.0f} steps")

# %% [markdown]
# ## 5. Step hooks and clipping statistics
# `optimizer.attach_step_hook(fn)` sets the function that runs after every real (noise-adding) step.  There is one slot,
# and the accountant lives in it, so chain to the previous hook rather than replacing it.  With ghost clipping the
# wrapped model keeps the per-sample gradient norms of the last batch in `per_sample_gradient_norms`: the quantity to
# look at when choosing `max_grad_norm`.

# %%
model, optimizer, loader = fresh()
engine = PrivacyEngine()
model, optimizer, criterion, loader = engine.make_private(
    module=model, optimizer=optimizer, data_loader=loader, criterion=nn.CrossEntropyLoss(), noise_multiplier=1.0,
    max_grad_norm=1.0, grad_sample_mode="ghost")
seen = []
accounting = optimizer.step_hook


def hook(opt):
    accounting(opt)
    seen.append(float(model.per_sample_gradient_norms.median()))


optimizer.attach_step_hook(hook)
run(model, optimizer, loader, criterion=criterion)
print(f"5. median per-sample gradient norm over the epoch: {min(seen):.2f} .. {max(seen):.2f}; "
      f"{steps_accounted(engine)} steps accounted")

# %% [markdown]
# ## 6. Random numbers
# `secure_mode=True` draws both the Poisson samples and the noise from a cryptographically secure generator (the
# `torchcsprng` package if it is installed, otherwise this package's ChaCha20 generator keyed from the OS entropy pool,
# which computes the same stream on CPU and GPU) and sums four draws per element to defeat floating-point attacks on the
# Gaussian sampler.  Use it for the final run.  For reproducible experiments pass your own `noise_generator` instead
# (the two are mutually exclusive: a seeded generator is the opposite of a secure one).

# %%
model, optimizer, loader = fresh()
engine = PrivacyEngine(secure_mode=True)
model, optimizer, loader = engine.make_private(module=model, optimizer=optimizer, data_loader=loader,
                                                noise_multiplier=1.0, max_grad_norm=1.0)
run(model, optimizer, loader)
print(f"6. secure mode: generator {type(engine.secure_rng).__name__}, eps = {engine.get_epsilon(1e-5):.2f}")

outs = []
for _ in range(2):
    torch.manual_seed(1)
    model, optimizer, loader = fresh()
    engine = PrivacyEngine()
    model, optimizer, loader = engine.make_private(
        module=model, optimizer=optimizer, data_loader=loader, noise_multiplier=1.0, max_grad_norm=1.0,
        noise_generator=torch.Generator().manual_seed(7), poisson_sampling=False)
    run(model, optimizer, loader, steps=3)
    outs.append(torch.cat([p.detach().flatten() for p in model.parameters()]))
print("6. same noise generator seed, same result:", torch.equal(outs[0], outs[1]))

# %% [markdown]
# ## 7. Checkpoints
# A checkpoint holds the model, the optimizer state, the accountant's history and the schedulers, so a resumed run keeps
# counting its budget where it stopped.  The file layout is the one of Opacus 1.6.

# %%
model, optimizer, loader = fresh()
engine = PrivacyEngine()
model, optimizer, loader = engine.make_private(module=model, optimizer=optimizer, data_loader=loader,
                                                noise_multiplier=1.0, max_grad_norm=1.0)
run(model, optimizer, loader)
buffer = io.BytesIO()
engine.save_checkpoint(path=buffer, module=model, optimizer=optimizer, checkpoint_dict={"epoch": 1})
before = engine.get_epsilon(1e-5)

model2, optimizer2, loader2 = fresh()
engine2 = PrivacyEngine()
model2, optimizer2, loader2 = engine2.make_private(module=model2, optimizer=optimizer2, data_loader=loader2,
                                                    noise_multiplier=1.0, max_grad_norm=1.0)
buffer.seek(0)
extra = engine2.load_checkpoint(path=buffer, module=model2, optimizer=optimizer2)
print(f"7. resumed at epoch {extra['epoch']} with eps = {engine2.get_epsilon(1e-5):.3f} (saved at {before:.3f})")

# %% [markdown]
# ## 8. Virtual steps by hand
# `BatchMemoryManager` splits logical batches for you.  The mechanism underneath: `optimizer.signal_skip_step(True)`
# makes the next `step()` only clip and accumulate; the following unsignalled `step()` adds noise for the whole logical
# batch and updates.  The accountant counts one step per logical batch.

# %%
model, optimizer, loader = fresh(batch_size=32)          # physical batches of 32, logical batch 4 x 32
engine = PrivacyEngine()
model, optimizer, loader = engine.make_private(module=model, optimizer=optimizer, data_loader=loader,
                                                noise_multiplier=1.0, max_grad_norm=1.0, poisson_sampling=False)
criterion = nn.CrossEntropyLoss()
for i, (x, y) in enumerate(loader):
    optimizer.zero_grad()
    criterion(model(x), y).backward()
    optimizer.signal_skip_step(do_skip=(i + 1) % 4 != 0)
    optimizer.step()
print(f"8. {i + 1} physical batches, {steps_accounted(engine)} accounted steps")
