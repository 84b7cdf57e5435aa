# %% [markdown]
# # Building an image classifier with differential privacy
#
# This guide trains a small ResNet on 32 x 32 colour images with DP-SGD and shows the four things every private
# training run needs:
#
# 1. a model without layers that mix samples (BatchNorm),
# 2. a `PrivacyEngine` that wraps model, optimizer and data loader,
# 3. a way to keep the *physical* batch small while the *logical* batch (the one the privacy analysis sees) stays large,
# 4. the privacy budget spent so far.
#
# It runs as a script (`python tutorials/building_image_classifier.py`) or cell by cell in an editor that understands
# `# %%` markers.  With `--data-root PATH` it uses torchvision's CIFAR-10 from that folder; without, it draws a synthetic
# stand-in of the same shape so that it runs anywhere in under a minute.
#
# Counterpart in the reference: `tutorials/building_image_classifier.ipynb`.

# %%
import argparse
import os
import sys

import torch
import torch.nn as nn
from torch.utils.data import DataLoader, TensorDataset

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))   # run from a source checkout

from opacus_b200 import PrivacyEngine  # noqa: E402
from opacus_b200.utils.batch_memory_manager import BatchMemoryManager  # noqa: E402
from opacus_b200.validators import ModuleValidator  # noqa: E402

ap = argparse.ArgumentParser()
ap.add_argument("--data-root", default=None)
ap.add_argument("--epochs", type=int, default=2)
ap.add_argument("--samples", type=int, default=2048, help="size of the synthetic training set")
ap.add_argument("--batch-size", type=int, default=256, help="logical batch: what the privacy analysis sees")
ap.add_argument("--max-physical-batch", type=int, default=64, help="what is in memory at once")
ap.add_argument("--epsilon", type=float, default=8.0)
ap.add_argument("--delta", type=float, default=1e-5)
ap.add_argument("--clip", type=float, default=1.2)
ap.add_argument("--lr", type=float, default=1e-3)
ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
args, _ = ap.parse_known_args()
device = torch.device(args.device)

# %% [markdown]
# ## Data
# Each sample must belong to one person for the guarantee to mean "per person"; here a sample is one image.

# %%
if args.data_root:
    from torchvision import datasets, transforms

    tf = transforms.Compose([transforms.ToTensor(),
                             transforms.Normalize((0.4914, 0.4822, 0.4465), (0.2470, 0.2435, 0.2616))])
    train_set = datasets.CIFAR10(args.data_root, train=True, transform=tf)
    test_set = datasets.CIFAR10(args.data_root, train=False, transform=tf)
else:
    gen = torch.Generator().manual_seed(0)
    prototypes = torch.randn(10, 3, 32, 32, generator=gen)

    def synthetic(n):
        y = torch.randint(0, 10, (n,), generator=gen)
        return TensorDataset(prototypes[y] + 1.5 * torch.randn(n, 3, 32, 32, generator=gen), y)

    train_set, test_set = synthetic(args.samples), synthetic(args.samples // 4)
train_loader = DataLoader(train_set, batch_size=args.batch_size)
test_loader = DataLoader(test_set, batch_size=512)

# %% [markdown]
# ## Model
# BatchNorm computes statistics over the batch, so one person's image changes another person's gradient and
# per-sample clipping loses its meaning.  `ModuleValidator.validate` lists such layers, `ModuleValidator.fix` replaces
# them (BatchNorm -> GroupNorm) and leaves everything else alone.


# %%
def block(c_in, c_out, stride):
    return nn.Sequential(nn.Conv2d(c_in, c_out, 3, stride=stride, padding=1, bias=False), nn.BatchNorm2d(c_out), nn.ReLU())


model = nn.Sequential(block(3, 32, 1), block(32, 64, 2), block(64, 128, 2), nn.AdaptiveAvgPool2d(1), nn.Flatten(),
                      nn.Linear(128, 10))
problems = ModuleValidator.validate(model, strict=False)
print(f"{len(problems)} layers are not compatible with DP training, e.g.: {problems[0]}")
model = ModuleValidator.fix(model)
assert ModuleValidator.validate(model, strict=False) == []
model = model.to(device)

# %% [markdown]
# ## Making it private
# The optimizer is created *after* the fix (it must hold the new parameters).  `make_private_with_epsilon` picks the
# noise multiplier that spends exactly `epsilon` over the planned number of epochs; `make_private` takes the noise
# multiplier directly.  The returned loader draws Poisson samples (every sample joins a batch independently with
# probability `batch_size / len(dataset)`), which is what the accountant assumes.

# %%
optimizer = torch.optim.RMSprop(model.parameters(), lr=args.lr)
engine = PrivacyEngine(accountant="rdp")
model, optimizer, train_loader = engine.make_private_with_epsilon(
    module=model, optimizer=optimizer, data_loader=train_loader, epochs=args.epochs,
    target_epsilon=args.epsilon, target_delta=args.delta, max_grad_norm=args.clip)
print(f"noise multiplier {optimizer.noise_multiplier:.3f} for clipping norm {args.clip}")

# %% [markdown]
# ## Training with a bounded physical batch
# Per-sample gradients cost `batch x parameters` memory.  `BatchMemoryManager` cuts a logical batch into physical
# ones of at most `max_physical_batch_size`; `optimizer.step()` only accumulates clipped sums until the logical batch is
# complete, then adds noise once and updates.  The training loop does not change.

# %%
criterion = nn.CrossEntropyLoss()


def accuracy(loader):
    model.eval()
    hit = n = 0
    with torch.no_grad():
        for x, y in loader:
            hit += (model(x.to(device)).argmax(1).cpu() == y).sum().item()
            n += len(y)
    return hit / max(n, 1)


for epoch in range(args.epochs):
    model.train()
    with BatchMemoryManager(data_loader=train_loader, max_physical_batch_size=args.max_physical_batch,
                            optimizer=optimizer) as loader:
        for x, y in loader:
            optimizer.zero_grad()
            loss = criterion(model(x.to(device)), y.to(device))
            loss.backward()
            optimizer.step()
    print(f"epoch {epoch}: loss {loss.item():.3f}  test accuracy {accuracy(test_loader):.3f}  "
          f"eps = {engine.get_epsilon(args.delta):.2f} at delta = {args.delta}")

# %% [markdown]
# ## What to tune
# * `max_grad_norm`: too small biases the gradient, too large means more noise for the same guarantee; values around
#   the median per-sample gradient norm work well (in ghost mode `model.per_sample_gradient_norms` holds the last batch's).
# * batch size: larger logical batches improve the signal-to-noise ratio per step at the price of fewer steps per epoch.
# * learning rate: usually lower than without privacy.
# * `grad_sample_mode="ghost"` never materialises per-sample gradients (one backward pass in this package); it is the
#   mode to use when the model is large.
