# %% [markdown]
# # A character-level LSTM classifier with differential privacy
#
# Task: guess the language of a surname from its characters.  The point of the guide is the recurrent layer:
# `torch.nn.LSTM` runs a fused cuDNN kernel whose internals cannot be hooked, so per-sample gradients are not available
# from it.  `opacus_b200.layers.DPLSTM` is the same network written as a loop over `Linear` cells (same parameters,
# same state-dict keys, same outputs); the package computes the per-sample gradients of all time steps of one cell in a
# single stacked kernel call.
#
#     python tutorials/building_lstm_name_classifier.py [--names-dir PATH]
#
# `--names-dir` is a folder of `Language.txt` files with one name per line (the data set of PyTorch's char-RNN tutorial);
# without it, names are synthesised from per-language character distributions.
#
# Counterpart in the reference: `tutorials/building_lstm_name_classifier.ipynb`.

# %%
import argparse
import glob
import os
import string
import sys

import torch
import torch.nn as nn
from torch.utils.data import DataLoader, Dataset

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from opacus_b200 import PrivacyEngine  # noqa: E402
from opacus_b200.layers import DPLSTM  # noqa: E402

ap = argparse.ArgumentParser()
ap.add_argument("--names-dir", default=None)
ap.add_argument("--epochs", type=int, default=3)
ap.add_argument("--batch-size", type=int, default=128)
ap.add_argument("--hidden", type=int, default=64)
ap.add_argument("--sigma", type=float, default=1.0)
ap.add_argument("--clip", type=float, default=1.5)
ap.add_argument("--lr", type=float, default=2.0)
ap.add_argument("--delta", type=float, default=8e-5)
ap.add_argument("--samples", type=int, default=3000)
ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
args, _ = ap.parse_known_args()
device = torch.device(args.device)

# %% [markdown]
# ## Data: names as byte sequences, padded to one length

# %%
ALPHABET = string.ascii_letters + " .,;'-#"           # '#' is the padding symbol
PAD = len(ALPHABET) - 1
MAX_LEN = 15


def encode(name):
    ids = [ALPHABET.find(ch) for ch in name[:MAX_LEN] if ch in ALPHABET[:-1]]
    return torch.tensor(ids + [PAD] * (MAX_LEN - len(ids)))


class Names(Dataset):
    def __init__(self, pairs):
        self.x = torch.stack([encode(n) for n, _ in pairs])
        self.y = torch.tensor([c for _, c in pairs])

    def __len__(self):
        return len(self.y)

    def __getitem__(self, i):
        return self.x[i], self.y[i]


if args.names_dir:
    files = sorted(glob.glob(os.path.join(args.names_dir, "*.txt")))
    languages = [os.path.splitext(os.path.basename(f))[0] for f in files]
    pairs = [(line.strip(), c) for c, f in enumerate(files) for line in open(f, encoding="utf-8") if line.strip()]
else:
    languages = ["north", "south", "east", "west"]
    gen = torch.Generator().manual_seed(0)
    letters = string.ascii_lowercase
    pairs = []
    for c in range(len(languages)):
        weights = torch.rand(26, generator=gen) ** 4 + 0.01          # a peaked letter distribution per language
        for _ in range(args.samples // len(languages)):
            n = int(torch.randint(4, 11, (1,), generator=gen))
            chars = torch.multinomial(weights, n, replacement=True, generator=gen)
            pairs.append(("".join(letters[i] for i in chars).capitalize(), c))
perm = torch.randperm(len(pairs), generator=torch.Generator().manual_seed(1)).tolist()
cut = int(0.8 * len(pairs))
train_set, test_set = Names([pairs[i] for i in perm[:cut]]), Names([pairs[i] for i in perm[cut:]])
train_loader = DataLoader(train_set, batch_size=args.batch_size)
print(f"{len(train_set)} training names, {len(languages)} languages, e.g. {pairs[perm[0]][0]!r}")

# %% [markdown]
# ## Model
# `DPLSTM` takes the arguments of `nn.LSTM`.  An `nn.LSTM` in an existing model can also be swapped in place with
# `ModuleValidator.fix(model)`, which copies the weights.


# %%
class CharLSTM(nn.Module):
    def __init__(self, vocab, hidden, classes):
        super().__init__()
        self.embed = nn.Embedding(vocab, 32)
        self.lstm = DPLSTM(32, hidden, num_layers=1, batch_first=True)
        self.head = nn.Linear(hidden, classes)

    def forward(self, ids):
        out, _ = self.lstm(self.embed(ids))
        return self.head(out[:, -1])


model = CharLSTM(len(ALPHABET), args.hidden, len(languages)).to(device)
optimizer = torch.optim.SGD(model.parameters(), lr=args.lr)

# %% [markdown]
# ## Private training
# Nothing here is specific to recurrent models: the engine finds the `Linear` cells inside `DPLSTM` and the embedding.

# %%
engine = PrivacyEngine(accountant="rdp")
model, optimizer, train_loader = engine.make_private(
    module=model, optimizer=optimizer, data_loader=train_loader, noise_multiplier=args.sigma, max_grad_norm=args.clip)
criterion = nn.CrossEntropyLoss()
for epoch in range(args.epochs):
    model.train()
    for ids, y in train_loader:
        optimizer.zero_grad()
        loss = criterion(model(ids.to(device)), y.to(device))
        loss.backward()
        optimizer.step()
    model.eval()
    with torch.no_grad():
        acc = (model(test_set.x.to(device)).argmax(1).cpu() == test_set.y).float().mean().item()
    print(f"epoch {epoch}: loss {loss.item():.3f}  test accuracy {acc:.3f}  eps = {engine.get_epsilon(args.delta):.2f}")

# %% [markdown]
# ## Notes
# * Variable-length input can be passed as a `PackedSequence`; `DPLSTM` accepts it like `nn.LSTM` does.
# * `DPGRU` and `DPRNN` follow the same pattern.
# * The state dict of `DPLSTM` uses `nn.LSTM`'s key names, so a privately trained model loads into a plain `nn.LSTM` for
#   inference.
