# %% [markdown]
# # Fine-tuning a text classifier with differential privacy
#
# The usual recipe for private NLP is: take a pretrained encoder, freeze most of it, train the top privately.  Frozen
# parameters need no per-sample gradients, so the cost of privacy falls with the share of the model that is trained, and
# the signal-to-noise ratio improves because the noise is spread over fewer coordinates.
#
# This guide has no network access to fetch a pretrained model, so it *makes* one: a small Transformer encoder is first
# trained without privacy on a public task (which of two topics a sentence is about), then its embeddings and lower block
# are frozen and the upper block and a new head are fine-tuned privately on a different, private task (a sentiment-like
# label: which of two sets of opinion words has the majority in the sentence).  With a real checkpoint, replace the first half by `from_pretrained(...)`.
#
#     python tutorials/building_text_classifier.py
#
# Counterpart in the reference: `tutorials/building_text_classifier.ipynb`.

# %%
import argparse
import os
import sys

import torch
import torch.nn as nn
from torch.utils.data import DataLoader, TensorDataset

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from opacus_b200 import PrivacyEngine  # noqa: E402
from opacus_b200.layers import DPMultiheadAttention  # noqa: E402
from opacus_b200.validators import ModuleValidator  # noqa: E402

ap = argparse.ArgumentParser()
ap.add_argument("--samples", type=int, default=4000)
ap.add_argument("--seq", type=int, default=24)
ap.add_argument("--vocab", type=int, default=200)
ap.add_argument("--d-model", type=int, default=64)
ap.add_argument("--epochs", type=int, default=3)
ap.add_argument("--batch-size", type=int, default=200)
ap.add_argument("--epsilon", type=float, default=6.0)
ap.add_argument("--delta", type=float, default=1e-4)
ap.add_argument("--clip", type=float, default=0.5)
ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
args, _ = ap.parse_known_args()
device = torch.device(args.device)
gen = torch.Generator().manual_seed(0)

# %% [markdown]
# ## A Transformer encoder made of DP-friendly parts
# `nn.MultiheadAttention` packs its projections into one parameter used in a fused call; `DPMultiheadAttention` has the
# same interface with separate `Linear` projections.  LayerNorm normalises within a sample and is fine as it is.


# %%
class Block(nn.Module):
    def __init__(self, d):
        super().__init__()
        self.n1, self.n2 = nn.LayerNorm(d), nn.LayerNorm(d)
        self.attn = DPMultiheadAttention(d, 4, batch_first=True)
        self.ff = nn.Sequential(nn.Linear(d, 2 * d), nn.GELU(), nn.Linear(2 * d, d))

    def forward(self, x):
        h = self.n1(x)
        x = x + self.attn(h, h, h, need_weights=False)[0]
        return x + self.ff(self.n2(x))


class Encoder(nn.Module):
    def __init__(self, vocab, d, seq, classes):
        super().__init__()
        self.tok, self.pos = nn.Embedding(vocab, d), nn.Embedding(seq, d)
        self.lower, self.upper = Block(d), Block(d)
        self.norm = nn.LayerNorm(d)
        self.head = nn.Linear(d, classes)

    def forward(self, ids):
        x = self.tok(ids) + self.pos(torch.arange(ids.shape[1], device=ids.device).expand_as(ids))
        return self.head(self.norm(self.upper(self.lower(x))).mean(dim=1))


# %% [markdown]
# ## "Pretraining" on public data (no privacy)

# %%
def topic_data(n):
    y = torch.randint(0, 2, (n,), generator=gen)
    upper_half = torch.rand(n, args.seq, generator=gen) < (0.3 + 0.4 * y[:, None].float())
    ids = torch.randint(0, args.vocab // 2, (n, args.seq), generator=gen) + upper_half.long() * (args.vocab // 2)
    return ids, y


def sentiment_data(n):
    """Six "opinion" words per sentence, drawn from a positive set (ids 0-9) and a negative one (10-19); the label says
    which set has the majority.  The other words are neutral filler."""
    ids = torch.randint(20, args.vocab, (n, args.seq), generator=gen)
    y = torch.randint(0, 2, (n,), generator=gen)
    n_pos = torch.where(y == 1, torch.randint(4, 6, (n,), generator=gen), torch.randint(1, 3, (n,), generator=gen))
    slots = torch.rand(n, args.seq, generator=gen).argsort(dim=1)[:, :6]          # six distinct positions
    is_pos = torch.arange(6)[None, :] < n_pos[:, None]
    words = torch.randint(0, 10, (n, 6), generator=gen) + (~is_pos).long() * 10
    ids.scatter_(1, slots, words)
    return ids, y


model = Encoder(args.vocab, args.d_model, args.seq, 2).to(device)
pub_x, pub_y = topic_data(args.samples)
opt = torch.optim.AdamW(model.parameters(), lr=2e-3)
for x, y in DataLoader(TensorDataset(pub_x, pub_y), batch_size=100, shuffle=True):
    opt.zero_grad()
    nn.functional.cross_entropy(model(x.to(device)), y.to(device)).backward()
    opt.step()
print("public pretraining done")

# %% [markdown]
# ## Freeze the bottom, put a new head on top
# Only parameters with `requires_grad=True` get per-sample gradients, are clipped and receive noise.

# %%
for part in (model.tok, model.pos, model.lower):
    for p in part.parameters():
        p.requires_grad_(False)
model.head = nn.Linear(args.d_model, 2).to(device)
trainable = [p for p in model.parameters() if p.requires_grad]
print(f"training {sum(p.numel() for p in trainable):,} of {sum(p.numel() for p in model.parameters()):,} parameters")
assert ModuleValidator.validate(model, strict=False) == []

# %% [markdown]
# ## Private fine-tuning with ghost clipping
# `grad_sample_mode="ghost"` computes per-sample gradient *norms* without the gradients and the clipped sum directly;
# `make_private` then also returns a wrapped loss function, and the loop keeps its usual shape.

# %%
priv_x, priv_y = sentiment_data(args.samples)
test_x, test_y = sentiment_data(1000)
loader = DataLoader(TensorDataset(priv_x, priv_y), batch_size=args.batch_size)
optimizer = torch.optim.AdamW(trainable, lr=3e-3)
engine = PrivacyEngine(accountant="prv")
model, optimizer, criterion, loader = engine.make_private_with_epsilon(
    module=model, optimizer=optimizer, data_loader=loader, criterion=nn.CrossEntropyLoss(),
    target_epsilon=args.epsilon, target_delta=args.delta, epochs=args.epochs, max_grad_norm=args.clip,
    grad_sample_mode="ghost")
for epoch in range(args.epochs):
    model.train()
    for x, y in loader:
        optimizer.zero_grad()
        loss = criterion(model(x.to(device)), y.to(device))
        loss.backward()
        optimizer.step()
    model.eval()
    with torch.no_grad():
        acc = (model(test_x.to(device)).argmax(1).cpu() == test_y).float().mean().item()
    print(f"epoch {epoch}: loss {loss.item():.3f}  test accuracy {acc:.3f}  eps = {engine.get_epsilon(args.delta):.2f}")
