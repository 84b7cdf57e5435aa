"""Private sentiment classifier (mean of word embeddings + MLP) with DP-Adam and a target epsilon.

    python examples/imdb.py [--epsilon 3.0] [--epochs 2]

Counterpart in the reference: ``examples/imdb.py``.
"""
import argparse
import os
import sys

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.data import DataLoader, TensorDataset

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))   # run from a source checkout

from opacus_b200 import PrivacyEngine  # noqa: E402


class BagOfEmbeddings(nn.Module):
    def __init__(self, vocab=5000, dim=32):
        super().__init__()
        self.emb = nn.Embedding(vocab, dim, padding_idx=0)
        self.fc = nn.Sequential(nn.Linear(dim, 32), nn.ReLU(), nn.Linear(32, 2))

    def forward(self, ids):
        mask = (ids != 0).unsqueeze(-1)
        return self.fc((self.emb(ids) * mask).sum(1) / mask.sum(1).clamp(min=1))


def synthetic(n, vocab=5000, length=64, seed=0):
    g = torch.Generator().manual_seed(seed)
    y = torch.randint(0, 2, (n,), generator=g)
    lo = torch.where(y[:, None] == 1, 1, vocab // 2)               # the two classes use different halves of the vocabulary
    ids = lo + torch.randint(0, vocab // 2 - 1, (n, length), generator=g)
    noise = torch.randint(1, vocab, (n, length), generator=g)
    ids = torch.where(torch.rand(n, length, generator=g) < 0.6, noise, ids)
    return TensorDataset(ids, y)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--epsilon", type=float, default=3.0)
    ap.add_argument("--epochs", type=int, default=2)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    args = ap.parse_args()
    torch.manual_seed(0)
    model = BagOfEmbeddings().to(args.device)
    optimizer = torch.optim.Adam(model.parameters(), lr=0.01)
    engine = PrivacyEngine(accountant="prv")
    model, optimizer, loader = engine.make_private_with_epsilon(
        module=model, optimizer=optimizer, data_loader=DataLoader(synthetic(4096), batch_size=256),
        target_epsilon=args.epsilon, target_delta=1e-5, epochs=args.epochs, max_grad_norm=1.0)
    print(f"calibrated noise multiplier: {optimizer.noise_multiplier:.3f}")
    test = synthetic(1024, seed=1)
    for epoch in range(args.epochs):
        model.train()
        for x, y in loader:
            optimizer.zero_grad()
            if len(x):
                F.cross_entropy(model(x.to(args.device)), y.to(args.device)).backward()
            optimizer.step()
        model.eval()
        with torch.no_grad():
            x, y = test.tensors
            acc = (model(x.to(args.device)).argmax(1).cpu() == y).float().mean().item()
        print(f"epoch {epoch + 1}: accuracy {acc:.3f}, epsilon spent {engine.get_epsilon(1e-5):.2f}")


if __name__ == "__main__":
    main()
