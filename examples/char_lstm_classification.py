"""Character-level name classification with a DP-compatible LSTM / GRU / RNN.

    python examples/char_lstm_classification.py [--cell lstm|gru|rnn] [--epochs 2]

Counterpart in the reference: ``examples/char-lstm-classification.py``.
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
from opacus_b200.layers import DPGRU, DPLSTM, DPRNN  # noqa: E402


class CharClassifier(nn.Module):
    def __init__(self, cell, vocab=64, emb=32, hidden=64, classes=8):
        super().__init__()
        self.emb = nn.Embedding(vocab, emb, padding_idx=0)
        self.rnn = {"lstm": DPLSTM, "gru": DPGRU, "rnn": DPRNN}[cell](emb, hidden, batch_first=True)
        self.out = nn.Linear(hidden, classes)

    def forward(self, x):
        h, _ = self.rnn(self.emb(x))
        last = (x != 0).sum(1).clamp(min=1) - 1                      # last real character of every name
        return self.out(h[torch.arange(len(x)), last])


def synthetic(n, vocab=64, classes=8, max_len=12, seed=0):
    """Names whose class is decided by which characters they favour."""
    g = torch.Generator().manual_seed(seed)
    y = torch.randint(0, classes, (n,), generator=g)
    lens = torch.randint(3, max_len + 1, (n,), generator=g)
    base = 1 + (y[:, None] * 7 + torch.randint(0, 9, (n, max_len), generator=g)) % (vocab - 1)
    x = torch.where(torch.arange(max_len)[None, :] < lens[:, None], base, torch.zeros_like(base))
    return TensorDataset(x, y)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--cell", default="lstm", choices=["lstm", "gru", "rnn"])
    ap.add_argument("--epochs", type=int, default=2)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    args = ap.parse_args()
    torch.manual_seed(0)
    model = CharClassifier(args.cell).to(args.device)
    optimizer = torch.optim.Adam(model.parameters(), lr=5e-3)
    engine = PrivacyEngine()
    model, optimizer, loader = engine.make_private(
        module=model, optimizer=optimizer, data_loader=DataLoader(synthetic(2048), batch_size=128),
        noise_multiplier=0.8, max_grad_norm=1.0)
    test = synthetic(512, seed=1)
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
        print(f"epoch {epoch + 1}: accuracy {acc:.3f}, epsilon {engine.get_epsilon(8e-5):.2f}")


if __name__ == "__main__":
    main()
