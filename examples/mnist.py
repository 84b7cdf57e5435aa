"""DP-SGD on MNIST (or synthetic digits): the basic training loop.

    python examples/mnist.py [--epochs 1] [--sigma 1.0] [--clip 1.0] [--data-root PATH] [--device cpu|cuda]

Counterpart in the reference: ``examples/mnist.py``.
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
from opacus_b200.models import SmallCNN  # noqa: E402


def load(root, n):
    if root:
        from torchvision import datasets, transforms

        tf = transforms.Compose([transforms.ToTensor(), transforms.Normalize((0.1307,), (0.3081,))])
        return datasets.MNIST(root, train=True, transform=tf), datasets.MNIST(root, train=False, transform=tf)
    g = torch.Generator().manual_seed(0)
    proto = torch.randn(10, 1, 28, 28, generator=g)                     # one blurry prototype per class
    def make(m):
        y = torch.randint(0, 10, (m,), generator=g)
        return TensorDataset(proto[y] + 0.7 * torch.randn(m, 1, 28, 28, generator=g), y)
    return make(n), make(n // 6)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--epochs", type=int, default=1)
    ap.add_argument("--batch-size", type=int, default=256)
    ap.add_argument("--lr", type=float, default=0.1)
    ap.add_argument("--sigma", type=float, default=1.0)
    ap.add_argument("--clip", type=float, default=1.0)
    ap.add_argument("--delta", type=float, default=1e-5)
    ap.add_argument("--samples", type=int, default=6000, help="synthetic training set size")
    ap.add_argument("--data-root", default=None)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    args = ap.parse_args()
    train, test = load(args.data_root, args.samples)
    model = SmallCNN().to(args.device)
    optimizer = torch.optim.SGD(model.parameters(), lr=args.lr)
    engine = PrivacyEngine(accountant="rdp")
    model, optimizer, loader = engine.make_private(
        module=model, optimizer=optimizer, data_loader=DataLoader(train, batch_size=args.batch_size),
        noise_multiplier=args.sigma, max_grad_norm=args.clip)
    for epoch in range(args.epochs):
        model.train()
        for x, y in loader:
            x, y = x.to(args.device), y.to(args.device)
            optimizer.zero_grad()
            if len(x):
                F.cross_entropy(model(x), y).backward()
            optimizer.step()
        model.eval()
        correct = 0
        with torch.no_grad():
            for x, y in DataLoader(test, batch_size=1024):
                correct += (model(x.to(args.device)).argmax(1).cpu() == y).sum().item()
        print(f"epoch {epoch + 1}: test accuracy {correct / len(test):.3f}, "
              f"epsilon {engine.get_epsilon(args.delta):.2f} at delta {args.delta}")


if __name__ == "__main__":
    main()
