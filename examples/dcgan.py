"""A small GAN whose discriminator -- the only network that sees real data -- is trained with DP-SGD.

    python examples/dcgan.py [--steps 30]

Counterpart in the reference: ``examples/dcgan.py``.
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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    args = ap.parse_args()
    torch.manual_seed(0)
    dev = args.device
    G = nn.Sequential(nn.ConvTranspose2d(16, 32, 4, 1, 0), nn.GroupNorm(4, 32), nn.ReLU(),
                      nn.ConvTranspose2d(32, 16, 4, 2, 1), nn.GroupNorm(4, 16), nn.ReLU(),
                      nn.ConvTranspose2d(16, 1, 4, 2, 1), nn.Tanh()).to(dev)            # z [N,16,1,1] -> [N,1,16,16]
    D = nn.Sequential(nn.Conv2d(1, 16, 4, 2, 1), nn.LeakyReLU(0.2), nn.Conv2d(16, 32, 4, 2, 1), nn.GroupNorm(4, 32),
                      nn.LeakyReLU(0.2), nn.Conv2d(32, 1, 4, 1, 0), nn.Flatten()).to(dev)
    real = TensorDataset(torch.tanh(torch.randn(1024, 1, 16, 16) * 0.3 + torch.linspace(-1, 1, 16)[None, None, None, :]))
    opt_g = torch.optim.Adam(G.parameters(), lr=2e-4, betas=(0.5, 0.999))
    opt_d = torch.optim.Adam(D.parameters(), lr=2e-4, betas=(0.5, 0.999))
    engine = PrivacyEngine()
    D, opt_d, loader = engine.make_private(module=D, optimizer=opt_d, data_loader=DataLoader(real, batch_size=64),
                                           noise_multiplier=0.7, max_grad_norm=1.0)
    step = 0
    while step < args.steps:
        for (x,) in loader:
            if not len(x):
                continue
            x = x.to(dev)
            # discriminator: real and fake batches go through SEPARATE private steps (each sample clipped once)
            opt_d.zero_grad()
            F.binary_cross_entropy_with_logits(D(x), torch.ones(len(x), 1, device=dev)).backward()
            opt_d.step()
            fake = G(torch.randn(len(x), 16, 1, 1, device=dev))
            opt_d.zero_grad()
            F.binary_cross_entropy_with_logits(D(fake.detach()), torch.zeros(len(x), 1, device=dev)).backward()
            opt_d.step()
            # generator: only touches the discriminator's outputs, no privacy cost (post-processing)
            opt_g.zero_grad()
            D.disable_hooks()
            loss_g = F.binary_cross_entropy_with_logits(D(fake), torch.ones(len(x), 1, device=dev))
            loss_g.backward()
            D.enable_hooks()
            opt_g.step()
            step += 1
            if step >= args.steps:
                break
    print(f"generator loss {loss_g.item():.3f}, epsilon {engine.get_epsilon(1e-5):.2f}")


if __name__ == "__main__":
    main()
