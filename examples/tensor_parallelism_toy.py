"""Column / row parallel MLP under ghost clipping (works with the gloo backend on CPU).

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 examples/tensor_parallelism_toy.py

Counterpart in the reference: ``examples/tensor_parallelism_toy.py``.
"""
import argparse
import os
import sys

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.data import DataLoader, TensorDataset

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))   # run from a source checkout

import torch.distributed as dist  # noqa: E402

from opacus_b200.grad_sample import GradSampleModuleFastGradientClippingTP  # noqa: E402
from opacus_b200.parallel.tensor_parallel import (ColumnParallelLinear, RowParallelLinear,  # noqa: E402
                                                  TensorParallelDPOptimizer)
from opacus_b200.utils.fast_gradient_clipping_utils import DPLossFastGradientClipping  # noqa: E402


class ToyMLP(nn.Module):
    def __init__(self):
        super().__init__()
        self.norm = nn.LayerNorm(32)                                  # replicated, trained (identical noise on all ranks)
        self.up = ColumnParallelLinear(32, 128)                       # output features split over the ranks
        self.down = RowParallelLinear(128, 10)                        # input features split, partial sums all-reduced

    def forward(self, x):
        return self.down(F.relu(self.up(self.norm(x))))


def main():
    cuda = torch.cuda.is_available()
    if cuda:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    dist.init_process_group("nccl" if cuda else "gloo")
    dev = "cuda" if cuda else "cpu"
    torch.manual_seed(0)                                              # same init and same data on every rank
    model = ToyMLP().to(dev)
    gsm = GradSampleModuleFastGradientClippingTP(model, max_grad_norm=1.0, single_pass=True)
    opt = TensorParallelDPOptimizer(torch.optim.SGD(model.parameters(), lr=0.1), noise_multiplier=1.0,
                                    max_grad_norm=1.0, expected_batch_size=16)
    crit = DPLossFastGradientClipping(gsm, opt, nn.CrossEntropyLoss(), "mean")
    x, y = torch.randn(16, 32, device=dev), torch.randint(0, 10, (16,), device=dev)
    for step in range(5):
        opt.zero_grad()
        loss = crit(gsm(x), y)
        loss.backward()
        opt.step()
        if dist.get_rank() == 0:
            print(f"step {step}: loss {loss.item():.3f}, first norms {gsm.per_sample_gradient_norms[:3].tolist()}")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
