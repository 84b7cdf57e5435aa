"""DP-SGD for a ResNet-18 with GroupNorm on 3x32x32 images: validator fix-up, virtual batches, optional DDP.

    python examples/cifar10.py [--logical-batch 1024] [--physical-batch 256] [--steps 4] [--device cuda]
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 examples/cifar10.py --device cuda

Counterpart in the reference: ``examples/cifar10.py``.
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
import torchvision  # noqa: E402

from opacus_b200 import PrivacyEngine  # noqa: E402
from opacus_b200.models import resnet18_gn  # noqa: E402
from opacus_b200.distributed import DifferentiallyPrivateDistributedDataParallel as DPDDP  # noqa: E402
from opacus_b200.utils.batch_memory_manager import BatchMemoryManager  # noqa: E402
from opacus_b200.validators import ModuleValidator  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--logical-batch", type=int, default=1024)
    ap.add_argument("--physical-batch", type=int, default=256)
    ap.add_argument("--steps", type=int, default=4, help="logical steps")
    ap.add_argument("--sigma", type=float, default=1.0)
    ap.add_argument("--clip", type=float, default=1.0)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if world > 1:
        if args.device == "cuda":
            torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
        dist.init_process_group("nccl" if args.device == "cuda" else "gloo")
    torch.manual_seed(0)
    stock = torchvision.models.resnet18(num_classes=10)            # BatchNorm inside: not DP compatible
    print("validator on the stock model:", sorted({type(e).__name__ for e in ModuleValidator.validate(stock, strict=False)}))
    assert ModuleValidator.is_valid(ModuleValidator.fix(stock))    # BatchNorm -> GroupNorm
    # the stock blocks add the residual in place on a hooked layer's output, which module backward hooks do
    # not allow; this package's ResNet-18-GN is the same network written without in-place arithmetic
    model = resnet18_gn(num_classes=10).to(args.device)
    n = args.logical_batch * world * args.steps
    g = torch.Generator().manual_seed(rank)
    data = TensorDataset(torch.randn(n, 3, 32, 32, generator=g), torch.randint(0, 10, (n,), generator=g))
    module = DPDDP(model) if world > 1 else model
    optimizer = torch.optim.SGD(model.parameters(), lr=0.1, momentum=0.9)
    engine = PrivacyEngine()
    module, optimizer, loader = engine.make_private(
        module=module, optimizer=optimizer, data_loader=DataLoader(data, batch_size=args.logical_batch * world),
        noise_multiplier=args.sigma, max_grad_norm=args.clip)
    with BatchMemoryManager(data_loader=loader, max_physical_batch_size=args.physical_batch,
                            optimizer=optimizer) as physical:
        for x, y in physical:
            x, y = x.to(args.device), y.to(args.device)
            optimizer.zero_grad()
            if len(x):
                loss = F.cross_entropy(module(x), y)
                loss.backward()
            optimizer.step()                                        # a real step only at logical-batch boundaries
    if rank == 0:
        print(f"done: loss {loss.item():.3f}, epsilon {engine.get_epsilon(1e-5):.2f}")
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
