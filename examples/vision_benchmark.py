"""Throughput and memory of DP training on synthetic images, one line per configuration.

    python examples/vision_benchmark.py --device cuda --architecture resnet18 --batch-size 256 --steps 20
    python examples/vision_benchmark.py --device cuda --modes none,hooks,ghost --dtype bf16
    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 examples/vision_benchmark.py --device cuda

For every requested mode (``none`` = plain SGD without privacy, ``hooks``, ``ghost``, ``functorch``, ``ew``) the same
model is trained for ``--steps`` steps on random ``3 x H x W`` images; the script prints samples per second (CUDA events
on a GPU, wall clock on the CPU; the first steps are warm-up), the peak CUDA memory of a step, and the ratio to the
non-private run.  Architectures: ``resnet18`` (GroupNorm instead of BatchNorm, this package's definition),
``cnn`` (the small MNIST / CIFAR network) and any ``torchvision.models`` name (BatchNorm is replaced by GroupNorm through
``ModuleValidator.fix``).  Under ``torch.distributed.run`` the model is wrapped for data parallelism
(``DifferentiallyPrivateDistributedDataParallel``); ``--clip-per-layer`` switches to per-layer clipping.

Counterpart in the reference: ``examples/vision_benchmark.py``.
"""
import argparse
import os
import sys
import time

import torch
import torch.nn as nn
from torch.utils.data import DataLoader, TensorDataset

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))   # run from a source checkout

from opacus_b200 import PrivacyEngine  # noqa: E402
from opacus_b200.validators import ModuleValidator  # noqa: E402


def build_model(name: str, gn_groups: int, classes: int, size: int) -> nn.Module:
    if name == "resnet18":
        from opacus_b200.models import resnet18_gn

        return resnet18_gn(num_classes=classes, groups=gn_groups)
    if name == "cnn":
        return nn.Sequential(nn.Conv2d(3, 32, 3, padding=1), nn.ReLU(), nn.AvgPool2d(2),
                             nn.Conv2d(32, 64, 3, padding=1), nn.ReLU(), nn.AdaptiveAvgPool2d(4), nn.Flatten(),
                             nn.Linear(64 * 16, classes))
    from torchvision import models

    return ModuleValidator.fix(getattr(models, name)(num_classes=classes))


def run_mode(mode: str, args, device, rank: int, world: int):
    torch.manual_seed(0)
    model = build_model(args.architecture, args.gn_groups, args.classes, args.height).to(device)
    dtype = torch.bfloat16 if args.dtype == "bf16" else torch.float32
    model = model.to(dtype)
    if world > 1:
        from opacus_b200.distributed import DifferentiallyPrivateDistributedDataParallel as DPDDP

        model = DPDDP(model) if mode != "none" else nn.parallel.DistributedDataParallel(model)
    optimizer = torch.optim.SGD(model.parameters(), lr=args.lr, momentum=args.momentum, weight_decay=args.weight_decay)
    B = args.batch_size
    data = TensorDataset(torch.zeros(B * 16 * world, 1))
    loader = DataLoader(data, batch_size=B * world)
    criterion = nn.CrossEntropyLoss()
    engine = None
    if mode != "none":
        engine = PrivacyEngine(accountant="rdp", secure_mode=args.secure_mode)
        clipping = "per_layer" if args.clip_per_layer else "flat"
        bound = args.max_per_sample_grad_norm
        if args.clip_per_layer:
            n_params = sum(1 for p in model.parameters() if p.requires_grad)
            bound = [bound / n_params ** 0.5] * n_params
        out = engine.make_private(module=model, optimizer=optimizer, criterion=criterion, data_loader=loader,
                                  noise_multiplier=args.sigma, max_grad_norm=bound, clipping=clipping,
                                  grad_sample_mode=mode, poisson_sampling=False)
        model, optimizer = out[0], out[1]
        if mode == "ghost":
            criterion = out[2]
    x = torch.randn(B, 3, args.height, args.width, device=device, dtype=dtype)
    y = torch.randint(0, args.classes, (B,), device=device)

    def step():
        optimizer.zero_grad(set_to_none=True)
        loss = criterion(model(x).float(), y)
        loss.backward()
        optimizer.step()

    warm = max(2, args.steps // 5)
    for _ in range(warm):
        step()
    if device.type == "cuda":
        torch.cuda.synchronize()
        base = torch.cuda.memory_allocated()
        torch.cuda.reset_peak_memory_stats()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(args.steps):
            step()
        t1.record()
        torch.cuda.synchronize()
        seconds = t0.elapsed_time(t1) / 1e3
        peak_mb = (torch.cuda.max_memory_allocated() - base) / 2 ** 20
    else:
        start = time.perf_counter()
        for _ in range(args.steps):
            step()
        seconds = time.perf_counter() - start
        peak_mb = float("nan")
    rate = args.steps * B * world / seconds
    eps = engine.get_epsilon(args.delta) if engine is not None else None
    return rate, peak_mb, eps


def main():
    ap = argparse.ArgumentParser(description="DP training throughput on synthetic images")
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--architecture", default="resnet18")
    ap.add_argument("--modes", default="none,hooks,ghost")
    ap.add_argument("--dtype", default="fp32", choices=["fp32", "bf16"])
    ap.add_argument("--batch-size", type=int, default=128, help="per process")
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--height", type=int, default=32)
    ap.add_argument("--width", type=int, default=32)
    ap.add_argument("--classes", type=int, default=10)
    ap.add_argument("--gn-groups", type=int, default=32)
    ap.add_argument("--lr", type=float, default=0.1)
    ap.add_argument("--momentum", type=float, default=0.9)
    ap.add_argument("--weight-decay", type=float, default=0.0)
    ap.add_argument("--sigma", type=float, default=1.0)
    ap.add_argument("--max-per-sample-grad-norm", type=float, default=1.0)
    ap.add_argument("--delta", type=float, default=1e-5)
    ap.add_argument("--secure-mode", action="store_true")
    ap.add_argument("--clip-per-layer", action="store_true")
    args = ap.parse_args()

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    device = torch.device(args.device)
    if world > 1:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if device.type == "cuda":
            torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
            device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
        dist.init_process_group("nccl" if device.type == "cuda" else "gloo")
    results = {}
    for mode in args.modes.split(","):
        results[mode] = run_mode(mode, args, device, rank, world)
        if rank == 0:
            rate, mem, eps = results[mode]
            rel = f"  {rate / results['none'][0]:5.2f}x of non-private" if "none" in results and mode != "none" else ""
            eps_s = f"  eps({args.delta:g}) = {eps:.2f}" if eps is not None else ""
            print(f"{args.architecture:12s} {args.dtype:5s} {mode:10s} {rate:12.1f} samples/s  "
                  f"peak {mem:9.1f} MB{rel}{eps_s}", flush=True)
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()


if __name__ == "__main__":
    main()
