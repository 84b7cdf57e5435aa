# %% [markdown]
# # Differentially private training on several GPUs (data parallel)
#
# With data parallelism every process holds the whole model and a share of each batch.  For DP-SGD three things have to
# be right, and the package takes care of all of them when it sees a distributed model:
#
# * **sampling**: every process draws its own Poisson sample of its own shard of the data, with the *same* rate
#   `q = logical batch / dataset size`, so the union is a Poisson sample of the whole data set;
# * **noise**: clipped gradient sums are added up over processes, and noise of standard deviation
#   `noise_multiplier * max_grad_norm` must be added to that total exactly **once** (not once per process);
# * **averaging**: the noisy total is divided by the *global* expected batch size.
#
# Two wrappers are offered:
#
# * `DifferentiallyPrivateDistributedDataParallel` (DPDDP): a marker without gradient hooks; the optimizer
#   (`DistributedDPOptimizer`) reduces the clipped sums itself.  On GPUs of one NVLink domain this is one fused kernel
#   (reduce + noise + update) over a flat gradient buffer in symmetric memory; elsewhere it is a bucketed all-reduce.
# * `torch.nn.parallel.DistributedDataParallel` with `clipping="per_layer"`: every layer is clipped to its own norm bound as
#   soon as its gradient exists, so the all-reduce of that layer overlaps the rest of the backward pass.
#
# Launch (any number of processes; gloo on CPUs, NCCL on GPUs):
#
#     python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 tutorials/ddp_tutorial.py
#     python tutorials/ddp_tutorial.py --spawn 2          # the script starts its own two CPU processes
#
# Counterpart in the reference: `tutorials/ddp_tutorial.ipynb`.

# %%
import argparse
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn as nn
from torch.utils.data import DataLoader, TensorDataset

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from opacus_b200 import PrivacyEngine  # noqa: E402
from opacus_b200.distributed import DifferentiallyPrivateDistributedDataParallel as DPDDP  # noqa: E402


def make_data(n=4096):
    gen = torch.Generator().manual_seed(0)            # the same data set in every process; the sampler shards it
    proto = torch.randn(10, 1, 28, 28, generator=gen)
    y = torch.randint(0, 10, (n,), generator=gen)
    return TensorDataset(proto[y] + 0.7 * torch.randn(n, 1, 28, 28, generator=gen), y)


def make_model():
    torch.manual_seed(0)                              # replicas must start identical
    return nn.Sequential(nn.Conv2d(1, 16, 8, 2, padding=3), nn.ReLU(), nn.MaxPool2d(2, 1),
                         nn.Conv2d(16, 32, 4, 2), nn.ReLU(), nn.MaxPool2d(2, 1), nn.Flatten(),
                         nn.Linear(32 * 4 * 4, 32), nn.ReLU(), nn.Linear(32, 10))


# %% [markdown]
# ## One process
# `make_private` recognises the DPDDP wrapper, returns a `DistributedDPOptimizer`, and builds a loader whose sampler knows
# rank and world size.  The loop is the single-process loop.

# %%
def worker(rank, world, args):
    use_cuda = torch.cuda.is_available() and not args.cpu
    if use_cuda:
        torch.cuda.set_device(rank % torch.cuda.device_count())
    device = torch.device("cuda", rank % torch.cuda.device_count()) if use_cuda else torch.device("cpu")
    if not dist.is_initialized():
        dist.init_process_group("nccl" if use_cuda else "gloo", rank=rank, world_size=world)

    model = DPDDP(make_model().to(device))
    optimizer = torch.optim.SGD(model.parameters(), lr=args.lr)
    loader = DataLoader(make_data(), batch_size=args.batch_size)          # the LOGICAL (global) batch size
    engine = PrivacyEngine(accountant="rdp")
    model, optimizer, loader = engine.make_private(
        module=model, optimizer=optimizer, data_loader=loader, noise_multiplier=args.sigma, max_grad_norm=args.clip)
    if rank == 0:
        print(f"{world} processes, optimizer {type(optimizer).__name__}, "
              f"expected batch per process {optimizer.expected_batch_size}")
    criterion = nn.CrossEntropyLoss()
    for epoch in range(args.epochs):
        for x, y in loader:
            optimizer.zero_grad()
            loss = criterion(model(x.to(device)), y.to(device))
            loss.backward()
            optimizer.step()
        # every process has accounted the same steps, so epsilon is the same everywhere
        if rank == 0:
            print(f"epoch {epoch}: loss {loss.item():.3f}  eps = {engine.get_epsilon(1e-5):.2f}")

    # replicas stay identical: same reduced gradient, same noise (drawn once, by the owner of each parameter range)
    flat = torch.cat([p.detach().float().flatten() for p in model.parameters()])
    gathered = [torch.empty_like(flat) for _ in range(world)]
    dist.all_gather(gathered, flat)
    if rank == 0:
        print("replicas identical:", all(torch.equal(gathered[0], t) for t in gathered))
    dist.barrier()
    dist.destroy_process_group()


def _spawned(rank, world, args):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(args.port), RANK=str(rank), WORLD_SIZE=str(world))
    worker(rank, world, args)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--spawn", type=int, default=0, help="start this many local processes instead of using torchrun")
    ap.add_argument("--cpu", action="store_true")
    ap.add_argument("--port", type=int, default=29533)
    ap.add_argument("--epochs", type=int, default=2)
    ap.add_argument("--batch-size", type=int, default=256)
    ap.add_argument("--sigma", type=float, default=1.0)
    ap.add_argument("--clip", type=float, default=1.0)
    ap.add_argument("--lr", type=float, default=0.2)
    args, _ = ap.parse_known_args()          # a notebook kernel passes arguments of its own
    if args.spawn:
        args.cpu = args.cpu or torch.cuda.device_count() < args.spawn
        mp.spawn(_spawned, args=(args.spawn, args), nprocs=args.spawn, join=True)
    else:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", str(args.port))
        worker(int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), args)
