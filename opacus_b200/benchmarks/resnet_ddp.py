"""ResNet-18 (GroupNorm, 32 groups) on 3x32x32 images with data-parallel DP-SGD:
logical batch 4096 per GPU step split into physical batches of 512 by
``BatchMemoryManager``, hooks mode, flat clipping C = 1.0, sigma = 1.0, SGD with
momentum 0.9, bf16 compute.  Reports samples/s (device-timed, max over ranks).

    python -m opacus_b200.benchmarks.resnet_ddp [--impl ours|reference] [--logical 4096] [--physical 512] [--steps 2]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        -m opacus_b200.benchmarks.resnet_ddp ...

``ours`` wraps the model in ``ShardedDataParallel`` (bf16 compute weights, fused
reduce + noise + momentum-SGD + publish kernel); ``reference`` uses ``DPDDP`` +
``DistributedDPOptimizer`` of the reference library under autocast.
"""
import argparse
import datetime
import json
import os
import sys

import torch
import torch.distributed as dist
import torch.nn as nn
from torch.utils.data import DataLoader, TensorDataset


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--logical", type=int, default=4096)
    ap.add_argument("--physical", type=int, default=512)
    ap.add_argument("--steps", type=int, default=2, help="timed logical steps")
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--channels-last", action="store_true", help="NHWC model and inputs (both libraries)")
    args = ap.parse_args()
    import warnings

    warnings.simplefilter("ignore")
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    sys.path.insert(0, root)
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29561")
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=datetime.timedelta(seconds=300))

    if args.impl == "reference":           # stock-PyTorch definition, nothing of this package on the reference's path
        sys.path.insert(0, os.path.join(root, "baseline"))
        from resnet_plain import resnet18_gn
    else:
        from opacus_b200.models import resnet18_gn

    torch.manual_seed(0)
    model = resnet18_gn().cuda()
    if args.channels_last:
        model = model.to(memory_format=torch.channels_last)
    n_batches = args.steps + args.warmup
    n_data = args.logical * world * n_batches
    # the loader only fixes the sampling rate and batch structure; samples are synthetic
    g = torch.Generator().manual_seed(rank)
    ds = TensorDataset(torch.randn(n_data, 3, 32, 32, generator=g), torch.randint(0, 10, (n_data,), generator=g))
    dl = DataLoader(ds, batch_size=args.logical * world)

    if args.impl == "reference":
        sys.path.insert(0, os.path.join(root, "baseline", "_ref"))
        from opacus import PrivacyEngine
        from opacus.distributed import DifferentiallyPrivateDistributedDataParallel as DPDDP
        from opacus.utils.batch_memory_manager import BatchMemoryManager

        module = DPDDP(model)
        autocast = True
    else:
        from opacus_b200 import PrivacyEngine
        from opacus_b200.parallel.sharded import ShardedDataParallel
        from opacus_b200.utils.batch_memory_manager import BatchMemoryManager

        module = ShardedDataParallel(model)
        autocast = False
    opt = torch.optim.SGD(model.parameters(), lr=0.1, momentum=0.9)
    pe = PrivacyEngine(accountant="rdp")
    module, opt, dl = pe.make_private(module=module, optimizer=opt, data_loader=dl, noise_multiplier=1.0,
                                      max_grad_norm=1.0, grad_sample_mode="hooks", poisson_sampling=True)
    crit = nn.CrossEntropyLoss()

    def logical_steps(count, timed):
        seen = 0
        done = 0
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with BatchMemoryManager(data_loader=dl, max_physical_batch_size=args.physical, optimizer=opt) as loader:
            torch.cuda.synchronize()
            start.record()
            for x, y in loader:
                x = x.cuda(non_blocking=True)
                y = y.cuda(non_blocking=True)
                if not autocast:
                    x = x.to(torch.bfloat16)
                if args.channels_last:
                    x = x.contiguous(memory_format=torch.channels_last)
                opt.zero_grad()
                if len(x):
                    if autocast:
                        with torch.autocast("cuda", dtype=torch.bfloat16):
                            out = module(x)
                    else:
                        out = module(x)
                    crit(out.float(), y).backward()
                    seen += len(x)
                skipped = opt._check_skip_next_step(pop_next=False)
                opt.step()
                if not skipped:
                    done += 1
                    if done >= count:
                        break
            end.record()
            torch.cuda.synchronize()
        return seen, start.elapsed_time(end)

    logical_steps(args.warmup, False)
    dist.barrier()
    seen, ms = logical_steps(args.steps, True)
    t = torch.tensor([ms, float(seen)], device="cuda", dtype=torch.float64)
    tmax = t.clone()
    dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    if rank == 0:
        total_seen = float(t[1])
        print(json.dumps({"impl": args.impl, "metric": "dp_resnet18gn_samples_per_s", "n_gpus": world,
                          "value": total_seen / (float(tmax[0]) / 1e3), "logical_batch_per_gpu": args.logical,
                          "physical_batch": args.physical, "logical_steps": args.steps, "samples": total_seen,
                          "ms": float(tmax[0]), "channels_last": bool(args.channels_last),
                          "epsilon_delta_1e-5": pe.get_epsilon(1e-5), "dtype": "bf16"}))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
