"""Kernel-time breakdown of one DP training step of the Llama benchmark model
(``torch.profiler`` CUDA activity; shares, not absolute times).

    python -m opacus_b200.benchmarks.step_profile [--layers N] [--impl ours|reference] [--top 40]
"""
import argparse
import os
import sys

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--vocab", type=int, default=None)
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--top", type=int, default=40)
    ap.add_argument("--engine", default="sharded", choices=["sharded", "plain"])
    ap.add_argument("--ce", default="fused", choices=["fused", "torch"])
    ap.add_argument("--cprofile", type=int, default=0, help="profile the host side of this many steps instead")
    args = ap.parse_args()
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    sys.path.insert(0, root)
    import bench

    args.gpus, args.steps, args.warmup = 1, 1, 2
    torch.cuda.set_device(0)
    build = bench.build_ours if args.impl == "ours" else bench.build_reference
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29534")
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    if args.impl == "ours" and args.engine == "sharded":
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", 0))
    step, cfg, engine, mode = build(args, 0, 1)
    ids_h, labels_h = bench.make_data(cfg, args, 1, 0)
    ids, labels = ids_h.cuda(), labels_h.cuda()
    for i in range(3):
        step(ids[i], labels[i])
    torch.cuda.synchronize()
    if args.cprofile:
        import cProfile
        import pstats
        import time

        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for i in range(args.cprofile):
            step(ids[i % len(ids)], labels[i % len(ids)])
        host = (time.perf_counter() - t0) / args.cprofile
        torch.cuda.synchronize()
        wall = (time.perf_counter() - t0) / args.cprofile
        print(f"host time to enqueue one step {host * 1e3:.1f} ms; wall {wall * 1e3:.1f} ms")
        pr = cProfile.Profile()
        pr.enable()
        for i in range(args.cprofile):
            step(ids[i % len(ids)], labels[i % len(ids)])
        pr.disable()
        torch.cuda.synchronize()
        pstats.Stats(pr).sort_stats("tottime").print_stats(args.top)
        return
    from torch.profiler import ProfilerActivity, profile

    with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
        step(ids[3], labels[3])
        torch.cuda.synchronize()
    ev = [e for e in prof.key_averages() if e.device_time_total > 0 and e.device_type.name == "CUDA"]
    total = sum(e.device_time_total for e in ev)
    ev.sort(key=lambda e: -e.device_time_total)
    print(f"total kernel time {total / 1e3:.2f} ms over {sum(e.count for e in ev)} launches")
    for e in ev[: args.top]:
        print(f"{e.device_time_total / 1e3:9.3f} ms {100 * e.device_time_total / total:5.1f}% x{e.count:5d}  {e.key[:110]}")


if __name__ == "__main__":
    main()
