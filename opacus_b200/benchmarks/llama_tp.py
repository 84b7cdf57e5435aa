"""Llama-3-8B-shaped decoder under N-way tensor parallelism with ghost clipping: tokens/s.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port P \
        -m opacus_b200.benchmarks.llama_tp [--layers 32] [--seq 2048] [--batch 64] [--micro 8] [--steps 3]

By default all ranks form one tensor-parallel group and see the same batch; ``--tp K`` (K dividing the number of
ranks) makes groups of K consecutive ranks and runs the ``ranks / K`` groups as sharded data parallelism over
``ShardedDataParallel`` (2-d layout: each group sees its own share of the logical batch; optimizer state and fp32
master weights are sharded over the ranks with the same position in their groups).  Linear layers are
column / row parallel, the output layer is split over the vocabulary and feeds
``VocabParallelCrossEntropy``; embedding and norm weights are replicated and
trained (identical noise on every rank).  ``--sp`` shards the activations between the
blocks over samples and uses the fused all-gather / reduce-scatter GEMMs.  The logical batch is processed in
micro-batches with ``signal_skip_step``.  Per-sample norms are summed over the
group by the peer-memory kernel (``csrc/peer_collectives.cu``); C = 1.0,
sigma = 1.0, DP-AdamW, bf16, synthetic token ids copied from pinned host memory
every micro-step.  Device-timed, max over ranks.
"""
import argparse
import datetime
import json
import os

import torch
import torch.distributed as dist


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--batch", type=int, default=64, help="logical (global) batch")
    ap.add_argument("--micro", type=int, default=8, help="samples per micro-step")
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--sp", action="store_true",
                    help="sequence parallel: activations sharded over samples between the blocks, fused collective GEMMs")
    ap.add_argument("--no-fused", action="store_true", help="with --sp: NCCL + cuBLAS instead of the fused GEMMs")
    ap.add_argument("--tp", type=int, default=0, help="tensor-parallel group size (default: all ranks)")
    ap.add_argument("--no-peer-norm", action="store_true", help="reduce the norms with NCCL instead of the peer kernel")
    args = ap.parse_args()
    import warnings

    warnings.simplefilter("ignore")
    local = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29583")
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=300))
    rank, world = dist.get_rank(), dist.get_world_size()

    from opacus_b200.grad_sample import GradSampleModuleFastGradientClippingTP
    from opacus_b200.models import Llama, llama_8b_config
    from opacus_b200.ops import _cuda
    from opacus_b200.parallel.tensor_parallel import (TensorParallelDPOptimizer, VocabParallelCrossEntropy,
                                                      parallelize_llama)
    from opacus_b200.utils.fast_gradient_clipping_utils import DPLossFastGradientClipping

    cfg = llama_8b_config(n_layers=args.layers)
    torch.manual_seed(0)
    torch.set_default_dtype(torch.bfloat16)
    with torch.device(dev):
        model = Llama(cfg)                       # same weights on every rank, then sharded in place
    torch.set_default_dtype(torch.float32)
    tp = args.tp or world
    assert world % tp == 0, "--tp must divide the number of ranks"
    dp = world // tp
    tp_group = dp_group = None
    if dp > 1:
        for k in range(dp):
            grp = dist.new_group(list(range(k * tp, (k + 1) * tp)))
            tp_group = grp if rank // tp == k else tp_group
        for j in range(tp):
            grp = dist.new_group(list(range(j, world, tp)))
            dp_group = grp if rank % tp == j else dp_group
    parallelize_llama(model, tp_group, sequence_parallel=args.sp, fused=not args.no_fused)   # explicit: the flag decides
    torch.cuda.empty_cache()
    if dp > 1:
        from opacus_b200.optimizers import FSDPOptimizerFastGradientClipping
        from opacus_b200.parallel.sharded import ShardedDataParallel

        engine = ShardedDataParallel(model, process_group=dp_group, tp_group=tp_group)
        gsm = GradSampleModuleFastGradientClippingTP(engine, max_grad_norm=1.0, single_pass=True, process_group=tp_group)
        opt = FSDPOptimizerFastGradientClipping(torch.optim.AdamW(model.parameters(), lr=1e-4), noise_multiplier=1.0,
                                                max_grad_norm=1.0, expected_batch_size=args.batch // dp, engine=engine)
    else:
        gsm = GradSampleModuleFastGradientClippingTP(model, max_grad_norm=1.0, single_pass=True)
        opt = TensorParallelDPOptimizer(torch.optim.AdamW(model.parameters(), lr=1e-4), noise_multiplier=1.0,
                                        max_grad_norm=1.0, expected_batch_size=args.batch)
    gsm.use_peer_memory = not args.no_peer_norm
    crit = DPLossFastGradientClipping(gsm, opt, VocabParallelCrossEntropy(tp_group), "mean")
    n_micro = args.batch // (args.micro * dp)
    T = args.seq
    g = torch.Generator().manual_seed(1 + rank // tp)       # one stream of samples per tensor-parallel group
    host = [torch.randint(0, cfg.vocab_size, (args.micro, T + 1), generator=g).pin_memory() for _ in range(n_micro)]
    losses = torch.zeros(1, device=dev)

    def logical_step():
        for i in range(n_micro):
            ids = host[i].to(dev, non_blocking=True)
            opt.zero_grad(set_to_none=True)
            opt.signal_skip_step(do_skip=i < n_micro - 1)
            logits = gsm(ids[:, :-1])
            loss = crit(logits.flatten(0, 1), ids[:, 1:].reshape(-1), shape=(args.micro, T))
            loss.backward()
            opt.step()
        return loss.item()

    for _ in range(args.warmup):
        logical_step()
    torch.cuda.synchronize()
    dist.barrier()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(args.steps):
        last = logical_step()
    e.record()
    torch.cuda.synchronize()
    _cuda.check_status()
    t = torch.tensor([s.elapsed_time(e)], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t) / args.steps
    if rank == 0:
        print(json.dumps({"metric": "dp_llama8b_tp_tokens_per_s", "value": args.batch * T / (ms / 1e3), "n_gpus": world,
                          "ms_per_logical_step": ms, "config": {"layers": args.layers, "seq": T, "global_batch": args.batch,
                                                                "micro_batch": args.micro, "parallelism": f"tp{tp}" + ("+sp" if args.sp else "") + (f" x sharded dp{dp}" if dp > 1 else ""),
                                                                "fused_collective_gemms": bool(args.sp and not args.no_fused)},
                          "peer_norm_kernel": not args.no_peer_norm, "loss": last, "dtype": "bf16",
                          "max_mem_gb": torch.cuda.max_memory_allocated() / 2 ** 30}))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
