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

``--impl reference`` runs the reference library (installed under ``baseline/_ref``) on the stock-PyTorch model
definition of ``baseline/llama_plain.py`` with the wiring of its own example
(``examples/tensor_parallelism_llama.py:104-198`` there): DTensor ``parallelize_module`` with Colwise / Rowwise plans,
norm weights frozen (its tensor-parallel controller rejects replicated trainable parameters),
``GradSampleModuleFastGradientClippingTP`` + ``FSDPOptimizerFastGradientClipping`` + ``DPLossFastGradientClipping``, the
same batch, micro-batching, sigma and clipping bound.  If the reference cannot run the configuration the script prints
``{"impl": "reference", "unavailable": ...}`` and exits 0.
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
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
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
    if args.impl == "reference":
        try:
            out = run_reference(args, dev, rank, world)
        except Exception as exc:                        # reported, never fatal for the caller
            import traceback

            traceback.print_exc()
            out = {"impl": "reference", "unavailable": f"{type(exc).__name__}: {str(exc)[:300]}"}
        if rank == 0:
            print(json.dumps(out))
        dist.barrier()
        dist.destroy_process_group()
        return

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


def run_reference(args, dev, rank, world):
    """The reference arm (see the module docstring); returns the JSON record."""
    import sys

    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    sys.path.insert(0, os.path.join(root, "baseline", "_ref"))
    sys.path.insert(0, os.path.join(root, "baseline"))
    import torch.nn as nn
    from llama_plain import Llama, llama_8b_config
    from opacus.grad_sample.grad_sample_module_fast_gradient_clipping_tp import GradSampleModuleFastGradientClippingTP
    from opacus.optimizers import FSDPOptimizerFastGradientClipping
    from opacus.utils.fast_gradient_clipping_utils import DPLossFastGradientClipping
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor import Replicate
    from torch.distributed.tensor.parallel import ColwiseParallel, RowwiseParallel, parallelize_module

    cfg = llama_8b_config(n_layers=args.layers)
    torch.manual_seed(0)
    torch.set_default_dtype(torch.bfloat16)
    with torch.device(dev):
        model = Llama(cfg)
    torch.set_default_dtype(torch.float32)
    mesh = init_device_mesh("cuda", (world,))
    for blk in model.layers:
        plan = {"self_attn.q_proj": ColwiseParallel(), "self_attn.k_proj": ColwiseParallel(),
                "self_attn.v_proj": ColwiseParallel(), "self_attn.o_proj": RowwiseParallel(),
                "mlp.gate_proj": ColwiseParallel(), "mlp.up_proj": ColwiseParallel(), "mlp.down_proj": RowwiseParallel()}
        blk.self_attn.n_heads //= world
        blk.self_attn.n_kv //= world
        for norm in (blk.input_layernorm, blk.post_attention_layernorm):
            for p in norm.parameters():
                p.requires_grad = False
        parallelize_module(module=blk, device_mesh=mesh, parallelize_plan=plan)
    model = parallelize_module(model, mesh, {"embed_tokens": RowwiseParallel(input_layouts=Replicate()),
                                             "lm_head": RowwiseParallel(input_layouts=Replicate())})
    for p in model.norm.parameters():
        p.requires_grad = False
    torch.cuda.empty_cache()
    gsm = GradSampleModuleFastGradientClippingTP(model, loss_reduction="mean", batch_first=True, max_grad_norm=1.0)
    opt = FSDPOptimizerFastGradientClipping(torch.optim.AdamW([p for p in gsm.parameters() if p.requires_grad], lr=1e-4),
                                            noise_multiplier=1.0, max_grad_norm=1.0, expected_batch_size=args.batch,
                                            loss_reduction="mean")
    crit = DPLossFastGradientClipping(gsm, opt, nn.CrossEntropyLoss(reduction="mean"), "mean")
    n_micro = args.batch // args.micro
    T = args.seq
    g = torch.Generator().manual_seed(1)
    host = [torch.randint(0, cfg.vocab_size, (args.micro, T + 1), generator=g).pin_memory() for _ in range(n_micro)]

    def logical_step():
        for i in range(n_micro):
            ids = host[i].to(dev, non_blocking=True)
            opt.zero_grad(set_to_none=True)
            opt.signal_skip_step(do_skip=i < n_micro - 1)
            logits = gsm(ids[:, :-1].contiguous())         # its embedding rule takes a view of the ids
            loss = crit(logits.float().flatten(0, 1), ids[:, 1:].reshape(-1), shape=(args.micro, T))
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
    t = torch.tensor([s.elapsed_time(e)], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t) / args.steps
    return {"metric": "dp_llama8b_tp_tokens_per_s", "impl": "reference", "value": args.batch * T / (ms / 1e3),
            "n_gpus": world, "ms_per_logical_step": ms,
            "config": {"layers": args.layers, "seq": T, "global_batch": args.batch, "micro_batch": args.micro,
                       "parallelism": f"tp{world} (DTensor)", "norm_weights": "frozen (required by the reference)"},
            "loss": last, "dtype": "bf16", "max_mem_gb": torch.cuda.max_memory_allocated() / 2 ** 30}


if __name__ == "__main__":
    main()
