"""Llama-style decoder trained with ghost clipping on sharded data parallelism.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 examples/fsdp_llama.py [--layers 4]
    ... examples/fsdp_llama.py --shard-params        # row-sharded Linear weights (parameters and gradients sharded too)
    ... examples/fsdp_llama.py --layers 32 --d-model 4096 --ffn 14336 --heads 32 --kv-heads 8 --vocab 128256 \
            --seq 2048 --batch 2 --untied [--shard-params]    # the Llama-3-8B shape on 8 GPUs

``FSDP2Wrapper`` returns this package's sharded engine: bf16 compute weights, fp32 master weights and optimizer
state sharded over the ranks, and ONE kernel per step for reduce-scatter + noise + AdamW + all-gather.  Works with one
process as well.  With ``--shard-params`` the eligible Linear weights are kept as row shards (1 / world per GPU) and
gathered inside the GEMM that consumes them; their gradients are reduce-scattered layer by layer and never exist whole.
The script prints tokens per second (CUDA events, max over ranks) and the memory in use per GPU.  Counterpart in the reference: ``examples/fsdp_llama3.py`` / ``examples/fsdp_example.py``.
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

from opacus_b200 import PrivacyEngine  # noqa: E402
from opacus_b200.layers import FusedCrossEntropyLoss  # noqa: E402
from opacus_b200.models import Llama, LlamaConfig  # noqa: E402
from opacus_b200.utils.fsdp_utils import FSDP2Wrapper  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--d-model", type=int, default=512)
    ap.add_argument("--seq", type=int, default=256)
    ap.add_argument("--batch", type=int, default=8, help="per GPU")
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--ffn", type=int, default=None, help="MLP width (default 4 x d-model)")
    ap.add_argument("--heads", type=int, default=8)
    ap.add_argument("--kv-heads", type=int, default=4)
    ap.add_argument("--vocab", type=int, default=32000)
    ap.add_argument("--shard-params", action="store_true")
    ap.add_argument("--untied", action="store_true", help="separate output layer (the Llama-3-8B layout)")
    args = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    for k, v in (("MASTER_ADDR", "127.0.0.1"), ("MASTER_PORT", "29544"), ("RANK", "0"), ("WORLD_SIZE", "1")):
        os.environ.setdefault(k, v)
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rank, world = dist.get_rank(), dist.get_world_size()
    torch.manual_seed(0)
    cfg = LlamaConfig(vocab_size=args.vocab, d_model=args.d_model, n_layers=args.layers, n_heads=args.heads,
                      n_kv_heads=args.kv_heads, ffn_dim=args.ffn or 4 * args.d_model,
                      tie_embeddings=not args.untied)                          # tied embeddings are supported
    with torch.device("cuda"):
        model = Llama(cfg)
    n_params = sum(p.numel() for p in model.parameters())
    module = FSDP2Wrapper(model, shard_params=args.shard_params)
    optimizer = torch.optim.AdamW(model.parameters(), lr=1e-4)
    n = args.batch * world * 64
    loader = DataLoader(TensorDataset(torch.zeros(n, 1, dtype=torch.long)), batch_size=args.batch * world)
    engine = PrivacyEngine()
    module, optimizer, criterion, _ = engine.make_private(
        module=module, optimizer=optimizer, criterion=FusedCrossEntropyLoss(), data_loader=loader,
        noise_multiplier=0.8, max_grad_norm=1.0, grad_sample_mode="ghost_fsdp", poisson_sampling=False)
    g = torch.Generator().manual_seed(rank)
    warm = min(2, args.steps - 1)
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for step in range(args.steps):
        if step == warm:
            dist.barrier()
            torch.cuda.synchronize()
            t0.record()
        ids = torch.randint(0, cfg.vocab_size, (args.batch, args.seq + 1), generator=g).cuda()
        optimizer.zero_grad(set_to_none=True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            logits = module(ids[:, :-1])
        loss = criterion(logits.flatten(0, 1), ids[:, 1:].reshape(-1), shape=(args.batch, args.seq))
        loss.backward()                      # ONE backward pass: norms, clip factors and clipped sums
        optimizer.step()                     # ONE kernel: reduce-scatter + noise + AdamW + all-gather
        if rank == 0:
            print(f"step {step}: loss {loss.item():.3f}")
    t1.record()
    torch.cuda.synchronize()
    free, total = torch.cuda.mem_get_info()
    stats = torch.tensor([t0.elapsed_time(t1), (total - free) / 2 ** 30, torch.cuda.max_memory_allocated() / 2 ** 30],
                         device="cuda")
    dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    if rank == 0:
        ms = stats[0].item() / max(args.steps - warm, 1)
        print(f"{n_params / 1e9:.2f} G parameters, {world} GPUs, shard_params={args.shard_params}: {ms:.1f} ms per step, "
              f"{args.batch * world * args.seq / ms * 1e3:,.0f} tokens/s; memory in use per GPU {stats[1].item():.1f} GB "
              f"(symmetric buffers included), peak of the caching allocator {stats[2].item():.1f} GB")
        print(f"epsilon {engine.get_epsilon(1e-5):.2f}; per-sample norms of the last batch: "
              f"{module.per_sample_gradient_norms[:4].tolist()}")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
