"""Llama-style decoder trained with ghost clipping on sharded data parallelism.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 examples/fsdp_llama.py [--layers 4]

``FSDP2Wrapper`` returns this package's sharded engine: bf16 compute weights, fp32 master weights and optimizer
state sharded over the ranks, and ONE kernel per step for reduce-scatter + noise + AdamW + all-gather.  Works with one
process as well.  Counterpart in the reference: ``examples/fsdp_llama3.py`` / ``examples/fsdp_example.py``.
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
    args = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    for k, v in (("MASTER_ADDR", "127.0.0.1"), ("MASTER_PORT", "29544"), ("RANK", "0"), ("WORLD_SIZE", "1")):
        os.environ.setdefault(k, v)
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rank, world = dist.get_rank(), dist.get_world_size()
    torch.manual_seed(0)
    cfg = LlamaConfig(vocab_size=32000, d_model=args.d_model, n_layers=args.layers, n_heads=8, n_kv_heads=4,
                      ffn_dim=4 * args.d_model, tie_embeddings=True)           # tied embeddings are supported
    model = Llama(cfg).cuda()
    module = FSDP2Wrapper(model)
    optimizer = torch.optim.AdamW(model.parameters(), lr=1e-4)
    n = args.batch * world * 64
    loader = DataLoader(TensorDataset(torch.zeros(n, 1, dtype=torch.long)), batch_size=args.batch * world)
    engine = PrivacyEngine()
    module, optimizer, criterion, _ = engine.make_private(
        module=module, optimizer=optimizer, criterion=FusedCrossEntropyLoss(), data_loader=loader,
        noise_multiplier=0.8, max_grad_norm=1.0, grad_sample_mode="ghost_fsdp", poisson_sampling=False)
    g = torch.Generator().manual_seed(rank)
    for step in range(args.steps):
        ids = torch.randint(0, cfg.vocab_size, (args.batch, args.seq + 1), generator=g).cuda()
        optimizer.zero_grad(set_to_none=True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            logits = module(ids[:, :-1])
        loss = criterion(logits.flatten(0, 1), ids[:, 1:].reshape(-1), shape=(args.batch, args.seq))
        loss.backward()                      # ONE backward pass: norms, clip factors and clipped sums
        optimizer.step()                     # ONE kernel: reduce-scatter + noise + AdamW + all-gather
        if rank == 0:
            print(f"step {step}: loss {loss.item():.3f}")
    if rank == 0:
        print(f"epsilon {engine.get_epsilon(1e-5):.2f}; per-sample norms of the last batch: "
              f"{module.per_sample_gradient_norms[:4].tolist()}")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
