"""Tensor-parallel Llama under ghost clipping, optionally sequence parallel (sample-sharded activations and the
fused all-gather / reduce-scatter GEMMs on NVLink-connected GPUs).

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 examples/tensor_parallelism_llama.py [--sp]

Counterpart in the reference: ``examples/tensor_parallelism_llama.py``.
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
from opacus_b200.models import Llama, LlamaConfig  # noqa: E402
from opacus_b200.parallel.tensor_parallel import (TensorParallelDPOptimizer, VocabParallelCrossEntropy,  # noqa: E402
                                                  parallelize_llama)
from opacus_b200.utils.fast_gradient_clipping_utils import DPLossFastGradientClipping  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--sp", action="store_true", help="sequence parallel between the tensor-parallel blocks")
    ap.add_argument("--steps", type=int, default=3)
    args = ap.parse_args()
    cuda = torch.cuda.is_available()
    if cuda:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    dist.init_process_group("nccl" if cuda else "gloo")
    dev = "cuda" if cuda else "cpu"
    rank, world = dist.get_rank(), dist.get_world_size()
    torch.manual_seed(0)
    cfg = LlamaConfig(vocab_size=1024, d_model=256, n_layers=2, n_heads=8, n_kv_heads=8, ffn_dim=512,
                      tie_embeddings=False)
    model = Llama(cfg).to(dev)
    if cuda:
        model = model.bfloat16()
    parallelize_llama(model, sequence_parallel=args.sp)               # in place; embedding and norms stay replicated
    gsm = GradSampleModuleFastGradientClippingTP(model, max_grad_norm=1.0, single_pass=True)
    B, T = 2 * world, 128
    opt = TensorParallelDPOptimizer(torch.optim.AdamW(model.parameters(), lr=1e-3), noise_multiplier=1.0,
                                    max_grad_norm=1.0, expected_batch_size=B)
    crit = DPLossFastGradientClipping(gsm, opt, VocabParallelCrossEntropy(), "mean")
    g = torch.Generator().manual_seed(1)                              # every rank sees the same batch
    for step in range(args.steps):
        ids = torch.randint(0, cfg.vocab_size, (B, T + 1), generator=g).to(dev)
        opt.zero_grad()
        logits = gsm(ids[:, :-1])                                     # [B, T, vocab / world]
        loss = crit(logits.flatten(0, 1), ids[:, 1:].reshape(-1), shape=(B, T))
        loss.backward()
        opt.step()
        if rank == 0:
            print(f"step {step}: loss {loss.item():.3f}")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
