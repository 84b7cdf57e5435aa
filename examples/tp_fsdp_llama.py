"""Llama under ghost clipping in the 2-d layout: groups of ``--tp`` consecutive GPUs are tensor parallel, the groups
among themselves are sharded data parallel (each group trains on its own samples; fp32 master weights and optimizer
state are sharded over the ranks with the same position in their groups).  Needs CUDA GPUs with peer access.

    python -m torch.distributed.run --nproc-per-node 4 --master-addr 127.0.0.1 examples/tp_fsdp_llama.py --tp 2

The reference has no counterpart (it offers tensor parallelism and FSDP separately:
``examples/tensor_parallelism_llama.py``, ``opacus/utils/fsdp_utils.py``).
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))   # run from a source checkout

import torch.distributed as dist  # noqa: E402

from opacus_b200.accountants import RDPAccountant  # noqa: E402
from opacus_b200.grad_sample import GradSampleModuleFastGradientClippingTP  # noqa: E402
from opacus_b200.models import Llama, LlamaConfig  # noqa: E402
from opacus_b200.optimizers import FSDPOptimizerFastGradientClipping  # noqa: E402
from opacus_b200.parallel.sharded import ShardedDataParallel  # noqa: E402
from opacus_b200.parallel.tensor_parallel import VocabParallelCrossEntropy, parallelize_llama  # noqa: E402
from opacus_b200.utils.fast_gradient_clipping_utils import DPLossFastGradientClipping  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tp", type=int, default=2, help="tensor-parallel group size")
    ap.add_argument("--sp", action="store_true", help="sequence parallel between the tensor-parallel blocks")
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--batch", type=int, default=4, help="samples per tensor-parallel group and step")
    args = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rank, world = dist.get_rank(), dist.get_world_size()
    tp, dp = args.tp, world // args.tp
    tp_group = dp_group = None
    for k in range(dp):                                   # every rank creates every group, in the same order
        g = dist.new_group(list(range(k * tp, (k + 1) * tp)))
        tp_group = g if rank // tp == k else tp_group
    for j in range(tp):
        g = dist.new_group(list(range(j, world, tp)))
        dp_group = g if rank % tp == j else dp_group

    torch.manual_seed(0)                                  # identical weights everywhere before sharding
    cfg = LlamaConfig(vocab_size=1024, d_model=256, n_layers=2, n_heads=8, n_kv_heads=8, ffn_dim=512,
                      tie_embeddings=False)
    model = Llama(cfg).cuda().bfloat16()
    parallelize_llama(model, tp_group, sequence_parallel=args.sp)
    engine = ShardedDataParallel(model, process_group=dp_group, tp_group=tp_group)
    gsm = GradSampleModuleFastGradientClippingTP(engine, max_grad_norm=1.0, single_pass=True, process_group=tp_group)
    opt = FSDPOptimizerFastGradientClipping(torch.optim.AdamW(model.parameters(), lr=1e-3), noise_multiplier=1.0,
                                            max_grad_norm=1.0, expected_batch_size=args.batch, engine=engine)
    crit = DPLossFastGradientClipping(gsm, opt, VocabParallelCrossEntropy(tp_group), "mean")
    accountant = RDPAccountant()
    n_data = 4096
    opt.attach_step_hook(accountant.get_optimizer_hook_fn(sample_rate=args.batch * dp / n_data))

    T = 64
    data = torch.Generator().manual_seed(1 + rank // tp)  # the ranks of a tensor-parallel group read the same samples
    for step in range(args.steps):
        ids = torch.randint(0, cfg.vocab_size, (args.batch, T + 1), generator=data).cuda()
        opt.zero_grad()
        logits = gsm(ids[:, :-1])
        loss = crit(logits.flatten(0, 1), ids[:, 1:].reshape(-1), shape=(args.batch, T))
        value = loss.item()
        loss.backward()
        opt.step()
        if rank == 0:
            print(f"step {step}: loss {value:.4f}  eps {accountant.get_epsilon(1e-5):.3f}")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
