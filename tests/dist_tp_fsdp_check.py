"""Multi-GPU check of tensor parallelism x sharded data parallelism (2-D); launched by ``test_gpu_multi.py`` as

    TP_SIZE=2 python -m torch.distributed.run --standalone --local-addr 127.0.0.1 --nproc-per-node N tests/dist_tp_fsdp_check.py

Ranks ``[k * TP_SIZE, (k + 1) * TP_SIZE)`` form tensor-parallel group ``k``; ranks with the same position in their
tensor-parallel group form a data-parallel group.  With N == TP_SIZE the data-parallel groups have one rank each.
"""
import datetime
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from opacus_b200.ops import _cuda  # noqa: E402


def make_groups(rank, world, tp):
    dp = world // tp
    tp_group = dp_group = None
    for k in range(dp):
        g = dist.new_group(list(range(k * tp, (k + 1) * tp)))
        if rank // tp == k:
            tp_group = g
    for j in range(tp):
        g = dist.new_group(list(range(j, world, tp)))
        if rank % tp == j:
            dp_group = g
    return tp_group, dp_group, dp


def build(dev, tp_group, dp_group, *, two_d, sigma, clip, lr, batch, sp=False):
    from opacus_b200.grad_sample import GradSampleModuleFastGradientClippingTP
    from opacus_b200.models import Llama, LlamaConfig
    from opacus_b200.optimizers import FSDPOptimizerFastGradientClipping
    from opacus_b200.parallel.sharded import ShardedDataParallel
    from opacus_b200.parallel.tensor_parallel import (TensorParallelDPOptimizer, VocabParallelCrossEntropy,
                                                      parallelize_llama)
    from opacus_b200.utils.fast_gradient_clipping_utils import DPLossFastGradientClipping

    torch.manual_seed(0)
    cfg = LlamaConfig(vocab_size=1024, d_model=256, n_layers=2, n_heads=8, n_kv_heads=8, ffn_dim=512,
                      tie_embeddings=False)
    model = Llama(cfg).to(dev).bfloat16()
    parallelize_llama(model, tp_group, sequence_parallel=sp)
    if two_d:
        wrapped = ShardedDataParallel(model, process_group=dp_group, tp_group=tp_group)
        gsm = GradSampleModuleFastGradientClippingTP(wrapped, max_grad_norm=clip, single_pass=True,
                                                     process_group=tp_group)
        opt = FSDPOptimizerFastGradientClipping(torch.optim.SGD(model.parameters(), lr=lr), noise_multiplier=sigma,
                                                max_grad_norm=clip, expected_batch_size=batch, engine=wrapped)
    else:
        gsm = GradSampleModuleFastGradientClippingTP(model, max_grad_norm=clip, single_pass=True,
                                                     process_group=tp_group)
        opt = TensorParallelDPOptimizer(torch.optim.SGD(model.parameters(), lr=lr), noise_multiplier=sigma,
                                        max_grad_norm=clip, expected_batch_size=batch, process_group=tp_group)
    crit = DPLossFastGradientClipping(gsm, opt, VocabParallelCrossEntropy(tp_group), "mean")
    return model, gsm, opt, crit


def train(gsm, opt, crit, ids, steps):
    B, T = ids.shape[0], ids.shape[1] - 1
    for _ in range(steps):
        opt.zero_grad()
        logits = gsm(ids[:, :-1])
        loss = crit(logits.flatten(0, 1), ids[:, 1:].reshape(-1), shape=(B, T))
        loss.backward()
        opt.step()
    torch.cuda.synchronize()
    _cuda.check_status()


def probes(model):
    return {"down_proj (row shard)": model.layers[0].mlp.down_proj.weight.detach().float().clone(),
            "q_proj (column shard)": model.layers[1].self_attn.q_proj.weight.detach().float().clone(),
            "norm (replicated)": model.layers[0].input_layernorm.weight.detach().float().clone(),
            "embedding (replicated)": model.embed_tokens.weight.detach().float().clone()}


def check_matches_tensor_parallel_alone(rank, world, tp, tp_group, dp_group, dp, sp):
    """Noise off: the 2-D job, whose data-parallel ranks each see a share of the batch, ends where one
    tensor-parallel group that sees the whole batch ends.  ``sp``: activations sharded over samples between the
    blocks, so the sums of the norm and embedding weights are completed over the tensor-parallel group first."""
    dev = torch.device("cuda", torch.cuda.current_device())
    per_rank, T = 4, 64
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, 1024, (per_rank * dp, T + 1), generator=g).to(dev)
    model, gsm, opt, crit = build(dev, tp_group, dp_group, two_d=False, sigma=0.0, clip=1.0, lr=0.1,
                                  batch=per_rank * dp, sp=sp)
    train(gsm, opt, crit, ids, 2)
    want = probes(model)
    k = rank // tp
    model, gsm, opt, crit = build(dev, tp_group, dp_group, two_d=True, sigma=0.0, clip=1.0, lr=0.1, batch=per_rank,
                                  sp=sp)
    train(gsm, opt, crit, ids[k * per_rank:(k + 1) * per_rank], 2)
    for name, got in probes(model).items():
        ref = want[name]
        assert (got - ref).abs().max() <= 2e-2 * ref.abs().max() + 1e-3, (rank, sp, name, (got - ref).abs().max().item())


def check_noise_layout(rank, world, tp, tp_group, dp_group, dp):
    """Noise on: replicas of a parameter stay identical over the tensor-parallel
    group, shards of one weight receive independent draws of the right scale."""
    dev = torch.device("cuda", torch.cuda.current_device())
    per_rank, T = 2, 32
    sigma, clip, lr = 1.0, 0.05, 1.0        # per coordinate the clipped signal (norm <= clip in all) is far below the noise
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(0, 1024, (per_rank, T + 1), generator=g).to(dev)
    model, gsm, opt, crit = build(dev, tp_group, dp_group, two_d=True, sigma=sigma, clip=clip, lr=lr, batch=per_rank)
    torch.cuda.manual_seed(100 + rank)      # different generator states per rank: the group has to agree by itself
    before = probes(model)
    train(gsm, opt, crit, ids, 1)
    after = probes(model)
    std = sigma * clip / (per_rank * dp)            # the noised sum is divided by the global expected batch
    for name in before:
        delta = after[name] - before[name]
        pieces = [torch.empty_like(delta) for _ in range(tp)]
        dist.all_gather(pieces, delta.contiguous(), group=tp_group)
        if "replicated" in name:
            assert all(torch.equal(p, pieces[0]) for p in pieces), (rank, name, "replicas diverged")
        else:
            a, b = pieces[0].flatten().double(), pieces[1].flatten().double()
            corr = float((a * b).mean() / (a.std() * b.std()))
            assert abs(corr) < 0.05, (rank, name, "shards received correlated noise", corr)
        if name != "norm (replicated)":                     # bf16 weights near 1.0 cannot show steps this small
            seen = float(delta.double().std())
            assert 0.5 * std < seen < 1.5 * std, (rank, name, seen, std)


def main():
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=datetime.timedelta(seconds=120))
    rank, world = dist.get_rank(), dist.get_world_size()
    tp = int(os.environ.get("TP_SIZE", "2"))
    assert world % tp == 0 and tp >= 2
    tp_group, dp_group, dp = make_groups(rank, world, tp)
    for sp in (False, True):
        check_matches_tensor_parallel_alone(rank, world, tp, tp_group, dp_group, dp, sp)
    check_noise_layout(rank, world, tp, tp_group, dp_group, dp)
    dist.barrier()
    if rank == 0:
        print(f"tp x fsdp check ok (tp {tp} x dp {dp})")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
