"""Multi-GPU check of the sharded engine; launched by ``test_gpu_multi.py`` as

    python -m torch.distributed.run --standalone --local-addr 127.0.0.1 --nproc-per-node N tests/dist_sharded_check.py

Every rank trains on its slice of a global batch for a few noise-free steps;
rank 0 then repeats the run alone on the whole batch (engine with a one-rank
group) and compares master weights -- once with the flat space in one piece and
plain peer loads / stores, once cut into four pieces that are stepped beside
the weight-gradient GEMMs, through the NVLink multicast address when the fabric
offers one.  A second phase checks that the noise added across ranks has the
variance of a single global draw, a third that a run resumed from the gathered
state dicts continues exactly like the uninterrupted one.
"""
import datetime
import os
import sys

import torch
import torch.distributed as dist
import torch.nn as nn

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from opacus_b200.grad_sample import GradSampleModuleFastGradientClippingFSDP  # noqa: E402
from opacus_b200.models import Llama, LlamaConfig  # noqa: E402
from opacus_b200.ops import _cuda  # noqa: E402
from opacus_b200.optimizers import FSDPOptimizerFastGradientClipping  # noqa: E402
from opacus_b200.parallel.sharded import ShardedDataParallel  # noqa: E402
from opacus_b200.utils.fast_gradient_clipping_utils import DPLossFastGradientClipping  # noqa: E402

B, T, C = 4, 64, 0.5


def build(group, expected, sigma, opt_cls, wide=False, **engine_kw):
    torch.manual_seed(0)
    cfg = LlamaConfig(vocab_size=512, d_model=512, n_layers=2, n_heads=8, n_kv_heads=4, ffn_dim=1024) if wide else \
        LlamaConfig(vocab_size=512, d_model=128, n_layers=2, n_heads=4, n_kv_heads=2, ffn_dim=256)
    model = Llama(cfg).cuda()
    eng = ShardedDataParallel(model, process_group=group, **engine_kw)
    gsm = GradSampleModuleFastGradientClippingFSDP(eng, max_grad_norm=C)
    inner = opt_cls(model.parameters(), lr=1e-2)
    opt = FSDPOptimizerFastGradientClipping(inner, noise_multiplier=sigma, max_grad_norm=C,
                                            expected_batch_size=expected, engine=eng)
    crit = DPLossFastGradientClipping(gsm, opt, nn.CrossEntropyLoss(), "mean")
    return eng, gsm, opt, crit


def run(gsm, opt, crit, ids, steps):
    for _ in range(steps):
        opt.zero_grad(set_to_none=True)
        logits = gsm(ids[:, :-1])
        crit(logits.float().flatten(0, 1), ids[:, 1:].reshape(-1), shape=(ids.shape[0], T)).backward()
        opt.step()
    torch.cuda.synchronize()
    _cuda.check_status()


def main():
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=datetime.timedelta(seconds=120))
    rank, world = dist.get_rank(), dist.get_world_size()
    solo = dist.new_group(ranks=[0])
    g = torch.Generator().manual_seed(5)
    ids_all = torch.randint(0, 512, (B * world, T + 1), generator=g).cuda()
    mine = ids_all[rank * B:(rank + 1) * B]

    used_multicast = False
    for opt_cls, engine_kw in ((torch.optim.AdamW, dict(step_pieces=1, multicast=False)),
                               (torch.optim.AdamW, dict(step_pieces=4, multicast=True)),
                               (torch.optim.SGD, dict(step_pieces=4))):
        eng, gsm, opt, crit = build(None, B, 0.0, opt_cls, **engine_kw)
        run(gsm, opt, crit, mine, 3)
        used_multicast = used_multicast or eng.multicast
        if engine_kw.get("step_pieces") == 4:
            assert eng.last_step_launches > 1, "the step did not run in pieces"
        got = eng.full_precision_state_dict()
        # every rank must also hold identical compute weights
        flat = eng._flat_param.tensor.float()
        ref_flat = flat.clone()
        dist.broadcast(ref_flat, 0)
        assert torch.equal(flat, ref_flat), "compute weights differ between ranks"
        if rank == 0:
            eng1, gsm1, opt1, crit1 = build(solo, B * world, 0.0, opt_cls)
            run(gsm1, opt1, crit1, ids_all, 3)
            want = eng1.full_precision_state_dict()
            for k in want:
                err = ((got[k] - want[k]).norm() / (want[k].norm() + 1e-12)).item()
                assert err < 5e-3, (opt_cls.__name__, k, err)
        dist.barrier()

    # noise: one global draw of std sigma*C on the summed gradient
    eng, gsm, opt, crit = build(None, B, 50.0, torch.optim.SGD)
    before = eng.master.clone()
    run(gsm, opt, crit, mine, 1)
    delta = (eng.master - before) * (B * world) / 1e-2
    std = delta.std().item()
    assert abs(std - 50.0 * C) / (50.0 * C) < 0.05, std
    pieces = [torch.empty_like(delta) for _ in range(world)]
    dist.all_gather(pieces, delta)
    if rank == 0 and world > 1:
        corr = (pieces[0] * pieces[1]).mean().item() / (std * std)
        assert abs(corr) < 0.02, corr
        print(f"sharded check ok on {world} GPUs (noise std {std:.2f}, cross-rank corr {corr:.4f}, "
              f"multicast {'used' if used_multicast else 'not available'})")
    dist.barrier()

    # resume: 2 steps, gather the state, load it into a fresh engine, 2 more steps == 4 steps in one go
    eng, gsm, opt, crit = build(None, B, 0.0, torch.optim.AdamW, step_pieces=4)
    run(gsm, opt, crit, mine, 2)
    saved = {"module": {k: v.clone() for k, v in eng.state_dict().items()}, "optimizer": opt.state_dict()}
    run(gsm, opt, crit, mine, 2)
    want = eng.full_precision_state_dict()
    eng2, gsm2, opt2, crit2 = build(None, B, 0.0, torch.optim.AdamW, step_pieces=2)     # another layout on purpose
    with torch.no_grad():
        for p in eng2.module.parameters():
            p.add_(1.0)                      # the start must come from the file, not from the seed
    eng2.load_state_dict(saved["module"])
    opt2.load_state_dict(saved["optimizer"])
    run(gsm2, opt2, crit2, mine, 2)
    got = eng2.full_precision_state_dict()
    for k in want:
        err = ((got[k] - want[k]).norm() / (want[k].norm() + 1e-12)).item()
        assert err < 1e-4, ("resume", k, err)
    if rank == 0:
        print("sharded resume ok")
    dist.barrier()

    # parameter sharding: Linear weights kept as row shards (fused all-gather -> GEMM forward, layer-by-layer
    # reduce-scatter + step) against the replicated layout run by rank 0 alone on the whole batch
    if world in (1, 2, 4):
        from opacus_b200.parallel.param_sharding import ShardedLinear

        eng, gsm, opt, crit = build(None, B, 0.0, torch.optim.AdamW, wide=True, shard_params=True)
        assert sum(isinstance(m, ShardedLinear) for m in eng.module.modules()) >= 4      # 10 on 2 ranks, 4 on 4
        run(gsm, opt, crit, mine, 3)
        got = eng.full_precision_state_dict()
        if rank == 0:
            eng1, gsm1, opt1, crit1 = build(solo, B * world, 0.0, torch.optim.AdamW, wide=True)
            run(gsm1, opt1, crit1, ids_all, 3)
            want = eng1.full_precision_state_dict()
            for k in want:
                err = ((got[k] - want[k]).norm() / (want[k].norm() + 1e-12)).item()
                assert err < 2e-2, ("shard_params", k, err)
        dist.barrier()
        # noise on a sharded weight: one draw of std sigma * C per element of the whole weight, rows independent
        eng, gsm, opt, crit = build(None, B, 50.0, torch.optim.SGD, wide=True, shard_params=True)
        layer = next(m for m in eng.module.modules() if isinstance(m, ShardedLinear))
        before = layer.master.clone()
        run(gsm, opt, crit, mine, 1)
        delta = (layer.master - before) * (B * world) / 1e-2
        std = delta.std().item()
        assert abs(std - 50.0 * C) / (50.0 * C) < 0.05, ("shard noise", std)
        parts = [torch.empty_like(delta) for _ in range(world)]
        dist.all_gather(parts, delta)
        if world > 1:
            corr = (parts[0] * parts[1]).mean().item() / (std * std)
            assert abs(corr) < 0.03, corr
        if rank == 0:
            print("sharded parameters ok")
        dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
