"""Multi-GPU check of the sharded engine; launched by ``test_gpu_multi.py`` as

    python -m torch.distributed.run --standalone --local-addr 127.0.0.1 --nproc-per-node N tests/dist_sharded_check.py

Every rank trains on its slice of a global batch for a few noise-free steps;
rank 0 then repeats the run alone on the whole batch (engine with a one-rank
group) and compares master weights.  A second phase checks that the noise
added across ranks has the variance of a single global draw.
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


def build(group, expected, sigma, opt_cls):
    torch.manual_seed(0)
    model = Llama(LlamaConfig(vocab_size=512, d_model=128, n_layers=2, n_heads=4, n_kv_heads=2, ffn_dim=256)).cuda()
    eng = ShardedDataParallel(model, process_group=group)
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

    for opt_cls in (torch.optim.AdamW, torch.optim.SGD):
        eng, gsm, opt, crit = build(None, B, 0.0, opt_cls)
        run(gsm, opt, crit, mine, 3)
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
        print(f"sharded check ok on {world} GPUs (noise std {std:.2f}, cross-rank corr {corr:.4f})")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
