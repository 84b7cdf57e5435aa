"""Multi-GPU check of the peer-memory collectives used by tensor parallelism; launched by ``test_gpu_multi.py`` as

    python -m torch.distributed.run --standalone --local-addr 127.0.0.1 --nproc-per-node N tests/dist_tp_check.py
"""
import datetime
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from opacus_b200.ops import _cuda  # noqa: E402
from opacus_b200.parallel import symm  # noqa: E402


def check_norm_reducer(rank, world):
    red = symm.PeerNormReducer(torch.device("cuda", torch.cuda.current_device()), capacity=1024)
    for it, n in enumerate([7, 1024, 300, 300, 64]):
        g = torch.Generator(device="cuda").manual_seed(100 * it + rank)
        part = torch.rand(n, device="cuda", generator=g)
        g0 = torch.Generator(device="cuda").manual_seed(999 + it)
        rep = torch.rand(n, device="cuda", generator=g0) if it % 2 == 0 else None
        total, clip = red(part, rep, 0.75)
        parts = [torch.empty_like(part) for _ in range(world)]
        dist.all_gather(parts, part)
        ref = torch.zeros_like(part)
        for p in parts:                      # rank order, like the kernel
            ref = ref + p
        if rep is not None:
            ref = ref + rep
        assert torch.equal(total, ref), (rank, it, (total - ref).abs().max().item())
        torch.testing.assert_close(clip, (0.75 / (ref.sqrt() + 1e-6)).clamp(max=1.0))
        both = [torch.empty_like(clip) for _ in range(world)]
        dist.all_gather(both, clip)
        assert all(torch.equal(b, both[0]) for b in both), "clip factors differ between ranks"
    torch.cuda.synchronize()
    _cuda.check_status()


def check_fused_gemms(rank, world):
    from opacus_b200.parallel.fused_tp import AllGatherGemm, GemmReduceScatter

    dev = torch.device("cuda", torch.cuda.current_device())
    K, N = 384, 1024
    rows = 256                                   # per rank
    g = torch.Generator(device="cuda").manual_seed(7)
    x_all = torch.randn(rows * world, K, device=dev, generator=g).bfloat16()      # same on every rank
    w = torch.randn(N, K, device=dev, generator=g).bfloat16()
    # all-gather(A) -> GEMM: column-parallel layer, this rank's weight columns
    w_mine = w[rank * (N // world):(rank + 1) * (N // world)].contiguous()
    ag = AllGatherGemm(rows, K, dev, gather="a")
    for it in range(3):
        xs = (x_all * (it + 1)).bfloat16()
        ag.shard.copy_(xs[rank * rows:(rank + 1) * rows])
        y = ag(w_mine)
        ref = xs.float() @ w_mine.float().t()
        assert (y.float() - ref).abs().max() <= 1e-2 * ref.abs().max(), (rank, it)
        assert torch.equal(ag.full, xs)
    # all-gather(B) -> GEMM: weights sharded by rows, activations local
    wr = N // world if (N // world) % 256 == 0 else 256
    w_all = torch.randn(wr * world, K, device=dev, generator=g).bfloat16()
    agb = AllGatherGemm(wr, K, dev, gather="b")
    agb.shard.copy_(w_all[rank * wr:(rank + 1) * wr])
    x_loc = x_all[:384].contiguous()
    y = agb(x_loc)
    ref = x_loc.float() @ w_all.float().t()
    assert (y.float() - ref).abs().max() <= 1e-2 * ref.abs().max()
    # GEMM -> reduce-scatter: row-parallel layer, K split over the ranks
    Kl = 128
    gr = torch.Generator(device="cuda").manual_seed(50 + rank)
    x_r = torch.randn(rows * world, Kl, device=dev, generator=gr).bfloat16()
    w_r = torch.randn(N, Kl, device=dev, generator=gr).bfloat16()
    rs = GemmReduceScatter(rows * world, N, dev)
    for it in range(3):
        y = rs(x_r, w_r)
        part = (x_r.float() @ w_r.float().t()).bfloat16().float()     # partials travel as bf16
        dist.all_reduce(part)
        ref = part[rank * rows:(rank + 1) * rows]
        assert (y.float() - ref).abs().max() <= 1e-2 * ref.abs().max(), (rank, it)
    torch.cuda.synchronize()
    _cuda.check_status()


def main():
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=datetime.timedelta(seconds=120))
    rank, world = dist.get_rank(), dist.get_world_size()
    check_norm_reducer(rank, world)
    check_fused_gemms(rank, world)
    dist.barrier()
    if rank == 0:
        print("tp check ok")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
