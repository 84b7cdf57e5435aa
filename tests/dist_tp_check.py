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
    # pull form: the partial sums are accumulated in this rank's slot of the symmetric buffer (as the ghost-norm
    # epilogues do) and the call reads every rank's slot from that rank's memory; then a longer vector (growth)
    for it, n in enumerate([40, 1024, 40]):
        g = torch.Generator(device="cuda").manual_seed(500 + 10 * it + rank)
        part = torch.rand(n, device="cuda", generator=g)
        acc = red.accumulator(n)
        assert acc is not None and float(acc.abs().sum()) == 0.0
        acc.add_(part * 0.25)
        acc.add_(part * 0.75)
        total, clip = red(acc, None, 0.5)
        parts = [torch.empty_like(part) for _ in range(world)]
        dist.all_gather(parts, part * 0.25 + part * 0.75)
        ref = torch.zeros_like(part)
        for p in parts:
            ref = ref + p
        assert torch.equal(total, ref), (rank, "pull", it, (total - ref).abs().max().item())
        torch.testing.assert_close(clip, (0.5 / (ref.sqrt() + 1e-6)).clamp(max=1.0))
    big = torch.rand(3000, device="cuda", generator=torch.Generator(device="cuda").manual_seed(rank))
    assert red.accumulator(3000) is None
    total, _ = red(big, None, 1.0)
    parts = [torch.empty_like(big) for _ in range(world)]
    dist.all_gather(parts, big)
    assert red.capacity >= 3000 and torch.equal(total, sum(parts[1:], parts[0]))
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


def check_sequence_parallel_llama(rank, world):
    """Tensor-parallel Llama with sample-sharded activations: fused collective GEMMs against NCCL + cuBLAS."""
    import torch.nn as nn  # noqa: F401

    from opacus_b200.grad_sample import GradSampleModuleFastGradientClippingTP
    from opacus_b200.models import Llama, LlamaConfig
    from opacus_b200.parallel.tensor_parallel import (TensorParallelDPOptimizer, VocabParallelCrossEntropy,
                                                      parallelize_llama)
    from opacus_b200.utils.fast_gradient_clipping_utils import DPLossFastGradientClipping

    dev = torch.device("cuda", torch.cuda.current_device())
    B, T = 2 * world, 128
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, 1024, (B, T + 1), generator=g).to(dev)
    results = {}
    for fused in (False, True):
        torch.manual_seed(0)
        cfg = LlamaConfig(vocab_size=1024, d_model=256, n_layers=2, n_heads=8, n_kv_heads=8, ffn_dim=512,
                          tie_embeddings=False)
        model = Llama(cfg).to(dev).bfloat16()
        parallelize_llama(model, sequence_parallel=True, fused=fused)
        gsm = GradSampleModuleFastGradientClippingTP(model, max_grad_norm=1.0, single_pass=True)
        opt = TensorParallelDPOptimizer(torch.optim.SGD(model.parameters(), lr=0.1), noise_multiplier=0.0,
                                        max_grad_norm=1.0, expected_batch_size=B)
        crit = DPLossFastGradientClipping(gsm, opt, VocabParallelCrossEntropy(), "mean")
        for _ in range(2):
            opt.zero_grad()
            logits = gsm(ids[:, :-1])
            loss = crit(logits.flatten(0, 1), ids[:, 1:].reshape(-1), shape=(B, T))
            value = loss.item()
            loss.backward()
            norms = gsm.per_sample_gradient_norms.clone()
            opt.step()
        torch.cuda.synchronize()
        _cuda.check_status()
        results[fused] = (value, norms, model.layers[0].mlp.down_proj.weight.detach().float().clone(),
                          model.embed_tokens.weight.detach().float().clone())
        if fused:
            assert "_ag" in model.lm_head.__dict__, "the output layer did not take the fused all-gather GEMM"
            assert "_rs" in model.layers[0].self_attn.o_proj.__dict__, "o_proj did not take the fused reduce-scatter GEMM"
            assert "_ag" in model.layers[0].self_attn.q_proj.__dict__, "q_proj did not take the fused all-gather GEMM"
            assert "_ag" in model.layers[1].mlp.gate_proj.__dict__, "gate_proj did not take the fused all-gather GEMM"
    (v0, n0, w0, e0), (v1, n1, w1, e1) = results[False], results[True]
    assert abs(v0 - v1) < 2e-2, (v0, v1)
    torch.testing.assert_close(n0, n1, rtol=3e-2, atol=1e-3)
    assert (w0 - w1).abs().max() <= 2e-2 * w0.abs().max() + 1e-3
    assert (e0 - e1).abs().max() <= 2e-2 * e0.abs().max() + 1e-3


def main():
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=datetime.timedelta(seconds=120))
    rank, world = dist.get_rank(), dist.get_world_size()
    check_norm_reducer(rank, world)
    check_fused_gemms(rank, world)
    check_sequence_parallel_llama(rank, world)
    dist.barrier()
    if rank == 0:
        print("tp check ok")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
