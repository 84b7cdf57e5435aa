"""Fused compute+collective kernels against the library composition (NCCL + cuBLAS) they replace.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        -m opacus_b200.benchmarks.tp_collectives [--tokens 8192] [--hidden 4096] [--ffn 14336] [--iters 20]

Shapes are those of a Llama-8B MLP under N-way tensor parallelism with sequence-sharded
activations: ``all-gather(x) -> x W_up^T`` (``[tokens, hidden] x [ffn/N, hidden]``) and
``h W_down^T -> reduce-scatter`` (``[tokens, ffn/N] x [hidden, ffn/N]``), plus the ``[B]``
per-sample-norm all-reduce.  Times are CUDA-event medians, max over ranks; a 256 MB buffer is
rewritten between iterations.  The roofline time is the larger of FLOPs / measured bf16 GEMM
peak and NVLink bytes per GPU / 770 GB/s (measured peer-copy bandwidth per direction).
"""
import argparse
import datetime
import json
import os

import torch
import torch.distributed as dist

from ..ops import _cuda
from ..parallel import symm
from ..parallel.fused_tp import AllGatherGemm, GemmReduceScatter, gemm_nt
from .kernels import _peaks

LINK_GBS = 770.0


def _timed(fn, iters, flush):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    ts = []
    for _ in range(iters):
        flush.add_(1.0)
        dist.barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    ts.sort()
    t = torch.tensor([ts[len(ts) // 2]], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--ffn", type=int, default=14336)
    ap.add_argument("--batch", type=int, default=64, help="length of the per-sample norm vector")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--json", default=None)
    args = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29581")
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=180))
    rank, world = dist.get_rank(), dist.get_world_size()
    tf_peak, _, src = _peaks()
    flush = torch.zeros(64 << 20, device=dev)
    T, H = args.tokens, args.hidden
    F = args.ffn // world // 256 * 256            # this rank's slice of the MLP width
    rows = T // world
    torch.manual_seed(rank)
    rows_out = []

    def report(name, ms_fused, ms_lib, flops, link_bytes):
        roof_ms = max(flops / (tf_peak * 1e9), link_bytes / (LINK_GBS * 1e6))
        rows_out.append(dict(op=name, world=world, fused_ms=ms_fused, library_ms=ms_lib, roofline_ms=roof_ms,
                             frac_of_roofline=roof_ms / ms_fused, speedup=ms_lib / ms_fused))
        if rank == 0:
            print(f"{name:34s} fused {ms_fused:8.4f} ms   NCCL+cuBLAS {ms_lib:8.4f} ms   x{ms_lib / ms_fused:5.2f}   "
                  f"roofline {roof_ms:7.4f} ms ({roof_ms / ms_fused:5.3f} of it, {src} GEMM peak / 770 GB/s link)",
                  flush=True)

    # ---- plain GEMM (no collective): the tensor-core core on its own
    a = torch.randn(T, H, device=dev).bfloat16()
    w_up = torch.randn(F, H, device=dev).bfloat16()
    out = torch.empty(T, F, device=dev, dtype=torch.bfloat16)
    ms_f = _timed(lambda: gemm_nt(a, w_up, out), args.iters, flush)
    ms_l = _timed(lambda: torch.matmul(a, w_up.t(), out=out), args.iters, flush)
    report("gemm_nt (no collective)", ms_f, ms_l, 2.0 * T * H * F, 0.0)

    # ---- all-gather(x) -> GEMM
    ag = AllGatherGemm(rows, H, dev, gather="a")
    ag.shard.copy_(a[:rows])
    full = torch.empty(T, H, device=dev, dtype=torch.bfloat16)

    def lib_ag():
        dist.all_gather_into_tensor(full, ag.shard)
        torch.matmul(full, w_up.t(), out=out)

    ms_f = _timed(lambda: ag(w_up, out), args.iters, flush)
    ms_l = _timed(lib_ag, args.iters, flush)
    report("all-gather(x) -> GEMM", ms_f, ms_l, 2.0 * T * H * F, (world - 1) * rows * H * 2.0)

    # ---- all-gather(W) -> GEMM (row-sharded weight)
    wrows = max(256, (args.ffn // world // world) // 256 * 256)
    agb = AllGatherGemm(wrows, H, dev, gather="b")
    agb.shard.copy_(torch.randn(wrows, H, device=dev).bfloat16())
    wfull = torch.empty(wrows * world, H, device=dev, dtype=torch.bfloat16)
    outb = torch.empty(T, wrows * world, device=dev, dtype=torch.bfloat16)

    def lib_agb():
        dist.all_gather_into_tensor(wfull, agb.shard)
        torch.matmul(a, wfull.t(), out=outb)

    ms_f = _timed(lambda: agb(a, outb), args.iters, flush)
    ms_l = _timed(lib_agb, args.iters, flush)
    report("all-gather(W) -> GEMM", ms_f, ms_l, 2.0 * T * H * wrows * world, (world - 1) * wrows * H * 2.0)

    # ---- GEMM -> reduce-scatter
    h = torch.randn(T, F, device=dev).bfloat16()
    w_down = torch.randn(H, F, device=dev).bfloat16()
    rs = GemmReduceScatter(T, H, dev)
    y = torch.empty(rows, H, device=dev, dtype=torch.bfloat16)
    part = torch.empty(T, H, device=dev, dtype=torch.bfloat16)

    def lib_rs():
        torch.matmul(h, w_down.t(), out=part)
        dist.reduce_scatter_tensor(y, part)

    ms_f = _timed(lambda: rs(h, w_down, y), args.iters, flush)
    ms_l = _timed(lib_rs, args.iters, flush)
    report("GEMM -> reduce-scatter", ms_f, ms_l, 2.0 * T * H * F, (world - 1) * rows * H * 2.0)

    # ---- per-sample norm all-reduce + clip factor
    red = symm.PeerNormReducer(dev, capacity=max(1024, args.batch))
    part_n = torch.rand(args.batch, device=dev)

    def lib_norm():
        t = part_n.clone()
        dist.all_reduce(t)
        return (1.0 / (t.sqrt() + 1e-6)).clamp(max=1.0)

    ms_f = _timed(lambda: red(part_n, None, 1.0), args.iters, flush)
    ms_l = _timed(lib_norm, args.iters, flush)
    report("norm all-reduce + clip factor", ms_f, ms_l, 0.0, 0.0)
    _cuda.check_status()
    if rank == 0 and args.json:
        with open(args.json, "w") as f:
            json.dump(rows_out, f, indent=1)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
