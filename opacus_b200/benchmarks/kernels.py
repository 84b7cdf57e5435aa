"""Micro-benchmark of the hot kernels at given shapes, timed with CUDA events.

    python -m opacus_b200.benchmarks.kernels --op ghost_norm --B 8 --T 1024 --din 2048 --dout 8192
    python -m opacus_b200.benchmarks.kernels --op wgrad --B 8 --T 1024 --din 2048 --dout 8192
    python -m opacus_b200.benchmarks.kernels --op wgrad_pair --B 8 --T 1024 --din 2048 --dout 8192
    python -m opacus_b200.benchmarks.kernels --op all
    python -m opacus_b200.benchmarks.kernels --op conv --B 512 --C 64 --O 64 --HW 32 --k 3

Reports time per call, achieved TFLOP/s (or GB/s) and the fraction of the
measured peak: ``MEASURED_PEAKS.json`` next to the repository root if present,
otherwise 1590 TFLOP/s bf16 and 6650 GB/s.  Between timed calls a buffer larger
than the L2 cache is rewritten so every call starts cold.
"""
import argparse
import json
import os

import torch

from .. import ops
from ..ops import _cuda


def _peaks():
    here = os.path.dirname(os.path.abspath(__file__))
    path = os.path.join(here, "..", "..", "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return float(d["bf16_tflops"]), float(d["hbm_gbs"]), "measured"
    except Exception:
        return 1590.0, 6650.0, "fallback"


def _time(fn, iters, flush):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        flush.add_(1.0)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    times.sort()
    return times[len(times) // 2]


def run(op, B, T, din, dout, iters=20):
    dev = torch.device("cuda")
    C = _cuda.load()
    flush = torch.zeros(64 << 20, device=dev)          # 256 MB > L2
    a = torch.randn(B, T, din, device=dev).bfloat16()
    g = (torch.randn(B, T, dout, device=dev) * 0.1).bfloat16()
    c = torch.rand(B, device=dev)
    tf_peak, bw_peak, src = _peaks()
    rows = []
    if op in ("ghost_norm", "all"):
        nT = (T + 127) // 128
        tiles = B * nT * (nT + 1) // 2
        flops = 2.0 * 128 * 128 * (din + dout) * tiles
        ms = _time(lambda: ops.linear_norm_sq(a, g, True, False), iters, flush)
        rows.append(("ghost_norm", ms, flops / ms / 1e9, "TFLOP/s", flops / ms / 1e9 / tf_peak))
    if op in ("wgrad", "all"):
        gs = g.reshape(B * T, dout).contiguous()
        a2 = a.reshape(B * T, din).contiguous()
        out = torch.empty(dout, din, device=dev)
        flops = 2.0 * B * T * din * dout
        ms = _time(lambda: C.wgrad_tn(gs, a2, out, 0.0), iters, flush)
        rows.append(("wgrad_tn", ms, flops / ms / 1e9, "TFLOP/s", flops / ms / 1e9 / tf_peak))
        ms = _time(lambda: torch.matmul(gs.t(), a2), iters, flush)
        rows.append(("cublas_tn (library, for scale)", ms, flops / ms / 1e9, "TFLOP/s", flops / ms / 1e9 / tf_peak))
    if op in ("wgrad_pair", "all"):
        # the same product on SM pairs (tcgen05 cta_group::2, clusters of two CTAs)
        gs = g.reshape(B * T, dout).contiguous()
        a2 = a.reshape(B * T, din).contiguous()
        out = torch.empty(dout, din, device=dev)
        flops = 2.0 * B * T * din * dout
        ms = _time(lambda: C.wgrad2_tn(gs, a2, out, 0.0, 1), iters, flush)
        rows.append(("wgrad2_tn (SM pairs)", ms, flops / ms / 1e9, "TFLOP/s", flops / ms / 1e9 / tf_peak))
    if op in ("weighted_grad", "all"):
        flops = 2.0 * B * T * din * dout
        ms = _time(lambda: ops.linear_weighted_grad(a, g, c), iters, flush)
        rows.append(("linear_weighted_grad (scale_rows + wgrad_tn)", ms, flops / ms / 1e9, "TFLOP/s",
                     flops / ms / 1e9 / tf_peak))
    if op in ("scale_rows", "all"):
        x = a.reshape(B * T, din)
        byts = x.numel() * 4.0
        ms = _time(lambda: C.scale_rows(x, c, T, 1.0), iters, flush)
        rows.append(("scale_rows", ms, byts / ms / 1e6, "GB/s", byts / ms / 1e6 / bw_peak))
    if op in ("embedding_norm", "all"):
        ids = torch.randint(0, 32000, (B, T), device=dev)
        nT = (T + 127) // 128
        flops = 2.0 * 128 * 128 * dout * B * nT * (nT + 1) // 2
        ms = _time(lambda: ops.embedding_norm_sq(ids, g), iters, flush)
        rows.append(("embedding_ghost_norm", ms, flops / ms / 1e9, "TFLOP/s", flops / ms / 1e9 / tf_peak))
    if op in ("secure_noise", "all"):
        # secure-mode noise: ChaCha20 block per thread -> Box-Muller -> four draws summed and halved per element
        from ..utils.secure_rng import SecureGenerator

        gen = SecureGenerator()
        ref = torch.empty(1 << 28, device=dev)
        for draws in (4, 1):
            ms = _time(lambda: gen.gaussian_like(ref, 1.0, draws=draws), max(2, iters // 4), flush)
            rows.append((f"chacha_normal (draws={draws}, 2^28 elements)", ms, ref.numel() / ms / 1e6, "Gelem/s",
                         ref.numel() * 4.0 / ms / 1e6 / bw_peak))
    if op in ("dp_step", "all"):
        n = 1 << 27
        p = torch.nn.Parameter(torch.zeros(n, device=dev))
        from ..optimizers import DPOptimizerFastGradientClipping

        dp = DPOptimizerFastGradientClipping(torch.optim.AdamW([p], lr=1e-3), noise_multiplier=1.0,
                                             max_grad_norm=1.0, expected_batch_size=8)
        grad = torch.zeros(n, device=dev)

        def one():
            p.summed_grad = grad
            dp._is_last_step_skipped = False
            if hasattr(grad, "_processed"):
                del grad._processed
            plan = dp._fused_plan()
            plan.run(dp, noise_std=1.0, denominator=8.0)

        byts = n * 4.0 * 8        # read+write of param, grad, exp_avg, exp_avg_sq
        ms = _time(one, iters, flush)
        rows.append(("fused_dp_adamw_step", ms, byts / ms / 1e6, "GB/s", byts / ms / 1e6 / bw_peak))
    if op in ("sharded_step", "all"):
        # the one-kernel reduce + noise + AdamW + publish step with a one-rank group (no peers: pure streaming)
        n = 1 << 27
        grad = torch.zeros(n, device=dev)
        param = torch.zeros(n, device=dev, dtype=torch.bfloat16)
        flags = torch.zeros(64, device=dev, dtype=torch.int32)
        master, m1, m2 = (torch.zeros(n, device=dev) for _ in range(3))
        epoch = [0]

        def sharded():
            epoch[0] += 1
            C.sharded_dp_step([grad.data_ptr()], [param.data_ptr()], [flags.data_ptr()], master, m1, m2, 0, n, 0, True,
                              epoch[0], 2, False, False, 1e-4, 0.0, 0.0, 0.01, 0.9, 0.999, 1e-8, 0.1, 0.0316, 1.0, 0.125,
                              1234, 4 * epoch[0] * n, 0, 0)

        byts = n * (4.0 * 7 + 2.0)     # read grad/master/m/v, write master/m/v (fp32) + bf16 weights
        ms = _time(sharded, iters, flush)
        rows.append(("sharded_step AdamW + noise (1 rank, 134 M)", ms, byts / ms / 1e6, "GB/s", byts / ms / 1e6 / bw_peak))
        del grad, param, master, m1, m2
    if op in ("cross_entropy", "all"):
        V = 128256
        logits = torch.randn(B * T, V, device=dev, dtype=torch.bfloat16, requires_grad=True)
        tgt = torch.randint(0, V, (B * T,), device=dev)
        gl = torch.rand(B * T, device=dev)
        ms = _time(lambda: C.cross_entropy_forward(logits.detach(), tgt, -100), iters, flush)
        byts = logits.numel() * 2.0
        rows.append(("cross_entropy forward (bf16 logits, V=128256)", ms, byts / ms / 1e6, "GB/s", byts / ms / 1e6 / bw_peak))
        loss, lse = C.cross_entropy_forward(logits.detach(), tgt, -100)
        ms = _time(lambda: C.cross_entropy_backward(logits.detach(), tgt, lse, gl, -100), iters, flush)
        rows.append(("cross_entropy backward", ms, 2 * byts / ms / 1e6, "GB/s", 2 * byts / ms / 1e6 / bw_peak))
        del logits
    if op in ("rope", "all"):
        x = torch.randn(B, T, 32, 64, device=dev, dtype=torch.bfloat16)
        byts = x.numel() * 4.0
        ms = _time(lambda: C.rope(x, 500000.0, False, False, 1.0), iters, flush)
        rows.append(("rope (32 heads x 64)", ms, byts / ms / 1e6, "GB/s", byts / ms / 1e6 / bw_peak))
    if op in ("swiglu", "all"):
        ga = torch.randn(B * T, dout, device=dev, dtype=torch.bfloat16)
        up = torch.randn(B * T, dout, device=dev, dtype=torch.bfloat16)
        byts = ga.numel() * 2.0
        ms = _time(lambda: C.swiglu_forward(ga, up), iters, flush)
        rows.append(("swiglu forward", ms, 3 * byts / ms / 1e6, "GB/s", 3 * byts / ms / 1e6 / bw_peak))
        ms = _time(lambda: C.swiglu_backward(ga, up, ga), iters, flush)
        rows.append(("swiglu backward", ms, 5 * byts / ms / 1e6, "GB/s", 5 * byts / ms / 1e6 / bw_peak))
    if op in ("rmsnorm", "all"):
        xs = torch.randn(B * T, din, device=dev, dtype=torch.bfloat16)
        dl = torch.randn(B * T, din, device=dev, dtype=torch.bfloat16)
        wn = torch.ones(din, device=dev, dtype=torch.bfloat16)
        byts = xs.numel() * 2.0
        if din % 8 == 0 and din <= 8192:
            ms = _time(lambda: C.add_rmsnorm_forward(xs, dl, wn, 1e-5), iters, flush)
            rows.append(("add + rmsnorm forward", ms, 4 * byts / ms / 1e6, "GB/s", 4 * byts / ms / 1e6 / bw_peak))
            _, hs, rs = C.add_rmsnorm_forward(xs, dl, wn, 1e-5)
            ms = _time(lambda: C.add_rmsnorm_backward(xs, dl, hs, rs, wn), iters, flush)
            rows.append(("add + rmsnorm backward", ms, 4 * byts / ms / 1e6, "GB/s", 4 * byts / ms / 1e6 / bw_peak))
    if op in ("norm_rule", "all") and din % 8 == 0 and din <= 4096:
        # LayerNorm / RMSNorm per-sample gradients + their norms in one launch: reads x and g once (x twice, L1)
        xs = torch.randn(B, T, din, device=dev, dtype=torch.bfloat16)
        gn = torch.randn(B, T, din, device=dev, dtype=torch.bfloat16)
        byts = xs.numel() * 2.0 * 2
        ms = _time(lambda: ops.norm_affine_grad_sample("rms", xs, gn, eps=1e-5, normalized_ndim=1, want_bias=False),
                   iters, flush)
        rows.append(("rmsnorm per-sample grad + norm (one launch)", ms, byts / ms / 1e6, "GB/s", byts / ms / 1e6 / bw_peak))
    if op in ("fp32_split", "all"):
        # fp32 operands through the three-plane bf16 split: 3x the bf16 FLOPs of the fp32 product
        a32, g32 = a.float(), g.float()
        flops = 2.0 * B * T * din * dout
        ms = _time(lambda: ops.linear_weighted_grad(a32, g32, c), iters, flush)
        rows.append(("fp32 clipped sum (split3 + wgrad_tn, 3 planes)", ms, flops / ms / 1e9, "TFLOP/s (fp32-equivalent)",
                     3 * flops / ms / 1e9 / tf_peak))
        ms = _time(lambda: torch.matmul((g32 * c[:, None, None]).reshape(B * T, dout).t(), a32.reshape(B * T, din)),
                   iters, flush)
        rows.append(("cuBLAS fp32/tf32 TN (library, for scale)", ms, flops / ms / 1e9, "TFLOP/s", flops / ms / 1e9 / tf_peak))
    _cuda.check_status()
    print(f"shape B={B} T={T} d_in={din} d_out={dout}; peaks: {tf_peak} TFLOP/s bf16, {bw_peak} GB/s ({src})")
    for name, ms, rate, unit, frac in rows:
        print(f"{name:48s} {ms:9.4f} ms  {rate:10.1f} {unit:8s} {frac:6.3f} of {src} peak")
    return rows


def run_conv(B, C, O, HW, k, stride=1, iters=20):
    """Conv2d per-sample weight gradient kernels at one layer shape (3x3 pad 1 or 1x1 pad 0)."""
    dev = torch.device("cuda")
    flush = torch.zeros(64 << 20, device=dev)
    conv = torch.nn.Conv2d(C, O, k, stride=stride, padding=k // 2, bias=False).to(dev).bfloat16()
    x = torch.randn(B, C, HW, HW, device=dev).bfloat16().contiguous(memory_format=torch.channels_last)
    OHW = (HW + 2 * (k // 2) - k) // stride + 1
    g = (torch.randn(B, O, OHW, OHW, device=dev) * 0.1).bfloat16().contiguous(memory_format=torch.channels_last)
    coef = torch.rand(B, device=dev)
    geom = _cuda.conv_geometry(conv, x, g)
    tf_peak, bw_peak, src = _peaks()
    flops = 2.0 * B * OHW * OHW * O * C * k * k
    in_bytes = (x.numel() + g.numel()) * 2.0
    out_bytes = B * O * C * k * k * 2.0
    rows = []
    ms = _time(lambda: _cuda.conv_grad_sample(x, g, geom), iters, flush)
    rows.append(("conv per-sample grad + norm (implicit)", ms, flops / ms / 1e9, (in_bytes + out_bytes) / ms / 1e6))
    ms = _time(lambda: _cuda.conv_grad_sample(x, g, geom, want_out=False), iters, flush)
    rows.append(("conv ghost norm (no output)", ms, flops / ms / 1e9, in_bytes / ms / 1e6))
    ms = _time(lambda: _cuda.conv_weighted_grad(x, g, coef, geom), iters, flush)
    rows.append(("conv clipped sum (one GEMM over the batch)", ms, flops / ms / 1e9, in_bytes / ms / 1e6))

    def unfold_bmm():
        cols = torch.nn.functional.unfold(x, k, padding=k // 2, stride=stride)
        return torch.bmm(g.reshape(B, O, -1), cols.transpose(1, 2))

    ms = _time(unfold_bmm, iters, flush)
    rows.append(("unfold + bmm (library, for scale)", ms, flops / ms / 1e9, (in_bytes + out_bytes) / ms / 1e6))
    _cuda.check_status()
    print(f"conv B={B} C={C} O={O} {HW}x{HW} k={k} stride={stride}; peaks: {tf_peak} TFLOP/s bf16, {bw_peak} GB/s ({src})")
    for name, ms, tf, gb in rows:
        print(f"{name:48s} {ms:9.4f} ms  {tf:8.1f} TFLOP/s ({tf / tf_peak:5.3f})  {gb:8.1f} GB/s algorithmic "
              f"({gb / bw_peak:5.3f} of {src} copy peak)")
    return rows


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--C", type=int, default=64)
    ap.add_argument("--O", type=int, default=64)
    ap.add_argument("--HW", type=int, default=32)
    ap.add_argument("--k", type=int, default=3)
    ap.add_argument("--stride", type=int, default=1)
    ap.add_argument("--op", default="all")
    ap.add_argument("--B", type=int, default=8)
    ap.add_argument("--T", type=int, default=1024)
    ap.add_argument("--din", type=int, default=2048)
    ap.add_argument("--dout", type=int, default=8192)
    ap.add_argument("--iters", type=int, default=20)
    args = ap.parse_args()
    if args.op == "conv":
        run_conv(args.B, args.C, args.O, args.HW, args.k, args.stride, args.iters)
    else:
        run(args.op, args.B, args.T, args.din, args.dout, args.iters)
