"""Per-layer DP step timing: forward + backward + clip + noise + SGD step of a
single layer at batch 64, in hooks and ghost-clipping modes, fp32 and bf16.

    python -m opacus_b200.benchmarks.layers [--impl ours|reference] [--dtype fp32|bf16|both] [--batch 64]
                                            [--layers linear,conv,...] [--iters 20] [--json out.json]

Layers and shapes: Linear 512->512 on [64,128,512]; Conv2d 64->64 k3 on
[64,64,32,32]; LayerNorm / GroupNorm(8) / InstanceNorm2d on [64,64,32,32];
Embedding 30000x512 on ids [64,128]; MultiheadAttention d=512 h=8 T=128;
RNN / GRU / LSTM in=hidden=512 T=128.  ``--impl reference`` runs the same
harness on the reference library found under ``baseline/_ref`` (its modes and
layers; protocol modelled on ``benchmarks/benchmark_layer.py:26-89`` there).
Times are CUDA-event medians in milliseconds; a 256 MB buffer is rewritten
between iterations so every iteration starts with a cold L2.  ``peak_mb`` is the
peak of CUDA memory allocated during one step above what was allocated before it
(layer, input and optimiser state excluded), the second metric of the
reference's layer benchmark (``benchmarks/utils.py:30-53``,
``benchmarks/layers.py:59-119`` there).  ``--kernels`` adds, per row, the names of
the GEMM-shaped kernels one step launched (``dpk::`` = this package's tensor-core
kernels; ``nvjet`` / ``gemm`` / ``cutlass`` / ``bmm`` = library GEMMs).
"""
import argparse
import json
import os
import sys

import torch
import torch.nn as nn

B = 64


class _Seq(nn.Module):
    """Recurrent layer returning only its output sequence."""

    def __init__(self, rnn):
        super().__init__()
        self.rnn = rnn

    def forward(self, x):
        return self.rnn(x)[0]


class _SelfAttn(nn.Module):
    def __init__(self, mha):
        super().__init__()
        self.mha = mha

    def forward(self, x):
        return self.mha(x, x, x, need_weights=False)[0]


def _specs(lib):
    """name -> (module factory, input factory)."""
    L = lib["layers"]
    dev = "cuda"
    return {
        "linear": (lambda: nn.Linear(512, 512), lambda dt: torch.randn(B, 128, 512, device=dev, dtype=dt)),
        "conv": (lambda: nn.Conv2d(64, 64, 3, padding=1), lambda dt: torch.randn(B, 64, 32, 32, device=dev, dtype=dt)),
        "layernorm": (lambda: nn.LayerNorm([64, 32, 32]), lambda dt: torch.randn(B, 64, 32, 32, device=dev, dtype=dt)),
        "groupnorm": (lambda: nn.GroupNorm(8, 64), lambda dt: torch.randn(B, 64, 32, 32, device=dev, dtype=dt)),
        "instancenorm": (lambda: nn.InstanceNorm2d(64, affine=True),
                         lambda dt: torch.randn(B, 64, 32, 32, device=dev, dtype=dt)),
        "embedding": (lambda: nn.Embedding(30000, 512), lambda dt: torch.randint(0, 30000, (B, 128), device=dev)),
        "mha": (lambda: _SelfAttn(L.DPMultiheadAttention(512, 8, batch_first=True)),
                lambda dt: torch.randn(B, 128, 512, device=dev, dtype=dt)),
        "rnn": (lambda: _Seq(L.DPRNN(512, 512, batch_first=True)), lambda dt: torch.randn(B, 128, 512, device=dev, dtype=dt)),
        "gru": (lambda: _Seq(L.DPGRU(512, 512, batch_first=True)), lambda dt: torch.randn(B, 128, 512, device=dev, dtype=dt)),
        "lstm": (lambda: _Seq(L.DPLSTM(512, 512, batch_first=True)), lambda dt: torch.randn(B, 128, 512, device=dev, dtype=dt)),
    }


def _load(impl):
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    if impl == "reference":
        sys.path.insert(0, os.path.join(root, "baseline", "_ref"))
        import opacus as pkg
        from opacus import layers
        from opacus.grad_sample import wrap_model
        from opacus.optimizers import DPOptimizer, DPOptimizerFastGradientClipping
        from opacus.utils.fast_gradient_clipping_utils import DPLossFastGradientClipping
    else:
        sys.path.insert(0, root)
        import opacus_b200 as pkg
        from opacus_b200 import layers
        from opacus_b200.grad_sample import wrap_model
        from opacus_b200.optimizers import DPOptimizer, DPOptimizerFastGradientClipping
        from opacus_b200.utils.fast_gradient_clipping_utils import DPLossFastGradientClipping
    return dict(pkg=pkg, layers=layers, wrap_model=wrap_model, DPOptimizer=DPOptimizer,
                DPOptimizerFGC=DPOptimizerFastGradientClipping, DPLoss=DPLossFastGradientClipping)


class _PerSampleSquare:
    """Criterion with a ``reduction`` attribute: mean of squares per sample."""

    def __init__(self, reduction="mean"):
        self.reduction = reduction

    def __call__(self, out, _target=None):
        per = out.float().pow(2).flatten(1).mean(dim=1)
        if self.reduction == "none":
            return per
        return per.mean() if self.reduction == "mean" else per.sum()


def _median_ms(fn, iters, flush):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        flush.add_(1.0)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    ts.sort()
    return ts[len(ts) // 2]


def time_layer(lib, impl, name, make, make_input, mode, dtype, iters, flush, want_kernels=False):
    torch.manual_seed(0)
    layer = make().cuda()
    if dtype == torch.bfloat16:
        layer = layer.to(torch.bfloat16)
    x = make_input(dtype)
    crit = _PerSampleSquare()
    if mode == "ghost":
        kw = {"single_pass": True} if impl == "ours" else {}
        model = lib["wrap_model"](layer, grad_sample_mode="ghost", max_grad_norm=1.0, **kw)
        opt = lib["DPOptimizerFGC"](torch.optim.SGD(layer.parameters(), lr=0.01), noise_multiplier=1.0,
                                    max_grad_norm=1.0, expected_batch_size=B)
        loss_fn = lib["DPLoss"](model, opt, crit, "mean")

        def step():
            opt.zero_grad()
            loss_fn(model(x), None).backward()
            opt.step()
    else:
        kw = {"skip_param_grads": True} if impl == "ours" else {}     # no wasted batch-gradient GEMM in autograd
        model = lib["wrap_model"](layer, grad_sample_mode="hooks", **kw)
        opt = lib["DPOptimizer"](torch.optim.SGD(layer.parameters(), lr=0.01), noise_multiplier=1.0,
                                 max_grad_norm=1.0, expected_batch_size=B)

        def step():
            opt.zero_grad()
            crit(model(x)).backward()
            opt.step()

    ms = _median_ms(step, iters, flush)
    torch.cuda.synchronize()
    base = torch.cuda.memory_allocated()
    torch.cuda.reset_peak_memory_stats()
    step()
    torch.cuda.synchronize()
    peak_mb = (torch.cuda.max_memory_allocated() - base) / 2 ** 20
    return ms, peak_mb, (_gemm_kernels(step) if want_kernels else None)


def _gemm_kernels(step):
    """Names (shortened) of the GEMM-shaped kernels of one step with their launch counts."""
    from torch.profiler import ProfilerActivity, profile

    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        step()
        torch.cuda.synchronize()
    marks = ("wgrad_tn", "gram_pair", "conv_psg", "tp_gemm", "nvjet", "gemm", "cutlass", "bmm", "xmma", "cudnn")
    out = {}
    for e in prof.key_averages():
        low = e.key.lower()
        if any(m in low for m in marks):
            out[e.key.split("(")[0][:60]] = int(e.count)
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--dtype", default="both", choices=["fp32", "bf16", "both"])
    ap.add_argument("--layers", default="all")
    ap.add_argument("--modes", default="hooks,ghost")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--batch", type=int, default=64, help="samples per step (the reference's suite sweeps 16 ... 512)")
    ap.add_argument("--json", default=None)
    ap.add_argument("--kernels", action="store_true", help="list the GEMM-shaped kernels of one step per row")
    args = ap.parse_args()
    import warnings

    warnings.simplefilter("ignore")
    global B
    B = args.batch
    lib = _load(args.impl)
    specs = _specs(lib)
    names = list(specs) if args.layers == "all" else args.layers.split(",")
    dtypes = {"fp32": [torch.float32], "bf16": [torch.bfloat16], "both": [torch.float32, torch.bfloat16]}[args.dtype]
    flush = torch.zeros(64 << 20, device="cuda")
    rows = []
    print(f"impl={args.impl}  batch={B}  (ms per DP step: fwd + bwd + clip + noise + SGD; peak CUDA MB of a step)")
    for name in names:
        make, make_input = specs[name]
        for dt in dtypes:
            for mode in args.modes.split(","):
                peak, kernels = None, None
                try:
                    ms, peak, kernels = time_layer(lib, args.impl, name, make, make_input, mode, dt, args.iters, flush,
                                                   args.kernels)
                    err = None
                except Exception as e:  # a layer/mode/dtype the library cannot run is reported, not fatal
                    ms, err = None, f"{type(e).__name__}: {str(e)[:120]}"
                rows.append({"impl": args.impl, "layer": name, "dtype": str(dt).split(".")[-1], "mode": mode, "batch": B,
                             "ms": ms, "peak_mb": peak, "gemm_kernels": kernels, "error": err})
                shown = f"{ms:9.3f} ms {peak:10.1f} MB" if ms is not None else f"   failed ({err})"
                print(f"{name:13s} {str(dt).split('.')[-1]:9s} {mode:6s} {shown}"
                      + (f"   {kernels}" if kernels else ""), flush=True)
    if args.impl == "ours":
        from opacus_b200.ops import _cuda

        _cuda.check_status()
    if args.json:
        with open(args.json, "w") as f:
            json.dump(rows, f, indent=1)


if __name__ == "__main__":
    main()
