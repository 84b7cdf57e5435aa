"""Race-detection substitutes on the GPU: (1) debug mode fills every kernel output buffer with NaN before the
launch, so a tile or an edge that a kernel does not write at an awkward size shows up in the result; (2) kernels whose
reduction order is fixed must give the same bits when run twice."""
import pytest
import torch
import torch.nn as nn

from opacus_b200 import ops

pytestmark = pytest.mark.gpu


@pytest.fixture()
def debug_mode():
    from opacus_b200.ops import _cuda

    _cuda.set_debug(True)
    yield
    _cuda.set_debug(False)


@pytest.mark.parametrize("B,T,din,dout", [(1, 1, 8, 8), (3, 77, 72, 40), (2, 129, 264, 136), (5, 300, 128, 520)])
def test_poisoned_outputs_are_fully_written_linear(debug_mode, B, T, din, dout):
    from opacus_b200.ops import _cuda

    assert _cuda.load().get_debug()
    torch.manual_seed(0)
    a = torch.randn(B, T, din, device="cuda").bfloat16()
    g = (torch.randn(B, T, dout, device="cuda") * 0.1).bfloat16()
    c = torch.rand(B, device="cuda")
    gs = ops.linear_grad_sample(a, g)
    assert torch.isfinite(gs.float()).all() and torch.isfinite(gs._dp_norm_sq).all()
    w, b = ops.linear_norm_sq(a, g, True, True)
    assert torch.isfinite(w).all() and torch.isfinite(b).all()
    ws, bs = ops.linear_weighted_grad(a, g, c, want_bias=True)
    assert torch.isfinite(ws).all() and torch.isfinite(bs).all()
    w32 = ops.linear_grad_sample(a.float(), g.float())
    assert torch.isfinite(w32).all()
    _cuda.check_status()


def test_poisoned_outputs_are_fully_written_other_kernels(debug_mode):
    from opacus_b200.grad_sample.conv import compute_conv_grad_sample, compute_conv_weighted_grad
    from opacus_b200.layers import FusedCrossEntropyLoss
    from opacus_b200.ops import _cuda

    torch.manual_seed(0)
    conv = nn.Conv2d(3, 20, 3, padding=1).cuda().bfloat16()
    x = torch.randn(3, 3, 13, 11, device="cuda").bfloat16()
    g = torch.randn_like(conv(x))
    out = compute_conv_grad_sample(conv, [x], g)
    assert all(torch.isfinite(v.float()).all() for v in out.values())
    wg = compute_conv_weighted_grad(conv, [x], g, torch.rand(3, device="cuda"), 1.0)
    assert all(torch.isfinite(v.float()).all() for v in wg.values())
    for kind, d in (("layer", 264), ("rms", 2048), ("layer", 100)):
        xs = torch.randn(3, 17, d, device="cuda").bfloat16()
        gw, gb = ops.norm_affine_grad_sample(kind, xs, torch.randn_like(xs), eps=1e-5, normalized_ndim=1,
                                             want_bias=kind == "layer")
        assert torch.isfinite(gw).all() and (gb is None or torch.isfinite(gb).all())
        assert torch.isfinite(ops.grad_sample_norm_sq(gw)).all()
    xg = torch.randn(3, 16, 7, 5, device="cuda")
    gw, gb = ops.norm_affine_grad_sample("group", xg, torch.randn_like(xg), eps=1e-5, num_groups=4)
    assert torch.isfinite(gw).all() and torch.isfinite(gb).all()
    ids = torch.randint(0, 90, (3, 37), device="cuda")
    ge = torch.randn(3, 37, 24, device="cuda").bfloat16()
    assert torch.isfinite(ops.embedding_norm_sq(ids, ge)).all()
    assert torch.isfinite(ops.embedding_weighted_grad(ids, ge, torch.rand(3, device="cuda"), 90)).all()
    logits = torch.randn(19, 1003, device="cuda").bfloat16().requires_grad_(True)
    loss = FusedCrossEntropyLoss(reduction="none")(logits, torch.randint(0, 1003, (19,), device="cuda"))
    loss.sum().backward()
    assert torch.isfinite(loss).all() and torch.isfinite(logits.grad.float()).all()
    n2 = torch.rand(11, device="cuda")
    assert torch.isfinite(ops.clip_factor(n2, 1.0)).all()
    gsx = torch.randn(11, 333, device="cuda")
    assert torch.isfinite(ops.grad_sample_norm_sq(gsx)).all() and torch.isfinite(ops.weighted_sum(gsx, n2)).all()
    _cuda.check_status()


def test_ghost_norm_kernels_are_bitwise_reproducible():
    """The Gram kernels write per-item partial sums and add them in a fixed order: same bits on every run.  (Shapes
    for which the Gram form is the cheaper one; the instantiate-and-square form for short sequences into wide layers
    adds its tiles' partial norms with atomics and is reproducible only to rounding.)"""
    from opacus_b200.ops import _cuda

    torch.manual_seed(0)
    a = torch.randn(4, 1024, 2048, device="cuda").bfloat16()
    g = (torch.randn(4, 1024, 1024, device="cuda") * 0.1).bfloat16()
    ids = torch.randint(0, 500, (4, 1024), device="cuda")
    first = [ops.linear_norm_sq(a, g, True, True), ops.embedding_norm_sq(ids, g)]
    for _ in range(3):
        again = [ops.linear_norm_sq(a, g, True, True), ops.embedding_norm_sq(ids, g)]
        assert torch.equal(first[0][0], again[0][0]) and torch.equal(first[0][1], again[0][1])
        assert torch.equal(first[1], again[1])
    # LayerNorm / RMSNorm rule: per-block partial sums added in chunk order
    xs = torch.randn(4, 1024, 2048, device="cuda").bfloat16()
    gn = torch.randn_like(xs)
    w1, _ = ops.norm_affine_grad_sample("rms", xs, gn, eps=1e-5, normalized_ndim=1, want_bias=False)
    w2, _ = ops.norm_affine_grad_sample("rms", xs, gn, eps=1e-5, normalized_ndim=1, want_bias=False)
    assert torch.equal(w1, w2) and torch.equal(w1._dp_norm_sq, w2._dp_norm_sq)
    # per-sample gradients of the batched kernel (no K split, no atomics on the output)
    gs1, gs2 = ops.linear_grad_sample(a, g), ops.linear_grad_sample(a, g)
    assert torch.equal(gs1, gs2)
    _cuda.check_status()


def test_step_kernel_is_bitwise_reproducible():
    """Same flat gradient, same generator state: the sharded step (noise included) gives the same bits twice."""
    C = __import__("opacus_b200.ops._cuda", fromlist=["load"]).load()
    n = 1 << 20
    torch.manual_seed(0)
    grad = torch.randn(n, device="cuda")
    start = torch.randn(n, device="cuda")
    results = []
    for _ in range(2):
        param = torch.zeros(n, device="cuda", dtype=torch.bfloat16)
        flags = torch.zeros(64, device="cuda", dtype=torch.int32)
        master, m, v = start.clone(), torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
        C.sharded_dp_step([grad.data_ptr()], [param.data_ptr()], [flags.data_ptr()], master, m, v, 0, n, 0, True, 1, 2,
                          False, False, 1e-2, 0.0, 0.0, 0.01, 0.9, 0.999, 1e-8, 0.1, 0.0316, 0.8, 0.125, 99, 4, 0, 0)
        torch.cuda.synchronize()
        results.append((master, m, v, param))
    for x, y in zip(*results):
        assert torch.equal(x, y)
    assert results[0][0].ne(start).any()
