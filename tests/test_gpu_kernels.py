"""Numerics of every CUDA kernel against the plain-PyTorch fp32 statement of
the same operation (``opacus_b200.ops._ref``)."""
import pytest
import torch

from opacus_b200 import ops
from opacus_b200.ops import _ref

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device("cuda")


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


@pytest.mark.parametrize("B,T,din,dout", [(3, 128, 64, 64), (2, 256, 128, 192), (5, 100, 72, 40), (2, 300, 200, 136),
                                           (4, 1024, 256, 512)])
@pytest.mark.parametrize("bias", [False, True])
def test_linear_ghost_norm(B, T, din, dout, bias):
    torch.manual_seed(0)
    a = torch.randn(B, T, din, device=_dev()).bfloat16()
    g = (torch.randn(B, T, dout, device=_dev()) * 0.1).bfloat16()
    w, b = ops.linear_norm_sq(a, g, True, bias, g_scale=3.0)
    gs = torch.bmm(g.float().transpose(1, 2), a.float()) * 3.0
    want_w = gs.pow(2).sum(dim=(1, 2))
    assert _rel(w, want_w) < 2e-3, (w, want_w)
    if bias:
        want_b = (g.float().sum(1) * 3.0).pow(2).sum(1)
        assert _rel(b, want_b) < 2e-3, (b, want_b)
    ops._cuda.check_status()


def test_linear_ghost_norm_2d():
    torch.manual_seed(0)
    a = torch.randn(7, 33, device=_dev())
    g = torch.randn(7, 10, device=_dev())
    w, b = ops.linear_norm_sq(a, g, True, True, g_scale=2.0)
    rw, rb = _ref.linear_norm_sq(a, g, True, True, g_scale=2.0)
    assert torch.allclose(w, rw, rtol=1e-5) and torch.allclose(b, rb, rtol=1e-5)


@pytest.mark.parametrize("B,T,D,V", [(3, 128, 64, 50), (2, 200, 128, 1000), (4, 512, 256, 32)])
def test_embedding_ghost_norm(B, T, D, V):
    torch.manual_seed(0)
    ids = torch.randint(0, V, (B, T), device=_dev())
    g = (torch.randn(B, T, D, device=_dev()) * 0.1).bfloat16()
    got = ops.embedding_norm_sq(ids, g, g_scale=2.0)
    dense = _ref.embedding_grad_sample(ids, g.float() * 2.0, V)
    want = dense.pow(2).sum(dim=(1, 2))
    assert _rel(got, want) < 2e-3, (got, want)
    ops._cuda.check_status()


@pytest.mark.parametrize("B,T,D,V", [(3, 128, 64, 50), (2, 200, 128, 1000), (4, 77, 40, 9)])
def test_embedding_ghost_norm_fp32_through_split_operands(B, T, D, V):
    """fp32 gradients: the mask-Gram kernel on (hi, hi, lo) x (hi, lo, hi) planes agrees with fp64 far inside bf16."""
    torch.manual_seed(0)
    ids = torch.randint(0, V, (B, T), device=_dev())
    g = torch.randn(B, T, D, device=_dev()) * 0.1
    got = ops.embedding_norm_sq(ids, g, g_scale=2.0)
    dense = _ref.embedding_grad_sample(ids, g.double() * 2.0, V)
    want = dense.pow(2).sum(dim=(1, 2))
    assert _rel(got.double(), want) < 1e-4, (got, want)
    ops._cuda.check_status()


@pytest.mark.parametrize("B,T,din,dout", [(2, 128, 64, 128), (3, 100, 72, 40), (4, 256, 256, 512), (2, 64, 512, 1000),
                                           (8, 1024, 2048, 512)])
@pytest.mark.parametrize("bias", [False, True])
def test_linear_weighted_grad(B, T, din, dout, bias):
    torch.manual_seed(0)
    a = torch.randn(B, T, din, device=_dev()).bfloat16()
    g = (torch.randn(B, T, dout, device=_dev()) * 0.1).bfloat16()
    c = torch.rand(B, device=_dev())
    w, b = ops.linear_weighted_grad(a, g, c, g_scale=1.5, want_bias=bias)
    rw, rb = _ref.linear_weighted_grad(a.float(), g.float(), c, g_scale=1.5, want_bias=bias)
    assert w.shape == rw.shape
    assert _rel(w, rw) < 6e-3, _rel(w, rw)
    if bias:
        assert _rel(b, rb) < 1e-3
    ops._cuda.check_status()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_sq_weighted_sum_clip(dtype):
    torch.manual_seed(0)
    gs = torch.randn(9, 37, 50, device=_dev()).to(dtype)
    n2 = ops.grad_sample_norm_sq(gs)
    assert torch.allclose(n2, _ref.grad_sample_norm_sq(gs), rtol=1e-4)
    c = ops.clip_factor(n2, 3.0)
    assert torch.allclose(c, _ref.clip_factor(n2, 3.0), rtol=1e-6)
    s = ops.weighted_sum(gs, c)
    assert torch.allclose(s.float(), _ref.weighted_sum(gs.float(), c), rtol=2e-2 if dtype != torch.float32 else 1e-4,
                          atol=1e-2 if dtype != torch.float32 else 1e-5)
    big = torch.randn(4, 1 << 16, device=_dev()).to(dtype)
    assert torch.allclose(ops.grad_sample_norm_sq(big), _ref.grad_sample_norm_sq(big), rtol=1e-3)
    assert torch.allclose(ops.weighted_sum(big, c[:4]).float(), _ref.weighted_sum(big.float(), c[:4]), rtol=2e-2, atol=2e-2)


def test_clip_factor_does_not_fail_open_on_nan():
    """A NaN squared norm (unfinished or aborted producer) must not come out as factor 1 = "unclipped"."""
    n2 = torch.tensor([4.0, float("nan"), 0.0, -1e-9, float("inf")], device=_dev())
    got = ops.clip_factor(n2, 1.0)
    want = _ref.clip_factor(n2.cpu(), 1.0)
    assert torch.isnan(got[1]) and torch.isnan(want[1])
    keep = torch.tensor([0, 2, 3, 4])
    assert torch.allclose(got.cpu()[keep], want[keep], rtol=1e-6)
    assert got[4] == 0 and got[0] < 0.5001
    from opacus_b200.parallel import symm

    red = symm.PeerNormReducer(torch.device("cuda", 0), capacity=16)
    _, clip = red(n2, None, 1.0)
    assert torch.isnan(clip[1]) and torch.allclose(clip.cpu()[keep], want[keep], rtol=1e-6)


@pytest.mark.parametrize("kind", ["layer", "rms", "group", "instance"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_layer_grads(kind, dtype):
    import torch.nn.functional as F

    torch.manual_seed(0)
    if kind in ("layer", "rms"):
        x = torch.randn(5, 17, 96, device=_dev()).to(dtype)
        g = torch.randn_like(x)
        gw, gb = ops.norm_affine_grad_sample(kind, x, g, eps=1e-5, normalized_ndim=1)
        xf, gf = x.float(), g.float()
        xhat = F.layer_norm(xf, (96,), eps=1e-5) if kind == "layer" else F.rms_norm(xf, (96,), eps=1e-5)
        assert torch.allclose(gw.float(), (xhat * gf).sum(1), rtol=1e-3, atol=1e-3)
        if kind == "layer":
            assert torch.allclose(gb.float(), gf.sum(1), rtol=1e-3, atol=1e-3)
    else:
        x = torch.randn(4, 16, 6, 5, device=_dev()).to(dtype)
        g = torch.randn_like(x)
        gw, gb = ops.norm_affine_grad_sample(kind, x, g, eps=1e-5, num_groups=4)
        xf, gf = x.float(), g.float()
        xhat = F.group_norm(xf, 4, eps=1e-5) if kind == "group" else F.instance_norm(xf, eps=1e-5)
        assert torch.allclose(gw.float(), (xhat * gf).sum((2, 3)), rtol=1e-3, atol=1e-3)
        assert torch.allclose(gb.float(), gf.sum((2, 3)), rtol=1e-3, atol=1e-3)


@pytest.mark.parametrize("kind", ["layer", "rms"])
@pytest.mark.parametrize("B,T,d", [(8, 1024, 2048), (3, 50, 4096), (2, 7, 264), (1, 1, 8), (4, 33, 100)])
def test_norm_layer_one_launch_grads_and_norms(kind, B, T, d):
    """The one-launch LayerNorm / RMSNorm rule: per-sample gradients and their squared norms (attached to the
    results) against fp32 torch; d = 100 (not a multiple of 8) and LayerNorm at d = 4096 take the two-kernel path."""
    import torch.nn.functional as F

    torch.manual_seed(1)
    x = torch.randn(B, T, d, device=_dev()).bfloat16()
    g = (torch.randn(B, T, d, device=_dev()) * 0.1).bfloat16()
    for _ in range(2):                                   # twice: the ticket counters must be left clean
        gw, gb = ops.norm_affine_grad_sample(kind, x, g, eps=1e-5, normalized_ndim=1, want_bias=kind == "layer")
        xf, gf = x.float(), g.float()
        xhat = F.layer_norm(xf, (d,), eps=1e-5) if kind == "layer" else F.rms_norm(xf, (d,), eps=1e-5)
        want_w = (xhat * gf).sum(1)
        assert torch.allclose(gw.float(), want_w, rtol=2e-3, atol=2e-3)
        n2 = ops.grad_sample_norm_sq(gw)
        assert torch.allclose(n2, want_w.pow(2).sum(1), rtol=2e-3), (n2, want_w.pow(2).sum(1))
        if kind == "layer":
            assert torch.allclose(gb.float(), gf.sum(1), rtol=2e-3, atol=2e-3)
            assert torch.allclose(ops.grad_sample_norm_sq(gb), gf.sum(1).pow(2).sum(1), rtol=2e-3)
    one_launch = d % 8 == 0 and (d <= 2048 or (kind == "rms" and d <= 4096))
    assert (getattr(gw, "_dp_norm_sq", None) is not None) == one_launch
    ops._cuda.check_status()


def test_weighted_sum_into_destination():
    gs = torch.randn(6, 40, 24, device=_dev())
    c = torch.rand(6, device=_dev())
    dst = torch.full((40, 24), 7.0, device=_dev())
    out = ops.weighted_sum(gs, c, out=dst)
    assert out.data_ptr() == dst.data_ptr()
    assert torch.allclose(dst, _ref.weighted_sum(gs, c), rtol=1e-5, atol=1e-5)


def test_embedding_weighted_grad():
    torch.manual_seed(0)
    ids = torch.randint(0, 40, (6, 33), device=_dev())
    g = torch.randn(6, 33, 24, device=_dev()).bfloat16()
    c = torch.rand(6, device=_dev())
    got = ops.embedding_weighted_grad(ids, g, c, 40, g_scale=2.0)
    want = _ref.embedding_weighted_grad(ids, g.float(), c, 40, g_scale=2.0)
    assert torch.allclose(got, want, rtol=1e-4, atol=1e-4)


def test_philox_normal_statistics():
    z = ops._cuda.philox_normal(1 << 22, 1234, 0, 2.0, "cuda")
    assert abs(z.mean().item()) < 5e-3
    assert abs(z.std().item() - 2.0) < 5e-3
    zz = (z / 2.0)
    assert abs((zz ** 4).mean().item() - 3.0) < 3e-2          # kurtosis of a Gaussian
    assert abs((zz[:-1] * zz[1:]).mean().item()) < 3e-3        # no lag-1 correlation
    z2 = ops._cuda.philox_normal(1 << 22, 1234, 4, 2.0, "cuda")
    assert abs((z * z2).mean().item()) / 4.0 < 3e-3            # different offsets are independent
    assert torch.equal(z, ops._cuda.philox_normal(1 << 22, 1234, 0, 2.0, "cuda"))


@pytest.mark.parametrize("opt_name", ["sgd", "sgd_momentum", "adam", "adamw"])
def test_fused_step_matches_torch_without_noise(opt_name):
    from opacus_b200.optimizers import DPOptimizerFastGradientClipping

    torch.manual_seed(0)

    def make():
        torch.manual_seed(1)
        ps = [torch.nn.Parameter(torch.randn(33, 17, device=_dev())), torch.nn.Parameter(torch.randn(5000, device=_dev()))]
        if opt_name == "sgd":
            o = torch.optim.SGD(ps, lr=0.1, weight_decay=0.01)
        elif opt_name == "sgd_momentum":
            o = torch.optim.SGD(ps, lr=0.1, momentum=0.9, nesterov=True)
        elif opt_name == "adam":
            o = torch.optim.Adam(ps, lr=0.01, weight_decay=0.1)
        else:
            o = torch.optim.AdamW(ps, lr=0.01, weight_decay=0.1)
        return ps, o

    ps_a, oa = make()
    ps_b, ob = make()
    dp = DPOptimizerFastGradientClipping(oa, noise_multiplier=0.0, max_grad_norm=1.0, expected_batch_size=4)
    for it in range(3):
        grads = [torch.randn_like(p) for p in ps_a]
        dp.zero_grad()
        for p, g in zip(ps_a, grads):
            p.grad = g.clone()
        dp.step()
        for p, g in zip(ps_b, grads):
            p.grad = g / 4
        ob.step()
        ob.zero_grad()
        for pa, pb in zip(ps_a, ps_b):
            assert torch.allclose(pa, pb, rtol=1e-5, atol=1e-6), (opt_name, it, (pa - pb).abs().max())
    assert dp._fused_plan() is not None


def test_fused_step_noise_level():
    from opacus_b200.optimizers import DPOptimizerFastGradientClipping

    p = torch.nn.Parameter(torch.zeros(1 << 20, device=_dev()))
    o = torch.optim.SGD([p], lr=1.0)
    dp = DPOptimizerFastGradientClipping(o, noise_multiplier=2.0, max_grad_norm=0.5, expected_batch_size=1)
    p.grad = torch.zeros_like(p)
    dp.step()
    assert abs(p.detach().std().item() - 1.0) < 1e-2
    assert abs(p.detach().mean().item()) < 5e-3
    first = p.detach().clone()
    dp.zero_grad()
    p.grad = torch.zeros_like(p)
    dp.step()
    second = p.detach() - first
    assert abs((first * second).mean().item()) < 5e-3        # fresh noise every step


@pytest.mark.parametrize("bm,bn,splits", [(128, 128, 1), (128, 256, 1), (256, 256, 1), (128, 128, 4), (256, 256, 2),
                                           (0, 0, 0)])
@pytest.mark.parametrize("K,M,N", [(512, 256, 512), (1000, 520, 264), (4096, 1024, 256)])
def test_wgrad_tile_shapes_and_split_k(bm, bn, splits, K, M, N):
    C = ops._cuda.load()
    torch.manual_seed(0)
    gs = (torch.randn(K, M, device=_dev()) * 0.1).bfloat16()
    a = torch.randn(K, N, device=_dev()).bfloat16()
    want = gs.float().t() @ a.float()
    if splits > 1 and (K + 63) // 64 < 8 * splits:
        pytest.skip("contraction too short to split")
    out = torch.full((M, N), 7.0, device=_dev())
    C.wgrad_tn_ex(gs, a, out, 0.0, None, bm, bn, splits)
    assert _rel(out, want) < 6e-3
    base = torch.randn(M, N, device=_dev())
    out2 = base.clone()
    C.wgrad_tn_ex(gs, a, out2, 1.0, None, bm, bn, splits)
    assert _rel(out2, want + base) < 6e-3
    ops._cuda.check_status()


@pytest.mark.parametrize("B,T,din,dout", [(4, 128, 256, 256), (3, 100, 136, 72), (16, 64, 512, 512)])
def test_linear_per_sample_grad_with_fused_norm(B, T, din, dout):
    torch.manual_seed(0)
    a = torch.randn(B, T, din, device=_dev()).bfloat16()
    g = (torch.randn(B, T, dout, device=_dev()) * 0.1).bfloat16()
    gs = ops.linear_grad_sample(a, g)
    want = torch.bmm(g.float().transpose(1, 2), a.float())
    assert gs.shape == want.shape and _rel(gs, want) < 8e-3
    n2 = ops.grad_sample_norm_sq(gs)
    assert n2 is gs._dp_norm_sq
    assert _rel(n2, want.pow(2).sum(dim=(1, 2))) < 2e-3
    ops._cuda.check_status()


def test_conv_per_sample_grad_tensor_core_path():
    import torch.nn as nn

    from opacus_b200.grad_sample.conv import compute_conv_grad_sample

    torch.manual_seed(0)
    conv = nn.Conv2d(16, 32, 3, stride=2, padding=1).to(_dev()).bfloat16()
    x = torch.randn(6, 16, 15, 14, device=_dev()).bfloat16()
    y = conv(x)
    g = (torch.randn_like(y) * 0.1)
    got = compute_conv_grad_sample(conv, [x], g)
    conv32 = nn.Conv2d(16, 32, 3, stride=2, padding=1).to(_dev())
    want_w = []
    for i in range(6):
        w = torch.nn.grad.conv2d_weight(x[i:i + 1].float(), conv32.weight.shape, g[i:i + 1].float(), stride=2, padding=1)
        want_w.append(w)
    want_w = torch.stack(want_w)
    gw = got[conv.weight]
    assert gw.shape == want_w.shape and _rel(gw, want_w) < 1e-2
    assert _rel(ops.grad_sample_norm_sq(gw), want_w.pow(2).sum(dim=(1, 2, 3, 4))) < 5e-3
    assert _rel(got[conv.bias], g.float().sum(dim=(2, 3))) < 1e-2


def _conv_oracle(conv, x, g):
    """fp32 per-sample weight gradients by one autograd call per sample."""
    out = []
    w = conv.weight.detach().float().requires_grad_(True)
    for b in range(x.shape[0]):
        y = torch.nn.functional.conv2d(x[b:b + 1].float(), w, None, conv.stride, conv.padding, conv.dilation) \
            if x.dim() == 4 else \
            torch.nn.functional.conv1d(x[b:b + 1].float(), w, None, conv.stride, conv.padding, conv.dilation)
        (gw,) = torch.autograd.grad(y, w, g[b:b + 1].float())
        out.append(gw)
    return torch.stack(out)


@pytest.mark.gpu
@pytest.mark.parametrize("cfg", [
    dict(C=64, O=64, H=32, W=32, k=3, s=1, p=1, d=1),
    dict(C=128, O=256, H=8, W=8, k=3, s=1, p=1, d=1),
    dict(C=24, O=40, H=14, W=14, k=3, s=1, p=1, d=1),     # partial channel block, odd width
    dict(C=64, O=128, H=16, W=16, k=1, s=1, p=0, d=1),
    dict(C=64, O=128, H=32, W=32, k=3, s=2, p=1, d=1),    # strided
    dict(C=64, O=128, H=17, W=17, k=1, s=2, p=0, d=1),
    dict(C=32, O=32, H=20, W=20, k=3, s=1, p=2, d=2),     # dilated
    dict(C=16, O=32, H=9, W=70, k=(3, 5), s=(1, 2), p=(1, 2), d=1),
])
def test_conv_implicit_per_sample_grad(cfg):
    from opacus_b200.ops import _cuda

    torch.manual_seed(0)
    B = 5
    conv = torch.nn.Conv2d(cfg["C"], cfg["O"], cfg["k"], stride=cfg["s"], padding=cfg["p"], dilation=cfg["d"],
                           bias=False).cuda().to(torch.bfloat16)
    x = torch.randn(B, cfg["C"], cfg["H"], cfg["W"], device="cuda", dtype=torch.bfloat16)
    y = conv(x)
    g = torch.randn_like(y)
    geom = _cuda.conv_geometry(conv, x, g)
    assert geom is not None
    gs = _cuda.conv_grad_sample(x, g, geom)
    ref = _conv_oracle(conv, x, g)
    assert gs.shape == ref.shape
    scale = ref.abs().max()
    assert (gs.float() - ref).abs().max() <= 1e-2 * scale
    nref = ref.flatten(1).square().sum(1)
    torch.testing.assert_close(gs._dp_norm_sq, nref, rtol=2e-3, atol=0)
    # norm only
    n2 = _cuda.conv_grad_sample(x, g, geom, want_out=False)
    torch.testing.assert_close(n2, nref, rtol=2e-3, atol=0)
    # clipped sum as one GEMM over the batch
    coef = torch.rand(B, device="cuda")
    ws = _cuda.conv_weighted_grad(x, g, coef, geom, g_scale=2.0)
    wref = (ref * (2.0 * coef)[:, None, None, None, None]).sum(0)
    assert (ws - wref).abs().max() <= 1e-2 * wref.abs().max()
    # weighted sum of the permuted per-sample view
    s = _cuda.weighted_sum(gs, coef)
    sref = (gs.float() * coef[:, None, None, None, None]).sum(0)
    assert s.shape == sref.shape and (s.float() - sref).abs().max() <= 2e-2 * sref.abs().max()
    _cuda.check_status()


def _conv_oracle_general(conv, x, g):
    """Per-sample weight gradients through the layer's own forward (groups, string padding included), computed in
    fp64 (fp32 convolutions of the library may run on tf32 tensor cores, which is coarser than the kernels under test)
    and returned in fp32."""
    import copy

    ref = copy.deepcopy(conv).double()
    out = []
    for b in range(x.shape[0]):
        ref.zero_grad()
        y = ref(x[b:b + 1].double())
        (gw,) = torch.autograd.grad(y, ref.weight, g[b:b + 1].double())
        out.append(gw)
    return torch.stack(out).float()


@pytest.mark.gpu
@pytest.mark.parametrize("cfg", [
    dict(C=3, O=64, H=32, W=32, k=3, s=1, p=1, groups=1, dtype=torch.bfloat16),       # ResNet stem: 3 channels
    dict(C=1, O=16, H=28, W=28, k=8, s=2, p=3, groups=1, dtype=torch.bfloat16),       # one channel, wide filter
    dict(C=32, O=64, H=12, W=12, k=3, s=1, p=1, groups=4, dtype=torch.bfloat16),      # grouped
    dict(C=12, O=20, H=9, W=11, k=3, s=1, p=1, groups=2, dtype=torch.bfloat16),       # grouped, 6 / 10 channels per group
    dict(C=16, O=32, H=10, W=10, k=(2, 4), s=1, p="same", groups=1, dtype=torch.bfloat16),   # odd padding totals
    dict(C=64, O=64, H=16, W=16, k=3, s=1, p=1, groups=1, dtype=torch.float32),       # fp32 as three bf16 passes
    dict(C=3, O=24, H=14, W=14, k=3, s=2, p=1, groups=1, dtype=torch.float32),
])
def test_conv_kernel_coverage_beyond_plain_bf16(cfg):
    """Channel counts that are not multiples of 8, groups, "same" padding with an odd total and fp32 data all run on
    the implicit-unfold kernel (no unfolded copy) and agree with per-sample autograd."""
    from opacus_b200.grad_sample.conv import compute_conv_grad_sample, compute_conv_norm_sq, compute_conv_weighted_grad
    from opacus_b200.ops import _cuda

    torch.manual_seed(0)
    B, dt = 4, cfg["dtype"]
    conv = torch.nn.Conv2d(cfg["C"], cfg["O"], cfg["k"], stride=cfg["s"], padding=cfg["p"], groups=cfg["groups"],
                           bias=True).cuda().to(dt)
    x = torch.randn(B, cfg["C"], cfg["H"], cfg["W"], device="cuda", dtype=dt)
    g = torch.randn_like(conv(x))
    assert _cuda.conv_geometry(conv, x, g) is not None
    ref = _conv_oracle_general(conv, x, g)
    tol = 1e-2 if dt == torch.bfloat16 else 2e-4
    out = compute_conv_grad_sample(conv, [x], g)
    gw = out[conv.weight]
    assert gw.shape == ref.shape
    assert (gw.float() - ref).abs().max() <= tol * ref.abs().max()
    nref = ref.flatten(1).square().sum(1)
    torch.testing.assert_close(ops.grad_sample_norm_sq(gw), nref, rtol=2e-3 if dt == torch.bfloat16 else 1e-4, atol=0)
    nsq = compute_conv_norm_sq(conv, [x], g, 2.0)
    torch.testing.assert_close(nsq[conv.weight], 4.0 * nref, rtol=2e-3 if dt == torch.bfloat16 else 1e-4, atol=0)
    coef = torch.rand(B, device="cuda")
    wg = compute_conv_weighted_grad(conv, [x], g, coef, 1.0)
    wref = (ref * coef[:, None, None, None, None]).sum(0)
    assert wg[conv.weight].shape == wref.shape
    assert (wg[conv.weight].float() - wref).abs().max() <= tol * wref.abs().max()
    _cuda.check_status()


@pytest.mark.gpu
@pytest.mark.parametrize("cfg", [
    dict(C=16, O=24, size=(6, 10, 12), k=3, s=1, p=1, d=1, groups=1, dtype=torch.bfloat16),
    dict(C=8, O=16, size=(7, 9, 8), k=(2, 3, 3), s=(2, 2, 1), p=(1, 0, 2), d=1, groups=1, dtype=torch.bfloat16),
    dict(C=16, O=16, size=(6, 8, 9), k=(3, 2, 3), s=(1, 3, 2), p=(2, 1, 1), d=(2, 1, 1), groups=2, dtype=torch.bfloat16),
    dict(C=3, O=8, size=(4, 6, 5), k=(2, 4, 3), s=1, p="same", d=1, groups=1, dtype=torch.bfloat16),
    dict(C=8, O=8, size=(5, 8, 8), k=3, s=1, p=1, d=1, groups=1, dtype=torch.float32),
])
def test_conv3d_on_the_implicit_kernel(cfg):
    """Conv3d per-sample gradients, ghost norms and clipped sums run on the 2-d implicit-unfold kernel (one call per
    kernel-depth offset over depth-stacked images) and agree with per-sample autograd."""
    from opacus_b200.grad_sample.conv import (_implicit_geometry, compute_conv_grad_sample, compute_conv_norm_sq,
                                              compute_conv_weighted_grad)
    from opacus_b200.ops import _cuda

    torch.manual_seed(0)
    B, dt = 3, cfg["dtype"]
    conv = torch.nn.Conv3d(cfg["C"], cfg["O"], cfg["k"], stride=cfg["s"], padding=cfg["p"], dilation=cfg["d"],
                           groups=cfg["groups"], bias=True).cuda().to(dt)
    x = torch.randn(B, cfg["C"], *cfg["size"], device="cuda", dtype=dt)
    g = torch.randn_like(conv(x))
    assert _implicit_geometry(conv, x, g) is not None
    ref = _conv_oracle_general(conv, x, g)
    tol = 1e-2 if dt == torch.bfloat16 else 2e-4
    rtol = 2e-3 if dt == torch.bfloat16 else 1e-4
    out = compute_conv_grad_sample(conv, [x], g)
    gw = out[conv.weight]
    assert gw.shape == ref.shape
    assert (gw.float() - ref).abs().max() <= tol * ref.abs().max()
    nref = ref.flatten(1).square().sum(1)
    torch.testing.assert_close(gw._dp_norm_sq, nref, rtol=rtol, atol=0)
    torch.testing.assert_close(out[conv.bias].float(), g.float().flatten(2).sum(2), rtol=1e-2, atol=1e-2)
    nsq = compute_conv_norm_sq(conv, [x], g, 2.0)
    torch.testing.assert_close(nsq[conv.weight], 4.0 * nref, rtol=rtol, atol=0)
    coef = torch.rand(B, device="cuda")
    wg = compute_conv_weighted_grad(conv, [x], g, coef, 1.0)
    wref = (ref * coef[:, None, None, None, None, None]).sum(0)
    assert wg[conv.weight].shape == wref.shape
    assert (wg[conv.weight].float() - wref).abs().max() <= tol * wref.abs().max()
    _cuda.check_status()


@pytest.mark.gpu
@pytest.mark.parametrize("K,M,N,splits,beta", [(64, 256, 256, 1, 0.0), (1024, 512, 768, 1, 0.0), (300, 264, 200, 1, 0.0),
                                                (4096, 512, 2048, 4, 0.0), (2048, 256, 512, 2, 1.0),
                                                (128, 128, 64, 1, 1.0), (8192, 2048, 2048, 1, 0.0)])
def test_wgrad_on_sm_pairs(K, M, N, splits, beta):
    """The cta_group::2 form of the clipped-sum GEMM (clusters of two CTAs per 256 x 256 tile) against fp32 torch and,
    without a K split, bit for bit against the one-CTA kernel."""
    C = ops._cuda.load()
    torch.manual_seed(0)
    gs = (torch.randn(K, M, device=_dev()) * 0.1).bfloat16()
    a = torch.randn(K, N, device=_dev()).bfloat16()
    start = torch.randn(M, N, device=_dev())
    out = start.clone()
    C.wgrad2_tn(gs, a, out, beta, splits)
    ref = gs.float().t() @ a.float() + beta * start
    assert _rel(out, ref) < 1e-4
    if splits == 1:
        one = start.clone()
        C.wgrad_tn_ex(gs, a, one, beta, None, 256, 256, 1)
        assert torch.equal(out, one)
    ops._cuda.check_status()


@pytest.mark.parametrize("B,T,din,dout", [(4, 128, 512, 512), (3, 50, 72, 40), (2, 1024, 256, 128)])
def test_fp32_linear_rules_run_on_split_bf16_operands(B, T, din, dout):
    """fp32 activations and gradients: per-sample gradient, ghost norm and clipped sum through the three-plane
    bf16 split agree with fp32 torch far inside what one bf16 rounding of the operands would give."""
    torch.manual_seed(0)
    a = torch.randn(B, T, din, device=_dev())
    g = torch.randn(B, T, dout, device=_dev()) * 0.1
    want = torch.bmm(g.double().transpose(1, 2), a.double())
    gs = ops.linear_grad_sample(a, g)
    assert gs.dtype == torch.float32 and gs.shape == (B, dout, din)
    assert _rel(gs.double(), want) < 5e-5
    assert _rel(gs._dp_norm_sq.double(), want.pow(2).sum(dim=(1, 2))) < 1e-4
    w, b = ops.linear_norm_sq(a, g, True, True, g_scale=2.0)
    assert _rel(w.double(), 4.0 * want.pow(2).sum(dim=(1, 2))) < 1e-4
    assert _rel(b.double(), 4.0 * g.double().sum(1).pow(2).sum(1)) < 1e-4
    c = torch.rand(B, device=_dev())
    ws, _ = ops.linear_weighted_grad(a, g, c, g_scale=1.5)
    wref = (want * (1.5 * c.double())[:, None, None]).sum(0)
    assert _rel(ws.double(), wref) < 5e-5
    ops._cuda.check_status()


@pytest.mark.gpu
def test_conv1d_implicit_and_rules():
    from opacus_b200.grad_sample.conv import compute_conv_grad_sample, compute_conv_norm_sq, compute_conv_weighted_grad
    from opacus_b200.ops import _cuda

    torch.manual_seed(1)
    conv = torch.nn.Conv1d(16, 24, 5, padding=2).cuda().to(torch.bfloat16)
    x = torch.randn(4, 16, 100, device="cuda", dtype=torch.bfloat16)
    g = torch.randn(4, 24, 100, device="cuda", dtype=torch.bfloat16)
    assert _cuda.conv_geometry(conv, x, g) is not None
    ref = _conv_oracle(conv, x, g)
    out = compute_conv_grad_sample(conv, [x], g)
    assert out[conv.weight].shape == ref.shape
    assert (out[conv.weight].float() - ref).abs().max() <= 1e-2 * ref.abs().max()
    torch.testing.assert_close(out[conv.bias].float(), g.float().sum(2), rtol=2e-2, atol=2e-1)
    nsq = compute_conv_norm_sq(conv, [x], g, 3.0)
    torch.testing.assert_close(nsq[conv.weight], 9.0 * ref.flatten(1).square().sum(1), rtol=2e-3, atol=0)
    coef = torch.rand(4, device="cuda")
    wg = compute_conv_weighted_grad(conv, [x], g, coef, 1.0)
    wref = (ref * coef[:, None, None, None]).sum(0)
    assert (wg[conv.weight] - wref).abs().max() <= 1e-2 * wref.abs().max()
    bref = (g.float().sum(2) * coef[:, None]).sum(0)
    torch.testing.assert_close(wg[conv.bias], bref, rtol=1e-2, atol=1e-1)
    _cuda.check_status()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,V", [(torch.bfloat16, 4096), (torch.float32, 1000), (torch.bfloat16, 1003), (torch.float16, 512)])
def test_fused_cross_entropy_matches_fp32(dtype, V):
    from opacus_b200.layers import FusedCrossEntropyLoss
    from opacus_b200.ops import _cuda

    torch.manual_seed(0)
    N = 37
    logits = (torch.randn(N, V, device="cuda") * 3).to(dtype).requires_grad_(True)
    target = torch.randint(0, V, (N,), device="cuda")
    target[5] = -100
    crit = FusedCrossEntropyLoss(reduction="none")
    loss = crit(logits, target)
    ref_in = logits.detach().float().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(ref_in, target, reduction="none")
    torch.testing.assert_close(loss, ref, rtol=1e-4, atol=1e-4)
    w = torch.rand(N, device="cuda")
    (loss * w).sum().backward()
    (ref * w).sum().backward()
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert logits.grad.dtype == dtype
    assert (logits.grad.float() - ref_in.grad).abs().max() <= tol
    assert logits.grad[5].abs().max() == 0
    mean = FusedCrossEntropyLoss()(logits.detach(), target)
    torch.testing.assert_close(mean, torch.nn.functional.cross_entropy(ref_in.detach(), target), rtol=1e-4, atol=1e-4)
    _cuda.check_status()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_fused_rope_and_swiglu_match_torch(dtype):
    from opacus_b200.models.llama import _apply_rope, _rope_tables, rope, swiglu
    from opacus_b200.ops import _cuda

    torch.manual_seed(0)
    B, T, H, hd = 2, 37, 4, 64
    x = torch.randn(B, T, H, hd, device="cuda", dtype=dtype, requires_grad=True)
    y = rope(x, 500000.0)
    xr = x.detach().float().requires_grad_(True)
    cos, sin = _rope_tables(T, hd, 500000.0, x.device, torch.float32)
    yr = _apply_rope(xr.transpose(1, 2), cos, sin).transpose(1, 2)
    assert y.shape == yr.shape and y.is_contiguous()
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-4
    assert (y.float() - yr).abs().max() <= tol
    w = torch.randn(yr.shape, device="cuda")
    (y.float() * w).sum().backward()
    (yr * w).sum().backward()
    assert x.grad.shape == x.shape and (x.grad.float() - xr.grad).abs().max() <= tol

    g = torch.randn(5, 7, 64, device="cuda", dtype=dtype, requires_grad=True)
    u = torch.randn(5, 7, 64, device="cuda", dtype=dtype, requires_grad=True)
    h = swiglu(g, u)
    gr, ur = g.detach().float().requires_grad_(True), u.detach().float().requires_grad_(True)
    hr = torch.nn.functional.silu(gr) * ur
    assert (h.float() - hr).abs().max() <= tol * 4
    w = torch.randn_like(hr)
    (h.float() * w).sum().backward()
    (hr * w).sum().backward()
    assert (g.grad.float() - gr.grad).abs().max() <= tol * 4 and (u.grad.float() - ur.grad).abs().max() <= tol * 4
    _cuda.check_status()


@pytest.mark.gpu
@pytest.mark.parametrize("B,T,D,V", [(3, 128, 64, 500), (2, 200, 72, 1000), (4, 384, 256, 4096)])
def test_tied_cross_norm_kernel(B, T, D, V):
    from opacus_b200.ops import _cuda

    torch.manual_seed(0)
    ids = torch.randint(0, V, (B, T), device="cuda")
    g_e = torch.randn(B, T, D, device="cuda").bfloat16()
    a_h = torch.randn(B, T, D, device="cuda").bfloat16()
    g_h = (torch.randn(B, T, V, device="cuda") * 0.1).bfloat16()
    got = _cuda.load().tied_cross_norm(ids, g_e, a_h, g_h, 1.5, None)
    # dense oracle: <scatter(G_E by ids), G_H^T A_H> per sample, fp32
    want = torch.empty(B, device="cuda")
    for b in range(B):
        ge = torch.zeros(V, D, device="cuda").index_add_(0, ids[b], g_e[b].float())
        gh = g_h[b].float().t() @ a_h[b].float()
        want[b] = 1.5 * (ge * gh).sum()
    torch.testing.assert_close(got, want, rtol=2e-2, atol=2e-2 * want.abs().max().item())
    total = torch.ones(B, device="cuda")
    _cuda.load().tied_cross_norm(ids, g_e, a_h, g_h, 1.5, total)
    torch.testing.assert_close(total, want + 1.0, rtol=2e-2, atol=2e-2 * want.abs().max().item())
    _cuda.check_status()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("D", [64, 2048, 4096, 1000])
@pytest.mark.parametrize("with_delta", [True, False])
def test_add_rms_norm_matches_torch(dtype, D, with_delta):
    """Residual add + RMSNorm in one kernel each way against the two statements in fp32."""
    from opacus_b200.layers.add_rms_norm import AddRMSNorm

    torch.manual_seed(0)
    rows = (3, 37)
    m = AddRMSNorm(D, eps=1e-5).to(_dev(), dtype)
    m.weight.data.uniform_(0.5, 1.5)
    x = torch.randn(*rows, D, device=_dev()).to(dtype).requires_grad_()
    d = torch.randn(*rows, D, device=_dev()).to(dtype).requires_grad_() if with_delta else None
    gy = torch.randn(*rows, D, device=_dev()).to(dtype)
    gh = torch.randn(*rows, D, device=_dev()).to(dtype)
    y, h = m(x, d)
    (y.float() * gy.float() + h.float() * gh.float()).sum().backward()

    xf = x.detach().float().requires_grad_()
    df = d.detach().float().requires_grad_() if with_delta else None
    wf = m.weight.detach().float().requires_grad_()
    hf = xf + df if with_delta else xf
    hf_seen = hf.to(dtype).float() if with_delta else hf          # the kernel normalises the rounded sum it returns
    yf = torch.nn.functional.rms_norm(hf_seen, (D,), wf, 1e-5)
    (yf * gy.float() + hf * gh.float()).sum().backward()
    tol = 1e-5 if dtype == torch.float32 else (2e-3 if dtype == torch.float16 else 1e-2)
    assert _rel(h, hf) < tol and _rel(y, yf) < tol
    assert _rel(x.grad, xf.grad) < tol
    if with_delta:
        assert _rel(d.grad, df.grad) < tol
    assert _rel(m.weight.grad, wf.grad) < 2 * tol
