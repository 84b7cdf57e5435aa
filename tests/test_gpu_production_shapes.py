"""The DP kernels at the shapes of the language-model benchmark (vocabulary 128256, width 2048, 1024 tokens) and at the
awkward ends of their index ranges (one sample, odd lengths), each against the fp32 PyTorch statement of the same op.

Reference math: ``opacus/grad_sample/linear.py:47,83-92`` (ghost norm of a Linear),
``opacus/utils/fast_gradient_clipping_utils.py:194-201`` (clipped sums), ``opacus/grad_sample/embedding.py:68-90``
(embedding ghost norm); the tied cross term has no counterpart there (shared parameters are rejected).
"""
import pytest
import torch

from opacus_b200 import ops

pytestmark = pytest.mark.gpu

V, D, T = 128256, 2048, 1024


def _rel(a, b):
    return ((a.double() - b.double()).norm() / (b.double().norm() + 1e-30)).item()


def _operands(B, t=T, d_in=D, d_out=V, seed=0):
    torch.manual_seed(seed)
    a = torch.randn(B, t, d_in, device="cuda").bfloat16()
    g = (torch.randn(B, t, d_out, device="cuda") * 0.05).bfloat16()
    return a, g


def test_lm_head_ghost_norm_at_vocabulary_width():
    a, g = _operands(2)
    got, _ = ops.linear_norm_sq(a, g, True, False, g_scale=2.0)
    want = torch.empty(2, device="cuda", dtype=torch.float64)
    for b in range(2):
        aa = a[b].float() @ a[b].float().t()
        gg = g[b].float() @ g[b].float().t()
        want[b] = 4.0 * (aa.double() * gg.double()).sum()
    assert _rel(got, want) < 2e-3, (got, want)
    ops._cuda.check_status()


def test_lm_head_ghost_norm_accumulates_into_running_total():
    a, g = _operands(2, seed=1)
    alone, _ = ops.linear_norm_sq(a, g, True, False, g_scale=1.0)
    total = torch.full((2,), 5.0, device="cuda")
    ops.linear_norm_sq(a, g, True, False, 1.0, total=total)
    torch.testing.assert_close(total, alone + 5.0, rtol=1e-5, atol=0)
    ops._cuda.check_status()


def test_lm_head_clipped_sum_at_vocabulary_width():
    a, g = _operands(2, seed=2)
    c = torch.tensor([0.25, 0.9], device="cuda")
    got, _ = ops.linear_weighted_grad(a, g, c, g_scale=1.5, want_bias=False)
    want = (g.float() * (1.5 * c)[:, None, None]).reshape(-1, V).t() @ a.float().reshape(-1, D)
    assert got.shape == (V, D)
    assert _rel(got, want) < 6e-3
    # spot-check the last rows and columns (the partial tiles of a width that is not a multiple of 256)
    assert _rel(got[-70:], want[-70:]) < 6e-3 and _rel(got[:, -9:], want[:, -9:]) < 6e-3
    ops._cuda.check_status()


def test_mlp_clipped_sums_at_model_width():
    """The two MLP shapes of the 1B model at the benchmark's batch: 8 x 1024 tokens, 2048 <-> 8192."""
    for d_in, d_out in ((2048, 8192), (8192, 2048)):
        a, g = _operands(8, d_in=d_in, d_out=d_out, seed=3)
        c = torch.rand(8, device="cuda")
        got, _ = ops.linear_weighted_grad(a, g, c, g_scale=1.0, want_bias=False)
        want = (g.float() * c[:, None, None]).reshape(-1, d_out).t() @ a.float().reshape(-1, d_in)
        assert _rel(got, want) < 6e-3
        n2, _ = ops.linear_norm_sq(a, g, True, False, g_scale=1.0)
        ref = torch.stack([((a[b].float() @ a[b].float().t()).double()
                            * (g[b].float() @ g[b].float().t()).double()).sum() for b in range(8)])
        assert _rel(n2, ref) < 2e-3
    ops._cuda.check_status()


def test_tied_cross_term_at_vocabulary_width():
    from opacus_b200.ops import _cuda

    torch.manual_seed(4)
    B = 2
    ids = torch.randint(0, V, (B, T), device="cuda")
    ids[:, ::7] = ids[:, :1]                  # repeated tokens: the scatter side has collisions
    g_e = torch.randn(B, T, D, device="cuda").bfloat16()
    a_h = torch.randn(B, T, D, device="cuda").bfloat16()
    g_h = (torch.randn(B, T, V, device="cuda") * 0.05).bfloat16()
    got = _cuda.load().tied_cross_norm(ids, g_e, a_h, g_h, 2.0, None)
    want = torch.empty(B, device="cuda", dtype=torch.float64)
    for b in range(B):
        # <scatter(G_E by ids), G_H^T A_H> = sum_t  G_E[t] . (G_H[:, ids[t]]^T A_H)
        cols = g_h[b].float()[:, ids[b]]                  # [T, T]: column ids[t] of G_H for every t
        rows = cols.t() @ a_h[b].float()                  # [T, D]
        want[b] = 2.0 * (rows.double() * g_e[b].double()).sum()
    torch.testing.assert_close(got.double(), want, rtol=2e-2, atol=2e-2 * want.abs().max().item())
    _cuda.check_status()


@pytest.mark.parametrize("B,t", [(1, 1), (1, 77), (1, 129), (3, 1023), (2, 257)])
def test_tied_cross_term_one_sample_and_odd_lengths(B, t):
    from opacus_b200.ops import _cuda

    torch.manual_seed(5)
    d, v = 72, 1000
    ids = torch.randint(0, v, (B, t), device="cuda")
    g_e = torch.randn(B, t, d, device="cuda").bfloat16()
    a_h = torch.randn(B, t, d, device="cuda").bfloat16()
    g_h = (torch.randn(B, t, v, device="cuda") * 0.1).bfloat16()
    got = _cuda.load().tied_cross_norm(ids, g_e, a_h, g_h, 1.0, None)
    want = torch.empty(B, device="cuda")
    for b in range(B):
        ge = torch.zeros(v, d, device="cuda").index_add_(0, ids[b], g_e[b].float())
        want[b] = (ge * (g_h[b].float().t() @ a_h[b].float())).sum()
    torch.testing.assert_close(got, want, rtol=2e-2, atol=2e-2 * want.abs().max().item() + 1e-3)
    _cuda.check_status()


@pytest.mark.parametrize("B,H,W", [(1, 7, 7), (1, 32, 32), (2, 13, 29), (3, 1, 40), (1, 5, 3)])
def test_conv_kernel_one_sample_and_odd_sizes(B, H, W):
    from opacus_b200.ops import _cuda

    torch.manual_seed(6)
    conv = torch.nn.Conv2d(16, 24, 3, padding=1, bias=False).cuda().to(torch.bfloat16)
    x = torch.randn(B, 16, H, W, device="cuda", dtype=torch.bfloat16)
    g = torch.randn_like(conv(x))
    geom = _cuda.conv_geometry(conv, x, g)
    assert geom is not None
    w = conv.weight.detach().float().requires_grad_()
    ref = torch.stack([torch.autograd.grad(torch.nn.functional.conv2d(x[b:b + 1].float(), w, padding=1), w,
                                           g[b:b + 1].float())[0] for b in range(B)])
    gs = _cuda.conv_grad_sample(x, g, geom)
    assert gs.shape == ref.shape
    assert (gs.float() - ref).abs().max() <= 1e-2 * ref.abs().max()
    nref = ref.flatten(1).square().sum(1)
    torch.testing.assert_close(_cuda.conv_grad_sample(x, g, geom, want_out=False), nref, rtol=2e-3, atol=0)
    coef = torch.rand(B, device="cuda")
    ws = _cuda.conv_weighted_grad(x, g, coef, geom, g_scale=1.0)
    wref = (ref * coef[:, None, None, None, None]).sum(0)
    assert (ws.float() - wref).abs().max() <= 1e-2 * wref.abs().max()
    _cuda.check_status()


def test_embedding_ghost_norm_at_vocabulary_width():
    torch.manual_seed(7)
    B = 4
    ids = torch.randint(0, V, (B, T), device="cuda")
    ids[:, 1::5] = ids[:, :1]
    g = (torch.randn(B, T, D, device="cuda") * 0.1).bfloat16()
    got = ops.embedding_norm_sq(ids, g, g_scale=1.0)
    same = (ids[:, :, None] == ids[:, None, :]).double()
    gg = torch.bmm(g.float(), g.float().transpose(1, 2)).double()
    want = (same * gg).sum(dim=(1, 2))
    assert _rel(got, want) < 2e-3
    ops._cuda.check_status()
