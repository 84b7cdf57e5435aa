"""Per-layer per-sample gradients against the micro-batch oracle (one
batch-of-one backward pass per sample), for hooks and functorch modes and both
loss reductions; plus ghost norms and clipped sums against the same oracle."""
import pytest
import torch
import torch.nn as nn
from torch.nn.utils.rnn import pack_padded_sequence

from opacus_b200.grad_sample import GradSampleModule, GradSampleModuleFastGradientClipping
from opacus_b200.layers import DPGRU, DPLSTM, DPRNN, DPMultiheadAttention, SequenceBias
from opacus_b200.utils.per_sample_gradients_utils import (
    check_per_sample_gradients_are_correct,
    compute_grad_samples_microbatch_and_opacus,
)

torch.manual_seed(0)


class _First(nn.Module):
    def __init__(self, m):
        super().__init__()
        self.m = m

    def forward(self, *a):
        out = self.m(*a)
        if isinstance(out, tuple) and not isinstance(out, torch.nn.utils.rnn.PackedSequence):
            return out[0]
        return out


CASES = [
    ("linear2d", lambda: nn.Linear(7, 5), lambda: torch.randn(6, 7), True),
    ("linear3d", lambda: nn.Linear(7, 5, bias=False), lambda: torch.randn(4, 9, 7), True),
    ("linear4d", lambda: nn.Linear(3, 4), lambda: torch.randn(3, 2, 5, 3), True),
    ("conv1d", lambda: nn.Conv1d(4, 6, 3, stride=2, padding=1), lambda: torch.randn(5, 4, 11), True),
    ("conv1d_same", lambda: nn.Conv1d(4, 4, 4, padding="same", dilation=2, groups=2), lambda: torch.randn(3, 4, 13), True),
    ("conv2d", lambda: nn.Conv2d(3, 8, (3, 2), stride=(1, 2), padding=(1, 0), dilation=(2, 1)), lambda: torch.randn(4, 3, 9, 8), True),
    ("conv2d_groups", lambda: nn.Conv2d(6, 9, 3, groups=3, bias=False), lambda: torch.randn(3, 6, 7, 7), True),
    ("conv3d", lambda: nn.Conv3d(2, 4, (2, 3, 2), stride=(1, 2, 1), padding=1), lambda: torch.randn(3, 2, 5, 6, 5), True),
    ("layernorm", lambda: nn.LayerNorm(12), lambda: torch.randn(5, 7, 12), True),
    ("layernorm2", lambda: nn.LayerNorm([7, 12]), lambda: torch.randn(5, 3, 7, 12), True),
    ("rmsnorm", lambda: nn.RMSNorm(12, eps=1e-5), lambda: torch.randn(5, 7, 12), True),
    ("groupnorm", lambda: nn.GroupNorm(2, 6), lambda: torch.randn(4, 6, 5, 3), True),
    ("instancenorm", lambda: nn.InstanceNorm2d(5, affine=True), lambda: torch.randn(4, 5, 6, 3), True),
    ("embedding", lambda: nn.Embedding(11, 6), lambda: torch.randint(0, 11, (5, 8)), True),
    ("seqbias", lambda: SequenceBias(6, batch_first=True), lambda: torch.randn(4, 5, 6), True),
    ("lstm", lambda: _First(DPLSTM(5, 6, num_layers=2, bidirectional=True, batch_first=True)), lambda: torch.randn(4, 7, 5), True),
    ("gru_tf", lambda: _First(DPGRU(5, 6, batch_first=False)), lambda: torch.randn(7, 4, 5), False),
    ("rnn", lambda: _First(DPRNN(5, 6, batch_first=True, nonlinearity="relu")), lambda: torch.randn(4, 7, 5), True),
]


@pytest.mark.parametrize("name,make,inp,batch_first", CASES, ids=[c[0] for c in CASES])
@pytest.mark.parametrize("mode", ["hooks", "functorch"])
def test_per_sample_grads(name, make, inp, batch_first, mode):
    if mode == "functorch" and name in ("embedding",):
        pass
    torch.manual_seed(1)
    assert check_per_sample_gradients_are_correct(inp(), make(), batch_first=batch_first, atol=1e-4, rtol=1e-3,
                                                  grad_sample_mode=mode)


class _SelfAttention(nn.Module):
    def __init__(self):
        super().__init__()
        self.att = DPMultiheadAttention(8, 2, add_bias_kv=True, batch_first=True)

    def forward(self, x):
        return self.att(x, x, x)[0]


def test_mha_per_sample_grads():
    assert check_per_sample_gradients_are_correct(torch.randn(3, 5, 8), _SelfAttention(), atol=1e-4, rtol=1e-3)


def test_packed_sequence_lstm():
    torch.manual_seed(2)
    x = pack_padded_sequence(torch.randn(4, 6, 5), [6, 4, 3, 1], batch_first=True)
    micro, ours = compute_grad_samples_microbatch_and_opacus(x, _First(DPLSTM(5, 4, batch_first=True)), batch_first=True)
    for k in micro:
        assert torch.allclose(micro[k], ours[k], atol=1e-4, rtol=1e-3), k


def test_embedding_bag():
    torch.manual_seed(3)
    for mode in ("sum", "mean"):
        import copy

        bag = nn.EmbeddingBag(13, 5, mode=mode)
        plain = copy.deepcopy(bag)
        idx = torch.randint(0, 13, (17,))
        off = torch.tensor([0, 3, 4, 9, 12])
        want = []
        for b in range(5):
            plain.zero_grad()
            end = off[b + 1] if b < 4 else 17
            plain(idx[off[b]:end], torch.tensor([0])).sum().backward()
            want.append(plain.weight.grad.clone())
        gsm = GradSampleModule(bag, loss_reduction="sum")
        gsm(idx, off).sum().backward()
        assert torch.allclose(bag.weight.grad_sample, torch.stack(want), atol=1e-5)
        gsm.to_standard_module()


def test_empty_batch_runs():
    for layer, x in [(nn.Linear(4, 3), torch.randn(0, 5, 4)), (nn.Conv2d(2, 3, 3), torch.randn(0, 2, 6, 6)),
                     (nn.Embedding(5, 3), torch.zeros(0, 4, dtype=torch.long)), (nn.GroupNorm(1, 2), torch.randn(0, 2, 3))]:
        gsm = GradSampleModule(layer)
        gsm(x).sum().backward()
        for p in layer.parameters():
            assert p.grad_sample.shape[0] == 0 or p.grad_sample.abs().sum() == 0


class _Net(nn.Module):
    """Embedding -> Linear -> LayerNorm -> Conv1d -> Linear, with a custom layer in the middle."""

    def __init__(self, tied=False):
        super().__init__()
        self.emb = nn.Embedding(20, 8)
        self.fc1 = nn.Linear(8, 8)
        self.ln = nn.LayerNorm(8)
        self.conv = nn.Conv1d(8, 8, 3, padding=1)
        self.rms = nn.RMSNorm(8, eps=1e-5)
        self.out = nn.Linear(8, 20, bias=False)
        if tied:
            self.out.weight = self.emb.weight

    def forward(self, ids):
        x = self.ln(torch.tanh(self.fc1(self.emb(ids))))
        x = x + self.conv(x.transpose(1, 2)).transpose(1, 2)
        return self.out(self.rms(x))


def _oracle(model, ids, y, C, token_mean=True):
    """Per-sample norms and clipped gradient sum by brute force."""
    crit = nn.CrossEntropyLoss(reduction="sum")
    params = [p for p in model.parameters()]
    grads, norms = [], []
    for i in range(ids.shape[0]):
        model.zero_grad()
        crit(model(ids[i:i + 1]).flatten(0, 1), y[i:i + 1].flatten()).div(ids.shape[1] if token_mean else 1).backward()
        g = [p.grad.detach().clone() for p in params]
        grads.append(g)
        norms.append(torch.sqrt(sum(t.pow(2).sum() for t in g)))
    norms = torch.stack(norms)
    coef = (C / (norms + 1e-6)).clamp(max=1.0)
    summed = [sum(coef[i] * grads[i][k] for i in range(len(grads))) for k in range(len(params))]
    return norms, summed


@pytest.mark.parametrize("tied", [False, True])
@pytest.mark.parametrize("single_pass", [True, False])
@pytest.mark.parametrize("reduction", ["mean", "sum"])
def test_ghost_matches_oracle(tied, single_pass, reduction):
    if tied and not single_pass:
        pytest.skip("two-pass ghost clipping rejects tied parameters (as the reference does)")
    from opacus_b200.optimizers import DPOptimizerFastGradientClipping
    from opacus_b200.utils.fast_gradient_clipping_utils import DPLossFastGradientClipping

    torch.manual_seed(4)
    model = _Net(tied)
    ids = torch.randint(0, 20, (5, 7))
    y = torch.randint(0, 20, (5, 7))
    C = 0.7
    norms, summed = _oracle(model, ids, y, C, token_mean=reduction == "mean")
    model.zero_grad()
    gsm = GradSampleModuleFastGradientClipping(model, max_grad_norm=C, loss_reduction=reduction, single_pass=single_pass)
    opt = DPOptimizerFastGradientClipping(torch.optim.SGD(model.parameters(), lr=0.0), noise_multiplier=0.0,
                                          max_grad_norm=C, expected_batch_size=5, loss_reduction=reduction)
    crit = DPLossFastGradientClipping(gsm, opt, nn.CrossEntropyLoss(reduction=reduction), reduction)
    loss = crit(gsm(ids).flatten(0, 1), y.flatten(), shape=(5, 7))
    loss.backward()
    assert torch.allclose(gsm.per_sample_gradient_norms, norms, rtol=1e-4, atol=1e-5)
    for p, want in zip(model.parameters(), summed):
        assert torch.allclose(p.grad, want, rtol=1e-3, atol=1e-5)
    gsm.to_standard_module()
    for p in model.parameters():
        assert not hasattr(p, "grad_sample") and not hasattr(p, "_forward_counter")


def test_hooks_controller_and_state_dict_prefix():
    from opacus_b200.grad_sample import GradSampleHooks

    m = nn.Sequential(nn.Linear(3, 4), nn.ReLU(), nn.Linear(4, 2))
    ctl = GradSampleHooks(m)
    m(torch.randn(5, 3)).sum().backward()
    assert m[0].weight.grad_sample.shape == (5, 4, 3)
    with pytest.raises(ValueError):
        GradSampleHooks(m)
    ctl.cleanup()
    assert not hasattr(m[0].weight, "grad_sample")
    w = GradSampleModule(m)
    assert all(k.startswith("_module.") for k in w.state_dict())
    assert w.to_standard_module() is m


def test_accumulation_list_and_poisson_guard():
    m = GradSampleModule(nn.Linear(3, 2))
    for _ in range(2):
        m(torch.randn(4, 3)).sum().backward()
    assert isinstance(m._module.weight.grad_sample, list) and len(m._module.weight.grad_sample) == 2
    m.zero_grad()
    assert m._module.weight.grad_sample is None
    m.forbid_grad_accumulation()
    m(torch.randn(4, 3)).sum().backward()
    with pytest.raises(ValueError):
        m(torch.randn(4, 3)).sum().backward()


def test_clip_factor_propagates_nan_on_cpu():
    from opacus_b200 import ops

    c = ops.clip_factor(torch.tensor([4.0, float("nan"), 0.0]), 1.0)
    assert torch.isnan(c[1]) and abs(float(c[0]) - 0.5) < 1e-5 and float(c[2]) == 1.0


def test_embedding_per_sample_gradient_stays_compact_through_a_dp_step():
    """Hooks mode on an embedding: ``p.grad_sample`` has the dense shape but holds (ids, G); clipping and the
    weighted sum run on the compact pair, the step equals the one computed from dense per-sample gradients, and
    reading the tensor any other way yields the dense values."""
    from opacus_b200 import ops
    from opacus_b200.grad_sample import GradSampleModule
    from opacus_b200.ops import _ref
    from opacus_b200.ops.lazy import LazyEmbeddingGradSample
    from opacus_b200.optimizers import DPOptimizer

    torch.manual_seed(0)
    emb = nn.Embedding(300, 16)
    model = GradSampleModule(nn.Sequential(emb, nn.Flatten(), nn.Linear(16 * 7, 3)))
    opt = DPOptimizer(torch.optim.SGD(model.parameters(), lr=1.0), noise_multiplier=0.0, max_grad_norm=0.1,
                      expected_batch_size=5)
    ids = torch.randint(0, 300, (5, 7))
    y = torch.randint(0, 3, (5,))
    before = emb.weight.detach().clone()
    nn.functional.cross_entropy(model(ids), y).backward()
    gs = emb.weight.grad_sample
    assert isinstance(gs, LazyEmbeddingGradSample) and gs.shape == (5, 300, 16) and not gs.is_materialized
    dense = _ref.embedding_grad_sample(gs._ids, gs._g, 300)
    others = [p.grad_sample.reshape(5, -1) for p in model.parameters() if p is not emb.weight]
    norms = torch.cat([dense.reshape(5, -1)] + others, dim=1).norm(dim=1)
    want = before - (dense * (0.1 / (norms + 1e-6)).clamp(max=1.0)[:, None, None]).sum(0) / 5
    opt.step()
    assert not gs.is_materialized
    assert torch.allclose(emb.weight, want, atol=1e-6)
    assert torch.allclose(gs * 1.0, dense) and gs.is_materialized
    assert torch.allclose(ops.grad_sample_norm_sq(gs), dense.pow(2).sum((1, 2)), rtol=1e-5)


def test_buffers_rejected():
    with pytest.raises(NotImplementedError):
        GradSampleModule(nn.BatchNorm1d(3))


def test_hooks_mode_without_autograd_weight_gradients():
    """skip_param_grads: same per-sample gradients, no batch gradient computed by autograd (first layer included)."""
    from opacus_b200.grad_sample import GradSampleModule

    torch.manual_seed(0)
    def make():
        torch.manual_seed(0)
        return nn.Sequential(nn.Conv2d(3, 4, 3, padding=1), nn.GroupNorm(2, 4), nn.ReLU(), nn.Flatten(),
                             nn.Linear(4 * 6 * 6, 5))
    x = torch.randn(7, 3, 6, 6)
    y = torch.randint(0, 5, (7,))
    a, b = GradSampleModule(make()), GradSampleModule(make(), skip_param_grads=True)
    for m in (a, b):
        nn.functional.cross_entropy(m(x), y).backward()
    for (n1, p1), (n2, p2) in zip(a.named_parameters(), b.named_parameters()):
        assert p2.grad is None and p1.grad is not None, n1
        torch.testing.assert_close(p1.grad_sample, p2.grad_sample)
    # a second pass accumulates nothing stale and evaluation mode passes through
    b.zero_grad()
    nn.functional.cross_entropy(b(x), y).backward()
    for (_, p1), (_, p2) in zip(a.named_parameters(), b.named_parameters()):
        torch.testing.assert_close(p1.grad_sample, p2.grad_sample)
    b.eval()
    assert b(x).shape == (7, 5)


def test_dense_axis_order_of_permuted_views():
    """The clip-weighted sum of a permuted dense view (the channels-last conv gradient) is taken in storage order."""
    from opacus_b200.ops._cuda import _dense_order

    base = torch.randn(5, 4, 3, 2, 6)                  # [B, O, kh, kw, C]
    view = base.permute(0, 1, 4, 2, 3)                 # [B, O, C, kh, kw]
    order = _dense_order(view)
    assert order == [0, 1, 3, 4, 2] and view.permute(order).is_contiguous()
    assert _dense_order(base) is None                  # already contiguous
    assert _dense_order(base[:, :, :, :, ::2]) is None  # strided, not a permutation of a dense buffer
    # the result mapped back to logical axes equals the plain weighted sum
    c = torch.rand(5)
    phys = view.permute(order)
    out = (phys * c.view(-1, 1, 1, 1, 1)).sum(0)
    inv = [0] * 4
    for pos, d in enumerate(order[1:]):
        inv[d - 1] = pos
    torch.testing.assert_close(out.permute(inv), (view * c.view(-1, 1, 1, 1, 1)).sum(0))


class _AddNormNet(torch.nn.Module):
    """Two residual additions, each inside the RMSNorm that follows it (or as separate statements)."""

    def __init__(self, fused):
        super().__init__()
        from opacus_b200.layers.add_rms_norm import AddRMSNorm

        cls = AddRMSNorm if fused else torch.nn.RMSNorm
        self.fused = fused
        self.a, self.n1, self.b, self.n2 = torch.nn.Linear(12, 12), cls(12, eps=1e-5), torch.nn.Linear(12, 12), cls(12, eps=1e-5)
        self.head = torch.nn.Linear(12, 3)

    def forward(self, x):
        if self.fused:
            y, h = self.n1(x)
            y, h = self.n2(h, self.a(y))
            return self.head(h + self.b(y)).mean(1)
        h = x
        h = h + self.a(self.n1(h))
        return self.head(h + self.b(self.n2(h))).mean(1)


@pytest.mark.parametrize("mode", ["hooks", "ghost", "ghost_single_pass"])
def test_add_rms_norm_matches_separate_statements(mode):
    from opacus_b200 import GradSampleModule
    from opacus_b200.grad_sample import GradSampleModuleFastGradientClipping

    torch.manual_seed(3)
    plain, fused = _AddNormNet(False), _AddNormNet(True)
    for p in plain.parameters():
        p.data.uniform_(-0.7, 0.7)
    fused.load_state_dict(plain.state_dict())
    x, y = torch.randn(5, 7, 12), torch.randint(0, 3, (5,))
    if mode == "hooks":
        got, want = GradSampleModule(fused), GradSampleModule(plain)
        for m in (got, want):
            torch.nn.functional.cross_entropy(m(x), y).backward()
        for (n, p), q in zip(got.named_parameters(), want.parameters()):
            assert torch.allclose(p.grad_sample, q.grad_sample, atol=1e-6), n
    else:
        norms = []
        for net in (fused, plain):
            m = GradSampleModuleFastGradientClipping(net, max_grad_norm=0.1, use_ghost_clipping=True,
                                                     single_pass=mode == "ghost_single_pass")
            loss = torch.nn.functional.cross_entropy(m(x), y, reduction="none").mean()
            loss.backward()
            norms.append(m.get_norm_sample().clone())
        assert torch.allclose(norms[0], norms[1], atol=1e-6)


def test_llama_matches_plain_definition():
    """The decoder with fused add+norm modules computes what the plain definition computes from the same state dict."""
    import dataclasses
    import os
    import sys

    sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline"))
    from llama_plain import Llama as PlainLlama, LlamaConfig as PlainConfig

    from opacus_b200.models.llama import Llama, LlamaConfig

    cfg = LlamaConfig(vocab_size=97, d_model=64, n_layers=3, n_heads=4, n_kv_heads=2, ffn_dim=128)
    torch.manual_seed(0)
    ours = Llama(cfg)
    for n, p in ours.named_parameters():
        if "norm" in n:
            p.data.uniform_(0.5, 1.5)
    plain = PlainLlama(PlainConfig(**{f.name: getattr(cfg, f.name) for f in dataclasses.fields(PlainConfig)}))
    plain.load_state_dict(ours.state_dict())
    ids = torch.randint(0, 97, (2, 11))
    a, b = ours(ids), plain(ids)
    assert torch.allclose(a, b, atol=1e-6)
    a.square().sum().backward()
    b.square().sum().backward()
    for (n, p), q in zip(ours.named_parameters(), plain.parameters()):
        assert torch.allclose(p.grad, q.grad, atol=1e-5), n


@pytest.mark.parametrize("cfg", [
    dict(k=3, s=1, p=1, d=1, groups=1, size=(5, 6, 7)),
    dict(k=(2, 3, 3), s=(2, 2, 1), p=(1, 0, 2), d=1, groups=1, size=(7, 9, 8)),
    dict(k=(3, 2, 3), s=(1, 3, 2), p=(2, 1, 1), d=(2, 1, 1), groups=2, size=(6, 8, 9)),
    dict(k=(2, 4, 3), s=1, p="same", d=1, groups=1, size=(4, 6, 5)),
    dict(k=(1, 3, 3), s=(1, 2, 2), p="valid", d=1, groups=1, size=(3, 7, 7)),
])
def test_conv3d_as_depth_stacked_conv2d(cfg):
    """The 2-d problems that carry a Conv3d onto the implicit-unfold kernel have exactly its weight gradient."""
    from opacus_b200.grad_sample.conv import depth_stacked_pairs

    torch.manual_seed(0)
    B, C, O = 3, 4, 6
    conv = torch.nn.Conv3d(C, O, cfg["k"], stride=cfg["s"], padding=cfg["p"], dilation=cfg["d"], groups=cfg["groups"],
                           bias=False).double()
    x = torch.randn(B, C, *cfg["size"], dtype=torch.float64)
    y = conv(x)
    g = torch.randn_like(y)
    for b in range(B):
        (want,) = torch.autograd.grad(conv(x[b:b + 1]), conv.weight, g[b:b + 1])
        for a, x2, g2 in depth_stacked_pairs(conv, x[b:b + 1], g[b:b + 1]):
            shape2 = (O, C // cfg["groups"]) + tuple(conv.kernel_size[1:])
            got = torch.nn.grad.conv2d_weight(x2, shape2, g2.contiguous(), stride=conv.stride[1:], padding=0,
                                              dilation=conv.dilation[1:], groups=cfg["groups"])
            torch.testing.assert_close(got, want[:, :, a], rtol=1e-10, atol=1e-10)
