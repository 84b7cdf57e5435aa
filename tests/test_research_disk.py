"""DiSK (Kalman-filtered DP optimizers): the filter recursion against a plain restatement."""
import copy
import math

import pytest
import torch
import torch.nn as nn
from torch.utils.data import DataLoader, TensorDataset

from opacus_b200.grad_sample import GradSampleModule
from opacus_b200.research.disk_optimizer import KF_DPOptimizer, KF_PrivacyEngine, get_optimizer_class


def _setup():
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(5, 4), nn.Tanh(), nn.Linear(4, 2))
    x = torch.randn(6, 5)
    y = torch.randint(0, 2, (6,))
    return model, x, y


def _clipped_mean_grad(model, x, y, C):
    """Per-sample clipped, averaged gradient at the model's current parameters (micro-batch oracle)."""
    params = list(model.parameters())
    total = [torch.zeros_like(p) for p in params]
    for i in range(len(x)):
        gs = torch.autograd.grad(nn.functional.cross_entropy(model(x[i:i + 1]), y[i:i + 1]), params)
        norm = math.sqrt(sum(float(g.pow(2).sum()) for g in gs))
        f = min(1.0, C / (norm + 1e-6))
        for t, g in zip(total, gs):
            t.add_(g, alpha=f)
    return [t / len(x) for t in total]


@pytest.mark.parametrize("kappa,gamma", [(0.7, 0.0), (0.7, 0.5)])
def test_kalman_filter_recursion(kappa, gamma):
    model, x, y = _setup()
    ref = copy.deepcopy(model)
    gsm = GradSampleModule(model)
    lr, C = 0.3, 0.8
    opt = KF_DPOptimizer(torch.optim.SGD(model.parameters(), lr=lr), noise_multiplier=0.0, max_grad_norm=C,
                         expected_batch_size=6, kappa=kappa, gamma=gamma)

    def closure():
        opt.zero_grad()
        loss = nn.functional.cross_entropy(gsm(x), y)
        loss.backward()
        return loss

    natural = (1 - kappa) / kappa
    one = gamma == 0 or abs(gamma - natural) < 1e-3
    g_eff = natural if one else gamma
    c = 1.0 if one else (1 - kappa) / (gamma * kappa)
    m = d = None
    rparams = list(ref.parameters())
    for step in range(4):
        opt.step(closure)
        # ---- restatement
        if d is None:
            obs = _clipped_mean_grad(ref, x, y, C)
        elif one:
            with torch.no_grad():
                for p, dd in zip(rparams, d):
                    p.add_(dd, alpha=g_eff)
            obs = _clipped_mean_grad(ref, x, y, C)
            with torch.no_grad():
                for p, dd in zip(rparams, d):
                    p.sub_(dd, alpha=g_eff)
        else:
            # clipping acts on the mixed per-sample gradient
            params = rparams
            total = [torch.zeros_like(p) for p in params]
            for i in range(len(x)):
                g0 = torch.autograd.grad(nn.functional.cross_entropy(ref(x[i:i + 1]), y[i:i + 1]), params)
                with torch.no_grad():
                    for p, dd in zip(params, d):
                        p.add_(dd, alpha=g_eff)
                g1 = torch.autograd.grad(nn.functional.cross_entropy(ref(x[i:i + 1]), y[i:i + 1]), params)
                with torch.no_grad():
                    for p, dd in zip(params, d):
                        p.sub_(dd, alpha=g_eff)
                mix = [c * b + (1 - c) * a for a, b in zip(g0, g1)]
                norm = math.sqrt(sum(float(g.pow(2).sum()) for g in mix))
                f = min(1.0, C / (norm + 1e-6))
                for t, g in zip(total, mix):
                    t.add_(g, alpha=f)
            obs = [t / len(x) for t in total]
        m = [o.clone() for o in obs] if m is None else [kappa * mm + (1 - kappa) * o for mm, o in zip(m, obs)]
        with torch.no_grad():
            old = [p.clone() for p in rparams]
            for p, mm in zip(rparams, m):
                p.sub_(mm, alpha=lr)
            d = [p - o for p, o in zip(rparams, old)]
        for p, q in zip(model.parameters(), rparams):
            torch.testing.assert_close(p, q, rtol=1e-4, atol=1e-5)


def test_noise_rescaling_and_factory():
    model, _, _ = _setup()
    kappa, gamma = 0.7, 0.5
    c = (1 - kappa) / (gamma * kappa)
    opt = KF_DPOptimizer(torch.optim.SGD(model.parameters(), lr=0.1), noise_multiplier=1.0, max_grad_norm=1.0,
                         expected_batch_size=4, kappa=kappa, gamma=gamma)
    assert abs(opt.noise_multiplier - 1.0 / math.sqrt(c * c + (1 - c) ** 2)) < 1e-12
    assert get_optimizer_class("flat", False, "hooks", kalman=True) is KF_DPOptimizer
    assert get_optimizer_class("flat", False, "hooks", kalman=False).__name__ == "DPOptimizer"
    with pytest.raises(ValueError):
        opt.step()


def test_kf_privacy_engine_trains():
    model, x, y = _setup()
    dl = DataLoader(TensorDataset(x.repeat(4, 1), y.repeat(4)), batch_size=6)
    pe = KF_PrivacyEngine()
    inner = torch.optim.SGD(model.parameters(), lr=0.1)
    m, opt, dl = pe.make_private(module=model, optimizer=inner, data_loader=dl, noise_multiplier=0.5,
                                 max_grad_norm=1.0, kalman=True, kappa=0.7, gamma=0.5, poisson_sampling=False)
    assert isinstance(opt, KF_DPOptimizer)
    for xb, yb in dl:
        def closure():
            opt.zero_grad()
            loss = nn.functional.cross_entropy(m(xb), yb)
            loss.backward()
            return loss

        opt.step(closure)
    assert pe.get_epsilon(1e-5) > 0
