"""End-to-end behaviour of PrivacyEngine / DPOptimizer on CPU
(model of ``opacus/tests/privacy_engine_test.py``)."""
import io
import os
import math

import pytest
import torch
import torch.nn as nn
from torch.utils.data import DataLoader, TensorDataset

from opacus_b200 import PrivacyEngine
from opacus_b200.optimizers import DPOptimizer
from opacus_b200.schedulers import ExponentialNoise, StepGradClip
from opacus_b200.utils.batch_memory_manager import BatchMemoryManager
from opacus_b200.validators import ModuleValidator


class ConvNet(nn.Module):
    def __init__(self):
        super().__init__()
        self.conv = nn.Conv2d(1, 4, 3, padding=1)
        self.gn = nn.GroupNorm(2, 4)
        self.fc = nn.Linear(4 * 8 * 8, 5)

    def forward(self, x):
        return self.fc(torch.relu(self.gn(self.conv(x))).flatten(1))


def _data(n=64, bs=16):
    g = torch.Generator().manual_seed(0)
    ds = TensorDataset(torch.randn(n, 1, 8, 8, generator=g), torch.randint(0, 5, (n,), generator=g))
    return ds, DataLoader(ds, batch_size=bs)


def _private(mode="hooks", sigma=1.0, C=1.0, poisson=False, opt_cls=torch.optim.SGD, accountant="rdp", **kw):
    torch.manual_seed(7)
    model = ConvNet()
    opt = opt_cls(model.parameters(), lr=0.1)
    ds, dl = _data()
    pe = PrivacyEngine(accountant=accountant)
    out = pe.make_private(module=model, optimizer=opt, data_loader=dl, noise_multiplier=sigma, max_grad_norm=C,
                          grad_sample_mode=mode, poisson_sampling=poisson, **kw)
    return pe, model, out


def _train(out, steps=3):
    if len(out) == 4:
        m, opt, crit, dl = out
    else:
        m, opt, dl = out
        crit = nn.CrossEntropyLoss()
    it = iter(dl)
    for _ in range(steps):
        x, y = next(it)
        opt.zero_grad()
        crit(m(x), y).backward()
        opt.step()
    return m, opt


@pytest.mark.parametrize("mode", ["hooks", "functorch", "ew", "ghost"])
def test_no_noise_no_clip_equals_plain_sgd(mode):
    pe, model, out = _private(mode, sigma=0.0, C=1e20)
    _train(out, 3)
    torch.manual_seed(7)
    ref = ConvNet()
    opt = torch.optim.SGD(ref.parameters(), lr=0.1)
    _, dl = _data()
    it = iter(dl)
    for _ in range(3):
        x, y = next(it)
        opt.zero_grad()
        nn.functional.cross_entropy(ref(x), y).backward()
        opt.step()
    for a, b in zip(model.parameters(), ref.parameters()):
        assert torch.allclose(a, b, atol=1e-6), mode


@pytest.mark.parametrize("mode", ["hooks", "ghost"])
def test_modes_agree_with_clipping(mode):
    _, base, out0 = _private("functorch", sigma=0.0, C=0.1)
    _train(out0, 2)
    _, model, out = _private(mode, sigma=0.0, C=0.1)
    _train(out, 2)
    for a, b in zip(model.parameters(), base.parameters()):
        assert torch.allclose(a, b, atol=1e-6)


def test_flat_clipping_bounds_the_sum():
    pe, model, (m, opt, dl) = _private("hooks", sigma=0.0, C=0.05)
    x, y = next(iter(dl))
    opt.zero_grad()
    nn.functional.cross_entropy(m(x), y).backward()
    opt.clip_and_accumulate()
    total = math.sqrt(sum(p.summed_grad.pow(2).sum().item() for p in model.parameters()))
    assert total <= 0.05 * len(x) + 1e-5


def test_per_layer_clipping():
    n = len(list(ConvNet().parameters()))
    pe, model, (m, opt, dl) = _private("hooks", sigma=0.0, C=[0.01] * n, clipping="per_layer")
    x, y = next(iter(dl))
    opt.zero_grad()
    nn.functional.cross_entropy(m(x), y).backward()
    opt.clip_and_accumulate()
    for p in model.parameters():
        assert p.summed_grad.norm().item() <= 0.01 * len(x) + 1e-6
    assert opt.max_grad_norm == pytest.approx(0.01 * math.sqrt(n))


def test_adaptive_clipping_moves_bound():
    pe, model, (m, opt, dl) = _private(
        "hooks", sigma=0.5, C=10.0, clipping="adaptive", target_unclipped_quantile=0.1,
        clipbound_learning_rate=0.5, max_clipbound=100.0, min_clipbound=0.01, unclipped_num_std=1.0)
    before = float(opt.max_grad_norm)
    _train((m, opt, dl), 2)
    assert float(opt.max_grad_norm) < before


def test_noise_level():
    """With zero gradients the parameters perform a random walk of known variance."""
    torch.manual_seed(0)
    model = nn.Linear(200, 50, bias=False)
    nn.init.zeros_(model.weight)
    opt = torch.optim.SGD(model.parameters(), lr=0.5)
    ds = TensorDataset(torch.zeros(40, 200), torch.zeros(40, 50))
    pe = PrivacyEngine(accountant="rdp")
    m, dpo, dl = pe.make_private(module=model, optimizer=opt, data_loader=DataLoader(ds, batch_size=8),
                                 noise_multiplier=1.3, max_grad_norm=2.0, poisson_sampling=False)
    steps = 0
    for x, y in dl:
        dpo.zero_grad()
        (m(x) - y).pow(2).mean().backward()
        dpo.step()
        steps += 1
    var = model.weight.detach().var().item()
    want = steps * (1.3 * 2.0 * 0.5 / 8) ** 2
    assert abs(var - want) / want < 0.1


def test_poisson_sampling_and_accounting():
    pe, model, (m, opt, dl) = _private("hooks", poisson=True)
    sizes = []
    for x, y in dl:
        sizes.append(len(x))
        opt.zero_grad()
        if len(x):
            nn.functional.cross_entropy(m(x), y).backward()
            opt.step()
    assert len(set(sizes)) > 1 and len(sizes) == 4
    assert pe.get_epsilon(1e-5) > 0
    assert pe.accountant.history[0][1] == pytest.approx(0.25)


def test_make_private_with_epsilon_hits_target():
    torch.manual_seed(0)
    model = ConvNet()
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    ds, dl = _data(256, 16)
    pe = PrivacyEngine(accountant="rdp")
    m, o, dl2 = pe.make_private_with_epsilon(module=model, optimizer=opt, data_loader=dl, target_epsilon=4.0,
                                             target_delta=1e-5, epochs=2, max_grad_norm=1.0, poisson_sampling=False)
    for _ in range(2):
        for x, y in dl2:
            o.zero_grad()
            nn.functional.cross_entropy(m(x), y).backward()
            o.step()
    eps = pe.get_epsilon(1e-5)
    assert eps <= 4.0 and eps > 3.5


def test_virtual_batches_update_only_at_logical_boundaries():
    pe, model, (m, opt, dl) = _private("hooks", sigma=0.0, C=1e20)
    snaps = []
    with BatchMemoryManager(data_loader=dl, max_physical_batch_size=4, optimizer=opt) as small:
        for x, y in small:
            assert len(x) <= 4
            opt.zero_grad()
            nn.functional.cross_entropy(m(x), y).backward()
            opt.step()
            snaps.append(model.fc.weight.detach().clone())
    changes = [not torch.equal(a, b) for a, b in zip(snaps[:-1], snaps[1:])]
    assert len(snaps) == 16 and sum(changes) == 4 and all(changes[i] for i in (2, 6, 10, 14))
    # and the result equals training on the logical batches directly
    _, ref, out = _private("hooks", sigma=0.0, C=1e20)
    _train(out, 4)
    for a, b in zip(model.parameters(), ref.parameters()):
        assert torch.allclose(a, b, atol=1e-6)


def test_virtual_batches_ghost():
    pe, model, (m, opt, crit, dl) = _private("ghost", sigma=0.0, C=0.3)
    with BatchMemoryManager(data_loader=dl, max_physical_batch_size=4, optimizer=opt) as small:
        for x, y in small:
            opt.zero_grad()
            crit(m(x), y).backward()
            opt.step()
    _, ref, out = _private("hooks", sigma=0.0, C=0.3)
    _train(out, 4)
    for a, b in zip(model.parameters(), ref.parameters()):
        assert torch.allclose(a, b, atol=1e-6)


def test_forgotten_zero_grad_is_detected():
    pe, model, (m, opt, dl) = _private("hooks")
    x, y = next(iter(dl))
    nn.functional.cross_entropy(m(x), y).backward()
    opt.step()
    with pytest.raises(ValueError):
        opt.step()


def test_checkpoint_round_trip():
    pe, model, (m, opt, dl) = _private("hooks", opt_cls=torch.optim.Adam)
    ns = ExponentialNoise(opt, gamma=0.9)
    gs = StepGradClip(opt, step_size=1, gamma=0.5)
    _train((m, opt, dl), 2)
    ns.step()
    gs.step()
    buf = io.BytesIO()
    pe.save_checkpoint(path=buf, module=m, optimizer=opt, noise_scheduler=ns, grad_clip_scheduler=gs,
                       checkpoint_dict={"epoch": 3})
    buf.seek(0)
    raw = torch.load(io.BytesIO(buf.getvalue()), weights_only=False)
    assert set(raw) >= {"module_state_dict", "privacy_accountant_state_dict", "optimizer_state_dict",
                        "noise_scheduler_state_dict", "grad_clip_scheduler_state_dict", "epoch"}
    assert all(k.startswith("_module.") for k in raw["module_state_dict"])
    assert raw["privacy_accountant_state_dict"]["mechanism"] == "rdp"

    pe2, model2, (m2, opt2, dl2) = _private("hooks", opt_cls=torch.optim.Adam, sigma=2.0, C=3.0)
    ns2 = ExponentialNoise(opt2, gamma=0.1)
    gs2 = StepGradClip(opt2, step_size=5, gamma=0.1)
    rest = pe2.load_checkpoint(path=buf, module=m2, optimizer=opt2, noise_scheduler=ns2, grad_clip_scheduler=gs2)
    assert rest["epoch"] == 3
    assert pe2.accountant.history == pe.accountant.history
    for a, b in zip(model.parameters(), model2.parameters()):
        assert torch.equal(a, b)
    assert ns2.gamma == 0.9 and gs2.step_size == 1
    # noise_multiplier / max_grad_norm are not part of the checkpoint
    assert opt2.noise_multiplier != opt.noise_multiplier


def test_validation_and_fix():
    bad = nn.Sequential(nn.Conv2d(1, 4, 3), nn.BatchNorm2d(4), nn.Flatten(), nn.LSTM(4, 4))
    assert not ModuleValidator.is_valid(bad)
    fixed = ModuleValidator.fix(bad)
    assert ModuleValidator.is_valid(fixed)
    assert isinstance(fixed[1], nn.GroupNorm) and type(fixed[3]).__name__ == "DPLSTM"
    pe = PrivacyEngine(accountant="rdp")
    with pytest.raises(Exception):
        pe.validate(module=bad, optimizer=None, data_loader=None)
    with pytest.raises(ValueError):
        other = nn.Linear(2, 2)
        pe.make_private(module=nn.Linear(2, 2), optimizer=torch.optim.SGD(other.parameters(), lr=0.1),
                        data_loader=_data()[1], noise_multiplier=1.0, max_grad_norm=1.0)


def test_seeded_runs_are_identical():
    results = []
    for _ in range(2):
        g = torch.Generator().manual_seed(123)
        pe, model, out = _private("hooks", noise_generator=g)
        _train(out, 2)
        results.append([p.detach().clone() for p in model.parameters()])
    for a, b in zip(*results):
        assert torch.equal(a, b)


def test_schedulers():
    pe, model, (m, opt, dl) = _private("hooks", sigma=2.0, C=4.0)
    ns = ExponentialNoise(opt, gamma=0.5)
    assert opt.noise_multiplier == 2.0
    ns.step()
    assert opt.noise_multiplier == 1.0
    gc = StepGradClip(opt, step_size=2, gamma=0.5)
    gc.step()
    assert opt.max_grad_norm == 4.0
    gc.step()
    assert opt.max_grad_norm == 2.0
    sd = gc.state_dict()
    assert "optimizer" not in sd and sd["step_size"] == 2


def test_dp_optimizer_is_transparent_to_state_dict():
    pe, model, (m, opt, dl) = _private("hooks", opt_cls=torch.optim.Adam)
    _train((m, opt, dl), 1)
    assert isinstance(opt, DPOptimizer)
    assert opt.state_dict().keys() == opt.original_optimizer.state_dict().keys()


# ------------------------------------------------------------------ checkpoint interchange with the reference library
_REF = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref")

_INTERCHANGE_SCRIPT = r"""
import sys, torch, torch.nn as nn
from torch.utils.data import DataLoader, TensorDataset
lib, action, path = sys.argv[1], sys.argv[2], sys.argv[3]
if lib == "reference":
    sys.path.insert(0, sys.argv[4])
    from opacus import PrivacyEngine
else:
    from opacus_b200 import PrivacyEngine
torch.manual_seed(0)
model = nn.Sequential(nn.Linear(6, 5), nn.ReLU(), nn.Linear(5, 3))
opt = torch.optim.Adam(model.parameters(), lr=0.01)
g = torch.Generator().manual_seed(1)
ds = TensorDataset(torch.randn(32, 6, generator=g), torch.randint(0, 3, (32,), generator=g))
pe = PrivacyEngine(accountant="rdp")
m, o, dl = pe.make_private(module=model, optimizer=opt, data_loader=DataLoader(ds, batch_size=8),
                           noise_multiplier=1.1, max_grad_norm=1.0, poisson_sampling=False)
if action == "save":
    for x, y in dl:
        o.zero_grad(); nn.functional.cross_entropy(m(x), y).backward(); o.step()
    pe.save_checkpoint(path=path, module=m, optimizer=o, checkpoint_dict={"epoch": 7})
    print("EPS", pe.get_epsilon(1e-5), "W", float(m._module[0].weight.sum()))
else:
    rest = pe.load_checkpoint(path=path, module=m, optimizer=o)
    st = o.state_dict()["state"]
    print("EPS", pe.get_epsilon(1e-5), "W", float(m._module[0].weight.sum()), "EPOCH", rest["epoch"],
          "STEPS", int(st[0]["step"]) if len(st) else -1)
"""


def _interchange(lib, action, path):
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, PYTHONPATH=root + os.pathsep + os.environ.get("PYTHONPATH", ""), CUDA_VISIBLE_DEVICES="")
    res = subprocess.run([sys.executable, "-c", _INTERCHANGE_SCRIPT, lib, action, path, _REF], capture_output=True,
                         text=True, timeout=300, env=env)
    assert res.returncode == 0, res.stderr[-2000:]
    line = [ln for ln in res.stdout.splitlines() if ln.startswith("EPS")][-1].split()
    return {line[i]: float(line[i + 1]) for i in range(0, len(line), 2)}


@pytest.mark.skipif(not os.path.isdir(os.path.join(_REF, "opacus")), reason="reference library not installed")
@pytest.mark.parametrize("writer,reader", [("reference", "ours"), ("ours", "reference")])
def test_checkpoint_interchange_with_reference(tmp_path, writer, reader):
    """A checkpoint written by either library restores weights, optimizer state, the
    accountant history (same epsilon) and the user's entries in the other."""
    path = str(tmp_path / "ckpt.pt")
    saved = _interchange(writer, "save", path)
    loaded = _interchange(reader, "load", path)
    assert abs(saved["EPS"] - loaded["EPS"]) < 1e-9
    assert abs(saved["W"] - loaded["W"]) < 1e-6
    assert loaded["EPOCH"] == 7 and loaded["STEPS"] == 4


def test_step_recorder_collects_phases_and_clipping():
    from opacus_b200.utils.tracing import StepRecorder

    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(6, 5), nn.ReLU(), nn.Linear(5, 3))
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    ds = TensorDataset(torch.randn(16, 6), torch.randint(0, 3, (16,)))
    pe = PrivacyEngine()
    m, o, crit, dl = pe.make_private(module=model, optimizer=opt, criterion=nn.CrossEntropyLoss(),
                                     data_loader=DataLoader(ds, batch_size=8), noise_multiplier=1.0, max_grad_norm=0.01,
                                     grad_sample_mode="ghost", poisson_sampling=False)
    x, y = next(iter(dl))
    with StepRecorder() as rec:
        o.zero_grad()
        crit(m(x), y).backward()
        o.step()
    s = rec.summary()
    assert {"dp/backward", "dp/norm", "dp/clipped_sum", "dp/optimizer_step"} <= set(s["phases_ms"])
    assert s["calls"]["dp/norm"] == 2 and s["batch"] == 8
    assert s["clip_fraction"] == 1.0 and s["norm_max"] >= s["norm_mean"] > 0.01
    # outside the recorder the markers are inert
    o.zero_grad()
    crit(m(x), y).backward()
    o.step()
    assert rec.summary()["calls"]["dp/norm"] == 2
