"""Golden values for the accountants (``opacus/tests/accountants_test.py:94-234``)."""
import warnings

import pytest

from opacus_b200.accountants import GaussianAccountant, PRVAccountant, RDPAccountant, create_accountant, register_accountant
from opacus_b200.accountants.utils import get_noise_multiplier


def _run(acc, steps, sigma=1.5, q=0.04):
    for _ in range(steps):
        acc.step(noise_multiplier=sigma, sample_rate=q)
    return acc


def test_rdp_golden():
    eps = _run(RDPAccountant(), int(90 / 0.04)).get_epsilon(delta=1e-5)
    assert eps == pytest.approx(7.32911117143, abs=1e-7)


def test_gdp_golden():
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        acc = GaussianAccountant()
    eps = _run(acc, int(90 // 0.04)).get_epsilon(delta=1e-5)
    assert 6.59 < eps < 6.6


def test_prv_golden():
    eps = _run(PRVAccountant(), int(90 // 0.04)).get_epsilon(delta=1e-5)
    assert eps == pytest.approx(6.777395712150674, abs=1e-6)


@pytest.mark.parametrize("kw,acc,want", [
    (dict(epochs=90), "rdp", 1.416), (dict(steps=2000), "rdp", 1.3562),
    (dict(epochs=90), "prv", 1.34765625), (dict(steps=2000), "prv", 1.2915),
    (dict(epochs=90), "gdp", 1.3232421875),
])
def test_get_noise_multiplier(kw, acc, want):
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        sigma = get_noise_multiplier(target_epsilon=8, target_delta=1e-5, sample_rate=0.04, accountant=acc, **kw)
    assert sigma == pytest.approx(want, abs=1e-3)


def test_noise_multiplier_never_overshoots():
    for eps in (0.5, 2.0, 11.0):
        sigma = get_noise_multiplier(target_epsilon=eps, target_delta=1e-5, sample_rate=0.01, steps=500)
        acc = RDPAccountant()
        acc.history = [(sigma, 0.01, 500)]
        assert acc.get_epsilon(1e-5) <= eps


def test_history_run_length_and_state_dict():
    acc = RDPAccountant()
    _run(acc, 3, 1.0, 0.1)
    _run(acc, 2, 1.1, 0.1)
    assert acc.history == [(1.0, 0.1, 3), (1.1, 0.1, 2)] and len(acc) == 2
    sd = acc.state_dict()
    assert sd["mechanism"] == "rdp"
    other = RDPAccountant()
    other.load_state_dict(sd)
    assert other.history == acc.history and other.get_epsilon(1e-5) == acc.get_epsilon(1e-5)
    with pytest.raises(ValueError):
        PRVAccountant().load_state_dict(sd)
    with pytest.raises(ValueError):
        RDPAccountant().load_state_dict({})


def test_gdp_requires_constant_parameters():
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        acc = GaussianAccountant()
    acc.step(noise_multiplier=1.0, sample_rate=0.1)
    with pytest.raises(ValueError):
        acc.step(noise_multiplier=2.0, sample_rate=0.1)


def test_registry():
    class Dummy(RDPAccountant):
        @classmethod
        def mechanism(cls):
            return "dummy"

    register_accountant("dummy", Dummy)
    assert isinstance(create_accountant("dummy"), Dummy)
    with pytest.raises(ValueError):
        register_accountant("dummy", Dummy)
    register_accountant("dummy", Dummy, force=True)
    with pytest.raises(ValueError):
        create_accountant("nope")
    from opacus_b200.accountants import registry

    del registry._ACCOUNTANTS["dummy"]


def test_cli(capsys):
    from opacus_b200.scripts.compute_dp_sgd_privacy import main

    main(["-r", "0.04", "-n", "1.5", "-e", "90", "-d", "1e-5"])
    out = capsys.readouterr().out
    assert "7.3" in out
