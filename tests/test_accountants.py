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


# ---- invariants (property-based): what any privacy accountant must satisfy
from hypothesis import given, settings  # noqa: E402
from hypothesis import strategies as st  # noqa: E402


def _eps(kind, sigma, q, steps, delta=1e-5):
    from opacus_b200.accountants import create_accountant

    acc = create_accountant(kind)
    acc.history = [(sigma, q, steps)]
    return acc.get_epsilon(delta)


@settings(max_examples=25, deadline=None, derandomize=True)
@given(sigma=st.floats(0.6, 4.0), q=st.floats(0.001, 0.2), steps=st.integers(1, 2000))
def test_rdp_epsilon_grows_with_steps_and_rate_and_falls_with_noise(sigma, q, steps):
    base = _eps("rdp", sigma, q, steps)
    assert base >= 0
    assert _eps("rdp", sigma, q, steps * 2) >= base - 1e-9
    assert _eps("rdp", sigma * 1.5, q, steps) <= base + 1e-9
    assert _eps("rdp", sigma, min(1.0, q * 1.5), steps) >= base - 1e-9
    # a weaker delta can only make epsilon smaller
    assert _eps("rdp", sigma, q, steps, delta=1e-3) <= base + 1e-9


@settings(max_examples=10, deadline=None, derandomize=True)
@given(sigma=st.floats(0.8, 3.0), q=st.floats(0.005, 0.1), steps=st.integers(10, 1000))
def test_prv_is_not_looser_than_rdp_by_more_than_its_error_and_both_agree_roughly(sigma, q, steps):
    rdp, prv = _eps("rdp", sigma, q, steps), _eps("prv", sigma, q, steps)
    assert prv <= rdp * 1.02 + 0.05           # the numerical composition is the tighter analysis
    assert prv >= 0.3 * rdp - 0.05            # and not wildly different


@settings(max_examples=8, deadline=None, derandomize=True)
@given(eps=st.floats(0.5, 10.0), q=st.floats(0.005, 0.1), steps=st.integers(50, 2000))
def test_noise_multiplier_search_meets_its_target(eps, q, steps):
    from opacus_b200.accountants.utils import get_noise_multiplier

    sigma = get_noise_multiplier(target_epsilon=eps, target_delta=1e-5, sample_rate=q, steps=steps, accountant="rdp",
                                 epsilon_tolerance=0.01)
    got = _eps("rdp", sigma, q, steps)
    assert got <= eps + 1e-6 and got >= eps - 0.05 - 0.02 * eps
