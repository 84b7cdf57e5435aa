"""Stream ordering of the sharded engine's piece-wise step, checked on the CPU with stand-ins for the CUDA objects.

What is checked is the order in which ``ShardedDataParallel._optimizer_step`` queues work, not the kernels: state that is
created in a step must be zero-filled on the stream that runs the pieces (the main stream still holds the clipped-sum
GEMMs of the pass at that point), every piece waits for the events of the gradients it reads, the main stream joins the
side stream at the end, and the one-launch paths stay on the main stream.
"""
import contextlib
import types

import pytest
import torch
import torch.nn as nn


class _Stream:
    def __init__(self, device=None, name="side"):
        self.device, self.name, self.log = device, name, []

    def wait_event(self, ev):
        self.log.append(("wait_event", ev))

    def wait_stream(self, other):
        self.log.append(("wait_stream", other.name))


class _Buf:
    def __init__(self, n):
        self.tensor, self.ptrs, self.mc_ptr = torch.full((n,), 0.0), [0], 0


@pytest.fixture
def world(monkeypatch):
    import opacus_b200.ops as ops
    import opacus_b200.parallel.sharded as sh
    from opacus_b200.ops import _cuda

    trace = []                       # ("zeros" | "launch" | "enter" | "exit", current stream name, detail)
    current = ["main"]
    main = _Stream(name="main")

    @contextlib.contextmanager
    def stream_ctx(s):
        previous = current[0]
        current[0] = s.name
        trace.append(("enter", s.name, None))
        try:
            yield
        finally:
            current[0] = previous
            trace.append(("exit", s.name, None))

    real_zeros = torch.zeros

    def zeros(*a, **k):
        k.pop("device", None)
        trace.append(("zeros", current[0], a[0] if a else None))
        return real_zeros(*a, **k)

    class Kernels:
        def sharded_dp_step(self, *a):
            trace.append(("launch", current[0], (a[6], a[7])))          # (first element, count)

    monkeypatch.setattr(torch.cuda, "Stream", lambda device=None: _Stream(device))
    monkeypatch.setattr(torch.cuda, "stream", stream_ctx)
    monkeypatch.setattr(torch.cuda, "current_stream", lambda dev=None: main)
    monkeypatch.setattr(sh.torch, "zeros", zeros)
    monkeypatch.setattr(_cuda, "load", lambda: Kernels())
    monkeypatch.setattr(_cuda, "_rng_state", lambda gen, dev, n: (1, 2))
    monkeypatch.setattr(ops, "gaussian_like", lambda ref, std, generator=None, secure_mode=False: torch.zeros_like(ref))

    def build(optimizer="adamw", fresh=False):
        eng = sh.ShardedDataParallel.__new__(sh.ShardedDataParallel)
        nn.Module.__init__(eng)
        params = [nn.Parameter(torch.full((64,), 0.0)) for _ in range(4)]
        for i, p in enumerate(params):
            p._dp_grad_fresh = fresh
            p._dp_ready = (i % 2, i, f"written-{i}")
        eng._params = params
        eng._offsets = {p: i * 64 for i, p in enumerate(params)}
        eng.pieces, eng.world, eng.stripe, eng.piece_len, eng.rank = 4, 1, 64, 64, 0
        eng.total = eng.used = eng.slice_len = 256
        eng.master, eng.state0, eng.state1 = torch.full((256,), 0.0), None, None
        eng._steps, eng._step_stream, eng._epoch = 0, None, 0
        eng.tp_group, eng.tp_world, eng.tp_rank, eng._tp_seed, eng.noise_split = None, 1, 0, None, None
        eng._flat_grad, eng._flat_param, eng._flags = _Buf(256), _Buf(256), _Buf(4)
        eng.multicast, eng.multicast_reduce, eng.multicast_publish = False, True, True
        eng.param_dtype, eng._segments = torch.bfloat16, None
        eng.finish_grads = eng.mark_grads_fresh = eng._finish_row_layers = lambda: None
        inner = torch.optim.AdamW(params, lr=1e-3) if optimizer == "adamw" else torch.optim.SGD(params, lr=0.1, momentum=0.9)
        return eng, inner

    def dp_optimizer(inner, secure=False):
        return types.SimpleNamespace(original_optimizer=inner, _check_skip_next_step=lambda: False, loss_reduction="mean",
                                     _grad_denominator=lambda: 8, step_hook=None, _noise_std=lambda: 1.0, generator=None,
                                     secure_mode=secure, _is_last_step_skipped=False)

    return types.SimpleNamespace(build=build, dp_optimizer=dp_optimizer, trace=trace, main=main)


@pytest.mark.parametrize("optimizer,n_state", [("adamw", 2), ("sgd", 1)])
def test_new_state_is_zeroed_on_the_stream_of_the_pieces(world, optimizer, n_state):
    eng, inner = world.build(optimizer)
    eng._optimizer_step(world.dp_optimizer(inner))
    zeros = [t for t in world.trace if t[0] == "zeros" and t[2] == 256]
    launches = [t for t in world.trace if t[0] == "launch"]
    assert len(zeros) == n_state and all(t[1] == "side" for t in zeros)
    assert len(launches) == 4 and all(t[1] == "side" for t in launches)
    first_launch = world.trace.index(launches[0])
    assert all(world.trace.index(z) < first_launch for z in zeros)           # filled in front of the first piece
    side = eng._step_stream
    assert [e for e in side.log if e[0] == "wait_event"] == [("wait_event", f"written-{i}") for i in range(4)]
    assert ("wait_stream", "main") not in side.log                             # pieces do not wait for the GEMM stream
    assert world.main.log[-1] == ("wait_stream", "side")                       # the next pass sees the new weights
    assert sorted(t[2][0] for t in launches) == [0, 64, 128, 192] and eng.last_step_launches == 4
    world.trace.clear()
    eng._optimizer_step(world.dp_optimizer(inner))                             # later steps allocate nothing
    assert not [t for t in world.trace if t[0] == "zeros" and t[2] == 256]


def test_one_launch_paths_stay_on_the_main_stream(world):
    eng, inner = world.build(fresh=True)                 # a parameter without a gradient: zero-filled on the main stream
    eng._optimizer_step(world.dp_optimizer(inner))
    launches = [t for t in world.trace if t[0] == "launch"]
    assert len(launches) == 1 and launches[0][1] == "main" and launches[0][2] == (0, 256)
    assert all(t[1] == "main" for t in world.trace if t[0] == "zeros")
    assert eng._step_stream is None


def test_secure_mode_joins_the_side_stream_before_its_single_launch(world):
    eng, inner = world.build()
    eng._optimizer_step(world.dp_optimizer(inner, secure=True))
    launches = [t for t in world.trace if t[0] == "launch"]
    assert len(launches) == 1 and launches[0][1] == "main"
    assert ("wait_stream", "side") in world.main.log     # the state was zeroed on the side stream: main waits for it
