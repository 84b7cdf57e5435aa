"""Phase markers of a DP training step: NVTX ranges and an optional per-step record.

``OPACUS_B200_NVTX=1`` in the environment turns every phase into an NVTX range (visible in Nsight Systems);
without it the markers cost one attribute lookup.  Independently, a :class:`StepRecorder` collects, for the code
run inside its ``with`` block, the device time of every phase (CUDA events on the current stream; wall clock on
CPU) and the clipping statistics of the ghost-clipping controller::

    with StepRecorder() as rec:
        loss = criterion(model(x), y); loss.backward(); optimizer.step()
    print(rec.summary())
    # {'phases_ms': {'dp/backward': ..., 'dp/norm': ..., 'dp/clipped_sum': ..., 'dp/optimizer_step': ...},
    #  'calls': {...}, 'clip_fraction': 0.93, 'norm_mean': 4.1, 'norm_max': 9.7, 'batch': 8}

The reference has no tracing of its own (its benchmarks time whole layers with ``torch.utils.benchmark``,
``benchmarks/benchmark_layer.py:72-77``).
"""
from __future__ import annotations

import os
import time
from contextlib import contextmanager
from typing import Dict, List, Optional

import torch

NVTX = os.environ.get("OPACUS_B200_NVTX", "0") not in ("", "0")
_active: Optional["StepRecorder"] = None


@contextmanager
def phase(name: str):
    rec = _active
    if rec is None and not NVTX:
        yield
        return
    nvtx = NVTX and torch.cuda.is_available()
    if nvtx:
        torch.cuda.nvtx.range_push(name)
    token = rec._begin() if rec is not None else None
    try:
        yield
    finally:
        if rec is not None:
            rec._end(name, token)
        if nvtx:
            torch.cuda.nvtx.range_pop()


def record_clipping(norms: torch.Tensor, max_grad_norm: float) -> None:
    """Called by the clipping controller with the per-sample norms of the batch (kept on the device)."""
    if _active is not None:
        _active._norms.append((norms.detach(), float(max_grad_norm)))


class StepRecorder:
    def __init__(self):
        self._cuda = torch.cuda.is_available()
        self._spans: List[tuple] = []
        self._norms: List[tuple] = []
        self._prev = None

    def __enter__(self):
        global _active
        self._prev, _active = _active, self
        return self

    def __exit__(self, *exc):
        global _active
        _active = self._prev
        return False

    def _begin(self):
        if self._cuda:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            return e
        return time.perf_counter()

    def _end(self, name, token):
        if self._cuda:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            self._spans.append((name, token, e))
        else:
            self._spans.append((name, token, time.perf_counter()))

    def summary(self) -> Dict:
        """Synchronises the device once and returns the record (nested phases are each counted in full)."""
        if self._cuda:
            torch.cuda.synchronize()
        ms: Dict[str, float] = {}
        calls: Dict[str, int] = {}
        for name, a, b in self._spans:
            dt = a.elapsed_time(b) if self._cuda else (b - a) * 1e3
            ms[name] = ms.get(name, 0.0) + dt
            calls[name] = calls.get(name, 0) + 1
        out = {"phases_ms": ms, "calls": calls}
        if self._norms:
            norms, c = self._norms[-1]
            n = norms.float()
            out.update(clip_fraction=float((n > c).float().mean()), norm_mean=float(n.mean()), norm_max=float(n.max()),
                       batch=int(n.numel()))
        return out
