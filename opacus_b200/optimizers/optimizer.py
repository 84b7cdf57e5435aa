"""``DPOptimizer``: wraps any ``torch.optim.Optimizer`` and turns per-sample
gradients into one private gradient per step.

A logical step is: clip every sample's gradient to ``max_grad_norm`` and sum
(``clip_and_accumulate``) -> add ``N(0, (noise_multiplier * max_grad_norm)^2)``
(``add_noise``) -> divide by ``expected_batch_size * accumulated_iterations``
for mean-reduced losses (``scale_grad``) -> privacy-accountant hook -> wrapped
optimizer's ``step``.  With virtual batches (``signal_skip_step``) the
non-final physical batches stop after ``clip_and_accumulate``.

On CUDA the three passes over per-sample gradients that the textbook
formulation needs (norm, factor, weighted sum) run as this package's kernels,
and when the wrapped optimiser is plain SGD/Adam/AdamW the noise draw, scaling
and parameter update run as **one** Philox-fused multi-tensor kernel
(``fused_step``); ``p.grad`` still ends up holding the noised, scaled gradient.

Behavioural parity: ``opacus/optimizers/optimizer.py:32-581``.
"""
from __future__ import annotations

import logging
from collections import defaultdict
from typing import Callable, List, Optional, Union

import torch
from torch import nn
from torch.optim import Optimizer

from ..utils.tracing import phase

from .. import ops
from .utils import params

logger = logging.getLogger(__name__)
logger.disabled = True

_STALE = (
    "Gradients haven't been cleared since the last optimizer step. "
    "In order to obtain privacy guarantees you must call optimizer.zero_grad()"
    "on each step"
)


def _each_tensor(obj):
    if isinstance(obj, torch.Tensor):
        yield obj
    elif isinstance(obj, list):
        yield from obj


def _mark_as_processed(obj: Union[torch.Tensor, List[torch.Tensor]]):
    """Tag gradient tensors that already went into a private sum, so that using
    them a second time (forgotten ``zero_grad``) is detected."""
    for t in _each_tensor(obj):
        t._processed = True


def _check_processed_flag_tensor(x: torch.Tensor):
    if hasattr(x, "_processed"):
        raise ValueError(_STALE)


def _check_processed_flag(obj: Union[torch.Tensor, List[torch.Tensor]]):
    for t in _each_tensor(obj):
        _check_processed_flag_tensor(t)


def _generate_noise(std: float, reference: torch.Tensor, generator=None, secure_mode: bool = False) -> torch.Tensor:
    """Gaussian noise shaped like ``reference`` (zeros when ``std == 0``)."""
    return ops.gaussian_like(reference, std, generator=generator, secure_mode=secure_mode)


class DPOptimizer(Optimizer):
    # Subclasses whose noise/scale stages differ from the base in a way the
    # fused kernel does not express set this to False.
    _fused_ok = True

    def __init__(self, optimizer: Optimizer, *, noise_multiplier: float, max_grad_norm: float,
                 expected_batch_size: Optional[int], loss_reduction: str = "mean", generator=None,
                 secure_mode: bool = False, fused_step: Union[bool, str] = "auto", **kwargs):
        if loss_reduction not in ("mean", "sum"):
            raise ValueError(f"Unexpected value for loss_reduction: {loss_reduction}")
        if loss_reduction == "mean" and expected_batch_size is None:
            raise ValueError("You must provide expected batch size of the loss reduction is mean")
        self.original_optimizer = optimizer
        self.noise_multiplier = noise_multiplier
        self.max_grad_norm = max_grad_norm
        self.loss_reduction = loss_reduction
        self.expected_batch_size = expected_batch_size
        self.step_hook = None
        self.generator = generator
        self.secure_mode = secure_mode
        self.fused_step = fused_step
        self._step_skip_queue = []
        self._is_last_step_skipped = False
        for p in self.params:
            p.summed_grad = None

    # ------------------------------------------------------------- bookkeeping
    def _get_flat_grad_sample(self, p: torch.Tensor):
        """``p.grad_sample`` as one ``[B_total, *p.shape]`` tensor."""
        if not hasattr(p, "grad_sample"):
            raise ValueError("Per sample gradient not found. Are you using GradSampleModule?")
        gs = p.grad_sample
        if gs is None:
            raise ValueError("Per sample gradient is not initialized. Not updated in backward pass?")
        if isinstance(gs, torch.Tensor):
            return gs
        if isinstance(gs, list):
            return torch.cat(gs, dim=0)
        raise ValueError(f"Unexpected grad_sample type: {type(gs)}")

    def signal_skip_step(self, do_skip=True):
        """Queue whether the next ``step()`` only accumulates (virtual batches)."""
        self._step_skip_queue.append(do_skip)

    def _check_skip_next_step(self, pop_next=True):
        if not self._step_skip_queue:
            return False
        return self._step_skip_queue.pop(0) if pop_next else self._step_skip_queue[0]

    @property
    def params(self) -> List[nn.Parameter]:
        return params(self)

    @property
    def grad_samples(self) -> List[torch.Tensor]:
        return [self._get_flat_grad_sample(p) for p in self.params]

    @property
    def accumulated_iterations(self) -> int:
        """How many batches were accumulated in ``grad_sample`` since ``zero_grad``."""
        counts = set()
        for p in self.params:
            if not hasattr(p, "grad_sample"):
                raise ValueError("Per sample gradient not found. Are you using GradSampleModule?")
            gs = p.grad_sample
            if isinstance(gs, torch.Tensor):
                counts.add(1)
            elif isinstance(gs, list):
                counts.add(len(gs))
            else:
                raise ValueError(f"Unexpected grad_sample type: {type(gs)}")
        if len(counts) > 1:
            raise ValueError("Number of accumulated steps is inconsistent across parameters")
        return counts.pop()

    # The wrapped optimiser owns groups, state and defaults.
    @property
    def param_groups(self) -> List[dict]:
        return self.original_optimizer.param_groups

    @param_groups.setter
    def param_groups(self, v: List[dict]):
        self.original_optimizer.param_groups = v

    @property
    def state(self) -> defaultdict:
        return self.original_optimizer.state

    @state.setter
    def state(self, v: defaultdict):
        self.original_optimizer.state = v

    @property
    def defaults(self) -> dict:
        return self.original_optimizer.defaults

    @defaults.setter
    def defaults(self, v: dict):
        self.original_optimizer.defaults = v

    def attach_step_hook(self, fn: Callable[["DPOptimizer"], None]):
        """``fn(self)`` runs once per *logical* step, right before the wrapped
        optimiser's update (the privacy accountant uses it)."""
        self.step_hook = fn

    # ------------------------------------------------------------------ stages
    def _per_sample_clip_factor(self) -> torch.Tensor:
        gss = self.grad_samples
        if len(gss[0]) == 0:
            return torch.zeros((0,), device=gss[0].device)
        dev = gss[0].device
        total = None
        for gs in gss:
            n2 = ops.grad_sample_norm_sq(gs).to(dev)
            total = n2 if total is None else total + n2
        return ops.clip_factor(total, float(self.max_grad_norm))

    def _accumulate_clipped(self, p, grad_sample, factor):
        gs = grad_sample if grad_sample.dtype == p.dtype else grad_sample.to(p.dtype)
        grad = ops.weighted_sum(gs, factor.to(gs.device))
        if p.summed_grad is not None:
            p.summed_grad += grad
        else:
            p.summed_grad = grad

    def clip_and_accumulate(self):
        """``summed_grad += sum_n min(1, C/||g_n||) g_n`` with the norm taken
        over all parameters of sample ``n``."""
        factor = self._per_sample_clip_factor()
        for p in self.params:
            _check_processed_flag(p.grad_sample)
            self._accumulate_clipped(p, self._get_flat_grad_sample(p), factor)
            _mark_as_processed(p.grad_sample)

    def _noise_std(self) -> float:
        return self.noise_multiplier * self.max_grad_norm

    def add_noise(self):
        std = self._noise_std()
        for p in self.params:
            _check_processed_flag(p.summed_grad)
            noise = _generate_noise(std=std, reference=p.summed_grad, generator=self.generator,
                                    secure_mode=self.secure_mode)
            p.grad = (p.summed_grad + noise).view_as(p)
            _mark_as_processed(p.summed_grad)

    def _grad_denominator(self) -> float:
        if self.loss_reduction == "mean":
            return float(self.expected_batch_size * self.accumulated_iterations)
        return 1.0

    def scale_grad(self):
        if self.loss_reduction == "mean":
            d = self._grad_denominator()
            for p in self.params:
                p.grad /= d

    def zero_grad(self, set_to_none: bool = False):
        """Clears ``grad_sample`` always, and ``summed_grad`` unless the last
        ``step()`` was a skipped (accumulate-only) one."""
        for p in self.params:
            p.grad_sample = None
            if not self._is_last_step_skipped:
                p.summed_grad = None
        self.original_optimizer.zero_grad(set_to_none)

    # ------------------------------------------------------------------- step
    def _collect(self) -> bool:
        """Stage 1 of a step.  Returns False when there is nothing to do."""
        gss = self.grad_samples
        if gss is None or len(gss) == 0:
            return False
        self.clip_and_accumulate()
        return True

    def pre_step(self, closure: Optional[Callable[[], float]] = None) -> Optional[float]:
        """Everything up to (excluding) the wrapped optimiser's update.
        Returns True if that update should run."""
        if not self._collect():
            return True
        if self._check_skip_next_step():
            self._is_last_step_skipped = True
            return False
        self.add_noise()
        self.scale_grad()
        if self.step_hook:
            self.step_hook(self)
        self._is_last_step_skipped = False
        return True

    def _fused_plan(self):
        """A fused noise+scale+update plan when the configuration allows it."""
        if self.fused_step is False or self.secure_mode or not self._fused_ok:
            return None
        from .fused import plan_for

        return plan_for(self)

    def step(self, closure: Optional[Callable[[], float]] = None) -> Optional[float]:
        with phase("dp/optimizer_step"):
            return self._step(closure)

    def _step(self, closure: Optional[Callable[[], float]] = None) -> Optional[float]:
        if closure is not None:
            with torch.enable_grad():
                closure()
        plan = self._fused_plan()
        if plan is None:
            if self.pre_step():
                return self.original_optimizer.step()
            return None
        # fused path: same stages, last three in one kernel
        if self._collect():
            if self._check_skip_next_step():
                self._is_last_step_skipped = True
                return None
            for p in self.params:
                _check_processed_flag(p.summed_grad)
            if self.step_hook:
                self.step_hook(self)
            plan.run(self, noise_std=self._noise_std(), denominator=self._grad_denominator())
            for p in self.params:
                _mark_as_processed(p.summed_grad)
            self._is_last_step_skipped = False
            return None
        return self.original_optimizer.step()

    def __repr__(self):
        return self.original_optimizer.__repr__()

    def state_dict(self):
        """Exactly the wrapped optimiser's state (checkpoint compatible with it).  Under a sharded engine the
        state lives on the engine, 1/world per rank; it is gathered into the same layout (a collective call)."""
        engine = getattr(self, "engine", None)
        if engine is not None and hasattr(engine, "optimizer_state_dict"):
            return engine.optimizer_state_dict(self.original_optimizer)
        return self.original_optimizer.state_dict()

    def load_state_dict(self, state_dict) -> None:
        engine = getattr(self, "engine", None)
        if engine is not None and hasattr(engine, "load_optimizer_state_dict"):
            return engine.load_optimizer_state_dict(self.original_optimizer, state_dict)
        self.original_optimizer.load_state_dict(state_dict)
