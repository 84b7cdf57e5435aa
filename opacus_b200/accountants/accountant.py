"""Accountant interface.

An accountant keeps ``history``: a list of ``(noise_multiplier, sample_rate,
num_steps)`` runs of the sampled Gaussian mechanism, and converts it to an
``epsilon`` at a given ``delta``.  The checkpoint form is
``{"history": [...], "mechanism": name}``.

Behavioural parity: ``opacus/accountants/accountant.py:26-134``.
"""
from __future__ import annotations

import abc
import copy
from collections import OrderedDict
from typing import Any, Callable, List, Mapping, Optional, Tuple

Run = Tuple[float, float, int]


def push_run(history: List[Run], noise_multiplier: float, sample_rate: float) -> None:
    """Append one step to a run-length encoded history (extends the last run
    when both parameters are unchanged)."""
    if history:
        sigma, q, n = history[-1]
        if sigma == noise_multiplier and q == sample_rate:
            history[-1] = (sigma, q, n + 1)
            return
    history.append((noise_multiplier, sample_rate, 1))


class IAccountant(abc.ABC):
    @abc.abstractmethod
    def __init__(self):
        self.history: List[Run] = []

    @abc.abstractmethod
    def step(self, *, noise_multiplier: float, sample_rate: float):
        """Record one optimisation step."""

    @abc.abstractmethod
    def get_epsilon(self, delta: float, *args, **kwargs) -> float:
        """Privacy budget spent so far at ``delta``."""

    @abc.abstractmethod
    def __len__(self) -> int:
        """Number of recorded runs."""

    @classmethod
    @abc.abstractmethod
    def mechanism(cls) -> str:
        """Short name used in checkpoints and the registry."""

    def get_optimizer_hook_fn(self, sample_rate: float) -> Callable[[Any], None]:
        """Callback for ``DPOptimizer.attach_step_hook``.

        The effective rate of a logical step that accumulated ``k`` physical
        batches is ``k * sample_rate``; the same rate holds per rank in
        data-parallel runs because every rank samples from its own slice.
        """

        def _on_step(optim) -> None:
            self.step(
                noise_multiplier=optim.noise_multiplier,
                sample_rate=sample_rate * optim.accumulated_iterations,
            )

        return _on_step

    def state_dict(self, destination: Optional[Mapping[str, Any]] = None):
        out = OrderedDict() if destination is None else destination
        out["history"] = copy.deepcopy(self.history)
        out["mechanism"] = self.mechanism()
        return out

    def load_state_dict(self, state_dict: Mapping[str, Any]):
        if not state_dict:
            raise ValueError(
                "state dict is either None or empty and hence cannot be loaded"
                " into Privacy Accountant."
            )
        for key in ("history", "mechanism"):
            if key not in state_dict:
                raise ValueError(
                    f"state_dict does not have the key `{key}`."
                    " Cannot be loaded into Privacy Accountant."
                )
        if state_dict["mechanism"] != self.mechanism():
            raise ValueError(
                f"state_dict of {state_dict['mechanism']} cannot be loaded into "
                f" Privacy Accountant with mechanism {self.mechanism()}"
            )
        self.history = state_dict["history"]
