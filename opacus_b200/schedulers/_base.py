"""One implementation for both scheduler families: a scheduler owns the name
of a float attribute of the DP optimizer and rewrites it on every ``step()``."""
from typing import Callable, Dict


class _OptimizerAttrScheduler:
    attr: str = ""          # optimizer attribute that is scheduled
    family: str = ""        # used in the error message

    def __init__(self, optimizer, *, last_epoch=-1):
        if not hasattr(optimizer, self.attr):
            raise ValueError(
                f"{self.family} require your optimizer to have a .{self.attr} attr. "
                "Are you sure you are using a DPOptimizer? Those have it added for you."
            )
        self.optimizer = optimizer
        self.last_epoch = last_epoch
        self.step()

    # -- value access -------------------------------------------------------
    @property
    def _current(self) -> float:
        return getattr(self.optimizer, self.attr)

    def _next_value(self) -> float:
        raise NotImplementedError

    def step(self):
        self.last_epoch += 1
        setattr(self.optimizer, self.attr, self._next_value())

    # -- checkpointing: everything but the optimizer reference ---------------
    def state_dict(self) -> Dict:
        return {k: v for k, v in self.__dict__.items() if k != "optimizer"}

    def load_state_dict(self, state_dict: Dict):
        self.__dict__.update(state_dict)


class _Exponential(_OptimizerAttrScheduler):
    """Multiply by ``gamma`` every epoch (not on the construction step)."""

    def __init__(self, optimizer, *, gamma: float, last_epoch: int = -1):
        self.gamma = gamma
        super().__init__(optimizer, last_epoch=last_epoch)

    def _next_value(self):
        return self._current if self.last_epoch == 0 else self._current * self.gamma


class _Lambda(_OptimizerAttrScheduler):
    """``base * fn(epoch)`` with ``base`` the value at construction."""

    _fn_name = "fn"
    _base_name = "base"

    def __init__(self, optimizer, fn: Callable[[int], float], last_epoch: int = -1):
        setattr(self, self._fn_name, fn)
        setattr(self, self._base_name, getattr(optimizer, self.attr))
        super().__init__(optimizer, last_epoch=last_epoch)

    def _next_value(self):
        return getattr(self, self._base_name) * getattr(self, self._fn_name)(self.last_epoch)


class _Step(_OptimizerAttrScheduler):
    """Multiply by ``gamma`` every ``step_size`` epochs."""

    def __init__(self, optimizer, *, step_size: int, gamma: float, last_epoch: int = -1):
        self.step_size = step_size
        self.gamma = gamma
        super().__init__(optimizer, last_epoch=last_epoch)

    def _next_value(self):
        if self.last_epoch == 0 or self.last_epoch % self.step_size:
            return self._current
        return self.gamma * self._current
