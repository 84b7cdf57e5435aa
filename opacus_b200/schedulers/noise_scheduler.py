"""Schedules for ``optimizer.noise_multiplier``, with the calling convention of
torch LR schedulers (``opacus/schedulers/noise_scheduler.py:20-177``)."""
from typing import Callable

from ._base import _Exponential, _Lambda, _OptimizerAttrScheduler, _Step


class _NoiseScheduler(_OptimizerAttrScheduler):
    attr = "noise_multiplier"
    family = "NoiseSchedulers"

    def get_noise_multiplier(self):
        return self._next_value()


class ExponentialNoise(_Exponential, _NoiseScheduler):
    pass


class LambdaNoise(_Lambda, _NoiseScheduler):
    _fn_name = "noise_lambda"
    _base_name = "base_noise_multiplier"

    def __init__(self, optimizer, *, noise_lambda: Callable[[int], float], last_epoch: int = -1):
        super().__init__(optimizer, noise_lambda, last_epoch=last_epoch)


class StepNoise(_Step, _NoiseScheduler):
    pass
