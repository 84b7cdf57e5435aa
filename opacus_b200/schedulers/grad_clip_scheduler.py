"""Schedules for ``optimizer.max_grad_norm``
(``opacus/schedulers/grad_clip_scheduler.py:20-174``)."""
from typing import Callable

from ._base import _Exponential, _Lambda, _OptimizerAttrScheduler, _Step


class _GradClipScheduler(_OptimizerAttrScheduler):
    attr = "max_grad_norm"
    family = "GradClipSchedulers"

    def get_max_grad_norm(self):
        return self._next_value()


class ExponentialGradClip(_Exponential, _GradClipScheduler):
    pass


class LambdaGradClip(_Lambda, _GradClipScheduler):
    _fn_name = "scheduler_function"
    _base_name = "base_max_grad_norm"

    def __init__(self, optimizer, *, scheduler_function: Callable[[int], float], last_epoch: int = -1):
        super().__init__(optimizer, scheduler_function, last_epoch=last_epoch)


class StepGradClip(_Step, _GradClipScheduler):
    pass
