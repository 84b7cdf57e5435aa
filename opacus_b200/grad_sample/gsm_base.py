"""Common base of the per-sample-gradient controllers.

Two flavours share every class in this package: a *controller* (``...Hooks``)
that instruments a model in place and leaves the user's module object as it is,
and a *wrapper* (``...Module``) that is itself an ``nn.Module`` holding the model
as ``_module`` (so ``state_dict`` keys gain the ``_module.`` prefix).

Behavioural parity: ``opacus/grad_sample/gsm_base.py:27-221``.
"""
import logging
from abc import ABC, abstractmethod
from typing import Optional

import torch.nn as nn
from torch.utils.hooks import RemovableHandle

from ..utils.module_utils import trainable_parameters

logger = logging.getLogger(__name__)

# Attributes this package attaches to ``nn.Parameter`` objects.
OPACUS_PARAM_MONKEYPATCH_ATTRS = ["grad_sample", "_forward_counter", "_current_grad_sample", "_norm_sample"]


class AbstractGradSampleHooks(ABC):
    def __init__(self, m: nn.Module, *, batch_first=True, loss_reduction="mean"):
        super().__init__()
        self._module = m
        self.batch_first = batch_first
        self.loss_reduction = loss_reduction
        for _, p in trainable_parameters(m):
            p.grad_sample = None
            p._forward_counter = 0

    def set_grad_sample_to_none(self):
        for p in self._module.parameters():
            p.grad_sample = None

    def del_grad_sample(self):
        for p in self._module.parameters():
            del p.grad_sample

    def forbid_grad_accumulation(self):
        pass

    def allow_grad_accumulation(self):
        pass

    @abstractmethod
    def remove_hooks(self) -> None:
        ...

    def cleanup(self):
        """Remove instrumentation and every attribute added to parameters."""
        try:
            self.remove_hooks()
        except Exception as e:  # still strip the attributes below
            logger.warning(f"Failed to remove hooks during cleanup: {e}. Attempting to clean up attributes anyway.")
        finally:
            for p in self._module.parameters():
                for attr in OPACUS_PARAM_MONKEYPATCH_ATTRS:
                    if hasattr(p, attr):
                        delattr(p, attr)


class AbstractGradSampleModule(nn.Module, AbstractGradSampleHooks, ABC):
    def __init__(self, m: nn.Module, *, batch_first=True, loss_reduction="mean"):
        nn.Module.__init__(self)
        AbstractGradSampleHooks.__init__(self, m, batch_first=batch_first, loss_reduction=loss_reduction)
        self.grad_accumulation_hook: Optional[RemovableHandle] = None

    def forward(self, *args, **kwargs):
        return self._module(*args, **kwargs)

    def __getattr__(self, item):
        """Fall through to submodules of the wrapped model by (dotted) name."""
        try:
            return super().__getattr__(item)
        except AttributeError:
            if item and item != "_module" and "_module" in self.__dict__.get("_modules", {}):
                for name, sub in self._modules["_module"].named_modules():
                    if name == item:
                        return sub
            raise

    def zero_grad(self, set_to_none: bool = False):
        """``grad_sample`` is always reset to ``None`` (zero-filling it would
        count as one accumulated batch)."""
        self.set_grad_sample_to_none()
        super().zero_grad(set_to_none)

    def to_standard_module(self) -> nn.Module:
        """Strip all instrumentation and hand back the user's module."""
        self._close()
        return self._module

    def _close(self):
        self.cleanup()

    def __repr__(self):
        return f"{type(self).__name__}({self._module.__repr__()})"
