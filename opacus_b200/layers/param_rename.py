"""Expose a module's nested parameters under alternative flat names.

Used by the DP recurrent layers so that their ``state_dict`` has the key layout
of ``torch.nn.LSTM``/``GRU``/``RNN`` (``weight_ih_l0`` ...), while the parameters
physically live in child ``Linear`` modules (``l0.ih.weight`` ...).

Behavioural parity: ``opacus/layers/param_rename.py:33-139``.
"""
from typing import Dict

import torch.nn as nn
from torch.nn.modules.module import _IncompatibleKeys


class RenameParamsMixin:
    """Mix in *before* ``nn.Module``.  After :meth:`set_rename_map`, each
    parameter reachable as ``old`` is also registered on ``self`` as ``new``;
    ``state_dict()`` reports only the new names and ``load_state_dict`` accepts them."""

    def set_rename_map(self, rename_map: Dict[str, str]):
        self.old_to_new = dict(rename_map)
        self.new_to_old = {new: old for old, new in rename_map.items()}
        self._register_state_dict_hook(_drop_nested_names)
        self._alias_parameters()

    def _alias_parameters(self):
        mapping = self.__dict__.get("old_to_new")
        if not mapping:
            return
        own = self.__dict__.get("_parameters", {})
        for old, param in list(nn.Module.named_parameters(self)):
            new = mapping.get(old)
            if new is not None and own.get(new) is not param:
                self.register_parameter(new, param)

    def _register_renamed_parameters(self):  # name kept for API compatibility
        self._alias_parameters()

    def __setattr__(self, name, value) -> None:
        super().__setattr__(name, value)
        # A child module (or one of its parameters) may have been replaced.
        if isinstance(value, (nn.Module, nn.Parameter)):
            self._alias_parameters()

    def _apply(self, fn, *args, **kwargs):
        # ``.to()``/``.half()`` may swap Parameter objects; re-tie the aliases.
        out = super()._apply(fn, *args, **kwargs)
        self._alias_parameters()
        return out

    def load_state_dict(self, state_dict, strict: bool = True, **kwargs):
        missing, unexpected = super().load_state_dict(state_dict, strict=False, **kwargs)
        missing = [k for k in missing if k not in self.old_to_new]
        if strict:
            problems = []
            if missing:
                problems.append("Missing key(s) in state_dict: {}. ".format(", ".join(f'"{k}"' for k in missing)))
            if unexpected:
                problems.append("Unexpected key(s) in state_dict: {}. ".format(", ".join(f'"{k}"' for k in unexpected)))
            if problems:
                raise RuntimeError(
                    "Error(s) in loading state_dict for {}:\n\t{}".format(type(self).__name__, "\n\t".join(problems))
                )
        return _IncompatibleKeys(missing, unexpected)


def _drop_nested_names(module, state_dict, prefix, local_metadata):
    for old in module.old_to_new:
        state_dict.pop(prefix + old, None)
    return state_dict


def filter_out_old_keys(self, state_dict, prefix, local_metadata):
    """State-dict hook under the reference's name (``opacus/layers/param_rename.py:24-30``): a copy of ``state_dict``
    without the pre-rename parameter names of ``self``."""
    return {name: value for name, value in state_dict.items() if name not in self.old_to_new}
