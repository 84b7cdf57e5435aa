"""InstanceNorm is per-sample, but its running statistics are not private
(``opacus/validators/instance_norm.py:28-51``)."""
from typing import List, Union

import torch.nn as nn

from ..utils.module_utils import clone_module
from .errors import IllegalModuleConfigurationError, UnsupportedModuleError
from .utils import register_module_fixer, register_module_validator

INSTANCENORM = Union[nn.InstanceNorm1d, nn.InstanceNorm2d, nn.InstanceNorm3d]
_IN_TYPES = [nn.InstanceNorm1d, nn.InstanceNorm2d, nn.InstanceNorm3d]


@register_module_validator(_IN_TYPES)
def validate(module: INSTANCENORM) -> List[UnsupportedModuleError]:
    if not module.track_running_stats:
        return []
    return [
        IllegalModuleConfigurationError(
            "We do not support tracking running stats with differential privacy: the running mean/variance "
            "aggregate information across samples and would need a privacy mechanism of their own."
        )
    ]


@register_module_fixer(_IN_TYPES)
def fix(module: INSTANCENORM, **kwargs) -> INSTANCENORM:
    if not validate(module):
        return module
    fixed = clone_module(module)
    fixed.track_running_stats = False
    return fixed
