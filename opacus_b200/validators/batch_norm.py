"""BatchNorm couples the samples of a batch, so it has no per-sample gradient;
it is replaced by GroupNorm (default) or InstanceNorm
(``opacus/validators/batch_norm.py:36-142``)."""
import logging
import math
from typing import List, Optional, Union

import torch.nn as nn

from .errors import ShouldReplaceModuleError, UnsupportableModuleError, UnsupportedModuleError
from .utils import register_module_fixer, register_module_validator

logger = logging.getLogger(__name__)

_BN_TYPES = [nn.BatchNorm1d, nn.BatchNorm2d, nn.BatchNorm3d, nn.SyncBatchNorm]
BATCHNORM = Union[nn.BatchNorm1d, nn.BatchNorm2d, nn.BatchNorm3d, nn.SyncBatchNorm]
INSTANCENORM = Union[nn.InstanceNorm1d, nn.InstanceNorm2d, nn.InstanceNorm3d]


@register_module_validator(_BN_TYPES)
def validate(module: BATCHNORM) -> List[UnsupportedModuleError]:
    return [
        ShouldReplaceModuleError(
            "BatchNorm cannot support training with differential privacy: it normalises each sample with "
            "statistics of the other samples in the batch, so a sample's output (and gradient) depends on its "
            "peers. LayerNorm, InstanceNorm and GroupNorm do not have this property and are privacy-safe; "
            "ModuleValidator.fix() replaces BatchNorm with GroupNorm."
        )
    ]


@register_module_fixer(_BN_TYPES)
def fix(module: BATCHNORM, **kwargs) -> Union[nn.GroupNorm, INSTANCENORM]:
    """kwargs: ``replace_bn_with_in`` (bool) or ``num_groups`` (int), not both."""
    to_instance = kwargs.get("replace_bn_with_in", False)
    num_groups = kwargs.get("num_groups", None)
    if to_instance and num_groups is not None:
        raise ValueError("is_replace_bn_with_in and num_groups are mutually exclusive")
    if to_instance:
        return _batchnorm_to_instancenorm(module)
    return _batchnorm_to_groupnorm(module, num_groups=num_groups)


def _batchnorm_to_groupnorm(module: BATCHNORM, *, num_groups: Optional[int] = None) -> nn.GroupNorm:
    """Default group count: the largest divisor of the channel count that also divides 32."""
    groups = math.gcd(32, module.num_features) if num_groups is None else num_groups
    return nn.GroupNorm(groups, module.num_features, affine=module.affine)


def _batchnorm_to_instancenorm(module: BATCHNORM) -> INSTANCENORM:
    for bn, inorm in ((nn.BatchNorm1d, nn.InstanceNorm1d), (nn.BatchNorm2d, nn.InstanceNorm2d),
                      (nn.BatchNorm3d, nn.InstanceNorm3d)):
        if isinstance(module, bn):
            return inorm(module.num_features)
    raise UnsupportableModuleError(
        "There is no equivalent InstanceNorm module to replace SyncBatchNorm with. "
        "Consider replacing it with GroupNorm instead."
    )


def _nullify_batch_norm():
    return nn.Identity()
