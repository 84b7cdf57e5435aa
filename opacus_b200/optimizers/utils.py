from typing import List

import torch.nn as nn
from torch.optim import Optimizer


def params(optimizer: Optimizer) -> List[nn.Parameter]:
    """Trainable parameters of all groups, in group order."""
    return [p for group in optimizer.param_groups for p in group["params"] if p.requires_grad]
