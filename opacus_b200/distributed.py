"""Data-parallel model wrapper.  Unlike ``torch``'s DDP it installs no gradient
hooks: private gradients only exist after clipping, so synchronisation belongs
to the optimiser (``opacus/distributed.py:20-57``)."""
import torch
import torch.distributed as dist
import torch.nn as nn


def average_gradients(model: nn.Module) -> None:
    """Legacy helper: all-reduce and average ``.grad`` of every trainable parameter."""
    from .optimizers._collectives import all_reduce_grads

    grads = [p.grad for p in model.parameters() if p.requires_grad]
    all_reduce_grads(grads, average_by=dist.get_world_size())


class DifferentiallyPrivateDistributedDataParallel(nn.Module):
    """Holds ``module`` and makes every rank start from rank 0's parameters
    (one flat broadcast per dtype instead of one per parameter)."""

    def __init__(self, model: nn.Module):
        super().__init__()
        with torch.no_grad():
            by_kind = {}
            for p in model.parameters():
                by_kind.setdefault((p.dtype, p.device), []).append(p)
            for ps in by_kind.values():
                flat = torch.cat([p.data.reshape(-1) for p in ps])
                dist.broadcast(flat, 0)
                ofs = 0
                for p in ps:
                    p.data.copy_(flat[ofs: ofs + p.numel()].view_as(p))
                    ofs += p.numel()
        self.module = model

    def forward(self, *args, **kwargs):
        return self.module(*args, **kwargs)
