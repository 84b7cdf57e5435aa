"""The correctness oracle for per-sample gradients: run every sample through
the model alone ("micro-batches" of size one), collect ``.grad``, and compare
with what the gradient engine produced for the whole batch.

Behavioural parity: ``opacus/utils/per_sample_gradients_utils.py:28-439``.
"""
from contextlib import contextmanager
from typing import Callable, Dict, Iterable, List, Union

import numpy as np
import torch
import torch.nn as nn
from torch.nn.utils.rnn import PackedSequence, pad_packed_sequence

from ..grad_sample import wrap_model
from .module_utils import clone_module as _clone_to_device
from .module_utils import trainable_parameters
from .packed_sequences import compute_seq_lengths


def clone_module(module: nn.Module) -> nn.Module:
    return _clone_to_device(module)


def is_batch_empty(batch: Union[torch.Tensor, Iterable[torch.Tensor]]):
    first = batch if type(batch) is torch.Tensor else batch[0]
    return first.numel() == 0


@contextmanager
def _deterministic(seed: int = 0):
    was = torch.are_deterministic_algorithms_enabled()
    torch.use_deterministic_algorithms(True)
    try:
        torch.manual_seed(seed)
        np.random.seed(seed)
        yield
    finally:
        torch.use_deterministic_algorithms(was)


class ModelWithLoss(nn.Module):
    """``module`` followed by an L1 loss against zeros (a loss whose gradient
    is non-trivial for every output element)."""

    supported_reductions = ["mean", "sum"]

    def __init__(self, module: nn.Module, loss_reduction: str = "mean"):
        super().__init__()
        if loss_reduction not in self.supported_reductions:
            raise ValueError(
                f"Passed loss_reduction={loss_reduction}. Only {self.supported_reductions} supported.")
        self.wrapped_module = module
        self.criterion = nn.L1Loss(reduction=loss_reduction)

    def forward(self, x):
        out = self.wrapped_module(*x) if type(x) is tuple else self.wrapped_module(x)
        if type(out) is PackedSequence:
            return _compute_loss_packedsequences(self.criterion, out)
        return self.criterion(out, torch.zeros_like(out))


def compute_microbatch_grad_sample(x, module: nn.Module, batch_first: bool = True, loss_reduction: str = "mean",
                                   chunk_method: Callable = iter) -> Dict[str, torch.Tensor]:
    """``{param_name: [B, *shape]}`` from ``B`` independent batch-of-one passes
    on a copy of ``module``."""
    with _deterministic():
        net = ModelWithLoss(clone_module(module), loss_reduction)
        collected: Dict[int, List[torch.Tensor]] = {id(p): [] for p in net.parameters()}
        if not batch_first and type(x) is not list:
            x = x.transpose(0, 1)
        for x_i in chunk_method(x):
            net.zero_grad()
            if type(x_i) is not tuple:
                x_i = x_i.unsqueeze(0 if batch_first else 1)
            net(x_i).backward()
            for p in net.parameters():
                collected[id(p)].append(p.grad.detach().clone())
    out = {}
    for name, p in trainable_parameters(net.wrapped_module):
        rows = collected[id(p)]
        out[name] = torch.stack(rows, dim=0) if batch_first else torch.stack(rows, dim=1).transpose(0, 1)
    return out


def compute_opacus_grad_sample(x, module: nn.Module, batch_first: bool = True, loss_reduction: str = "mean",
                               grad_sample_mode: str = "hooks") -> Dict[str, torch.Tensor]:
    """``{param_name: grad_sample}`` from the gradient engine on a copy of ``module``."""
    with _deterministic():
        gsm = wrap_model(model=clone_module(module), grad_sample_mode=grad_sample_mode, batch_first=batch_first,
                         loss_reduction=loss_reduction)
        net = ModelWithLoss(gsm, loss_reduction)
        net.zero_grad()
        net(x).backward()
        return {name: p.grad_sample for name, p in trainable_parameters(net.wrapped_module._module)}


def check_torch_version_for_ew_sample() -> bool:
    return True


def get_grad_sample_modes(use_ew: bool = False):
    return ["hooks", "functorch"] + (["ew"] if use_ew else [])


def unpack_packedsequences(X: PackedSequence) -> List[torch.Tensor]:
    """Sequences of a packed batch in *packed (sorted) order*, un-padded."""
    padded, _ = pad_packed_sequence(X)
    padded = padded.permute(1, 0, 2)
    if X.sorted_indices is not None:
        padded = padded[X.sorted_indices]
    return [padded[i][:n, :] for i, n in enumerate(compute_seq_lengths(X.batch_sizes))]


def _compute_loss_packedsequences(criterion: nn.L1Loss, x: PackedSequence) -> torch.Tensor:
    if criterion.reduction == "sum":
        return criterion(x[0], torch.zeros_like(x[0]))
    seqs = unpack_packedsequences(x)
    total = 0
    for s in seqs:
        total = total + criterion(s, torch.zeros_like(s))
    return total / len(seqs)


def compute_microbatch_grad_sample_tensor_or_seq(x, module: nn.Module, batch_first: bool = True,
                                                 loss_reduction: str = "mean"):
    data = unpack_packedsequences(x) if type(x) is PackedSequence else x
    return compute_microbatch_grad_sample(data, module, batch_first=batch_first, loss_reduction=loss_reduction)


def compute_grad_samples_microbatch_and_opacus(x, module: nn.Module, batch_first: bool = True,
                                               loss_reduction: str = "mean", grad_sample_mode: str = "hooks",
                                               chunk_method: Callable = iter):
    if type(x) is PackedSequence:
        data = unpack_packedsequences(x)
    elif is_batch_empty(x):
        raise RuntimeError("x is expected to be non-empty.")
    else:
        data = x
    micro = compute_microbatch_grad_sample(data, module, batch_first=batch_first, loss_reduction=loss_reduction,
                                           chunk_method=chunk_method)
    ours = compute_opacus_grad_sample(x, module, batch_first=batch_first, loss_reduction=loss_reduction,
                                      grad_sample_mode=grad_sample_mode)
    if micro.keys() != ours.keys():
        raise ValueError(
            f"Keys not matching! Keys only in microbatch: {micro.keys() - ours.keys()}; "
            f"Keys only in Opacus: {ours.keys() - micro.keys()}")
    return micro, ours


def _check_per_sample_gradients_are_correct_with_reduction(x, module: nn.Module, batch_first: bool = True,
                                                           loss_reduction: str = "mean", atol: float = 1e-5,
                                                           rtol: float = 1e-4,
                                                           grad_sample_mode: str = "hooks") -> bool:
    micro, ours = compute_grad_samples_microbatch_and_opacus(
        x, module, batch_first=batch_first, loss_reduction=loss_reduction, grad_sample_mode=grad_sample_mode)
    for name, got in ours.items():
        want = micro[name]
        if got.shape != want.shape or not torch.allclose(want, got, atol, rtol):
            return False
    return True


def check_per_sample_gradients_are_correct(x, module: nn.Module, *, batch_first: bool = True, atol: float = 1e-5,
                                           rtol: float = 1e-4, grad_sample_mode: str = "hooks") -> bool:
    """True if the engine's per-sample gradients equal the micro-batch ones for
    both ``sum`` and ``mean`` loss reductions."""
    if grad_sample_mode == "ew" and not batch_first:
        raise RuntimeError("Batch should be first dimension.")
    return all(
        _check_per_sample_gradients_are_correct_with_reduction(
            x, module, batch_first=batch_first, loss_reduction=r, atol=atol, rtol=rtol,
            grad_sample_mode=grad_sample_mode)
        for r in ("sum", "mean"))
