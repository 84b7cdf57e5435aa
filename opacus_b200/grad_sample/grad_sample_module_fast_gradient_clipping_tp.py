"""Ghost clipping under 1-d tensor parallelism ("ghost_tp").

Every rank holds a shard of each parallel weight, so a layer's sampler yields
the squared norm of the local shard of the per-sample gradient.  The global
squared norm is the sum over tensor-parallel ranks.  Parameters that are *not*
sharded (plain tensors, or an Embedding sharded along its rows where every rank
sees the same per-sample gradient rows) must be counted once: only rank 0 of
the group contributes them (``param.merge_flag = False``).

Accepted parameter kinds: ``DTensor`` parameters from
``torch.distributed.tensor.parallel.parallelize_module`` and the
``ColumnParallelLinear``/``RowParallelLinear`` layers of
:mod:`opacus_b200.parallel.tensor_parallel`, which mark their weights with
``tp_sharded = True``.

Behavioural parity: ``opacus/grad_sample/grad_sample_module_fast_gradient_clipping_tp.py:33-147``.
"""
from __future__ import annotations

import logging
import warnings

import torch
import torch.nn as nn

from .grad_sample_module_fast_gradient_clipping import GradSampleHooksFastGradientClipping
from .gsm_base import AbstractGradSampleModule

logger = logging.getLogger(__name__)


def _is_dtensor(p) -> bool:
    try:
        from torch.distributed.tensor import DTensor
    except Exception:  # pragma: no cover
        return False
    return isinstance(p, DTensor)


class GradSampleHooksFastGradientClippingTP(GradSampleHooksFastGradientClipping):
    def __init__(self, m: nn.Module, *, batch_first=True, loss_reduction="mean", strict: bool = True,
                 force_functorch=False, max_grad_norm=1, use_ghost_clipping=True, single_pass: bool = False,
                 process_group=None):
        self.process_group = process_group
        super().__init__(m, batch_first=batch_first, loss_reduction=loss_reduction, strict=strict,
                         force_functorch=force_functorch, max_grad_norm=max_grad_norm,
                         use_ghost_clipping=use_ghost_clipping, single_pass=single_pass)
        self.set_pattern_param_sample_norm_sum()
        warnings.warn("Opacus TP is currently in beta. Custom model output placements may cause unexpected behavior.")

    def set_pattern_param_sample_norm_sum(self):
        """Decide per parameter whether every rank's norm counts (sharded) or only rank 0's."""
        for module in self.iterate_submodules(self._module):
            for _, p in module.named_parameters():
                if not p.requires_grad:
                    continue
                if getattr(p, "tp_sharded", False):
                    p.merge_flag = True
                elif not _is_dtensor(p):
                    p.merge_flag = False
                elif isinstance(module, nn.Embedding) and p.placements[0].is_shard(0):
                    p.merge_flag = False
                elif p.placements[0].is_replicate():
                    p.merge_flag = False
                    raise NotImplementedError(
                        "We currently do not support replicated model parameters, due to the constraint of "
                        "fsdpoptimizwer. This means that nn.Linear.bias must be disabled or configured to be sharded."
                    )
                else:
                    p.merge_flag = True

    # ---- single-pass bookkeeping: sharded and replicated parameters are kept apart
    _use_total_fastpath = False

    def _total_fastpath_ok(self, module) -> bool:
        """Layers all of whose parameters are shards add their norms inside the ghost-norm kernel straight into the
        running sum of the sharded part -- which, with peer memory, is this rank's slot of the symmetric buffer the
        group's all-reduce reads (``PeerNormReducer.accumulator``): no separate copy, no separate add."""
        ps = [p for p in module.parameters(recurse=False) if p.requires_grad]
        return bool(ps) and all(getattr(p, "merge_flag", False) and not getattr(p, "sp_local", False) for p in ps)

    def _new_total(self, n: int, device) -> torch.Tensor:
        reducer = self._peer_reducer(torch.empty(0, device=device)) if device.type == "cuda" else None
        if reducer is not None:
            acc = reducer.accumulator(n)
            if acc is not None:
                return acc
        return super()._new_total(n, device)
    overlap_norms = False        # the rules of this controller issue collectives; keep them on the main stream

    # ---- activations sharded over samples between the tensor-parallel blocks (sequence parallelism)
    def _world(self) -> int:
        return torch.distributed.get_world_size(self.process_group)

    def _batch_share(self, module) -> int:
        return self._world() if getattr(module, "sp_local_input", False) else 1

    def _prepare_site(self, module, activations, backprops):
        activations, backprops = super()._prepare_site(module, activations, backprops)   # a layer's own gathered input
        if getattr(module, "scatter_output", False):  # the output gradient arrives for this rank's samples only
            from ..parallel.tensor_parallel import _all_gather0

            backprops = _all_gather0(backprops, self.process_group)
            module.__dict__["_sp_grad_full"] = backprops
        return activations, backprops

    def _local_slice(self, n_local: int) -> slice:
        r = self._group_rank()
        return slice(r * n_local, (r + 1) * n_local)

    def _align_norm(self, p, v):
        if getattr(p, "sp_local", False) and self._batch_len and v.shape[0] * self._world() == self._batch_len:
            out = v.new_zeros(self._batch_len)
            out[self._local_slice(v.shape[0])] = v
            return out
        return super()._align_norm(p, v)

    def _site_coef(self, site, coef):
        n = site.backprops.shape[0]
        if getattr(site.module, "sp_local_region", False) and n * self._world() == coef.shape[0]:
            return coef[self._local_slice(n)].to(site.backprops.device)
        return super()._site_coef(site, coef)

    def _reset_single_pass_state(self):
        super()._reset_single_pass_state()
        self._norm_sq_replicated = None

    def _add_norm_sq(self, p, v):
        if getattr(p, "merge_flag", False) or getattr(p, "sp_local", False):
            # sharded weights and sample-local parameters: every rank holds a partial value, sum over the group
            super()._add_norm_sq(p, v)
        else:
            self._norm_sq_replicated = v.clone() if self._norm_sq_replicated is None else \
                self._norm_sq_replicated.add_(v)

    def _group_sum(self, sharded, replicated) -> torch.Tensor:
        """``sum_ranks sharded + replicated``.  On NVLink-connected GPUs this is one
        peer-memory kernel that also yields the clip factors (kept in
        ``_peer_clip``), bit-identical on all ranks; elsewhere an all-reduce."""
        ref = sharded if sharded is not None else replicated
        self._peer_clip = None
        reducer = self._peer_reducer(ref)
        if reducer is not None:
            total, clip = reducer(sharded, replicated, float(self.max_grad_norm))
            self._peer_clip = clip
            return total
        total = sharded.clone() if sharded is not None else torch.zeros_like(ref)
        torch.distributed.all_reduce(total, op=torch.distributed.ReduceOp.SUM, group=self.process_group)
        if replicated is not None:
            total = total + replicated
        return total

    def _peer_reducer(self, ref):
        """The peer-memory reducer, created on first use (collectively), or None."""
        if getattr(self, "_reducer", None) is None:
            self._reducer = False
            if ref.is_cuda and self.use_peer_memory:
                from ..parallel import symm

                if symm.available(self.process_group) is None:
                    self._reducer = symm.PeerNormReducer(ref.device, self.process_group)
        r = self._reducer
        return r if r and ref.numel() <= r.capacity else None

    use_peer_memory = True

    def _single_pass_norm_sq(self) -> torch.Tensor:
        return self._group_sum(self._norm_sq_total, self._norm_sq_replicated)

    def _group_rank(self) -> int:
        return torch.distributed.get_rank(self.process_group)

    def get_norm_sample(self) -> torch.Tensor:
        if self.single_pass and (self._norm_sq_total is not None or self._norm_sq_replicated is not None):
            norm = self._single_pass_norm_sq().clamp(min=0).sqrt()
            self.per_sample_gradient_norms = norm
            return norm
        sharded = replicated = None
        for p in self.trainable_parameters:
            v = p._norm_sample.float().square()
            if p.merge_flag:
                sharded = v if sharded is None else sharded + v
            else:
                replicated = v if replicated is None else replicated + v
        norm = self._group_sum(sharded, replicated).sqrt()
        self.per_sample_gradient_norms = norm
        return norm

    def get_clipping_coef(self) -> torch.Tensor:
        norm = self.get_norm_sample()
        clip = getattr(self, "_peer_clip", None)
        if clip is not None and clip.shape == norm.shape:
            return clip
        return (self.max_grad_norm / (norm + 1e-6)).clamp(max=1.0)


class GradSampleModuleFastGradientClippingTP(GradSampleHooksFastGradientClippingTP, AbstractGradSampleModule):
    def __init__(self, m: nn.Module, *, batch_first=True, loss_reduction="mean", strict: bool = True,
                 force_functorch=False, max_grad_norm=1, process_group=None, single_pass: bool = False):
        nn.Module.__init__(self)
        GradSampleHooksFastGradientClippingTP.__init__(
            self, m, batch_first=batch_first, loss_reduction=loss_reduction, strict=strict,
            force_functorch=force_functorch, max_grad_norm=max_grad_norm, process_group=process_group,
            single_pass=single_pass)
        self.grad_accumulation_hook = None
