"""1-d tensor parallelism for DP training: column- and row-parallel Linear
layers whose weight shards are ordinary parameters, so the ghost-clipping
engine treats them like any Linear (a shard's per-sample gradient only needs
the local activations and output gradients), plus the optimizer that knows
which parameters are sharded and which are replicated.

``ColumnParallelLinear`` splits the output features, ``RowParallelLinear`` the
input features; a column layer followed by a row layer needs one all-reduce in
forward (after the row layer) and one in backward (before the column layer).
Sharded parameters carry ``tp_sharded = True``; the "ghost_tp" controller sums
their squared per-sample norms over the group and counts replicated
parameters once (``opacus/grad_sample/grad_sample_module_fast_gradient_clipping_tp.py:65-115``).

The reference obtains the same layout from ``parallelize_module`` with
``ColwiseParallel`` / ``RowwiseParallel`` DTensors
(``examples/tensor_parallelism_llama.py:104-152``) and cannot train replicated
parameters; here they are supported (identical noise on every rank).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from ..grad_sample.linear import (
    compute_linear_grad_sample,
    compute_linear_norm_sample,
    compute_linear_norm_sq,
    compute_linear_weighted_grad,
)
from ..grad_sample.utils import (
    register_grad_sampler,
    register_norm_sampler,
    register_norm_sq_sampler,
    register_wgrad_sampler,
)
from ..optimizers.optimizer import _check_processed_flag, _generate_noise, _mark_as_processed
from ..optimizers.optimizer_fast_gradient_clipping import DPOptimizerFastGradientClipping


class _CopyToGroup(torch.autograd.Function):
    """Identity in forward, all-reduce of the gradient in backward (input of a column-parallel layer)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        dist.all_reduce(g, op=dist.ReduceOp.SUM, group=ctx.group)
        return g, None


class _ReduceFromGroup(torch.autograd.Function):
    """All-reduce in forward, identity in backward (output of a row-parallel layer)."""

    @staticmethod
    def forward(ctx, x, group):
        x = x.contiguous().clone()
        dist.all_reduce(x, op=dist.ReduceOp.SUM, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


class _GatherLastDim(torch.autograd.Function):
    """All-gather along the last axis in forward, take the local slice in backward."""

    @staticmethod
    def forward(ctx, x, group):
        world = dist.get_world_size(group)
        ctx.rank, ctx.world = dist.get_rank(group), world
        parts = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(parts, x.contiguous(), group=group)
        return torch.cat(parts, dim=-1)

    @staticmethod
    def backward(ctx, g):
        return g.chunk(ctx.world, dim=-1)[ctx.rank].contiguous(), None


def _group_size(group) -> int:
    return dist.get_world_size(group)


class ColumnParallelLinear(nn.Linear):
    """``y[..., shard] = x W_shard^T + b_shard``: this rank owns rows
    ``[rank*out/W, (rank+1)*out/W)`` of the full weight.  ``x`` is replicated.
    With ``gather_output`` the shards of ``y`` are concatenated on every rank."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, *, process_group=None,
                 gather_output: bool = False, device=None, dtype=None):
        world = _group_size(process_group)
        if out_features % world:
            raise ValueError(f"out_features={out_features} is not divisible by the group size {world}")
        super().__init__(in_features, out_features // world, bias=bias, device=device, dtype=dtype)
        self.process_group = process_group
        self.gather_output = gather_output
        self.full_out_features = out_features
        self.weight.tp_sharded = True
        if self.bias is not None:
            self.bias.tp_sharded = True

    def forward(self, x):
        y = F.linear(_CopyToGroup.apply(x, self.process_group), self.weight, self.bias)
        return _GatherLastDim.apply(y, self.process_group) if self.gather_output else y

    @classmethod
    def from_linear(cls, lin: nn.Linear, process_group=None, gather_output: bool = False):
        """Shard an existing (replicated) ``nn.Linear``."""
        rank, world = dist.get_rank(process_group), _group_size(process_group)
        out = cls(lin.in_features, lin.out_features, lin.bias is not None, process_group=process_group,
                  gather_output=gather_output, device=lin.weight.device, dtype=lin.weight.dtype)
        with torch.no_grad():
            out.weight.copy_(lin.weight.chunk(world, dim=0)[rank])
            if lin.bias is not None:
                out.bias.copy_(lin.bias.chunk(world, dim=0)[rank])
        return out


class RowParallelLinear(nn.Linear):
    """``y = sum_ranks x[..., shard] W[:, shard]^T + b``: this rank owns columns
    ``[rank*in/W, (rank+1)*in/W)`` of the full weight and sees the matching
    slice of the input (``input_is_parallel``), e.g. a column-parallel layer's
    output.  The bias is replicated and added once, after the reduction."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, *, process_group=None,
                 input_is_parallel: bool = True, device=None, dtype=None):
        world = _group_size(process_group)
        if in_features % world:
            raise ValueError(f"in_features={in_features} is not divisible by the group size {world}")
        super().__init__(in_features // world, out_features, bias=bias, device=device, dtype=dtype)
        self.process_group = process_group
        self.input_is_parallel = input_is_parallel
        self.full_in_features = in_features
        self.weight.tp_sharded = True

    def forward(self, x):
        if not self.input_is_parallel:
            rank, world = dist.get_rank(self.process_group), _group_size(self.process_group)
            x = x.chunk(world, dim=-1)[rank]
        y = _ReduceFromGroup.apply(F.linear(x, self.weight, None), self.process_group)
        return y if self.bias is None else y + self.bias

    @classmethod
    def from_linear(cls, lin: nn.Linear, process_group=None, input_is_parallel: bool = True):
        rank, world = dist.get_rank(process_group), _group_size(process_group)
        out = cls(lin.in_features, lin.out_features, lin.bias is not None, process_group=process_group,
                  input_is_parallel=input_is_parallel, device=lin.weight.device, dtype=lin.weight.dtype)
        with torch.no_grad():
            out.weight.copy_(lin.weight.chunk(world, dim=1)[rank])
            if lin.bias is not None:
                out.bias.copy_(lin.bias)
        return out


def _row_parallel_rules():
    """For the row-parallel layer the captured output gradient is that of the
    *reduced* output, which is also the gradient of the local partial product
    and of the bias, so the Linear rules apply unchanged."""
    for cls in (ColumnParallelLinear, RowParallelLinear):
        register_grad_sampler(cls)(compute_linear_grad_sample)
        register_norm_sampler(cls)(compute_linear_norm_sample)
        register_norm_sq_sampler(cls)(compute_linear_norm_sq)
        register_wgrad_sampler(cls)(compute_linear_weighted_grad)


_row_parallel_rules()


class TensorParallelDPOptimizer(DPOptimizerFastGradientClipping):
    """Ghost-clipping optimizer for a tensor-parallel group.

    Every rank sees the same batch.  A sharded parameter's noise is drawn
    locally (the shards are disjoint pieces of one tensor, so the draws are
    independent coordinates of one Gaussian); a replicated parameter must
    receive the *same* noise on every rank, so rank 0 of the group draws it and
    broadcasts.  No gradient collective is needed: sharded gradients are
    complete locally and replicated ones are identical by construction.
    """

    _fused_ok = False

    def __init__(self, optimizer, *, noise_multiplier, max_grad_norm, expected_batch_size, loss_reduction="mean",
                 generator=None, secure_mode=False, process_group=None, **kwargs):
        kwargs.pop("engine", None)
        super().__init__(optimizer, noise_multiplier=noise_multiplier, max_grad_norm=max_grad_norm,
                         expected_batch_size=expected_batch_size, loss_reduction=loss_reduction,
                         generator=generator, secure_mode=secure_mode, **kwargs)
        self.process_group = process_group

    def add_noise(self):
        std = self._noise_std()
        group = self.process_group
        src = dist.get_global_rank(group, 0) if group is not None else 0
        for p in self.params:
            _check_processed_flag(p.summed_grad)
            noise = _generate_noise(std=std, reference=p.summed_grad, generator=self.generator,
                                    secure_mode=self.secure_mode)
            if not getattr(p, "tp_sharded", False) and std != 0:
                dist.broadcast(noise, src, group=group)
            p.grad = (p.summed_grad + noise).view_as(p).to(p.dtype)
            _mark_as_processed(p.summed_grad)


class _VocabParallelCE(torch.autograd.Function):
    """Token-wise cross entropy over logits whose vocabulary axis is split across the group."""

    @staticmethod
    def forward(ctx, logits, target, group, vocab_start):
        lf = logits.float()
        m = lf.max(dim=-1).values
        dist.all_reduce(m, op=dist.ReduceOp.MAX, group=group)
        e = torch.exp(lf - m[:, None])
        z = e.sum(dim=-1)
        local = target - vocab_start
        mine = (local >= 0) & (local < logits.shape[-1])
        picked = torch.where(mine, lf.gather(1, local.clamp(0, logits.shape[-1] - 1)[:, None])[:, 0],
                             torch.zeros_like(m))
        packed = torch.stack([z, picked])
        dist.all_reduce(packed, op=dist.ReduceOp.SUM, group=group)
        z, picked = packed[0], packed[1]
        ctx.save_for_backward(e, z, local, mine)
        ctx.dtype = logits.dtype
        return torch.log(z) + m - picked

    @staticmethod
    def backward(ctx, g):
        e, z, local, mine = ctx.saved_tensors
        grad = e / z[:, None]
        rows = torch.nonzero(mine)[:, 0]
        grad[rows, local[rows]] -= 1.0
        return (grad * g[:, None]).to(ctx.dtype), None, None, None


class VocabParallelCrossEntropy(nn.Module):
    """``CrossEntropyLoss`` for logits ``[tokens, vocab / world]`` produced by a
    column-parallel output layer without gathering: only per-token maxima, partition
    sums and target logits (three ``[tokens]`` vectors) cross the group.  Works as the
    criterion of ``DPLossFastGradientClipping`` (has ``reduction``)."""

    def __init__(self, process_group=None, reduction: str = "mean"):
        super().__init__()
        self.process_group = process_group
        self.reduction = reduction

    def forward(self, logits, target):
        rank = dist.get_rank(self.process_group)
        loss = _VocabParallelCE.apply(logits, target, self.process_group, rank * logits.shape[-1])
        if self.reduction == "none":
            return loss
        return loss.mean() if self.reduction == "mean" else loss.sum()


def parallelize_llama(model, process_group=None, shard_lm_head: bool = True):
    """Turn a :class:`opacus_b200.models.Llama` (replicated, identical on all ranks) into its
    1-d tensor-parallel form in place: q/k/v/gate/up become column-parallel, o/down
    row-parallel, heads are divided over the ranks; embedding and norm weights stay
    replicated; with ``shard_lm_head`` the output layer is split over the vocabulary
    (use :class:`VocabParallelCrossEntropy`).  Same layout as the reference's plan
    (``examples/tensor_parallelism_llama.py:104-152``)."""
    world = _group_size(process_group)
    for blk in model.layers:
        att, mlp = blk.self_attn, blk.mlp
        if att.n_heads % world or att.n_kv % world:
            raise ValueError(f"{att.n_heads} query / {att.n_kv} key-value heads do not divide over {world} ranks")
        for name in ("q_proj", "k_proj", "v_proj"):
            setattr(att, name, ColumnParallelLinear.from_linear(getattr(att, name), process_group))
        att.o_proj = RowParallelLinear.from_linear(att.o_proj, process_group)
        att.n_heads //= world
        att.n_kv //= world
        for name in ("gate_proj", "up_proj"):
            setattr(mlp, name, ColumnParallelLinear.from_linear(getattr(mlp, name), process_group))
        mlp.down_proj = RowParallelLinear.from_linear(mlp.down_proj, process_group)
    if shard_lm_head:
        if model.lm_head.weight is model.embed_tokens.weight:
            raise ValueError("a tied output layer cannot be sharded over the vocabulary")
        model.lm_head = ColumnParallelLinear.from_linear(model.lm_head, process_group)
    return model
