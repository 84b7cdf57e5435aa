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

Sequence-parallel form (``parallelize_llama(sequence_parallel=True)``): between
two tensor-parallel blocks the activations are sharded over *samples*; a
column-parallel layer with ``input_mode="local"`` gathers its input inside its
GEMM and a row-parallel layer with ``scatter_output`` reduce-scatters inside its
GEMM (``parallel/fused_tp.py``), so the two all-reduces become an all-gather
and a reduce-scatter that overlap the matrix products, and everything outside
the blocks (norms, residual stream, embedding) runs on ``1 / world`` of the
batch.  Parameters of those outside modules carry ``sp_local = True``: their
per-sample norms are partial per rank and their clipped sums are completed by
an all-reduce in :class:`TensorParallelDPOptimizer`.

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


def _all_gather0(x: torch.Tensor, group) -> torch.Tensor:
    """Concatenation of every rank's ``x`` along dim 0."""
    x = x.contiguous()
    world = _group_size(group)
    if x.is_cuda:
        out = x.new_empty((world * x.shape[0],) + tuple(x.shape[1:]))
        dist.all_gather_into_tensor(out, x, group=group)
        return out
    parts = [torch.empty_like(x) for _ in range(world)]
    dist.all_gather(parts, x, group=group)
    return torch.cat(parts, dim=0)


def _reduce_scatter0(x: torch.Tensor, group) -> torch.Tensor:
    """This rank's dim-0 chunk of the sum of every rank's ``x``."""
    x = x.contiguous()
    world, rank = _group_size(group), dist.get_rank(group)
    if x.is_cuda:
        out = x.new_empty((x.shape[0] // world,) + tuple(x.shape[1:]))
        dist.reduce_scatter_tensor(out, x, group=group)
        return out
    x = x.clone()
    dist.all_reduce(x, group=group)
    return x.chunk(world, dim=0)[rank].contiguous()


class _GatherSamples(torch.autograd.Function):
    """All-gather over the sample axis in forward, reduce-scatter of the gradient in backward:
    the boundary from the sample-sharded region (residual stream, norms) into a tensor-parallel block."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _all_gather0(x, group)

    @staticmethod
    def backward(ctx, g):
        return _reduce_scatter0(g, ctx.group), None


class SampleGather(nn.Module):
    """``[B / world, ...] -> [B, ...]`` (see :class:`_GatherSamples`)."""

    def __init__(self, process_group=None):
        super().__init__()
        self.process_group = process_group

    def forward(self, x):
        return _GatherSamples.apply(x, self.process_group)


class SampleSlice(nn.Module):
    """This rank's share of the batch: ``[B, ...] -> [B / world, ...]`` (no gradient flows through token ids)."""

    def __init__(self, process_group=None):
        super().__init__()
        self.process_group = process_group

    def forward(self, x):
        world, rank = _group_size(self.process_group), dist.get_rank(self.process_group)
        if x.shape[0] % world:
            raise ValueError(f"batch of {x.shape[0]} does not divide over {world} tensor-parallel ranks")
        return x.chunk(world, dim=0)[rank]


def _fused_ok(x: torch.Tensor, rows: int, unit: int, world: int) -> bool:
    return x.is_cuda and x.dtype == torch.bfloat16 and rows % (unit * world) == 0


class _GatherLinear(torch.autograd.Function):
    """``y = all_gather(x_local) W^T`` as ONE kernel on NVLink-connected GPUs (``AllGatherGemm``): the peers'
    rows are pulled while the tensor cores already work on the rows that arrived.  Backward: input
    gradient by GEMM + reduce-scatter; the weight gradient only when autograd asks for it."""

    @staticmethod
    def forward(ctx, x, weight, layer):
        group = layer.process_group
        world = _group_size(group)
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1])
        rows, K = x2.shape
        full = None
        if layer.fused and _fused_ok(x2, rows * world, 128, world) and weight.dtype == torch.bfloat16 \
                and (128 * K * 2) % 8192 == 0 and weight.shape[0] % 8 == 0:
            from .fused_tp import AllGatherGemm

            ag = layer.__dict__.get("_ag")
            if ag is None or ag.rows_per_rank != rows or ag.K != K:
                ag = AllGatherGemm(rows, K, x.device, group, gather="a")
                layer.__dict__["_ag"] = ag
            ag.shard.copy_(x2)
            y = ag(weight.detach().contiguous())
            full = ag.full
        else:
            full = _all_gather0(x2, group)
            y = full @ weight.t()
        full_shape = (lead[0] * world,) + tuple(lead[1:])
        full_view = full.view(full_shape + (K,))
        layer.__dict__["_dp_activation"] = full_view
        ctx.save_for_backward(full, weight)
        ctx.group, ctx.x_shape = group, x.shape
        # the gathered input is a second output: layers that consume the same activations (k/v next to q,
        # up next to gate) take it from here and their input gradients join the one reduce-scatter below
        return y.view(full_shape + (weight.shape[0],)), full_view

    @staticmethod
    def backward(ctx, gy, gfull):
        full, weight = ctx.saved_tensors
        g2 = gy.reshape(-1, gy.shape[-1])
        gx = gw = None
        if ctx.needs_input_grad[0]:
            gin = g2 @ weight
            if gfull is not None:
                gin = gin + gfull.reshape(gin.shape)
            gx = _reduce_scatter0(gin, ctx.group).view(ctx.x_shape)
        if ctx.needs_input_grad[1]:
            gw = g2.t() @ full
        return gx, gw, None


class _LinearScatter(torch.autograd.Function):
    """``y_local = reduce_scatter(x W^T)`` over the sample axis as ONE kernel (``GemmReduceScatter``): finished
    output tiles are pushed to their owner while the rest is computed.  Backward gathers the output gradient
    (or takes the copy the per-sample-gradient rule already gathered)."""

    @staticmethod
    def forward(ctx, x, weight, layer):
        group = layer.process_group
        world = _group_size(group)
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1])
        M = x2.shape[0]
        if layer.fused and _fused_ok(x2, M, 128, world) and weight.dtype == torch.bfloat16 and weight.shape[0] % 8 == 0 \
                and x2.shape[1] % 8 == 0:
            from .fused_tp import GemmReduceScatter

            rs = layer.__dict__.get("_rs")
            if rs is None or rs.M != M or rs.N != weight.shape[0]:
                rs = GemmReduceScatter(M, weight.shape[0], x.device, group)
                layer.__dict__["_rs"] = rs
            y = rs(x2.contiguous(), weight.detach().contiguous())
        else:
            y = _reduce_scatter0(x2 @ weight.t(), group)
        ctx.save_for_backward(x2, weight)
        ctx.group, ctx.layer, ctx.x_shape = group, layer, x.shape
        return y.view((lead[0] // world,) + tuple(lead[1:]) + (weight.shape[0],))

    @staticmethod
    def backward(ctx, gy):
        x2, weight = ctx.saved_tensors
        g_full = ctx.layer.__dict__.pop("_sp_grad_full", None)
        if g_full is None:
            g_full = _all_gather0(gy.reshape(-1, gy.shape[-1]), ctx.group)
        g2 = g_full.reshape(-1, g_full.shape[-1])
        gx = gw = None
        if ctx.needs_input_grad[0]:
            gx = (g2 @ weight).view(ctx.x_shape)
        if ctx.needs_input_grad[1]:
            gw = g2.t() @ x2
        return gx, gw, None


class ColumnParallelLinear(nn.Linear):
    """``y[..., shard] = x W_shard^T + b_shard``: this rank owns rows
    ``[rank*out/W, (rank+1)*out/W)`` of the full weight.  ``x`` is replicated.
    With ``gather_output`` the shards of ``y`` are concatenated on every rank."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, *, process_group=None,
                 gather_output: bool = False, input_mode: str = "replicated", fused: bool = True,
                 return_gathered: bool = False, device=None, dtype=None):
        world = _group_size(process_group)
        if out_features % world:
            raise ValueError(f"out_features={out_features} is not divisible by the group size {world}")
        if input_mode not in ("replicated", "gathered", "local"):
            raise ValueError("input_mode must be 'replicated', 'gathered' or 'local'")
        super().__init__(in_features, out_features // world, bias=bias, device=device, dtype=dtype)
        self.process_group = process_group
        self.gather_output = gather_output
        self.full_out_features = out_features
        # "replicated": every rank holds the same input, the input gradient is all-reduced;
        # "gathered":   the input was produced by SampleGather (its backward reduce-scatters), nothing to add;
        # "local":      the input holds this rank's samples only and the layer gathers it itself, fused with
        #               the GEMM when ``fused`` and the shapes allow
        self.input_mode = input_mode
        self.fused = fused
        # with input_mode "local": forward returns ``(y, gathered_input)`` so that sibling layers reuse the gather
        self.return_gathered = return_gathered and input_mode == "local"
        if self.return_gathered and gather_output:
            raise ValueError("return_gathered and gather_output cannot be combined")
        self.sp_local_input = input_mode == "local"
        self.weight.tp_sharded = True
        if self.bias is not None:
            self.bias.tp_sharded = True

    def forward(self, x):
        if self.input_mode == "local":
            y, gathered = _GatherLinear.apply(x, self.weight, self)
            if self.bias is not None:
                y = y + self.bias
            if self.return_gathered:
                return y, gathered
        elif self.input_mode == "gathered":
            y = F.linear(x, self.weight, self.bias)
        else:
            y = F.linear(_CopyToGroup.apply(x, self.process_group), self.weight, self.bias)
        return _GatherLastDim.apply(y, self.process_group) if self.gather_output else y

    @classmethod
    def from_linear(cls, lin: nn.Linear, process_group=None, gather_output: bool = False,
                    input_mode: str = "replicated", fused: bool = True, return_gathered: bool = False):
        """Shard an existing (replicated) ``nn.Linear``."""
        rank, world = dist.get_rank(process_group), _group_size(process_group)
        out = cls(lin.in_features, lin.out_features, lin.bias is not None, process_group=process_group,
                  gather_output=gather_output, input_mode=input_mode, fused=fused, return_gathered=return_gathered,
                  device=lin.weight.device, dtype=lin.weight.dtype)
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
                 input_is_parallel: bool = True, scatter_output: bool = False, fused: bool = True, device=None,
                 dtype=None):
        world = _group_size(process_group)
        if in_features % world:
            raise ValueError(f"in_features={in_features} is not divisible by the group size {world}")
        super().__init__(in_features // world, out_features, bias=bias, device=device, dtype=dtype)
        self.process_group = process_group
        self.input_is_parallel = input_is_parallel
        # scatter_output: the sum over ranks is reduce-scattered over the sample axis (each rank keeps its
        # own samples) instead of all-reduced; fused with the GEMM when ``fused`` and the shapes allow
        self.scatter_output = scatter_output
        self.fused = fused
        self.full_in_features = in_features
        self.weight.tp_sharded = True

    def forward(self, x):
        if not self.input_is_parallel:
            rank, world = dist.get_rank(self.process_group), _group_size(self.process_group)
            x = x.chunk(world, dim=-1)[rank]
        if self.scatter_output:
            y = _LinearScatter.apply(x, self.weight, self)
        else:
            y = _ReduceFromGroup.apply(F.linear(x, self.weight, None), self.process_group)
        return y if self.bias is None else y + self.bias

    @classmethod
    def from_linear(cls, lin: nn.Linear, process_group=None, input_is_parallel: bool = True,
                    scatter_output: bool = False, fused: bool = True):
        rank, world = dist.get_rank(process_group), _group_size(process_group)
        out = cls(lin.in_features, lin.out_features, lin.bias is not None, process_group=process_group,
                  input_is_parallel=input_is_parallel, scatter_output=scatter_output, fused=fused,
                  device=lin.weight.device, dtype=lin.weight.dtype)
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

    Every rank sees the same batch.  The shards of a sharded parameter are
    disjoint pieces of one tensor, so their noise must be *independent*: each
    rank draws it from a generator of its own whose seed folds the rank of the
    group into the seed of the optimizer's generator (ranks that call
    ``torch.manual_seed(0)`` alike would otherwise hand every shard the same
    values, and a full weight with noise ``[Z, Z, ..., Z]`` is not the Gaussian
    mechanism).  A replicated parameter must receive the *same* noise on every
    rank, so rank 0 of the group draws it from the optimizer's generator and
    broadcasts; the other ranks do not draw for it at all.  No gradient
    collective is needed: sharded gradients are complete locally and replicated
    ones are identical by construction.
    """

    _fused_ok = False

    def __init__(self, optimizer, *, noise_multiplier, max_grad_norm, expected_batch_size, loss_reduction="mean",
                 generator=None, secure_mode=False, process_group=None, **kwargs):
        kwargs.pop("engine", None)
        super().__init__(optimizer, noise_multiplier=noise_multiplier, max_grad_norm=max_grad_norm,
                         expected_batch_size=expected_batch_size, loss_reduction=loss_reduction,
                         generator=generator, secure_mode=secure_mode, **kwargs)
        self.process_group = process_group
        self._shard_generators = {}

    def _shard_generator(self, device):
        """This rank's generator for the noise of its shards (one per device, created at first use)."""
        if self.secure_mode:
            return self.generator          # a CSPRNG seeded from the OS: already independent between ranks
        gen = self._shard_generators.get(device)
        if gen is None:
            if self.generator is not None:
                base = int(self.generator.initial_seed())
            elif device.type == "cuda":
                base = int(torch.cuda.default_generators[device.index].initial_seed())
            else:
                base = int(torch.initial_seed())
            rank = dist.get_rank(self.process_group) if dist.is_initialized() else 0
            # splitmix-style fold: distinct ranks land on unrelated 63-bit seeds even for base seeds 0, 1, 2, ...
            z = (base + (rank + 1) * 0x9E3779B97F4A7C15) & 0xFFFFFFFFFFFFFFFF
            z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & 0xFFFFFFFFFFFFFFFF
            z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & 0xFFFFFFFFFFFFFFFF
            gen = torch.Generator(device=device)
            gen.manual_seed((z ^ (z >> 31)) & 0x7FFFFFFFFFFFFFFF)
            self._shard_generators[device] = gen
        return gen

    def add_noise(self):
        std = self._noise_std()
        group = self.process_group
        src = dist.get_global_rank(group, 0) if group is not None else 0
        first = (dist.get_rank(group) if dist.is_initialized() else 0) == 0
        for p in self.params:
            _check_processed_flag(p.summed_grad)
            if getattr(p, "sp_local", False):
                # each rank clipped and summed its own samples only: complete the sum over the group
                dist.all_reduce(p.summed_grad, op=dist.ReduceOp.SUM, group=group)
            if getattr(p, "tp_sharded", False):
                noise = _generate_noise(std=std, reference=p.summed_grad,
                                        generator=self._shard_generator(p.summed_grad.device),
                                        secure_mode=self.secure_mode)
            elif std == 0:
                noise = torch.zeros_like(p.summed_grad)
            else:
                if first:
                    noise = _generate_noise(std=std, reference=p.summed_grad, generator=self.generator,
                                            secure_mode=self.secure_mode)
                else:
                    noise = torch.empty_like(p.summed_grad)
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


def parallelize_llama(model, process_group=None, shard_lm_head: bool = True, sequence_parallel: bool = False,
                      fused: Optional[bool] = None):
    """Turn a :class:`opacus_b200.models.Llama` (replicated, identical on all ranks) into its
    1-d tensor-parallel form in place: q/k/v/gate/up become column-parallel, o/down
    row-parallel, heads are divided over the ranks; embedding and norm weights stay
    replicated; with ``shard_lm_head`` the output layer is split over the vocabulary
    (use :class:`VocabParallelCrossEntropy`).  Same layout as the reference's plan
    (``examples/tensor_parallelism_llama.py:104-152``).

    ``sequence_parallel``: between the tensor-parallel blocks (embedding, residual stream, norms) every rank
    keeps only its ``B / world`` samples.  ``q_proj`` / ``gate_proj`` and the output layer gather their input
    inside their GEMM (``AllGatherGemm``) and hand the gathered copy to ``k_proj`` / ``v_proj`` / ``up_proj``; the
    output projections reduce-scatter inside their GEMM (``GemmReduceScatter``) instead of all-reducing -- as fused
    kernels when ``fused`` (default: groups of 4 or more ranks) and the shapes allow, as NCCL + cuBLAS otherwise.  Embedding and
    norm weights then see only local samples: their per-sample norms are partial (``sp_local``) and their
    clipped sums are completed by an all-reduce in :class:`TensorParallelDPOptimizer`.  Needs
    ``shard_lm_head`` and a batch divisible by the group size."""
    world = _group_size(process_group)
    sp = sequence_parallel
    if fused is None:
        # measured on B200/NVLink 5: with 8 ranks the fused kernels beat NCCL + cuBLAS by 1.3-1.5x on these
        # shapes, with 2 ranks the collective is a small share and the library GEMM core wins
        fused = world >= 4
    if sp and not shard_lm_head:
        raise ValueError("sequence_parallel needs the output layer sharded over the vocabulary")
    for blk in model.layers:
        att, mlp = blk.self_attn, blk.mlp
        if att.n_heads % world or att.n_kv % world:
            raise ValueError(f"{att.n_heads} query / {att.n_kv} key-value heads do not divide over {world} ranks")
        for name in ("q_proj", "k_proj", "v_proj", "gate_proj", "up_proj"):
            owner = att if name in ("q_proj", "k_proj", "v_proj") else mlp
            first = name in ("q_proj", "gate_proj")            # gathers for its siblings (fused into its GEMM)
            layer = ColumnParallelLinear.from_linear(
                getattr(owner, name), process_group, input_mode=("local" if first else "gathered") if sp else "replicated",
                fused=fused, return_gathered=sp and first)
            setattr(owner, name, layer)
        att.o_proj = RowParallelLinear.from_linear(att.o_proj, process_group, scatter_output=sp, fused=fused)
        att.n_heads //= world
        att.n_kv //= world
        mlp.down_proj = RowParallelLinear.from_linear(mlp.down_proj, process_group, scatter_output=sp, fused=fused)
        if sp:
            for norm in (blk.input_layernorm, blk.post_attention_layernorm):
                _mark_sample_local(norm)
    if shard_lm_head:
        if model.lm_head.weight is model.embed_tokens.weight:
            raise ValueError("a tied output layer cannot be sharded over the vocabulary")
        model.lm_head = ColumnParallelLinear.from_linear(model.lm_head, process_group,
                                                         input_mode="local" if sp else "replicated", fused=fused)
    if sp:
        model.sp_slice = SampleSlice(process_group)
        _mark_sample_local(model.embed_tokens)
        _mark_sample_local(model.norm)
    return model


def _mark_sample_local(module):
    """``module`` runs on this rank's samples only: its per-sample quantities are partial over the group."""
    module.sp_local_input = True
    module.sp_local_region = True
    for p in module.parameters(recurse=False):
        p.sp_local = True
