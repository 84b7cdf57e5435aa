"""Linear layers whose weight is sharded over the data-parallel ranks at rest (the parameter-sharding half of
FSDP / ZeRO-3), for models whose bf16 weights plus fp32 gradients should not be replicated.

``ShardedLinear`` keeps ``out_features / world`` rows of the weight, in symmetric (peer-visible) memory.

* forward: ONE kernel (``csrc/tp_gemm.cu``, mode "all-gather of B's rows") pulls the peers' rows over NVLink into a
  local scratch copy while its tensor-core warps already multiply the rows that have arrived -- the parameter
  all-gather of FSDP fused into the first GEMM that consumes it.  The scratch copy belongs to a pool shared by all
  layers of the same shape, so at most a few whole weights exist per GPU at any time.
* backward: the input gradient needs the whole weight again; it is gathered a second time (same kernel, on a
  128-row dummy operand) and multiplied by the library GEMM (the operand is MN-major for that product).
* DP step: the layer's clipped gradient sum ``G^T diag(c) A`` is written into a symmetric fp32 scratch of the
  layer's shape, and the step kernel (``csrc/sharded_step.cu``) runs for this layer at once: every rank sums ITS
  rows over all ranks' scratch copies (reduce-scatter by peer loads or ``multimem.ld_reduce``), draws the noise for
  them, updates its fp32 master rows and moments and writes the new bf16 rows into its shard.  Neither a whole
  gradient nor a whole weight of such a layer is ever kept.

The reference gets parameter sharding from ``torch.distributed.fsdp.fully_shard`` applied per module
(``opacus/utils/fsdp_utils.py:39-61``) with NCCL all-gathers in front of every forward and backward and
reduce-scatters behind every backward (``opacus/optimizers/fsdpoptimizer_fast_gradient_clipping.py:138-181``).

Built by ``ShardedDataParallel(model, shard_params=True)`` / ``FSDP2Wrapper(model, shard_params=True)``; a layer
qualifies when it is a plain ``nn.Linear`` whose weight is not shared with another module,
``out_features % (256 * world) == 0`` and ``in_features % 16 == 0``.  Others stay in the engine's replicated
compute buffer.  Training such a model needs the single-pass ghost-clipping controller (``"ghost_fsdp"``); logical
batches split into several physical ones (``signal_skip_step``) are not supported in this mode.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from . import symm


def _kernels():
    from ..ops import _cuda

    return _cuda.load()


class _GatherSlot:
    """One whole-weight scratch buffer with the ready counters and flag words of the fused gather kernel; shared by
    all layers of one shape (they use it one after the other, in the same order on every rank)."""

    def __init__(self, N: int, K: int, device, group):
        self.full = torch.zeros(N, K, dtype=torch.bfloat16, device=device)
        self.ready = torch.zeros(N // 256, dtype=torch.int32, device=device)
        self.flags = symm.alloc(64, torch.int32, device, group)
        self.dummy = torch.zeros(128, K, dtype=torch.bfloat16, device=device)
        self.dummy_out = torch.empty(128, N, dtype=torch.bfloat16, device=device)
        self.epoch = 0
        self.holder = None          # the layer whose weight the buffer holds right now


class _ShardedLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight_shard, layer):
        ctx.layer = layer
        ctx.in_shape = x.shape
        ctx.in_dtype = x.dtype
        x2 = x.reshape(-1, layer.in_features).to(torch.bfloat16).contiguous()
        y = layer._gather_gemm(x2)
        return y.view(*x.shape[:-1], layer.out_features)

    @staticmethod
    def backward(ctx, gy):
        layer = ctx.layer
        full = layer._gathered_weight()
        gx = gy.reshape(-1, layer.out_features).to(torch.bfloat16) @ full
        # the weight's own gradient is the business of the DP engine (clipped sum from activations and output gradients)
        return gx.view(ctx.in_shape).to(ctx.in_dtype), None, None


class ShardedLinear(nn.Module):
    """``nn.Linear`` whose weight rows are divided over ``group``; ``weight`` is this rank's ``[out / world, in]``
    bf16 shard.  ``full_shape`` is the shape of the whole weight."""

    def __init__(self, linear: nn.Linear, group, slots: Dict[tuple, "_GatherSlot"]):
        super().__init__()
        self.group = group
        self.rank, self.world = symm.world_info(group)
        self.in_features, self.out_features = linear.in_features, linear.out_features
        N, K = self.out_features, self.in_features
        self.rows = N // self.world
        dev = linear.weight.device
        self._shard = symm.alloc(self.rows * K, torch.bfloat16, dev, group)
        mine = linear.weight.detach()[self.rank * self.rows:(self.rank + 1) * self.rows]
        self._shard.tensor.view(self.rows, K).copy_(mine.to(torch.bfloat16))
        self.weight = nn.Parameter(self._shard.tensor.view(self.rows, K), requires_grad=linear.weight.requires_grad)
        self.weight._dp_row_shard = self            # the engine keeps such parameters out of its flat space
        self.full_shape = (N, K)
        self.initial_master_rows = mine.float().clone()       # taken over (and dropped) by the engine
        self.bias = linear.bias
        key = (N, K)
        if key not in slots:
            slots[key] = _GatherSlot(N, K, dev, group)
        self._slot = slots[key]

    def extra_repr(self):
        return f"in_features={self.in_features}, out_features={self.out_features}, rows_here={self.rows}"

    # ---- the fused all-gather(W) -> GEMM
    def _launch(self, x2: torch.Tensor, out: torch.Tensor):
        slot = self._slot
        slot.epoch += 1
        slot.holder = None
        _kernels().tp_gemm(x2, slot.full, out, 2, self._shard.ptrs, [], slot.flags.ptrs, slot.ready, self.rank,
                           self.world, slot.epoch, 0)
        slot.holder = self

    def _gather_gemm(self, x2: torch.Tensor) -> torch.Tensor:
        out = torch.empty(x2.shape[0], self.out_features, dtype=torch.bfloat16, device=x2.device)
        self._launch(x2, out)
        return out

    def _gathered_weight(self) -> torch.Tensor:
        """The whole weight in the pool buffer (gathered again unless this layer was the buffer's last user)."""
        slot = self._slot
        if slot.holder is not self:
            self._launch(slot.dummy, slot.dummy_out)
        return slot.full

    def forward(self, x):
        y = _ShardedLinearFn.apply(x, self.weight, self)
        return y if self.bias is None else y + self.bias.to(y.dtype)


def eligible(module: nn.Linear, world: int, shared: set) -> bool:
    return (type(module) is nn.Linear and module.weight.is_cuda and id(module.weight) not in shared
            and module.out_features % (256 * world) == 0 and module.in_features % 16 == 0
            and module.weight.requires_grad)


def shard_linears(model: nn.Module, group) -> List[ShardedLinear]:
    """Replace every eligible ``nn.Linear`` of ``model`` in place; returns the new layers in module order."""
    _, world = symm.world_info(group)
    seen, shared = {}, set()
    for m in model.modules():
        for p in m.parameters(recurse=False):
            seen[id(p)] = seen.get(id(p), 0) + 1
    shared = {k for k, v in seen.items() if v > 1}
    slots: Dict[tuple, _GatherSlot] = {}
    made: List[ShardedLinear] = []

    def walk(parent):
        for name, child in list(parent.named_children()):
            if isinstance(child, nn.Linear) and eligible(child, world, shared):
                new = ShardedLinear(child, group, slots)
                setattr(parent, name, new)
                made.append(new)
            else:
                walk(child)

    walk(model)
    if world > 1:
        dist.barrier(group=group)           # every shard is written before any rank's first gather
    return made


def _register_rules():
    """Ghost-clipping rules of :class:`ShardedLinear`: the per-sample norm is the Linear one (it needs activations
    and output gradients only); the clipped sum goes through the engine, which reduce-scatters and steps the layer
    at once.  Materialised per-sample gradients (hooks mode) are not offered for sharded weights."""
    from ..grad_sample.utils import register_grad_sampler, register_norm_sq_sampler, register_wgrad_sampler

    def norm_sq(layer, activations, backprops, g_scale: float = 1.0, total=None):
        from .. import ops

        want_b = layer.bias is not None and layer.bias.requires_grad
        if total is not None:
            ops.linear_norm_sq(activations[0], backprops, True, want_b, g_scale, total=total)
            return {}
        nw, nb = ops.linear_norm_sq(activations[0], backprops, True, want_b, g_scale)
        out = {layer.weight: nw}
        if want_b:
            out[layer.bias] = nb
        return out

    def wgrad(layer, activations, backprops, coef, g_scale: float = 1.0):
        engine = getattr(layer, "_dp_engine", None)
        if engine is None:
            raise RuntimeError("a ShardedLinear can only be trained under the ShardedDataParallel engine that made it")
        engine.step_row_layer(layer, activations[0], backprops, coef, g_scale)
        out = {}
        if layer.bias is not None and layer.bias.requires_grad:
            B = backprops.shape[0]
            per = backprops.reshape(B, -1, backprops.shape[-1]).sum(dim=1).float()
            out[layer.bias] = (per * (coef.float() * g_scale)[:, None]).sum(dim=0)
        return out

    def grad_sample(layer, activations, backprops):
        raise NotImplementedError("per-sample gradients of a row-sharded weight are not materialised; use "
                                  "grad_sample_mode='ghost_fsdp'")

    register_norm_sq_sampler(ShardedLinear)(norm_sq)
    register_wgrad_sampler(ShardedLinear)(wgrad)
    register_grad_sampler(ShardedLinear)(grad_sample)


_register_rules()
