"""Sharded data-parallel engine (the native form of "FSDP + ghost clipping").

Layout, sized for GPUs with far more memory than a billion-parameter model
needs: the *compute* copy of the parameters (bf16 by default) is whole on every
GPU, in one flat buffer that peers can write; the fp32 master weights and the
optimiser state exist only for the slice of the flat space a rank owns
(``1/world`` each); clipped gradient sums are written by the ghost-clipping
engine straight into a flat fp32 buffer that peers can read.

A training step then needs no collective during forward or backward, and one
kernel at the end (``csrc/sharded_step.cu``): reduce-scatter of the gradient
sums over NVLink, one Gaussian draw per owned element, scaling, the SGD / Adam /
AdamW update of the owned slice, and the all-gather of the new weights into
every GPU's compute buffer -- all inside the same launch.

The reference obtains the same state sharding from ``torch`` FSDP2 at the cost
of three parameter all-gathers and two gradient reduce-scatters per step
(``opacus/utils/fsdp_utils.py:39-61``,
``opacus/optimizers/fsdpoptimizer_fast_gradient_clipping.py:32-181``).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from . import symm

_ALIGN = 64           # every parameter starts on a 64-element boundary of the flat space
_SLICE_QUANTUM = 1024


class ShardedDataParallel(nn.Module):
    """``process_group`` is the data-parallel group (ranks that hold the same parameters and see different
    samples).  ``tp_group`` is the tensor-parallel group this rank also belongs to, when the module was sharded
    by :mod:`opacus_b200.parallel.tensor_parallel` (2-D layout: every tensor-parallel rank runs this engine over
    its own data-parallel group).  Parameters marked ``tp_sharded`` then draw their noise from a Philox range of
    their tensor-parallel rank, all others from a range common to the tensor-parallel group under a seed the
    group agrees on, so that shards get independent noise and replicas stay bit-identical."""

    def __init__(self, module: nn.Module, *, param_dtype: torch.dtype = torch.bfloat16, process_group=None,
                 tp_group=None, **unused):
        super().__init__()
        first = next(module.parameters())
        if not first.is_cuda:
            raise ValueError("ShardedDataParallel needs the model on a CUDA device")
        self.module = module
        self.process_group = process_group
        self.rank, self.world = symm.world_info(process_group)
        if self.world > 8:
            raise NotImplementedError("one NVLink domain of at most 8 GPUs is supported")
        why = symm.available(process_group)
        if why is not None:
            raise RuntimeError(f"ShardedDataParallel cannot set up peer memory: {why}")
        if param_dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("param_dtype must be torch.bfloat16 or torch.float32")
        self.param_dtype = param_dtype
        dev = first.device

        # ---- flat layout over the distinct trainable parameters
        self._params: List[nn.Parameter] = []
        self._offsets: Dict[nn.Parameter, int] = {}
        self.tp_group = tp_group
        self.tp_rank, self.tp_world = symm.world_info(tp_group) if tp_group is not None else (0, 1)
        distinct = []
        for p in module.parameters():
            if p.requires_grad and not any(p is q for q in distinct):
                distinct.append(p)
        shards = [p for p in distinct if getattr(p, "tp_sharded", False)]
        if shards and tp_group is None:
            # Ranks of a tensor-parallel group run this engine with the same flat layout; under one seed two shards
            # of one weight would receive the SAME noise values, and correlated noise is not the Gaussian mechanism.
            raise ValueError("the module holds tensor-parallel shards: pass tp_group= so that they draw independent noise")
        total = 0
        self.noise_split = None
        # replicated parameters first, shards behind them: one split point separates the two noise ranges
        for p in [q for q in distinct if not getattr(q, "tp_sharded", False)] + shards:
            if shards and p is shards[0]:
                self.noise_split = total
            self._offsets[p] = total
            self._params.append(p)
            total += (p.numel() + _ALIGN - 1) // _ALIGN * _ALIGN
        # sums of parameters that saw only this tensor-parallel rank's samples are completed before the step
        self._tp_partial = [p for p in distinct if getattr(p, "sp_local", False)] if tp_group is not None else []
        self._tp_seed = None
        self.slice_len = (math.ceil(total / self.world) + _SLICE_QUANTUM - 1) // _SLICE_QUANTUM * _SLICE_QUANTUM
        self.total = self.slice_len * self.world
        self.slice_begin = self.rank * self.slice_len

        self._flat_param = symm.alloc(self.total, param_dtype, dev, process_group)
        self._flat_grad = symm.alloc(self.total, torch.float32, dev, process_group)
        self._flags = symm.alloc(64, torch.int32, dev, process_group)

        # ---- identical start on every rank, then adopt the flat storage
        full = torch.zeros(self.total, dtype=torch.float32, device=dev)
        for p in self._params:
            o = self._offsets[p]
            full[o: o + p.numel()].copy_(p.data.reshape(-1).float())
        if self.world > 1:
            dist.broadcast(full, dist.get_global_rank(process_group, 0) if process_group is not None else 0,
                           group=process_group)
        self.master = full[self.slice_begin: self.slice_begin + self.slice_len].clone()
        self._flat_param.tensor.copy_(full.to(param_dtype))
        del full
        for p in self._params:
            o = self._offsets[p]
            p.data = self._flat_param.tensor[o: o + p.numel()].view(p.shape)
            p._dp_grad_out = self._flat_grad.tensor[o: o + p.numel()].view(p.shape)
            p._dp_grad_fresh = True
        for p in module.parameters():        # frozen parameters follow the compute dtype
            if not p.requires_grad and p.is_floating_point():
                p.data = p.data.to(param_dtype)
        for b in module.buffers():
            if b.is_floating_point():
                b.data = b.data.to(param_dtype)
        self.state0: Optional[torch.Tensor] = None
        self.state1: Optional[torch.Tensor] = None
        self._epoch = 0
        self._steps = 0
        if self.world > 1:
            dist.barrier(group=process_group)

    # ------------------------------------------------------------------ module API
    def forward(self, *args, **kwargs):
        return self.module(*args, **kwargs)

    def mark_grads_fresh(self):
        """The next clipped-gradient write overwrites instead of accumulating."""
        for p in self._params:
            p._dp_grad_fresh = True

    def flat_grad(self) -> torch.Tensor:
        return self._flat_grad.tensor

    def finish_grads(self):
        """Zero the gradient of parameters that received none in this step."""
        for p in self._params:
            if p._dp_grad_fresh:
                p._dp_grad_out.zero_()
                p._dp_grad_fresh = False

    def full_precision_state_dict(self) -> Dict[str, torch.Tensor]:
        """fp32 master weights of the whole model, gathered from their owners (collective)."""
        if self.world > 1:
            pieces = [torch.empty_like(self.master) for _ in range(self.world)]
            dist.all_gather(pieces, self.master, group=self.process_group)
            full = torch.cat(pieces)
        else:
            full = self.master
        out = {}
        for name, p in self.module.named_parameters():
            if p in self._offsets:
                o = self._offsets[p]
                out[name] = full[o: o + p.numel()].view(p.shape).clone()
            else:
                out[name] = p.detach().clone()
        return out

    # ------------------------------------------------------------------ the step
    def optimizer_step(self, dpopt, closure=None):
        """Tail of ``FSDPOptimizerFastGradientClipping.step`` when this engine owns the parameters."""
        from ..utils.tracing import phase

        with phase("dp/optimizer_step"):
            return self._optimizer_step(dpopt, closure)

    def _optimizer_step(self, dpopt, closure=None):
        from ..ops import _cuda

        if closure is not None:
            with torch.enable_grad():
                closure()
        self.finish_grads()
        if dpopt._check_skip_next_step():
            dpopt._is_last_step_skipped = True
            return None
        inner = dpopt.original_optimizer
        groups = inner.param_groups
        g0 = groups[0]
        kind = {torch.optim.SGD: "sgd", torch.optim.Adam: "adam", torch.optim.AdamW: "adamw"}.get(type(inner))
        if kind is None:
            raise NotImplementedError(f"the sharded engine implements SGD, Adam and AdamW, not {type(inner).__name__}")
        keys = ("lr", "weight_decay", "momentum", "dampening", "nesterov", "betas", "eps")
        for g in groups[1:]:
            if any(g.get(k) != g0.get(k) for k in keys):
                raise NotImplementedError("the sharded engine needs identical hyper-parameters in all param groups")
        if g0.get("amsgrad") or g0.get("maximize"):
            raise NotImplementedError("amsgrad / maximize are not implemented in the sharded engine")
        if kind == "adam" and g0.get("decoupled_weight_decay"):
            kind = "adamw"

        self._steps += 1
        self._epoch += 1
        t = self._steps
        dev = self.master.device
        h = dict(lr=float(g0["lr"]), momentum=0.0, dampening=0.0, weight_decay=float(g0.get("weight_decay", 0.0)),
                 beta1=0.0, beta2=0.0, eps=0.0, bias_c1=1.0, bias_c2_sqrt=1.0)
        first_step, nesterov, kcode = False, False, 0
        if kind == "sgd":
            h["momentum"] = float(g0.get("momentum", 0.0))
            h["dampening"] = float(g0.get("dampening", 0.0))
            nesterov = bool(g0.get("nesterov", False))
            if h["momentum"] != 0.0 and self.state0 is None:
                self.state0 = torch.zeros(self.slice_len, dtype=torch.float32, device=dev)
                first_step = True
        else:
            b1, b2 = g0["betas"]
            if self.state0 is None:
                self.state0 = torch.zeros(self.slice_len, dtype=torch.float32, device=dev)
                self.state1 = torch.zeros(self.slice_len, dtype=torch.float32, device=dev)
            h.update(beta1=float(b1), beta2=float(b2), eps=float(g0["eps"]), bias_c1=1.0 - float(b1) ** t,
                     bias_c2_sqrt=math.sqrt(1.0 - float(b2) ** t))
            kcode = 2 if kind == "adamw" else 1

        # per-worker expected batch (times accumulated batches in hooks mode), summed over the workers
        denom = float(dpopt._grad_denominator()) * (self.world if dpopt.loss_reduction == "mean" else 1)
        if dpopt.step_hook:
            dpopt.step_hook(dpopt)
        seed, offset = _cuda._rng_state(dpopt.generator, dev, self.total * self.tp_world)
        noise_shift = 0
        if self.tp_group is not None:
            for p in self._tp_partial:
                dist.all_reduce(p._dp_grad_out, op=dist.ReduceOp.SUM, group=self.tp_group)
            if self._tp_seed is None:      # the group adopts its first rank's generator state, once
                state = torch.tensor([seed, offset], dtype=torch.int64, device=dev)
                dist.broadcast(state, dist.get_global_rank(self.tp_group, 0), group=self.tp_group)
                self._tp_seed = (int(state[0]), int(state[1]) - offset)
            seed, offset = self._tp_seed[0], offset + self._tp_seed[1]
            noise_shift = self.tp_rank * self.total if self.noise_split is not None else 0
        C = _cuda.load()
        C.sharded_dp_step(self._flat_grad.ptrs, self._flat_param.ptrs, self._flags.ptrs, self.master, self.state0,
                          self.state1, self.slice_begin, self.slice_len, self.rank,
                          self.param_dtype == torch.bfloat16, self._epoch, kcode, nesterov, first_step,
                          h["lr"], h["momentum"], h["dampening"], h["weight_decay"], h["beta1"], h["beta2"], h["eps"],
                          h["bias_c1"], h["bias_c2_sqrt"], float(dpopt._noise_std()), 1.0 / denom, seed, offset,
                          self.noise_split if noise_shift else 0, noise_shift)
        dpopt._is_last_step_skipped = False
        self.mark_grads_fresh()
        return None
