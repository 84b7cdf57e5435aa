"""Sharded data-parallel engine (the native form of "FSDP + ghost clipping").

Layout, sized for GPUs with far more memory than a billion-parameter model
needs: the *compute* copy of the parameters (bf16 by default) is whole on every
GPU, in one flat buffer that peers can write; the fp32 master weights and the
optimiser state exist only for the share of the flat space a rank owns
(``1/world`` each); clipped gradient sums are written by the ghost-clipping
engine straight into a flat fp32 buffer that peers can read.

The flat space is cut into ``pieces`` equal pieces and every rank owns one
*stripe* (``1/world``) of every piece.  A training step needs no collective
during forward or backward.  Its tail is the kernel of ``csrc/sharded_step.cu``:
reduce-scatter of the gradient sums over NVLink (one ``multimem.ld_reduce`` per
16 bytes when the buffers are bound to an NVLink multicast object, plain peer
loads otherwise), one Gaussian draw per owned element, scaling, the SGD / Adam /
AdamW update of the owned stripes, and the all-gather of the new weights into
every GPU's compute buffer (``multimem.st`` or peer stores).  With several ranks
the kernel is launched piece by piece on a side stream, each piece as soon as
the clipped sums that land in it are complete, so that the NVLink traffic runs
beside the remaining weight-gradient GEMMs instead of after them.

The reference obtains the same state sharding from ``torch`` FSDP2 at the cost
of three parameter all-gathers and two gradient reduce-scatters per step
(``opacus/utils/fsdp_utils.py:39-61``,
``opacus/optimizers/fsdpoptimizer_fast_gradient_clipping.py:32-181``).

Checkpoints: :meth:`state_dict` returns the fp32 master weights under the wrapped
module's own keys, :meth:`optimizer_state_dict` the optimiser state in the
``torch.optim`` layout (both gather from the owners: collective calls);
loading either refreshes the sharded fp32 state, so a resumed run continues
bit for bit (``opacus/privacy_engine.py:618-696`` is the file format).
"""
from __future__ import annotations

import math
import os
from typing import Dict, List, Optional

import numpy as np
import torch
import torch.distributed as dist
import torch.nn as nn

from . import symm

_ALIGN = 64           # every parameter starts on a 64-element boundary of the flat space
_STRIPE_QUANTUM = 1024
_KINDS = {torch.optim.SGD: "sgd", torch.optim.Adam: "adam", torch.optim.AdamW: "adamw"}
_SEGMENT = np.dtype([("end", "<i8"), ("lr", "<f4"), ("weight_decay", "<f4")])


class ShardedDataParallel(nn.Module):
    """``process_group`` is the data-parallel group (ranks that hold the same parameters and see different
    samples).  ``tp_group`` is the tensor-parallel group this rank also belongs to, when the module was sharded
    by :mod:`opacus_b200.parallel.tensor_parallel` (2-D layout: every tensor-parallel rank runs this engine over
    its own data-parallel group).  Parameters marked ``tp_sharded`` then draw their noise from a Philox range of
    their tensor-parallel rank, all others from a range common to the tensor-parallel group under a seed the
    group agrees on, so that shards get independent noise and replicas stay bit-identical.

    ``step_pieces``: into how many pieces the flat space is cut (default: 16 with several ranks and a model of
    at least a few million parameters, else 1).  ``multicast``: use the NVLink multicast address of the buffers
    when there is one (default: for groups of 4 or more ranks; ``True`` / ``False`` or ``OPACUS_B200_MULTICAST=1`` /
    ``0`` force it on where available / off)."""

    def __init__(self, module: nn.Module, *, param_dtype: torch.dtype = torch.bfloat16, process_group=None,
                 tp_group=None, step_pieces: Optional[int] = None, multicast: Optional[bool] = None,
                 shard_params: bool = False, **unused):
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
        # ---- optional parameter sharding: eligible Linear layers keep only their rows of the weight (see
        # parallel/param_sharding.py); their parameters live outside the flat space and are stepped layer by layer
        self._row_layers = []
        if shard_params:
            if tp_group is not None:
                raise NotImplementedError("shard_params together with a tensor-parallel group")
            from .param_sharding import shard_linears

            self._row_layers = shard_linears(module, process_group)
        distinct = []
        for p in module.parameters():
            if getattr(p, "_dp_row_shard", None) is not None:
                continue
            if p.requires_grad and not any(p is q for q in distinct):
                distinct.append(p)
        shards = [p for p in distinct if getattr(p, "tp_sharded", False)]
        if shards and tp_group is None:
            # Ranks of a tensor-parallel group run this engine with the same flat layout; under one seed two shards
            # of one weight would receive the SAME noise values, and correlated noise is not the Gaussian mechanism.
            raise ValueError("the module holds tensor-parallel shards: pass tp_group= so that they draw independent noise")
        used = 0
        self.noise_split = None
        # replicated parameters first, shards behind them: one split point separates the two noise ranges
        for p in [q for q in distinct if not getattr(q, "tp_sharded", False)] + shards:
            if shards and p is shards[0]:
                self.noise_split = used
            self._offsets[p] = used
            self._params.append(p)
            used += (p.numel() + _ALIGN - 1) // _ALIGN * _ALIGN
        self.used = used
        # sums of parameters that saw only this tensor-parallel rank's samples are completed before the step
        self._tp_partial = [p for p in distinct if getattr(p, "sp_local", False)] if tp_group is not None else []
        self._tp_seed = None

        # ---- pieces and stripes: piece k is [k * piece_len, (k + 1) * piece_len), rank r owns its r-th stripe
        if step_pieces is None:
            step_pieces = int(os.environ.get("OPACUS_B200_STEP_PIECES", "0")) or (16 if self.world > 1 else 1)
            step_pieces = max(1, min(step_pieces, used // (self.world * (1 << 18))))
        self.pieces = int(step_pieces)
        if self.pieces < 1:
            raise ValueError("step_pieces must be at least 1")
        cells = self.pieces * self.world
        self.stripe = (math.ceil(max(used, 1) / cells) + _STRIPE_QUANTUM - 1) // _STRIPE_QUANTUM * _STRIPE_QUANTUM
        self.piece_len = self.stripe * self.world
        self.total = self.piece_len * self.pieces
        self.slice_len = self.stripe * self.pieces            # elements this rank owns

        self._flat_param = symm.alloc(self.total, param_dtype, dev, process_group)
        self._flat_grad = symm.alloc(self.total, torch.float32, dev, process_group)
        self._flags = symm.alloc(64, torch.int32, dev, process_group)
        if multicast is None:
            # measured on NVLink 5 / NVSwitch: with 2 ranks the in-switch reduction is slower than plain peer loads
            # (every rank's own copy crosses its link too); from 4 ranks on it is at least as fast
            env = os.environ.get("OPACUS_B200_MULTICAST", "")
            multicast = self.world >= 4 if env == "" else env != "0"
        self.multicast = bool(multicast) and self.world > 1 and self._flat_param.mc_ptr != 0 \
            and self._flat_grad.mc_ptr != 0
        if self.world > 1:                 # all ranks take the same path or none
            flag = torch.tensor([1 if self.multicast else 0], device=dev)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=process_group)
            self.multicast = bool(flag.item())
        # the two uses of the multicast address can be chosen separately: the in-switch reduction of the gradient
        # (multimem.ld_reduce) and the replicated store of the new weights (multimem.st)
        self.multicast_reduce = os.environ.get("OPACUS_B200_MC_REDUCE", "1") != "0"
        self.multicast_publish = os.environ.get("OPACUS_B200_MC_PUBLISH", "1") != "0"

        # ---- identical start on every rank, then adopt the flat storage
        full = torch.zeros(self.total, dtype=torch.float32, device=dev)
        for p in self._params:
            o = self._offsets[p]
            full[o: o + p.numel()].copy_(p.data.reshape(-1).float())
        if self.world > 1:
            dist.broadcast(full, dist.get_global_rank(process_group, 0) if process_group is not None else 0,
                           group=process_group)
        self.master = self._share_of(full).clone()
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
        self._init_row_layers(dev)
        self._epoch = 0
        self._steps = 0
        self._step_stream = None
        self._segments = None            # (key, device table) of the per-group hyper-parameter ranges
        self._loading = None
        self.last_step_launches = 0
        self.register_load_state_dict_pre_hook(self._before_load)
        self.register_load_state_dict_post_hook(self._after_load)
        module.register_load_state_dict_post_hook(self._after_inner_load)
        if self.world > 1:
            dist.barrier(group=process_group)

    # ------------------------------------------------------------------ row-sharded layers
    def _init_row_layers(self, dev):
        self._row_scratch: Dict[tuple, symm.SymmetricBuffer] = {}
        self._row_flags = None
        self._row_epoch = 0
        self._row_pass = None            # per logical step: the launch arguments shared by all layers
        self._dpopt = None
        base = self.total
        for layer in self._row_layers:
            layer.__dict__["_dp_engine"] = self           # plain attribute: the engine is not a submodule of the layer
            layer.master = layer.initial_master_rows.reshape(-1).contiguous()
            del layer.initial_master_rows
            layer.state0 = layer.state1 = None
            layer.noise_base = base                       # Philox counters of this weight: noise_base + index in it
            layer.stepped = False
            base += layer.full_shape[0] * layer.full_shape[1]
            key = tuple(layer.full_shape)
            if key not in self._row_scratch:
                self._row_scratch[key] = symm.alloc(key[0] * key[1], torch.float32, dev, self.process_group, zero=False)
        if self._row_layers:
            self._row_flags = symm.alloc(64, torch.int32, dev, self.process_group)

    def attach_optimizer(self, dpopt):
        """The DP optimizer whose hyper-parameters the layer-by-layer steps of row-sharded layers read."""
        self._dpopt = dpopt

    def _row_pass_args(self):
        """Launch arguments common to the row-sharded layers of one logical step (made at the first layer)."""
        if self._row_pass is not None:
            return self._row_pass
        from ..ops import _cuda

        dpopt = self._dpopt
        if dpopt is None:
            raise RuntimeError("row-sharded layers need the optimizer attached to the engine "
                               "(FSDPOptimizerFastGradientClipping(..., engine=engine) does it)")
        if dpopt._check_skip_next_step(pop_next=False):
            raise NotImplementedError("logical batches split into several physical ones are not supported with "
                                      "shard_params=True (the clipped sums of a sharded layer are consumed at once)")
        if getattr(dpopt, "secure_mode", False):
            raise NotImplementedError("secure_mode with shard_params=True")
        inner = dpopt.original_optimizer
        kind, g0, _ = self._hyper(inner)
        t = self._steps + 1
        h = dict(momentum=0.0, dampening=0.0, beta1=0.0, beta2=0.0, eps=0.0, bias_c1=1.0, bias_c2_sqrt=1.0)
        nesterov, kcode = False, 0
        if kind == "sgd":
            h["momentum"] = float(g0.get("momentum", 0.0))
            h["dampening"] = float(g0.get("dampening", 0.0))
            nesterov = bool(g0.get("nesterov", False))
        else:
            b1, b2 = g0["betas"]
            h.update(beta1=float(b1), beta2=float(b2), eps=float(g0["eps"]), bias_c1=1.0 - float(b1) ** t,
                     bias_c2_sqrt=math.sqrt(1.0 - float(b2) ** t))
            kcode = 2 if kind == "adamw" else 1
        group_of = {}
        for g in inner.param_groups:
            for p in g["params"]:
                group_of[p] = g
        denom = float(dpopt._grad_denominator()) * (self.world if dpopt.loss_reduction == "mean" else 1)
        n_row = sum(l.full_shape[0] * l.full_shape[1] for l in self._row_layers)
        seed, offset = _cuda._rng_state(dpopt.generator, self.master.device, n_row)
        self._row_pass = dict(kind=kind, kcode=kcode, nesterov=nesterov, h=h, group_of=group_of,
                              noise_std=float(dpopt._noise_std()), inv_scale=1.0 / denom, seed=seed, offset=offset)
        return self._row_pass

    def step_row_layer(self, layer, activations, backprops, coef, g_scale: float):
        """Clipped sum of a row-sharded layer into the symmetric scratch of its shape, then at once the step
        kernel for this layer: reduce-scatter over the ranks (each rank sums its rows), noise, update of the fp32
        master rows and moments, new bf16 rows into the shard."""
        from .. import ops
        from ..ops import _cuda

        a = self._row_pass_args()
        N, K = layer.full_shape
        scratch = self._row_scratch[(N, K)]
        ops.linear_weighted_grad(activations, backprops, coef, g_scale, want_bias=False,
                                 out=scratch.tensor.view(N, K), accumulate=False)
        dev = layer.master.device
        h, kind = a["h"], a["kind"]
        first_step = False
        if kind == "sgd":
            if h["momentum"] != 0.0 and layer.state0 is None:
                layer.state0 = torch.zeros_like(layer.master)
                first_step = True
        elif layer.state0 is None:
            layer.state0, layer.state1 = torch.zeros_like(layer.master), torch.zeros_like(layer.master)
        group = a["group_of"].get(layer.weight)
        if group is None:
            raise RuntimeError("a row-sharded weight is missing from the optimizer's parameter groups")
        begin = self.rank * layer.rows * K
        n = layer.rows * K
        # the kernel addresses the compute copy as param[r] + index in the whole weight: every entry is this rank's
        # shard moved back by the offset of its first row, so all writes land in the shard itself
        shifted = layer.weight.data_ptr() - begin * layer.weight.element_size()
        self._row_epoch += 1
        mc = scratch.mc_ptr if (self.multicast and self.multicast_reduce) else 0
        _cuda.load().sharded_dp_step(
            scratch.ptrs, [shifted] * self.world, self._row_flags.ptrs, layer.master, layer.state0, layer.state1,
            begin, n, self.rank, True, self._row_epoch, a["kcode"], a["nesterov"], first_step, float(group["lr"]),
            h["momentum"], h["dampening"], float(group.get("weight_decay", 0.0)), h["beta1"], h["beta2"], h["eps"],
            h["bias_c1"], h["bias_c2_sqrt"], a["noise_std"], a["inv_scale"], a["seed"], a["offset"], 0,
            layer.noise_base, mc, 0, None, 0, 0, 0)
        layer.stepped = True
        layer._slot.holder = None if layer._slot.holder is layer else layer._slot.holder   # the pool copy is stale

    def _finish_row_layers(self):
        """End of a logical step: every row-sharded layer must have been stepped in this pass."""
        if not self._row_layers:
            return
        missing = [l for l in self._row_layers if not l.stepped]
        if missing and any(l.stepped for l in self._row_layers):
            raise RuntimeError(f"{len(missing)} row-sharded layers received no gradient in this step")
        for l in self._row_layers:
            l.stepped = False
        self._row_pass = None

    def _gather_rows(self, layer, rows: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """Whole ``[N, K]`` fp32 tensor from every rank's ``[rows * K]`` vector (collective)."""
        if rows is None:
            return None
        if self.world == 1:
            return rows.view(layer.full_shape).clone()
        parts = [torch.empty_like(rows) for _ in range(self.world)]
        dist.all_gather(parts, rows.contiguous(), group=self.process_group)
        return torch.cat(parts).view(layer.full_shape)

    # ------------------------------------------------------------------ layout helpers
    def _share_of(self, full: torch.Tensor) -> torch.Tensor:
        """This rank's stripes of a ``[total]`` tensor, concatenated in piece order (a view when ``world == 1``)."""
        return full.view(self.pieces, self.world, self.stripe)[:, self.rank].reshape(-1)

    def _gather(self, share: torch.Tensor) -> torch.Tensor:
        """``[total]`` tensor in flat order from every rank's share (collective)."""
        if self.world == 1:
            return share
        parts = [torch.empty_like(share) for _ in range(self.world)]
        dist.all_gather(parts, share.contiguous(), group=self.process_group)
        return torch.stack(parts).view(self.world, self.pieces, self.stripe).permute(1, 0, 2).reshape(-1)

    def _named_trainable(self):
        """(name, parameter) for every name under which a parameter of the flat space is reachable."""
        for name, p in self.module.named_parameters(remove_duplicate=False):
            if p in self._offsets:
                yield name, p

    # ------------------------------------------------------------------ module API
    def forward(self, *args, **kwargs):
        return self.module(*args, **kwargs)

    def mark_grads_fresh(self):
        """The next clipped-gradient write overwrites instead of accumulating."""
        for p in self._params:
            p._dp_grad_fresh = True
            p.__dict__.pop("_dp_ready", None)

    def flat_grad(self) -> torch.Tensor:
        return self._flat_grad.tensor

    def flat_param(self) -> torch.Tensor:
        return self._flat_param.tensor

    def finish_grads(self):
        """Zero the gradient of parameters that received none in this step."""
        for p in self._params:
            if p._dp_grad_fresh:
                p._dp_grad_out.zero_()
                p._dp_grad_fresh = False

    # ------------------------------------------------------------------ checkpoints
    def full_precision_state_dict(self) -> Dict[str, torch.Tensor]:
        """fp32 master weights of the whole model, gathered from their owners (collective)."""
        full = self._gather(self.master)
        out = {}
        for name, p in self.module.named_parameters():
            layer = getattr(p, "_dp_row_shard", None)
            if p in self._offsets:
                o = self._offsets[p]
                out[name] = full[o: o + p.numel()].view(p.shape).clone()
            elif layer is not None:
                out[name] = self._gather_rows(layer, layer.master)       # the whole [N, K] weight
            else:
                out[name] = p.detach().clone()
        return out

    def state_dict(self, *args, destination=None, prefix="", keep_vars=False):
        """The wrapped module's ``state_dict`` (its own keys, no extra prefix) with every trainable parameter in
        fp32 master precision.  The module's own ``state_dict`` runs while its parameters point at the gathered
        fp32 values, so key renaming or packing done by a layer (``DPMultiheadAttention`` writes ``in_proj_weight``)
        applies to the master weights as well.  Collective: all ranks of the group call it."""
        full = self._gather(self.master)
        if full.data_ptr() == self.master.data_ptr():
            full = full.clone()
        rows = {l.weight: self._gather_rows(l, l.master) for l in self._row_layers}
        with self._parameters_as(full, rows):
            sd = self.module.state_dict(*args, destination=destination, prefix=prefix, keep_vars=keep_vars)
            if not keep_vars:
                for k, v in list(sd.items()):      # nothing in the result may alias a Parameter that is switched back
                    if isinstance(v, nn.Parameter):
                        sd[k] = v.detach()
        return sd

    class _Swap:
        def __init__(self, engine, full, rows=None):
            self.engine, self.full, self.rows, self.saved = engine, full, rows or {}, []

        def __enter__(self):
            eng = self.engine
            for p in eng._params:
                o = eng._offsets[p]
                self.saved.append((p, p.data))
                p.data = self.full[o: o + p.numel()].view(p.shape)
            for p, whole in self.rows.items():           # row-sharded weights appear with their whole shape
                self.saved.append((p, p.data))
                p.data = whole
            return self

        def __exit__(self, *exc):
            for p, data in self.saved:
                p.data = data
            self.saved = []
            return False

    def _parameters_as(self, full: torch.Tensor, rows=None):
        """Context: every trainable parameter's ``.data`` is its range of the fp32 ``[total]`` tensor ``full``
        (row-sharded weights: the whole fp32 ``[N, K]`` tensor given for them in ``rows``)."""
        return ShardedDataParallel._Swap(self, full, rows)

    def _before_load(self, module, state_dict, prefix, *unused):
        """Keys come without the ``module.`` level (as :meth:`state_dict` writes them, and as a checkpoint of the
        bare model has them).  While the wrapped module loads, its parameters point at an ordinary fp32 buffer:
        the values arrive in full precision whatever the layers' own loading code does with the keys, and the
        copies never target the peer-mapped compute buffer (a copy from another GPU of this process into it would
        be executed by that GPU, which has no access to the mapping)."""
        own = prefix + "module."
        for key in [k for k in state_dict if k.startswith(prefix) and not k.startswith(own)]:
            state_dict[own + key[len(prefix):]] = state_dict.pop(key)
        full = self._flat_param.tensor.float()
        self._share_of(full).copy_(self.master)          # what this rank owns keeps its full precision
        rows = {l.weight: torch.zeros(l.full_shape, dtype=torch.float32, device=full.device) for l in self._row_layers}
        for l in self._row_layers:                       # rows this rank owns start from their current values
            rows[l.weight][self.rank * l.rows:(self.rank + 1) * l.rows].copy_(l.master.view(l.rows, -1))
        self._loading = self._parameters_as(full, rows)
        self._loading.__enter__()

    def _after_load(self, module, incompatible_keys):
        loading, self._loading = self._loading, None
        if loading is None:
            return
        loading.__exit__()
        with torch.no_grad():
            self.master.copy_(self._share_of(loading.full))
            self._flat_param.tensor.copy_(loading.full.to(self.param_dtype))
            for l in self._row_layers:
                mine = loading.rows[l.weight][self.rank * l.rows:(self.rank + 1) * l.rows]
                l.master.copy_(mine.reshape(-1))
                l.weight.data.copy_(mine.to(l.weight.dtype))
                l._slot.holder = None
        if self._row_layers and self.world > 1:
            dist.barrier(group=self.process_group)       # every shard is rewritten before any rank gathers again

    def _after_inner_load(self, module, incompatible_keys):
        if self._loading is None:            # loaded through the wrapped module directly: compute precision only
            self.refresh_master(None)

    @torch.no_grad()
    def refresh_master(self, values: Optional[Dict[str, torch.Tensor]] = None):
        """Make the fp32 master weights (and the compute copy) equal to ``values`` (name -> tensor) where given
        and to the current compute copy elsewhere.  Call it after changing parameter values by hand: the next
        step otherwise publishes the old master weights again."""
        full = self._flat_param.tensor.float()
        if values:
            for name, p in self._named_trainable():
                v = values.get(name)
                if v is not None:
                    o = self._offsets[p]
                    full[o: o + p.numel()].copy_(v.detach().reshape(-1).to(device=full.device, dtype=torch.float32))
        self.master.copy_(self._share_of(full))
        self._flat_param.tensor.copy_(full.to(self.param_dtype))

    def _state_names(self, inner):
        kind = _KINDS.get(type(inner))
        if kind is None:
            raise NotImplementedError(f"the sharded engine implements SGD, Adam and AdamW, not {type(inner).__name__}")
        return ("momentum_buffer",) if kind == "sgd" else ("exp_avg", "exp_avg_sq")

    def optimizer_state_dict(self, inner) -> dict:
        """State of the sharded optimiser in the layout ``inner.state_dict()`` would have had with whole fp32
        parameters (per-parameter ``step`` / ``exp_avg`` / ``exp_avg_sq`` or ``momentum_buffer``), so the file is
        interchangeable with ``torch.optim``'s.  Collective."""
        names = self._state_names(inner)
        sd = inner.state_dict()
        if self.state0 is None:
            return sd
        fulls = [self._gather(t) for t in (self.state0, self.state1) if t is not None]
        index = {}
        for gi, g in enumerate(inner.param_groups):
            for pi, p in enumerate(g["params"]):
                index[sd["param_groups"][gi]["params"][pi]] = p
        state = {}
        for idx, p in index.items():
            layer = getattr(p, "_dp_row_shard", None)
            if layer is not None and layer.state0 is not None:     # row-sharded weight: whole [N, K] state
                entry = {} if len(names) == 1 else {"step": torch.tensor(float(self._steps))}
                for name, rows in zip(names, (layer.state0, layer.state1)):
                    entry[name] = self._gather_rows(layer, rows)
                state[idx] = entry
                continue
            if p not in self._offsets:
                continue
            o = self._offsets[p]
            entry = {} if len(names) == 1 else {"step": torch.tensor(float(self._steps))}
            for name, full in zip(names, fulls):
                entry[name] = full[o: o + p.numel()].view(p.shape)
            state[idx] = entry
        sd["state"] = state
        return sd

    @torch.no_grad()
    def load_optimizer_state_dict(self, inner, sd: dict) -> None:
        """Inverse of :meth:`optimizer_state_dict`; also accepts a file written by a plain ``torch.optim``
        optimiser over the same parameters."""
        names = self._state_names(inner)
        inner.load_state_dict({"state": {}, "param_groups": sd["param_groups"]})
        state = sd.get("state", {})
        if not state:
            self.state0 = self.state1 = None
            self._steps = 0
            return
        dev = self.master.device
        fulls = [torch.zeros(self.total, dtype=torch.float32, device=dev) for _ in names]
        steps = 0
        for gi, g in enumerate(inner.param_groups):
            for pi, p in enumerate(g["params"]):
                entry = state.get(sd["param_groups"][gi]["params"][pi])
                layer = getattr(p, "_dp_row_shard", None)
                if entry is not None and layer is not None:
                    mine = slice(self.rank * layer.rows, (self.rank + 1) * layer.rows)
                    vals = [entry[name].to(device=dev, dtype=torch.float32).view(layer.full_shape)[mine].reshape(-1)
                            .clone() for name in names if name in entry]
                    layer.state0 = vals[0] if vals else None
                    layer.state1 = vals[1] if len(vals) > 1 else None
                    if "step" in entry:
                        steps = max(steps, int(float(entry["step"])))
                    continue
                if entry is None or p not in self._offsets:
                    continue
                o = self._offsets[p]
                for name, full in zip(names, fulls):
                    v = entry.get(name)
                    if v is not None:
                        full[o: o + p.numel()].copy_(v.reshape(-1).to(device=dev, dtype=torch.float32))
                if "step" in entry:
                    steps = max(steps, int(float(entry["step"])))
        shares = [self._share_of(f).clone() for f in fulls]
        self.state0 = shares[0]
        self.state1 = shares[1] if len(shares) > 1 else None
        self._steps = steps if len(names) > 1 else max(self._steps, 1)

    # ------------------------------------------------------------------ the step
    def optimizer_step(self, dpopt, closure=None):
        """Tail of ``FSDPOptimizerFastGradientClipping.step`` when this engine owns the parameters."""
        from ..utils.tracing import phase

        with phase("dp/optimizer_step"):
            return self._optimizer_step(dpopt, closure)

    def _hyper(self, inner):
        """(kind, common hyper-parameters, per-group (lr, weight_decay) or None)."""
        groups = inner.param_groups
        g0 = groups[0]
        kind = _KINDS.get(type(inner))
        if kind is None:
            raise NotImplementedError(f"the sharded engine implements SGD, Adam and AdamW, not {type(inner).__name__}")
        for g in groups:
            if g.get("amsgrad") or g.get("maximize"):
                raise NotImplementedError("amsgrad / maximize are not implemented in the sharded engine")
            if isinstance(g["lr"], torch.Tensor):
                raise NotImplementedError("a tensor learning rate is not implemented in the sharded engine")
        for g in groups[1:]:
            if any(g.get(k) != g0.get(k) for k in ("momentum", "dampening", "nesterov", "betas", "eps",
                                                    "decoupled_weight_decay")):
                raise NotImplementedError("parameter groups may differ in lr and weight_decay only "
                                          "(momentum / betas / eps must be common) in the sharded engine")
        if kind == "adam" and g0.get("decoupled_weight_decay"):
            kind = "adamw"
        per_group = [(float(g["lr"]), float(g.get("weight_decay", 0.0))) for g in groups]
        return kind, g0, (per_group if len(set(per_group)) > 1 else None)

    def _segment_table(self, inner, per_group):
        """Device table of the ranges of the flat space that share (lr, weight_decay), rebuilt when a value
        changes (a scheduler moves lr every step; the table is a few hundred bytes)."""
        key = tuple(per_group)
        if self._segments is not None and self._segments[0] == key:
            return self._segments[1]
        spans = []
        for g, hp in zip(inner.param_groups, per_group):
            for p in g["params"]:
                if p in self._offsets:
                    spans.append((self._offsets[p], hp))
        spans.sort(key=lambda t: t[0])
        rows = []
        for i, (begin, hp) in enumerate(spans):
            end = spans[i + 1][0] if i + 1 < len(spans) else self.total
            if rows and rows[-1][1] == hp:
                rows[-1][0] = end
            else:
                rows.append([end, hp])
        table = np.zeros(len(rows), dtype=_SEGMENT)
        for i, (end, hp) in enumerate(rows):
            table[i] = (end, hp[0], hp[1])
        dev_table = torch.from_numpy(table.view(np.uint8).copy()).to(self.master.device)
        self._segments = (key, dev_table)
        return dev_table

    # Pieces that run beside the weight-gradient GEMMs leave those the SMs.
    # One block per SM fits beside a GEMM CTA (registers and threads; the step kernel uses no shared memory) and the
    # step is bound by memory and link latency, not by issue slots.
    overlap_step = True
    overlap_blocks_multicast = 148
    overlap_blocks_peer = 148
    single_launch_blocks = 0         # grid cap of the one-launch step (0: whole grid); benchmarks set it

    def _optimizer_step(self, dpopt, closure=None):
        from ..ops import _cuda

        if closure is not None:
            with torch.enable_grad():
                closure()
        had_fresh = any(p._dp_grad_fresh for p in self._params)   # such gradients are zero-filled here, on this stream
        self.finish_grads()
        if dpopt._check_skip_next_step():
            dpopt._is_last_step_skipped = True
            return None
        inner = dpopt.original_optimizer
        kind, g0, per_group = self._hyper(inner)

        self._steps += 1
        t = self._steps
        dev = self.master.device
        h = dict(lr=float(g0["lr"]), momentum=0.0, dampening=0.0, weight_decay=float(g0.get("weight_decay", 0.0)),
                 beta1=0.0, beta2=0.0, eps=0.0, bias_c1=1.0, bias_c2_sqrt=1.0)
        runs = self._ready_runs(had_fresh) if self.overlap_step else None
        side = None
        if runs is not None:
            side = self._step_stream
            if side is None:
                side = self._step_stream = torch.cuda.Stream(device=dev)

        def zeros_for_state():
            # Optimiser state that is born in this step is zero-filled on the stream that runs the step: on the
            # main stream the fill would queue behind every weight-gradient GEMM of this pass, i.e. after the
            # pieces of the side stream had already read and written the state.
            if side is None:
                return torch.zeros(self.slice_len, dtype=torch.float32, device=dev)
            with torch.cuda.stream(side):
                return torch.zeros(self.slice_len, dtype=torch.float32, device=dev)

        first_step, nesterov, kcode = False, False, 0
        if kind == "sgd":
            h["momentum"] = float(g0.get("momentum", 0.0))
            h["dampening"] = float(g0.get("dampening", 0.0))
            nesterov = bool(g0.get("nesterov", False))
            if h["momentum"] != 0.0 and self.state0 is None:
                self.state0 = zeros_for_state()
                first_step = True
        else:
            b1, b2 = g0["betas"]
            if self.state0 is None:
                self.state0 = zeros_for_state()
                self.state1 = zeros_for_state()
            h.update(beta1=float(b1), beta2=float(b2), eps=float(g0["eps"]), bias_c1=1.0 - float(b1) ** t,
                     bias_c2_sqrt=math.sqrt(1.0 - float(b2) ** t))
            kcode = 2 if kind == "adamw" else 1
        # The table of per-group ranges is uploaded on the stream that will run the step: the main stream still holds
        # every weight-gradient GEMM of this pass, and waiting for it would undo the overlap of the pieces.
        if per_group is None:
            segments = None
        elif side is not None:
            with torch.cuda.stream(side):
                segments = self._segment_table(inner, per_group)
        else:
            segments = self._segment_table(inner, per_group)

        # per-worker expected batch (times accumulated batches in hooks mode), summed over the workers
        denom = float(dpopt._grad_denominator()) * (self.world if dpopt.loss_reduction == "mean" else 1)
        if dpopt.step_hook:
            dpopt.step_hook(dpopt)
        noise_std, inv_scale = float(dpopt._noise_std()), 1.0 / denom
        secure = bool(getattr(dpopt, "secure_mode", False)) and noise_std != 0.0
        if secure:
            # The noise comes from the optimizer's cryptographic generator through the five-draw rule
            # (opacus/optimizers/optimizer.py:143-160), not from the kernel's Philox stream: each rank adds it to
            # its own copy of the gradient on the stripes it owns, so the sum over ranks holds one draw per element.
            if self.tp_group is not None:
                raise NotImplementedError("secure_mode with a tensor-parallel group: replicas need one common draw")
            from .. import ops

            mine = self._flat_grad.tensor.view(self.pieces, self.world, self.stripe)[:, self.rank]
            mine.add_(ops.gaussian_like(mine, noise_std, generator=dpopt.generator, secure_mode=True))
            noise_std = 0.0
        seed, offset = (0, 0) if secure else _cuda._rng_state(dpopt.generator, dev, self.used * self.tp_world)
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
        grad_mc = self._flat_grad.mc_ptr if self.multicast and self.multicast_reduce else 0
        param_mc = self._flat_param.mc_ptr if self.multicast and self.multicast_publish else 0

        def launch(first_piece, n_pieces, max_blocks):
            """One launch (one flag epoch) over this rank's stripes of ``n_pieces`` consecutive pieces."""
            self._epoch += 1
            lo, n = first_piece * self.stripe, n_pieces * self.stripe
            cut = lambda x: None if x is None else x[lo: lo + n]
            C.sharded_dp_step(self._flat_grad.ptrs, self._flat_param.ptrs, self._flags.ptrs, cut(self.master),
                              cut(self.state0), cut(self.state1), first_piece * self.piece_len + self.rank * self.stripe,
                              n, self.rank, self.param_dtype == torch.bfloat16, self._epoch, kcode, nesterov,
                              first_step, h["lr"], h["momentum"], h["dampening"], h["weight_decay"], h["beta1"],
                              h["beta2"], h["eps"], h["bias_c1"], h["bias_c2_sqrt"], noise_std, inv_scale, seed,
                              offset, self.noise_split if noise_shift else 0, noise_shift, grad_mc, param_mc,
                              segments, max_blocks, self.stripe if n_pieces > 1 else 0, self.piece_len)

        if secure:
            runs = None                       # the host-side noise was added on the main stream, behind all GEMMs
            if side is not None:              # what was prepared on the side stream (segment table, new state)
                torch.cuda.current_stream(dev).wait_stream(side)
        if runs is None:
            launch(0, self.pieces, self.single_launch_blocks)
            self.last_step_launches = 1
        else:
            # Nothing this method queued on the main stream concerns the pieces (no gradient was zero-filled: that
            # case takes the one-launch path), so the side stream waits for the events of the writes only.
            main = torch.cuda.current_stream(dev)
            cap = int(os.environ.get("OPACUS_B200_OVERLAP_BLOCKS", "0")) or (
                self.overlap_blocks_multicast if self.multicast else self.overlap_blocks_peer)
            for k, (first_piece, n_pieces, events) in enumerate(runs):
                for ev in events:
                    side.wait_event(ev)
                with torch.cuda.stream(side):
                    launch(first_piece, n_pieces, cap if k + 1 < len(runs) else 0)
            main.wait_stream(side)
            self.last_step_launches = len(runs)
        dpopt._is_last_step_skipped = False
        self.mark_grads_fresh()
        self._finish_row_layers()
        return None

    def _ready_runs(self, had_fresh: bool):
        """``[(first_piece, n_pieces, events)]`` in the order in which the ghost-clipping pass completes the pieces
        (neighbouring pieces that complete together form one run), or None when the step has to be one launch: a
        single piece, a tensor-parallel group (sums are exchanged first), gradients that did not come from the
        single-pass controller.  The order depends only on the model's structure: all ranks compute the same."""
        if self.pieces < 2 or self.tp_group is not None or had_fresh:
            return None
        marks = [getattr(p, "_dp_ready", None) for p in self._params]
        if any(m is None for m in marks):
            return None
        latest = [dict() for _ in range(self.pieces)]   # per piece: stream -> (position, event) of its last write
        for p, (lane, order, event) in zip(self._params, marks):
            o = self._offsets[p]
            for k in range(o // self.piece_len, (o + p.numel() - 1) // self.piece_len + 1):
                if lane not in latest[k] or latest[k][lane][0] < order:
                    latest[k][lane] = (order, event)
        keyed = []
        for k, per_lane in enumerate(latest):
            when = max((v[0] for v in per_lane.values()), default=-1)
            keyed.append((when, k, [v[1] for v in per_lane.values()]))
        keyed.sort(key=lambda t: (t[0], t[1]))
        runs = []
        for when, k, events in keyed:
            if runs and runs[-1][3] == when and runs[-1][0] + runs[-1][1] == k:
                runs[-1][1] += 1
            else:
                runs.append([k, 1, events, when])
        return [(a, n, ev) for a, n, ev, _ in runs]
