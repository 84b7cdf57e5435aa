"""Ghost clipping / fast gradient clipping: per-sample gradient *norms* without
keeping per-sample gradients, and the clipped sum ``sum_n c_n g_n`` computed
from them.

Two execution strategies share this class:

``single_pass=False`` (the default when the class is constructed directly)
    The classic protocol: the caller back-propagates the plain loss once (hooks
    fill ``param._norm_sample``), reads :meth:`get_clipping_coef`, and
    back-propagates ``sum_n c_n loss_n`` with hooks disabled.

``single_pass=True`` (chosen by ``PrivacyEngine.make_private``)
    One backward pass only.  During forward the layer's parameters are swapped
    for detached views, so autograd computes input gradients but **no weight
    gradients**.  A tap on each layer's output sees the output gradient ``G``,
    accumulates the layer's squared per-sample norm into one ``[B]`` fp32
    buffer, and keeps ``(A, G)``.  When backward is finished,
    :meth:`finish_single_pass` turns the norms into clip factors and produces
    every parameter's clipped gradient sum directly as ``A^T diag(c) G`` (one
    GEMM with ``K = B*T`` per Linear) into ``param.grad``.  This is exact
    because each per-sample gradient is linear in that sample's rows of ``G``
    with the activations held fixed.  Tied parameters are supported: the cross
    terms ``2<g_i, g_j>`` between the uses of a shared parameter are added to
    the norm.

Registries (filled by the decorators in :mod:`.utils`): ``GRAD_SAMPLERS`` and
``NORM_SAMPLERS`` have the public signatures; ``NORM_SQ_SAMPLERS`` and
``WGRAD_SAMPLERS`` are the fused forms used by the single-pass path.

Behavioural parity: ``opacus/grad_sample/grad_sample_module_fast_gradient_clipping.py:42-363``
and ``opacus/utils/fast_gradient_clipping_utils.py:179-201`` (the two-pass protocol).
"""
from __future__ import annotations

import logging
from typing import Dict, List, Optional

import torch
import torch.nn as nn

from .. import ops
from ..layers.dp_rnn import DPGRU, DPLSTM, DPRNN, RNNLinear
from ..utils.module_utils import requires_grad, trainable_modules, trainable_parameters
from ..utils.tracing import phase, record_clipping
from .functorch import ft_compute_per_sample_gradient
from .grad_sample_module import (
    _OutputTap,
    _STACKED_TYPES,
    GradSampleHooks,
    captured_inputs,
    create_or_accumulate_grad_sample,
    promote_current_grad_sample,
)
from .gsm_base import AbstractGradSampleModule

logger = logging.getLogger(__name__)
logger.disabled = True


def create_norm_sample(*, param: torch.Tensor, grad_sample: torch.Tensor, max_batch_len: int) -> None:
    """``param._norm_sample`` <- per-sample L2 norm of ``grad_sample``."""
    if not param.requires_grad:
        return
    if max_batch_len == 0:
        param._norm_sample = torch.tensor([], device=grad_sample.device, dtype=grad_sample.dtype)
    else:
        param._norm_sample = ops.grad_sample_norm_sq(grad_sample).sqrt().to(grad_sample.dtype)


class _OnStream:
    """``with torch.cuda.stream(s)`` without its device look-ups: the caller knows both streams."""

    __slots__ = ("side", "back")

    def __init__(self, side, back):
        self.side, self.back = side, back

    def __enter__(self):
        torch.cuda.set_stream(self.side)

    def __exit__(self, *exc):
        torch.cuda.set_stream(self.back)
        return False


class _Site:
    """What the single-pass path keeps about one layer call until the clip
    factors are known."""

    __slots__ = ("module", "inputs", "backprops", "g_scale", "kept_grad_samples", "params")

    def __init__(self, module, inputs, backprops, g_scale, kept_grad_samples=None):
        self.params = None
        self.module = module
        self.inputs = inputs
        self.backprops = backprops
        self.g_scale = g_scale
        self.kept_grad_samples = kept_grad_samples


class GradSampleHooksFastGradientClipping(GradSampleHooks):
    NORM_SAMPLERS = {}
    NORM_SQ_SAMPLERS = {}
    WGRAD_SAMPLERS = {}
    CROSS_NORM_SAMPLERS = {}

    def __init__(self, m: nn.Module, *, batch_first=True, loss_reduction="mean", strict: bool = True,
                 force_functorch=False, max_grad_norm=1, use_ghost_clipping=True, single_pass: bool = False):
        self.single_pass = single_pass
        if logger.isEnabledFor(logging.INFO):
            self.log_module_gradient_sample_mode(
                module=m, force_functorch=force_functorch, use_ghost_clipping=use_ghost_clipping)
        super().__init__(m, batch_first=batch_first, loss_reduction=loss_reduction, strict=strict,
                         force_functorch=force_functorch)
        self.trainable_parameters = [p for _, p in trainable_parameters(self._module)]
        self.max_grad_norm = max_grad_norm
        self.use_ghost_clipping = use_ghost_clipping
        self._per_sample_gradient_norms = None
        self._reset_single_pass_state()

    # ------------------------------------------------------------- public API
    def get_clipping_coef(self) -> torch.Tensor:
        """``min(1, C / (norm + 1e-6))`` per sample."""
        self._join_norm_stream()
        if self.single_pass and self._norm_sq_total is not None:
            self.per_sample_gradient_norms = self._norm_sq_total.clamp(min=0).sqrt()
            return ops.clip_factor(self._norm_sq_total, float(self.max_grad_norm))
        norm = self.get_norm_sample()
        return (self.max_grad_norm / (norm + 1e-6)).clamp(max=1.0)

    def get_norm_sample(self) -> torch.Tensor:
        """Per-sample gradient norm over all parameters."""
        self._join_norm_stream()
        if self.single_pass and self._norm_sq_total is not None:
            norm = self._norm_sq_total.clamp(min=0).sqrt()
        else:
            per_param = [p._norm_sample for p in self.trainable_parameters]
            if per_param:
                dev = per_param[0].device
                per_param = [n.to(dev) for n in per_param]
            norm = torch.stack(per_param, dim=0).norm(2, dim=0)
        self.per_sample_gradient_norms = norm
        return norm

    @property
    def per_sample_gradient_norms(self) -> torch.Tensor:
        if self._per_sample_gradient_norms is None:
            raise AttributeError(
                "per_sample_gradient_norms is not set. Please call forward and backward on the model "
                "before accessing this property."
            )
        return self._per_sample_gradient_norms

    @per_sample_gradient_norms.setter
    def per_sample_gradient_norms(self, value):
        self._per_sample_gradient_norms = value

    # --------------------------------------------------------- instrumentation
    def add_hooks(self, *, loss_reduction: str = "mean", batch_first: bool = True,
                  force_functorch: bool = False) -> None:
        if not self.single_pass:
            return super().add_hooks(loss_reduction=loss_reduction, batch_first=batch_first,
                                     force_functorch=force_functorch)
        if hasattr(self._module, "autograd_grad_sample_hooks"):
            raise ValueError("Trying to add hooks twice to the same model")
        handles = []
        self._module.autograd_grad_sample_hooks = handles
        self.autograd_grad_sample_hooks = handles
        self._anchor = None
        for sub in self.iterate_submodules(self._module):
            if type(sub) in (DPRNN, DPLSTM, DPGRU):
                continue
            handles.append(sub.register_forward_pre_hook(self._detach_params_hook))
            handles.append(sub.register_forward_hook(self._single_pass_forward_hook, always_call=True))
        self.enable_hooks()

    def _reset_single_pass_state(self):
        self._sites: List[_Site] = []
        self._norm_sq_total: Optional[torch.Tensor] = None
        self._batch_len: Optional[int] = None
        self._uses: Dict[nn.Parameter, List[_Site]] = {}
        self._backward_stream = None

    # ---- single pass: forward side
    def _active(self, module) -> bool:
        return self.hooks_enabled and module.training and torch.is_grad_enabled() and requires_grad(module, recurse=True)

    def _detach_params_hook(self, module, _inputs):
        """Swap trainable parameters for detached views for the duration of
        ``module.forward`` so that autograd skips their gradients."""
        if not self._active(module):
            return
        saved = []
        for sub in module.modules():
            for name, p in sub._parameters.items():
                if p is not None and p.requires_grad:
                    saved.append((sub, name, p))
                    sub._parameters[name] = p.detach()
        module.__dict__["_dp_saved_params"] = saved

    def _single_pass_forward_hook(self, module, inputs, output):
        saved = module.__dict__.pop("_dp_saved_params", None)
        if saved is None:
            return None
        for sub, name, p in saved:
            sub._parameters[name] = p
        if output is None:
            return None
        if not hasattr(module, "activations"):
            module.activations = []
        module.activations.append(captured_inputs(module, inputs, output))
        for sub, name, p in saved:
            p._forward_counter += 1
        first = output[0] if isinstance(output, (tuple, list)) else output
        if self._anchor is None or self._anchor.device != first.device:
            self._anchor = torch.zeros((), device=first.device, requires_grad=True)
        tapped = _OutputTap.apply(first, self._anchor, self, module)
        if isinstance(output, tuple):
            return (tapped,) + tuple(output[1:])
        if isinstance(output, list):
            return [tapped] + list(output[1:])
        return tapped

    # ---- single pass: backward side
    def _on_output_grad(self, module, grad_out):
        if not self.hooks_enabled:
            return
        with phase("dp/norm"):
            if self.overlap_norms and grad_out.is_cuda:
                # norm kernels run beside the rest of the backward pass; finish_single_pass() joins the streams
                main = self._backward_stream
                if main is None or main.device != grad_out.device:
                    # the stream autograd runs this device's backward on, looked up once per pass
                    main = self._backward_stream = torch.cuda.current_stream(grad_out.device)
                side = getattr(self, "_norm_stream", None)
                if side is None or side.device != grad_out.device:
                    side = self._norm_stream = torch.cuda.Stream(device=grad_out.device)
                side.wait_stream(main)
                with _OnStream(side, main):
                    self._capture_site(module, grad_out)
                self._norm_stream_busy = True
            else:
                self._capture_site(module, grad_out)

    # The norm kernels (persistent, one CTA per SM) and the library GEMMs of the backward pass fill each other's
    # partial waves when they run on two streams.
    overlap_norms = True

    def _join_norm_stream(self):
        if getattr(self, "_norm_stream_busy", False):
            torch.cuda.current_stream(self._norm_stream.device).wait_stream(self._norm_stream)
            self._norm_stream_busy = False

    def _capture_site(self, module, grad_out):
        backprops = grad_out.detach()
        batch_dim = 0 if self.batch_first or type(module) is RNNLinear else 1
        if not hasattr(module, "max_batch_len"):
            from .grad_sample_module import _get_batch_size

            module.max_batch_len = _get_batch_size(module=module, batch_dim=batch_dim)
        # the module may see only a share of the batch (activations sharded over samples)
        n = module.max_batch_len * self._batch_share(module)
        activations = module.activations.pop()
        if self.loss_reduction == "mean":
            g_scale = float(n)
        elif self.loss_reduction == "sum":
            g_scale = 1.0
        else:
            raise ValueError(
                f"loss_reduction = {self.loss_reduction}. Only 'sum' and 'mean' losses are supported")
        if batch_dim != 0:
            activations = [t.transpose(0, batch_dim) if isinstance(t, torch.Tensor) else t for t in activations]
            backprops = backprops.transpose(0, batch_dim)
        activations = [t.to_local() if hasattr(t, "to_local") else t for t in activations]

        activations, backprops = self._prepare_site(module, activations, backprops)

        uses = 1
        if isinstance(module, _STACKED_TYPES) and self._has_rule(module):
            ready = self._queue_stacked_call(module, activations, backprops)
            if ready is None:
                return
            activations, backprops, uses = ready

        if self._batch_len is None:
            self._batch_len = n
        mtype = self._get_module_type(module)
        kept = None
        if n == 0:
            norm_sq = {}
        elif self.use_ghost_clipping and not self.force_functorch and mtype in self.NORM_SQ_SAMPLERS:
            fn = self.NORM_SQ_SAMPLERS[mtype]
            if (self._total_fastpath_ok(module) and backprops.shape[0] == self._batch_len
                    and getattr(fn, "_accepts_total", None) is not False):
                # built-in rules add straight into the running [B] buffer inside their kernel
                if self._norm_sq_total is None:
                    self._norm_sq_total = self._new_total(self._batch_len, backprops.device)
                try:
                    norm_sq = fn(module, activations, backprops, g_scale, total=self._norm_sq_total)
                except TypeError:
                    fn._accepts_total = False
                    norm_sq = fn(module, activations, backprops, g_scale)
            else:
                norm_sq = fn(module, activations, backprops, g_scale)
        elif self.use_ghost_clipping and mtype in self.NORM_SAMPLERS:
            scaled = backprops * g_scale if g_scale != 1.0 else backprops
            norm_sq = {p: v.float().square() for p, v in self.NORM_SAMPLERS[mtype](module, activations, scaled).items()}
        else:
            sampler = self.GRAD_SAMPLERS[mtype] if self._has_rule(module) else ft_compute_per_sample_gradient
            scaled = backprops * g_scale if g_scale != 1.0 else backprops
            kept = {p: gs for p, gs in sampler(module, activations, scaled).items() if p.requires_grad}
            norm_sq = {p: ops.grad_sample_norm_sq(gs) for p, gs in kept.items()}

        site = _Site(module, activations, backprops, g_scale, kept)
        self._sites.append(site)
        for p, v in norm_sq.items():
            if not p.requires_grad:
                continue
            self._add_norm_sq(p, self._align_norm(p, v.float()))
        for p in self._site_params(site):
            self._uses.setdefault(p, []).append(site)
            p._forward_counter -= uses
        if len(module.activations) == 0 and hasattr(module, "max_batch_len"):
            del module.max_batch_len

    # Built-in rules may add their norms straight into ``_norm_sq_total`` inside the
    # kernel; subclasses that need to tell parameters apart switch this off.
    _use_total_fastpath = True

    def _total_fastpath_ok(self, module) -> bool:
        return self._use_total_fastpath

    def _new_total(self, n: int, device) -> torch.Tensor:
        """The zeroed ``[B]`` fp32 buffer that collects the squared norms of a pass."""
        return torch.zeros(n, dtype=torch.float32, device=device)

    # ---- extension points for parallel layouts (identity here)
    def _batch_share(self, module) -> int:
        """How many times larger the whole batch is than what ``module`` sees."""
        return 1

    def _prepare_site(self, module, activations, backprops):
        """Last chance to exchange the captured tensors (e.g. gather a sharded output gradient).  A module that
        computes the tensor its parameters act on inside its own forward (a fused residual add, a gathered
        input) leaves it in ``_dp_activation``; it then stands in for the first module input."""
        own = module.__dict__.pop("_dp_activation", None)
        if own is not None:
            activations = [own.detach()] + list(activations[1:])
        return activations, backprops

    def _align_norm(self, p, v):
        """Bring a squared-norm vector to batch length (a short step of a packed sequence is padded at the end)."""
        if v.shape[0] < (self._batch_len or 0):
            v = torch.cat([v, v.new_zeros(self._batch_len - v.shape[0])])
        return v

    def _site_coef(self, site, coef):
        """Clip factors of the samples that ``site`` holds."""
        return coef[: site.backprops.shape[0]].to(site.backprops.device)

    def _add_norm_sq(self, p, v):
        """Account the squared per-sample norm ``v`` of parameter ``p``."""
        if self._norm_sq_total is None:
            self._norm_sq_total = self._new_total(v.shape[0], v.device)
        self._norm_sq_total.add_(v.to(self._norm_sq_total.device))

    def _add_cross_terms(self):
        """``||sum_i g_i||^2 = sum_i ||g_i||^2 + 2 sum_{i<j} <g_i, g_j>`` for a
        parameter used by several layer calls."""
        for p, sites in self._uses.items():
            if len(sites) < 2:
                continue
            for i in range(len(sites)):
                for j in range(i + 1, len(sites)):
                    cross = self._cross_term(p, sites[i], sites[j])
                    self._norm_sq_total.add_(cross.float().to(self._norm_sq_total.device), alpha=2.0)

    def _cross_term(self, p, s1: _Site, s2: _Site) -> torch.Tensor:
        key = (self._get_module_type(s1.module), self._get_module_type(s2.module))
        if key in self.CROSS_NORM_SAMPLERS:
            return self.CROSS_NORM_SAMPLERS[key](p, s1, s2)
        if (key[1], key[0]) in self.CROSS_NORM_SAMPLERS:
            return self.CROSS_NORM_SAMPLERS[(key[1], key[0])](p, s2, s1)
        gs = []
        for s in (s1, s2):
            if s.kept_grad_samples is not None and p in s.kept_grad_samples:
                gs.append(s.kept_grad_samples[p])
                continue
            mtype = self._get_module_type(s.module)
            sampler = self.GRAD_SAMPLERS[mtype] if self._has_rule(s.module) else ft_compute_per_sample_gradient
            scaled = s.backprops * s.g_scale if s.g_scale != 1.0 else s.backprops
            gs.append(sampler(s.module, s.inputs, scaled)[p])
        b = min(gs[0].shape[0], gs[1].shape[0])
        return (gs[0][:b].reshape(b, -1).float() * gs[1][:b].reshape(b, -1).float()).sum(dim=1)

    def finish_single_pass(self) -> Optional[torch.Tensor]:
        """Call after the (only) backward pass: writes ``sum_n c_n g_n`` into
        ``param.grad`` (accumulating, like autograd) and returns the clip factors."""
        if not self.single_pass:
            raise RuntimeError("finish_single_pass() needs single_pass=True")
        self._join_norm_stream()
        if not self._sites or self._norm_sq_total is None:
            coef = torch.zeros(0, device=self.trainable_parameters[0].device) if self.trainable_parameters else None
            for p in self.trainable_parameters:
                if (p.grad is None and getattr(p, "_dp_grad_out", None) is None
                        and getattr(p, "_dp_row_shard", None) is None):
                    p.grad = torch.zeros_like(p)
            self._reset_single_pass_state()
            return coef
        self._add_cross_terms()
        coef = self.get_clipping_coef()
        norms = getattr(self, "per_sample_gradient_norms", None)
        if norms is not None and not isinstance(self.max_grad_norm, (list, tuple)):
            record_clipping(norms, float(self.max_grad_norm))
        with phase("dp/clipped_sum"):
            self._write_clipped_sums(coef)
        for p in self.trainable_parameters:
            if (p.grad is None and getattr(p, "_dp_grad_out", None) is None
                    and getattr(p, "_dp_row_shard", None) is None):      # stepped by its engine, layer by layer
                p.grad = torch.zeros_like(p)
        self._reset_single_pass_state()
        return coef

    # Clipped sums of different layers are independent GEMMs.  Issued alternately on two CUDA streams, the
    # tail of one (persistent CTAs that run out of tiles: 256 tiles on 148 SMs is 1.73 waves) is filled by the
    # head of the next.  Sites that write the same parameter stay on one stream, in order.
    overlap_clipped_sums = True
    clipped_sum_streams = 2

    def _write_clipped_sums(self, coef):
        lanes = None
        if self.overlap_clipped_sums and coef.is_cuda and len(self._sites) > 2:
            main = torch.cuda.current_stream(coef.device)
            sides = getattr(self, "_side_streams", None)
            if sides is None or sides[0].device != coef.device or len(sides) != self.clipped_sum_streams - 1:
                sides = self._side_streams = [torch.cuda.Stream(device=coef.device)
                                              for _ in range(self.clipped_sum_streams - 1)]
            for st in sides:
                st.wait_stream(main)
            lanes = [main] + sides
        lane_of = {}
        for order, site in enumerate(self._sites_by_parameter()):
            if lanes is not None:
                owned = self._site_params(site)
                ps = [id(p) for p in owned]
                lane = next((lane_of[i] for i in ps if i in lane_of), len(lane_of) % len(lanes))
                for i in ps:
                    lane_of[i] = lane
                with _OnStream(lanes[lane], main):
                    self._write_site(site, coef)
                    if any(getattr(p, "_dp_grad_out", None) is not None for p in owned):
                        # an engine that owns the gradient storage may step the parts of the flat space written so
                        # far while later sums still run: (stream, position, event) of each parameter's last write
                        done = torch.cuda.Event()
                        done.record(lanes[lane])
                        for p in owned:
                            p._dp_ready = (lane, order, done)
            else:
                self._write_site(site, coef)
        if lanes is not None:
            for st in lanes[1:]:
                lanes[0].wait_stream(st)

    def _site_params(self, site):
        if site.params is None:
            site.params = [p for _, p in trainable_parameters(site.module)]
        return site.params

    def _sites_by_parameter(self):
        """The captured sites in backward order, except that the later uses of a shared parameter follow its first
        use directly: the parameter's sum is then complete early instead of only when the last site is written."""
        if all(len(v) < 2 for v in self._uses.values()):
            return self._sites
        out, seen = [], set()
        for site in self._sites:
            if id(site) in seen:
                continue
            seen.add(id(site))
            out.append(site)
            for p in self._site_params(site):
                for other in self._uses.get(p, ()):
                    if id(other) not in seen:
                        seen.add(id(other))
                        out.append(other)
        return out

    def _write_site(self, site, coef):
        mtype = self._get_module_type(site.module)
        c = self._site_coef(site, coef)
        if site.kept_grad_samples is not None:
            grads = {}
            for p, gs in site.kept_grad_samples.items():
                dst = getattr(p, "_dp_grad_out", None)
                if dst is not None and getattr(p, "_dp_grad_fresh", True) and gs.shape[1:] == p.shape:
                    # engine-owned gradient storage that holds nothing yet: the sum is written there directly
                    grads[p] = ops.weighted_sum(gs, c[: gs.shape[0]], out=dst)
                    p._dp_grad_fresh = False
                else:
                    grads[p] = ops.weighted_sum(gs, c[: gs.shape[0]])
        elif mtype in self.WGRAD_SAMPLERS and not self.force_functorch:
            grads = self.WGRAD_SAMPLERS[mtype](site.module, site.inputs, site.backprops, c, site.g_scale)
        else:
            sampler = self.GRAD_SAMPLERS[mtype] if self._has_rule(site.module) else ft_compute_per_sample_gradient
            scaled = site.backprops * site.g_scale if site.g_scale != 1.0 else site.backprops
            grads = {p: ops.weighted_sum(gs, c[: gs.shape[0]])
                     for p, gs in sampler(site.module, site.inputs, scaled).items()}
        for p, g in grads.items():
            if not p.requires_grad:
                continue
            dst = getattr(p, "_dp_grad_out", None)
            if dst is not None:
                # engine-owned gradient storage (fp32, independent of the parameter dtype)
                if g.data_ptr() != dst.data_ptr():
                    if getattr(p, "_dp_grad_fresh", True):
                        dst.copy_(g.reshape(p.shape))
                        p._dp_grad_fresh = False
                    else:
                        dst.add_(g.reshape(p.shape))
                continue
            g = g.reshape(p.shape).to(p.dtype)
            if p.grad is None:
                p.grad = g if g._base is None else g.clone()
            else:
                p.grad.add_(g)

    # ------------------------------------------------------- two-pass protocol
    def capture_activations_hook(self, module: nn.Module, forward_input: List[torch.Tensor],
                                 _forward_output: torch.Tensor):
        if not self.hooks_enabled or not module.training or not torch.is_grad_enabled() or not requires_grad(module):
            return
        if not hasattr(module, "activations"):
            module.activations = []
        module.activations.append(captured_inputs(module, forward_input, _forward_output))
        ghost_layer = self.use_ghost_clipping and type(module) in self.NORM_SAMPLERS
        for _, p in trainable_parameters(module):
            p._forward_counter += 1
            if ghost_layer and p._forward_counter > 1:
                raise NotImplementedError(
                    "Parameter tying is not supported with Ghost Clipping in two-pass mode; "
                    "use single_pass=True (PrivacyEngine.make_private does)."
                )

    def capture_backprops_hook(self, module: nn.Module, _forward_input, forward_output, loss_reduction: str,
                               batch_first: bool):
        if not self.hooks_enabled:
            return
        backprops = forward_output[0].detach()
        activations, backprops = self.rearrange_grad_samples(
            module=module, backprops=backprops, loss_reduction=loss_reduction, batch_first=batch_first)
        activations = [t.to_local() if hasattr(t, "to_local") else t for t in activations]
        mtype = type(module)
        if self.use_ghost_clipping and mtype in self.NORM_SAMPLERS:
            for param, ns in self.NORM_SAMPLERS[mtype](module, activations, backprops).items():
                if param.requires_grad:
                    param._norm_sample = ns
                    param._forward_counter -= 1
        else:
            uses = 1
            if isinstance(module, _STACKED_TYPES) and self._has_rule(module):
                ready = self._queue_stacked_call(module, activations, backprops)
                if ready is None:
                    return
                activations, backprops, uses = ready
            sampler = self.GRAD_SAMPLERS[mtype] if self._has_rule(module) else ft_compute_per_sample_gradient
            grad_samples = sampler(module, activations, backprops)
            for param, gs in grad_samples.items():
                create_or_accumulate_grad_sample(param=param, grad_sample=gs, max_batch_len=module.max_batch_len)
            del grad_samples
            for _, p in trainable_parameters(module):
                p._forward_counter -= uses
                if p._forward_counter == 0:
                    promote_current_grad_sample(p)
                    create_norm_sample(param=p, grad_sample=p.grad_sample, max_batch_len=module.max_batch_len)
                    p.grad_sample = None
        if len(module.activations) == 0 and hasattr(module, "max_batch_len"):
            del module.max_batch_len

    def log_module_gradient_sample_mode(self, module: nn.Module, *, force_functorch=False, use_ghost_clipping=True):
        """Log (INFO) which path every trainable submodule will take."""
        for name, m in trainable_modules(module):
            if type(m) in (DPRNN, DPLSTM, DPGRU):
                how = "No hook or functorch is added."
            elif use_ghost_clipping and type(m) in self.NORM_SAMPLERS:
                how = "under Ghost Clipping."
            elif not force_functorch and type(m) in self.GRAD_SAMPLERS:
                how = "under Fast Gradient Clipping (hook mode)."
            else:
                how = "under Fast Gradient Clipping (functorch mode)."
            logger.info(f"Module name: {name}, module type: {type(m)}, {how}")


class GradSampleModuleFastGradientClipping(GradSampleHooksFastGradientClipping, AbstractGradSampleModule):
    """``nn.Module`` wrapper flavour."""

    def __init__(self, m: nn.Module, *, batch_first=True, loss_reduction="mean", strict: bool = True,
                 force_functorch=False, max_grad_norm=1, use_ghost_clipping=True, single_pass: bool = False):
        nn.Module.__init__(self)
        GradSampleHooksFastGradientClipping.__init__(
            self, m, batch_first=batch_first, loss_reduction=loss_reduction, strict=strict,
            force_functorch=force_functorch, max_grad_norm=max_grad_norm,
            use_ghost_clipping=use_ghost_clipping, single_pass=single_pass)
        self.grad_accumulation_hook = None
