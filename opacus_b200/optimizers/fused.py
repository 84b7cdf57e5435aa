"""Fused noise + scale + update for SGD / Adam / AdamW inner optimisers.

One multi-tensor kernel launch per step reads every ``summed_grad`` once,
draws the Gaussian noise from a counter-based Philox stream (seeded from the
torch generator, so ``torch.manual_seed`` / ``noise_generator=`` keep their
meaning), writes the private gradient back (it is exposed as ``p.grad``) and
updates the parameter and the optimiser state in the layout
``torch.optim`` itself uses, so ``state_dict()`` stays interchangeable.

Replaces ``opacus/optimizers/optimizer.py:477-504,570`` (three elementwise
passes plus the inner optimiser's own kernels per parameter).
"""
from __future__ import annotations

from typing import Optional

import torch


class _FusedPlan:
    def __init__(self, kind: str):
        self.kind = kind  # "sgd" | "adam" | "adamw"

    def run(self, opt, *, noise_std: float, denominator: float):
        from ..ops import _k

        inner = opt.original_optimizer
        gen = opt.generator
        k = _k()
        for group in inner.param_groups:
            ps = [p for p in group["params"] if p.requires_grad and getattr(p, "summed_grad", None) is not None]
            if not ps:
                continue
            k.fused_dp_step(self.kind, inner, group, ps, noise_std=noise_std, inv_scale=1.0 / denominator,
                            generator=gen)
            for p in ps:
                g = p.summed_grad.view_as(p)
                # the private gradient is kept in fp32; a low-precision parameter gets a rounded view of it
                p.grad = g if g.dtype == p.dtype else g.to(p.dtype)


_GROUP_FLAGS = ("maximize", "differentiable", "amsgrad", "capturable", "decoupled_weight_decay", "foreach", "fused")


def _config_key(opt):
    """What the decision depends on; recomputed every step (cheap) so that ``add_param_group`` or an edited
    group flag is seen."""
    inner = opt.original_optimizer
    groups = tuple((len(g["params"]), isinstance(g.get("lr"), torch.Tensor)) + tuple(bool(g.get(k, False))
                                                                                   for k in _GROUP_FLAGS)
                   for g in inner.param_groups)
    gen = opt.generator
    return (type(inner), groups, None if gen is None else gen.device.type)


def plan_for(opt) -> Optional[_FusedPlan]:
    """A plan if every parameter is a CUDA tensor, the noise generator (if one was given) lives on the GPU and
    the wrapped optimiser is a configuration the kernel implements; else ``None`` (the staged path runs).
    Optimiser state is created in fp32 also for bf16 parameters (the update is done in fp32)."""
    key = _config_key(opt)
    cached = getattr(opt, "_fused_plan_cache", None)
    if cached is not None and cached[0] == key:
        return cached[1]
    inner = opt.original_optimizer
    plan = None
    ps = opt.params
    ok = bool(ps) and all(p.is_cuda and p.dtype in (torch.float32, torch.bfloat16) for p in ps)
    if ok and opt.generator is not None and opt.generator.device.type != "cuda":
        ok = False                    # the kernel's Philox stream is keyed by a CUDA generator's (seed, offset)
    if ok:
        t = type(inner)
        if t is torch.optim.SGD:
            ok = all(not g.get("maximize", False) and not g.get("differentiable", False) for g in inner.param_groups)
            plan = _FusedPlan("sgd") if ok else None
        elif t in (torch.optim.Adam, torch.optim.AdamW):
            ok = all(
                not g.get("amsgrad", False) and not g.get("maximize", False) and not g.get("capturable", False)
                and not g.get("differentiable", False) and not isinstance(g["lr"], torch.Tensor)
                for g in inner.param_groups
            )
            decoupled = t is torch.optim.AdamW or any(g.get("decoupled_weight_decay", False)
                                                      for g in inner.param_groups)
            plan = _FusedPlan("adamw" if decoupled else "adam") if ok else None
    opt._fused_plan_cache = (key, plan)
    return plan
