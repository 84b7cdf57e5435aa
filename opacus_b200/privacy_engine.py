"""``PrivacyEngine``: the one object a training script talks to.

``make_private`` takes the usual (module, optimizer, data_loader) triple and
returns DP counterparts: the model instrumented for per-sample gradients, a
``DPOptimizer`` that clips, noises and steps, and a Poisson-sampling loader.
In the ghost-clipping modes a wrapped criterion is returned as well, and the
model runs this package's single-backward-pass engine.

Behavioural parity: ``opacus/privacy_engine.py:42-696`` (same signatures,
defaults and checkpoint layout).
"""
import os
import warnings
from typing import IO, Any, BinaryIO, Dict, List, Optional, Union

import torch
from torch import nn, optim
from torch.nn.parallel import DistributedDataParallel as DDP
from torch.utils.data import DataLoader

from .accountants import create_accountant
from .accountants.utils import get_noise_multiplier
from .data_loader import DPDataLoader, switch_generator
from .distributed import DifferentiallyPrivateDistributedDataParallel as DPDDP
from .grad_sample import AbstractGradSampleModule, GradSampleHooks, GradSampleModule, get_gsm_class, prepare_module
from .optimizers import DPOptimizer, get_optimizer_class
from .schedulers import _GradClipScheduler, _NoiseScheduler
from .utils.fast_gradient_clipping_utils import DPLossFastGradientClipping
from .validators.module_validator import ModuleValidator


def _distributed_kinds():
    kinds = [DPDDP, DDP]
    try:
        from torch.distributed.fsdp import FSDPModule

        kinds.append(FSDPModule)
    except Exception:  # pragma: no cover
        pass
    from .parallel.sharded import ShardedDataParallel

    kinds.append(ShardedDataParallel)
    return tuple(kinds)


class PrivacyEngine:
    """
    Example
        >>> import torch
        >>> from torch.utils.data import DataLoader, TensorDataset
        >>> model = torch.nn.Linear(4, 2)
        >>> opt = torch.optim.SGD(model.parameters(), lr=0.1)
        >>> dl = DataLoader(TensorDataset(torch.randn(32, 4), torch.randint(0, 2, (32,))), batch_size=8)
        >>> engine = PrivacyEngine(accountant="rdp")
        >>> model, opt, dl = engine.make_private(module=model, optimizer=opt, data_loader=dl,
        ...                                      noise_multiplier=1.0, max_grad_norm=1.0)
        >>> for x, y in dl:
        ...     opt.zero_grad()
        ...     torch.nn.functional.cross_entropy(model(x), y).backward()
        ...     opt.step()
        >>> engine.get_epsilon(delta=1e-5) > 0
        True
    """

    def __init__(self, *, accountant: str = "prv", secure_mode: bool = False):
        self.accountant = create_accountant(mechanism=accountant)
        self.secure_mode = secure_mode
        self.secure_rng = None
        self.dataset = None
        if secure_mode:
            try:
                import torchcsprng as csprng

                self.secure_rng = csprng.create_random_device_generator("/dev/urandom")
            except ImportError:
                # the reference stops here; this package carries its own generator (ChaCha20 keyed from the OS
                # entropy pool, the same stream on CPU and GPU)
                from .utils.secure_rng import SecureGenerator

                self.secure_rng = SecureGenerator()
        else:
            warnings.warn(
                "Secure RNG turned off. This is perfectly fine for experimentation as it allows for much faster "
                "training performance, but remember to turn it on and retrain one last time before production "
                "with ``secure_mode`` turned on."
            )

    # ---------------------------------------------------------------- pieces
    def _prepare_optimizer(self, *, optimizer: optim.Optimizer, noise_multiplier: float,
                           max_grad_norm: Union[float, List[float]], expected_batch_size: int,
                           loss_reduction: str = "mean", distributed: bool = False, clipping: str = "flat",
                           noise_generator=None, grad_sample_mode="hooks", **kwargs) -> DPOptimizer:
        if isinstance(optimizer, DPOptimizer):
            optimizer = optimizer.original_optimizer
        generator = self.secure_rng if self.secure_mode else noise_generator
        cls = get_optimizer_class(clipping=clipping, distributed=distributed, grad_sample_mode=grad_sample_mode,
                                  **({"engine": kwargs["engine"]} if grad_sample_mode == "ghost_tp" and "engine" in kwargs
                                     else {}))
        return cls(optimizer=optimizer, noise_multiplier=noise_multiplier, max_grad_norm=max_grad_norm,
                   expected_batch_size=expected_batch_size, loss_reduction=loss_reduction, generator=generator,
                   secure_mode=self.secure_mode, **kwargs)

    def _prepare_data_loader(self, data_loader: DataLoader, *, poisson_sampling: bool, distributed: bool,
                             batch_first: bool = True, rand_on_empty: bool = False,
                             replica: Optional[tuple] = None) -> DataLoader:
        if self.dataset is None:
            self.dataset = data_loader.dataset
        elif self.dataset != data_loader.dataset:
            warnings.warn(
                f"PrivacyEngine detected new dataset object. Was: {self.dataset}, got: {data_loader.dataset}. "
                "Privacy accounting works per dataset, please initialize new PrivacyEngine if you're using "
                "different dataset. You can ignore this warning if two datasets above represent the same "
                "logical dataset"
            )
        if poisson_sampling:
            if replica is not None:         # 2-d layout: (data-parallel groups, this rank's group, shared generator)
                return DPDataLoader.from_data_loader(data_loader, generator=replica[2], distributed=True,
                                                     batch_first=batch_first, rand_on_empty=rand_on_empty,
                                                     num_replicas=replica[0], rank=replica[1])
            return DPDataLoader.from_data_loader(data_loader, generator=self.secure_rng, distributed=distributed,
                                                 batch_first=batch_first, rand_on_empty=rand_on_empty)
        if self.secure_mode:
            return switch_generator(data_loader=data_loader, generator=self.secure_rng)
        return data_loader

    def _tensor_parallel_replica(self, engine):
        """Sharded data parallelism over tensor-parallel groups: the ranks of one tensor-parallel group must draw
        the same Poisson sample, different groups disjoint ones.  Returns ``(groups, this rank's group, generator)``
        with a generator state common to the tensor-parallel group (rank 0 of the job draws a base seed and
        broadcasts it; collective), or None for every other layout."""
        if engine is None or getattr(engine, "tp_world", 1) <= 1:
            return None
        if self.secure_mode:
            raise NotImplementedError("secure_mode with tensor-parallel groups: the sampling generator must be shared")
        import torch.distributed as dist

        base = torch.randint(0, 2 ** 62, (1,), dtype=torch.int64)
        dev = next(engine.parameters()).device
        base = base.to(dev)
        dist.broadcast(base, 0)
        groups, mine = engine.world, engine.rank
        return groups, mine, torch.Generator().manual_seed((int(base.item()) + 7919 * mine) % (2 ** 63 - 1))

    def _prepare_model(self, module: nn.Module, *, batch_first: bool = True,
                       max_grad_norm: Union[float, List[float]] = 1.0, loss_reduction: str = "mean",
                       grad_sample_mode: str = "hooks", wrap_model: bool = True,
                       single_pass: Optional[bool] = None,
                       skip_param_grads: bool = False) -> Union[AbstractGradSampleModule, GradSampleHooks]:
        self.validate(module=module, optimizer=None, data_loader=None)
        if wrap_model and isinstance(module, AbstractGradSampleModule):
            if (module.batch_first != batch_first or module.loss_reduction != loss_reduction
                    or type(module) is not get_gsm_class(grad_sample_mode)):
                raise ValueError(
                    "Pre-existing GradSampleModule doesn't match new arguments."
                    f"Got: module.batch_first: {module.batch_first}, module.loss_reduction: "
                    f"{module.loss_reduction}, type(module): {type(module)}"
                    f"Requested: batch_first:{batch_first}, loss_reduction: {loss_reduction}, "
                    f"grad_sample_mode: {grad_sample_mode} Please pass vanilla nn.Module instead"
                )
            return module
        extra = {}
        if "ghost" in grad_sample_mode:
            extra["max_grad_norm"] = max_grad_norm
            if grad_sample_mode == "ghost":
                extra["single_pass"] = True if single_pass is None else single_pass
            elif single_pass is not None:
                extra["single_pass"] = single_pass
            tp_group = getattr(module, "tp_group", None)
            if grad_sample_mode == "ghost_tp" and tp_group is not None:     # 2-d: the sharded engine knows the group
                extra["process_group"] = tp_group
                extra.setdefault("single_pass", True)
        elif grad_sample_mode in ("hooks", "functorch") and skip_param_grads:
            extra["skip_param_grads"] = True
        return prepare_module(module, grad_sample_mode=grad_sample_mode, batch_first=batch_first,
                              loss_reduction=loss_reduction, wrap_model=wrap_model, **extra)

    def _prepare_criterion(self, *, module, optimizer: DPOptimizer, criterion, loss_reduction: str = "mean",
                           **kwargs) -> DPLossFastGradientClipping:
        return DPLossFastGradientClipping(module, optimizer, criterion, loss_reduction)

    # ------------------------------------------------------------- validation
    def is_compatible(self, *, module: nn.Module, optimizer: Optional[optim.Optimizer],
                      data_loader: Optional[DataLoader]) -> bool:
        return ModuleValidator.is_valid(module)

    def validate(self, *, module: nn.Module, optimizer: Optional[optim.Optimizer],
                 data_loader: Optional[DataLoader]):
        ModuleValidator.validate(module, strict=True)

    @classmethod
    def get_compatible_module(cls, module: nn.Module) -> nn.Module:
        module = ModuleValidator.fix(module)
        ModuleValidator.validate(module, strict=True)
        return module

    # ------------------------------------------------------------ entry points
    def make_private(self, *, module: nn.Module, optimizer: optim.Optimizer, criterion=nn.CrossEntropyLoss(),
                     data_loader: DataLoader, noise_multiplier: float, max_grad_norm: Union[float, List[float]],
                     batch_first: bool = True, loss_reduction: str = "mean", poisson_sampling: bool = True,
                     clipping: str = "flat", noise_generator=None, grad_sample_mode: str = "hooks",
                     wrap_model: bool = True, rand_on_empty: bool = False, **kwargs):
        """Returns ``(module, optimizer, data_loader)`` or, for ghost modes,
        ``(module, optimizer, criterion, data_loader)``.

        ``expected_batch_size`` is ``int(len(dataset) / len(data_loader))``,
        per worker when distributed.  Extra keyword arguments reach the
        optimizer (and the criterion wrapper) constructor; ``single_pass`` is
        consumed here and selects the ghost execution strategy.
        """
        if noise_generator and self.secure_mode:
            raise ValueError("Passing seed is prohibited in secure mode")
        owned = {id(p) for p in module.parameters()}
        for group in optimizer.param_groups:
            for p in group["params"]:
                if id(p) not in owned:
                    raise ValueError("Module parameters are different than optimizer Parameters")

        distributed = isinstance(module, _distributed_kinds())
        single_pass = kwargs.pop("single_pass", None)
        engine = module if type(module).__name__ == "ShardedDataParallel" else None
        # hooks mode: skip autograd's own (non-private) weight gradients.  Always with the sharded engine, whose
        # gradients live in its own buffer anyway; elsewhere on request (``p.grad`` then stays None until step()).
        skip_param_grads = kwargs.pop("skip_param_grads", engine is not None)

        module = self._prepare_model(module, batch_first=batch_first, max_grad_norm=max_grad_norm,
                                     loss_reduction=loss_reduction, grad_sample_mode=grad_sample_mode,
                                     wrap_model=wrap_model, single_pass=single_pass,
                                     skip_param_grads=skip_param_grads)
        if poisson_sampling:
            module.forbid_grad_accumulation()

        data_loader = self._prepare_data_loader(data_loader, distributed=distributed,
                                                poisson_sampling=poisson_sampling, batch_first=batch_first,
                                                rand_on_empty=rand_on_empty,
                                                replica=self._tensor_parallel_replica(engine))
        sample_rate = 1 / len(data_loader)
        expected_batch_size = int(len(data_loader.dataset) * sample_rate)
        if distributed:
            # workers that see different samples: all ranks, or one per tensor-parallel group in a 2-d layout
            expected_batch_size /= torch.distributed.get_world_size() // getattr(engine, "tp_world", 1)

        opt_kwargs = dict(kwargs)
        if engine is not None and clipping == "flat":
            opt_kwargs["engine"] = engine
        optimizer = self._prepare_optimizer(
            optimizer=optimizer, noise_multiplier=noise_multiplier, max_grad_norm=max_grad_norm,
            expected_batch_size=expected_batch_size, loss_reduction=loss_reduction,
            noise_generator=noise_generator, distributed=distributed, clipping=clipping,
            grad_sample_mode=grad_sample_mode, **opt_kwargs)
        optimizer.attach_step_hook(self.accountant.get_optimizer_hook_fn(sample_rate=sample_rate))

        if "ghost" in grad_sample_mode:
            criterion = self._prepare_criterion(module=module, optimizer=optimizer, criterion=criterion,
                                                loss_reduction=loss_reduction, **kwargs)
            return module, optimizer, criterion, data_loader
        return module, optimizer, data_loader

    def make_private_with_epsilon(self, *, module: nn.Module, optimizer: optim.Optimizer,
                                  criterion=nn.CrossEntropyLoss(), data_loader: DataLoader, target_epsilon: float,
                                  target_delta: float, epochs: int, max_grad_norm: Union[float, List[float]],
                                  batch_first: bool = True, loss_reduction: str = "mean",
                                  poisson_sampling: bool = True, clipping: str = "flat", noise_generator=None,
                                  grad_sample_mode: str = "hooks", wrap_model: bool = True, **kwargs):
        """``make_private`` with the noise multiplier calibrated so that
        ``epochs`` epochs cost at most ``(target_epsilon, target_delta)``."""
        sample_rate = 1 / len(data_loader)
        if len(self.accountant) > 0:
            warnings.warn(
                "You're calling make_private_with_epsilon with non-zero privacy budget already spent. "
                "Returned noise_multiplier assumes zero starting point, so your overall privacy budget will be higher."
            )
        sigma = get_noise_multiplier(target_epsilon=target_epsilon, target_delta=target_delta,
                                     sample_rate=sample_rate, epochs=epochs,
                                     accountant=self.accountant.mechanism(), **kwargs)
        return self.make_private(module=module, optimizer=optimizer, data_loader=data_loader, criterion=criterion,
                                 noise_multiplier=sigma, max_grad_norm=max_grad_norm, batch_first=batch_first,
                                 loss_reduction=loss_reduction, noise_generator=noise_generator,
                                 grad_sample_mode=grad_sample_mode, poisson_sampling=poisson_sampling,
                                 clipping=clipping, wrap_model=wrap_model, **kwargs)

    def get_epsilon(self, delta):
        return self.accountant.get_epsilon(delta)

    # ------------------------------------------------------------ checkpoints
    def save_checkpoint(self, *, path: Union[str, os.PathLike, BinaryIO, IO[bytes]], module: nn.Module,
                        optimizer: Optional[DPOptimizer] = None, noise_scheduler: Optional[_NoiseScheduler] = None,
                        grad_clip_scheduler: Optional[_GradClipScheduler] = None,
                        checkpoint_dict: Optional[Dict[str, Any]] = None,
                        module_state_dict_kwargs: Optional[Dict[str, Any]] = None,
                        torch_save_kwargs: Optional[Dict[str, Any]] = None):
        """One ``torch.save`` dict: ``module_state_dict``,
        ``privacy_accountant_state_dict`` and, when given, ``optimizer_state_dict``,
        ``noise_scheduler_state_dict``, ``grad_clip_scheduler_state_dict``, plus
        the caller's own entries.  ``noise_multiplier``/``max_grad_norm`` are
        not stored."""
        out = checkpoint_dict or {}
        out["module_state_dict"] = module.state_dict(**(module_state_dict_kwargs or {}))
        out["privacy_accountant_state_dict"] = self.accountant.state_dict()
        for key, obj in (("optimizer_state_dict", optimizer), ("noise_scheduler_state_dict", noise_scheduler),
                         ("grad_clip_scheduler_state_dict", grad_clip_scheduler)):
            if obj is not None:
                out[key] = obj.state_dict()
        torch.save(out, path, **(torch_save_kwargs or {}))

    def load_checkpoint(self, *, path: Union[str, os.PathLike, BinaryIO, IO[bytes]], module: nn.Module,
                        optimizer: Optional[DPOptimizer] = None, noise_scheduler: Optional[_NoiseScheduler] = None,
                        grad_clip_scheduler: Optional[_GradClipScheduler] = None,
                        module_load_dict_kwargs: Optional[Dict[str, Any]] = None,
                        torch_load_kwargs: Optional[Dict[str, Any]] = None) -> Dict:
        """Inverse of :meth:`save_checkpoint`; returns what is left of the dict."""
        ckpt = torch.load(path, **(torch_load_kwargs or {}), weights_only=False)
        module.load_state_dict(ckpt["module_state_dict"], **(module_load_dict_kwargs or {}))
        self.accountant.load_state_dict(ckpt["privacy_accountant_state_dict"])

        opt_sd = ckpt.pop("optimizer_state_dict", {})
        if optimizer is not None and len(opt_sd) > 0:
            optimizer.load_state_dict(opt_sd)
        elif (optimizer is not None) ^ (len(opt_sd) > 0):
            warnings.warn(
                f"optimizer_state_dict has {len(opt_sd)} items but optimizer is "
                f"{'' if optimizer else 'not'} provided."
            )
        for key, obj in (("noise_scheduler_state_dict", noise_scheduler),
                         ("grad_clip_scheduler_state_dict", grad_clip_scheduler)):
            sd = ckpt.pop(key, {})
            if obj is not None and len(sd) > 0:
                obj.load_state_dict(sd)
        return ckpt
