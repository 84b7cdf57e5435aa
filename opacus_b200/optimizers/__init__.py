"""DP optimizers and the (clipping, distributed, mode) -> class table
(``opacus/optimizers/__init__.py:15-71``)."""
from .adaclipoptimizer import AdaClipDPOptimizer
from .ddp_perlayeroptimizer import DistributedPerLayerOptimizer, SimpleDistributedPerLayerOptimizer
from .ddpoptimizer import DistributedDPOptimizer
from .ddpoptimizer_fast_gradient_clipping import DistributedDPOptimizerFastGradientClipping
from .fsdpoptimizer_fast_gradient_clipping import FSDPOptimizerFastGradientClipping
from .optimizer import DPOptimizer
from .optimizer_fast_gradient_clipping import DPOptimizerFastGradientClipping
from .perlayeroptimizer import DPPerLayerOptimizer

__all__ = [
    "AdaClipDPOptimizer",
    "DistributedDPOptimizer",
    "DPOptimizer",
    "DPOptimizerFastGradientClipping",
    "DistributedDPOptimizerFastGradientClipping",
    "FSDPOptimizerFastGradientClipping",
    "DPPerLayerOptimizer",
    "SimpleDistributedPerLayerOptimizer",
    "DistributedPerLayerOptimizer",
    "get_optimizer_class",
]

_GHOST = {("flat", False): DPOptimizerFastGradientClipping, ("flat", True): DistributedDPOptimizerFastGradientClipping}
_PLAIN = {
    ("flat", False): DPOptimizer,
    ("flat", True): DistributedDPOptimizer,
    ("per_layer", False): DPPerLayerOptimizer,
    ("adaptive", False): AdaClipDPOptimizer,
}


def get_optimizer_class(clipping: str, distributed: bool, grad_sample_mode: str = None, engine=None):
    key = (clipping, bool(distributed))
    if grad_sample_mode == "ghost_tp" and engine is not None and clipping == "flat":
        # tensor parallel x sharded data parallel: the engine's step kernel draws the noise (one Philox range per
        # tensor-parallel rank for the shards), so the optimizer is the one that hands the step to the engine
        return FSDPOptimizerFastGradientClipping
    if grad_sample_mode == "ghost":
        if key in _GHOST:
            return _GHOST[key]
        raise ValueError(
            f"Unsupported combination of parameters. Clipping: {clipping} and grad_sample_mode: {grad_sample_mode}")
    if grad_sample_mode == "ghost_tp":
        if clipping == "flat":
            from ..parallel.tensor_parallel import TensorParallelDPOptimizer

            return TensorParallelDPOptimizer
        raise ValueError(f"Unsupported combination of parameters. Clipping: {clipping} and grad_sample_mode: ghost_tp")
    if grad_sample_mode == "ghost_fsdp":
        if key == ("flat", True):
            return FSDPOptimizerFastGradientClipping
        raise ValueError(
            f"Unsupported combination of parameters. Clipping: {clipping}, distributed: {distributed}, "
            f"and grad_sample_mode: {grad_sample_mode}")
    if key in _PLAIN:
        return _PLAIN[key]
    if key == ("per_layer", True):
        if grad_sample_mode in ("hooks", "ew"):
            return SimpleDistributedPerLayerOptimizer
        raise ValueError(f"Unexpected grad_sample_mode: {grad_sample_mode}")
    raise ValueError(f"Unexpected optimizer parameters. Clipping: {clipping}, distributed: {distributed}")
