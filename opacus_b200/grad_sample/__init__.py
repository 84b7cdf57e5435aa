"""Per-sample gradient engine: controllers, wrappers, registries and the
built-in layer rules (importing this package registers them)."""
from .gsm_base import AbstractGradSampleHooks, AbstractGradSampleModule  # noqa: I001
from .grad_sample_module import GradSampleHooks, GradSampleModule, create_or_accumulate_grad_sample
from .grad_sample_module_fast_gradient_clipping import (
    GradSampleHooksFastGradientClipping,
    GradSampleModuleFastGradientClipping,
)
from .grad_sample_module_fast_gradient_clipping_fsdp import (
    GradSampleHooksFastGradientClippingFSDP,
    GradSampleModuleFastGradientClippingFSDP,
)
from .grad_sample_module_fast_gradient_clipping_tp import (
    GradSampleHooksFastGradientClippingTP,
    GradSampleModuleFastGradientClippingTP,
)
from .gsm_exp_weights import GradSampleModuleExpandedWeights
from .gsm_no_op import GradSampleHooksNoOp, GradSampleModuleNoOp
from .utils import (
    get_gsm_class,
    get_hooks_class,
    prepare_module,
    register_cross_norm_sampler,
    register_grad_sampler,
    register_norm_sampler,
    register_norm_sq_sampler,
    register_wgrad_sampler,
    wrap_model,
)
from .conv import compute_conv_grad_sample
from .dp_multihead_attention import compute_sequence_bias_grad_sample
from .dp_rnn import compute_rnn_linear_grad_sample
from .embedding import compute_embedding_grad_sample, compute_embedding_norm_sample
from .group_norm import compute_group_norm_grad_sample
from .instance_norm import compute_instance_norm_grad_sample
from .layer_norm import compute_layer_norm_grad_sample
from .linear import compute_linear_grad_sample
from .rms_norm import compute_rms_norm_grad_sample
from . import tied  # noqa: F401  (cross-term rules for shared parameters)

__all__ = [
    "AbstractGradSampleHooks",
    "AbstractGradSampleModule",
    "GradSampleHooks",
    "GradSampleModule",
    "GradSampleHooksFastGradientClipping",
    "GradSampleModuleFastGradientClipping",
    "GradSampleHooksFastGradientClippingFSDP",
    "GradSampleModuleFastGradientClippingFSDP",
    "GradSampleHooksFastGradientClippingTP",
    "GradSampleModuleFastGradientClippingTP",
    "GradSampleModuleExpandedWeights",
    "GradSampleHooksNoOp",
    "GradSampleModuleNoOp",
    "register_grad_sampler",
    "register_norm_sampler",
    "register_norm_sq_sampler",
    "register_wgrad_sampler",
    "register_cross_norm_sampler",
    "create_or_accumulate_grad_sample",
    "prepare_module",
    "wrap_model",
    "get_gsm_class",
    "get_hooks_class",
]
