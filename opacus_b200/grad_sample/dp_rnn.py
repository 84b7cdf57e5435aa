"""The linear maps inside the DP recurrent cells use the Linear rules.  The
engine stacks their per-time-step calls, so each rule sees ``[B, T, d]`` once
(``opacus/grad_sample/dp_rnn.py:26-51`` computes one outer product per step)."""
from ..layers.dp_rnn import RNNLinear
from .linear import (
    compute_linear_grad_sample,
    compute_linear_norm_sq,
    compute_linear_weighted_grad,
)
from .utils import register_grad_sampler, register_norm_sq_sampler, register_wgrad_sampler

compute_rnn_linear_grad_sample = register_grad_sampler(RNNLinear)(compute_linear_grad_sample)
register_norm_sq_sampler(RNNLinear)(compute_linear_norm_sq)
register_wgrad_sampler(RNNLinear)(compute_linear_weighted_grad)
