"""The public names of the Opacus 1.6 modules exist under the same paths in this package.

The table lists, per module path below ``opacus``, the names that module defines or exports (``__all__`` where it
has one); a user who replaces ``opacus`` by ``opacus_b200`` in an import statement must find each of them.
"""
import importlib

import pytest

API = {
    "": [
        "GradSampleModule", "GradSampleModuleFastGradientClipping", "PrivacyEngine", "__version__", "utils"
    ],
    "grad_sample": [
        "AbstractGradSampleHooks", "AbstractGradSampleModule", "GradSampleHooks",
        "GradSampleHooksFastGradientClipping", "GradSampleHooksFastGradientClippingFSDP",
        "GradSampleHooksFastGradientClippingTP", "GradSampleHooksNoOp", "GradSampleModule",
        "GradSampleModuleExpandedWeights", "GradSampleModuleFastGradientClipping",
        "GradSampleModuleFastGradientClippingFSDP", "GradSampleModuleFastGradientClippingTP",
        "GradSampleModuleNoOp", "create_or_accumulate_grad_sample", "get_gsm_class", "prepare_module",
        "register_grad_sampler", "register_norm_sampler", "wrap_model"
    ],
    "optimizers": [
        "AdaClipDPOptimizer", "DPOptimizer", "DPOptimizerFastGradientClipping", "DPPerLayerOptimizer",
        "DistributedDPOptimizer", "FSDPOptimizerFastGradientClipping", "SimpleDistributedPerLayerOptimizer",
        "DistributedPerLayerOptimizer", "DistributedDPOptimizerFastGradientClipping", "get_optimizer_class"
    ],
    "accountants": [
        "GaussianAccountant", "IAccountant", "PRVAccountant", "RDPAccountant", "create_accountant",
        "register_accountant"
    ],
    "accountants.utils": [
        "get_noise_multiplier"
    ],
    "accountants.analysis.rdp": [
        "compute_rdp", "get_privacy_spent"
    ],
    "accountants.analysis.gdp": [
        "compute_eps_poisson", "compute_eps_uniform", "compute_mu_poisson", "compute_mu_uniform",
        "delta_eps_mu", "eps_from_mu"
    ],
    "data_loader": [
        "CollateFnWithEmpty", "DPDataLoader", "dtype_safe", "shape_safe", "switch_generator",
        "wrap_collate_with_empty"
    ],
    "distributed": [
        "DifferentiallyPrivateDistributedDataParallel", "average_gradients"
    ],
    "layers": [
        "DPGRU", "DPLSTM", "DPMultiheadAttention", "DPRNN", "RenameParamsMixin", "SequenceBias"
    ],
    "validators": [
        "ModuleValidator", "register_module_fixer", "register_module_validator"
    ],
    "validators.errors": [
        "IllegalModuleConfigurationError", "NotYetSupportedModuleError", "ShouldReplaceModuleError",
        "UnsupportableModuleError", "UnsupportedError", "UnsupportedModuleError"
    ],
    "schedulers": [
        "ExponentialGradClip", "ExponentialNoise", "LambdaGradClip", "LambdaNoise", "StepGradClip",
        "StepNoise", "_GradClipScheduler", "_NoiseScheduler"
    ],
    "utils.uniform_sampler": [
        "DistributedUniformWithReplacementSampler", "UniformWithReplacementSampler"
    ],
    "utils.batch_memory_manager": [
        "BatchMemoryManager", "BatchSplittingSampler", "wrap_data_loader"
    ],
    "utils.fast_gradient_clipping_utils": [
        "DPLossFastGradientClipping", "DPTensorFastGradientClipping"
    ],
    "utils.module_utils": [
        "are_state_dict_equal", "clone_module", "get_submodule", "has_trainable_params",
        "parametrized_modules", "requires_grad", "trainable_modules", "trainable_parameters"
    ],
    "utils.tensor_utils": [
        "calc_sample_norms", "calc_sample_norms_one_layer", "filter_dilated_rows",
        "sum_over_all_but_batch_and_last_n", "unfold2d", "unfold3d"
    ],
    "utils.packed_sequences": [
        "compute_seq_lengths"
    ],
    "utils.per_sample_gradients_utils": [
        "ModelWithLoss", "check_per_sample_gradients_are_correct", "check_torch_version_for_ew_sample",
        "clone_module", "compute_grad_samples_microbatch_and_opacus", "compute_microbatch_grad_sample",
        "compute_microbatch_grad_sample_tensor_or_seq", "compute_opacus_grad_sample",
        "get_grad_sample_modes", "is_batch_empty", "unpack_packedsequences"
    ],
    "utils.fsdp_utils": [
        "FSDP2Wrapper", "has_params", "iterate_submodules"
    ],
    "privacy_engine": [
        "PrivacyEngine"
    ],
    "layers.dp_rnn": [
        "DPGRU", "DPGRUCell", "DPLSTM", "DPLSTMCell", "DPRNN", "DPRNNBase", "DPRNNCell", "DPRNNCellBase",
        "RNNLinear", "apply_permutation"
    ],
    "layers.dp_multihead_attention": [
        "DPMultiheadAttention", "SequenceBias"
    ],
    "layers.param_rename": [
        "RenameParamsMixin", "filter_out_old_keys"
    ],
    "optimizers.utils": [
        "params"
    ],
    "grad_sample.utils": [
        "get_gsm_class", "get_hooks_class", "prepare_module", "register_grad_sampler",
        "register_norm_sampler", "wrap_model"
    ],
}


@pytest.mark.parametrize("module", sorted(API))
def test_public_names_exist(module):
    mod = importlib.import_module("opacus_b200" + ("." + module if module else ""))
    missing = [name for name in API[module] if not hasattr(mod, name)]
    assert not missing, f"opacus_b200{'.' + module if module else ''} lacks {missing}"


def test_signatures_of_the_entry_points():
    import inspect

    from opacus_b200 import PrivacyEngine

    want = ["module", "optimizer", "criterion", "data_loader", "noise_multiplier", "max_grad_norm", "batch_first",
            "loss_reduction", "poisson_sampling", "clipping", "noise_generator", "grad_sample_mode"]
    have = list(inspect.signature(PrivacyEngine.make_private).parameters)
    assert [p for p in want if p not in have] == []
    eps = list(inspect.signature(PrivacyEngine.make_private_with_epsilon).parameters)
    assert all(p in eps for p in ("target_epsilon", "target_delta", "epochs", "max_grad_norm"))
    assert list(inspect.signature(PrivacyEngine.__init__).parameters)[1:] == ["accountant", "secure_mode"]
    for method in ("get_epsilon", "save_checkpoint", "load_checkpoint", "validate", "is_compatible", "get_compatible_module"):
        assert hasattr(PrivacyEngine, method), method
