"""mixtureofexperts_b200: the MoE-layer forward pass of MixtureOfExperts.jl on NVIDIA B200.

The names mirror the reference package (create_moe_config, MoELayer, TopKGating, SwitchGating,
GatedExpert, SwitchTransformerLoss, convert_to_moe, sample_moe, ...); the arithmetic runs in
hand-written CUDA kernels behind the C ABI of ``lib/libmoe_b200.so`` (include/moe_b200.h).
Using any of these names requires that library; there is no CPU or PyTorch fallback.  Names
are resolved on first use so that ``python -m mixtureofexperts_b200.build`` can (re)build the
library before it is loaded.
"""
import importlib

_EXPORTS = {
    "LIB_PATH": "_lib", "MoEError": "_lib", "version": "_lib",
    "Expert": "experts", "GatedExpert": "experts", "StandardExpert": "experts", "gelu": "experts", "identity": "experts", "relu": "experts",
    "silu": "experts", "swish": "experts",
    "GatingMechanism": "gating", "JitterGating": "gating", "SharedExpertGating": "gating", "SwitchGating": "gating", "TopKGating": "gating",
    "compute_gates": "gating",
    "MoEConfig": "layer", "MoELayer": "layer", "Router": "layer", "create_moe_config": "layer",
    "create_moe_layer": "layer", "load_balance_score": "layer", "reset_stats": "layer",
    "AuxiliaryFreeLoss": "losses", "LoadBalancingLoss": "losses", "SwitchTransformerLoss": "losses",
    "ZLoss": "losses", "compute_loss": "losses",
    "convert_to_moe": "llama2", "sample_moe": "llama2", "save_moe_model": "llama2", "usage_balance_score": "llama2", "expert_stats_lines": "llama2", "load_moe_model": "llama2", "moe_transformer": "llama2", "MoERunState": "llama2",
    "MoELanguageModel": "llama2", "MoEExpertWeights": "llama2", "LanguageModel": "llama2", "ModelConfig": "llama2",
    "random_language_model": "llama2", "count_parameters": "llama2", "count_active_parameters": "llama2",
}

__all__ = sorted(_EXPORTS)


def __getattr__(name):
    mod = _EXPORTS.get(name)
    if mod is None:
        raise AttributeError(f"module 'mixtureofexperts_b200' has no attribute '{name}'")
    value = getattr(importlib.import_module(f".{mod}", __name__), name)
    globals()[name] = value
    return value


def __dir__():
    return __all__
