"""mixtureofexperts_b200: the MoE-layer forward pass of MixtureOfExperts.jl on NVIDIA B200.

The names mirror the reference package (create_moe_config, MoELayer, TopKGating, SwitchGating,
GatedExpert, SwitchTransformerLoss, convert_to_moe, sample_moe, ...); the arithmetic runs in
hand-written CUDA kernels behind the C ABI of ``lib/libmoe_b200.so`` (include/moe_b200.h).
Importing the package requires that library; there is no CPU or PyTorch fallback.
"""
from ._lib import LIB_PATH, MoEError, version
from .experts import Expert, GatedExpert, gelu, identity, relu, silu, swish
from .gating import GatingMechanism, SharedExpertGating, SwitchGating, TopKGating, compute_gates
from .layer import (MoEConfig, MoELayer, Router, create_moe_config, create_moe_layer, load_balance_score,
                    reset_stats)
from .losses import AuxiliaryFreeLoss, LoadBalancingLoss, SwitchTransformerLoss, ZLoss, compute_loss

__all__ = [
    "LIB_PATH", "MoEError", "version", "Expert", "GatedExpert", "gelu", "identity", "relu", "silu", "swish",
    "GatingMechanism", "SharedExpertGating", "SwitchGating", "TopKGating", "compute_gates", "MoEConfig",
    "MoELayer", "Router", "create_moe_config", "create_moe_layer", "load_balance_score", "reset_stats",
    "AuxiliaryFreeLoss", "LoadBalancingLoss", "SwitchTransformerLoss", "ZLoss", "compute_loss",
]
