"""Load-balancing losses with the reference's names (src/balancing/)."""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

from . import _lib


class LoadBalancingLoss:
    """abstract type LoadBalancingLoss (src/gating/base.jl:14)."""


@dataclass
class SwitchTransformerLoss(LoadBalancingLoss):
    """SwitchTransformerLoss(alpha): alpha * N * sum_i f_i P_i (src/balancing/losses.jl:11-36)."""
    alpha: float = 0.01


@dataclass
class ZLoss(LoadBalancingLoss):
    """ZLoss(beta): beta * mean(logsumexp(logits)^2) (src/balancing/losses.jl:99-108)."""
    beta: float = 0.001


@dataclass
class AuxiliaryFreeLoss(LoadBalancingLoss):
    """AuxiliaryFreeLoss(num_experts; ...) (src/balancing/auxiliary_free.jl:11-34).  The layer
    adds ``bias`` to the router logits before selecting experts (moe_layer.jl:137-140); the
    momentum update of the bias (auxiliary_free.jl:36-71) runs on the host from the per-call
    expert counts."""
    num_experts: int
    bias_init: float = 0.0
    learning_rate: float = 0.01
    momentum: float = 0.9
    update_freq: int = 1
    use_complementary_loss: bool = True
    complementary_weight: float = 0.001
    bias: np.ndarray = field(default=None)
    bias_momentum: np.ndarray = field(default=None)
    update_counter: int = 0

    def __post_init__(self):
        if self.bias is None:
            self.bias = np.full(self.num_experts, self.bias_init, dtype=np.float32)
        if self.bias_momentum is None:
            self.bias_momentum = np.zeros(self.num_experts, dtype=np.float32)

    def update_bias(self, expert_counts) -> None:
        """update_bias! (src/balancing/auxiliary_free.jl:36-71) from per-expert counts."""
        self.update_counter += 1
        if self.update_counter % self.update_freq != 0:
            return
        counts = np.asarray(expert_counts, dtype=np.float32)
        total = float(counts.sum())
        if total == 0:
            return
        target = total / self.num_experts
        grad = (counts - np.float32(target)) / np.float32(total)
        self.bias_momentum = (np.float32(self.momentum) * self.bias_momentum
                              + np.float32(1 - self.momentum) * grad).astype(np.float32)
        self.bias = (self.bias - np.float32(self.learning_rate) * self.bias_momentum).astype(np.float32)
        self.bias = (self.bias - self.bias.mean(dtype=np.float32)).astype(np.float32)


def compute_loss(loss_fn, expert_indices, router_probs=None):
    """compute_loss(loss, expert_indices, router_probs) for SwitchTransformerLoss, and
    compute_loss(ZLoss(beta), router_logits) (src/balancing/losses.jl:15-36, :103-108) on CUDA
    tensors laid out like the reference's: expert_indices (k, T) 1-based, router_probs (E, T).
    Returns a 0-d CUDA float32 tensor."""
    import torch

    if isinstance(loss_fn, ZLoss):
        logits_t = expert_indices.t().contiguous()
        T, E = logits_t.shape
        dummy_idx = torch.ones((T, 1), dtype=torch.int32, device=logits_t.device)
        dummy_p = torch.zeros((T, 1), dtype=torch.float32, device=logits_t.device)
        out = torch.empty((), dtype=torch.float32, device=logits_t.device)
        with torch.cuda.device(logits_t.device):
            _lib.check(_lib.lib.moe_compute_loss(0.0, float(loss_fn.beta), 1, 1, 1, dummy_idx.data_ptr(),
                                                 dummy_p.data_ptr(), logits_t.data_ptr(), E, T, out.data_ptr(),
                                                 torch.cuda.current_stream().cuda_stream))
        return out
    if not isinstance(loss_fn, SwitchTransformerLoss):
        raise _lib.MoEError(_lib.ERR_UNSUPPORTED, f"loss {type(loss_fn).__name__} is not accelerated")
    idx_t = expert_indices.t().contiguous().to(torch.int32)
    p_t = router_probs.t().contiguous()
    T, k = idx_t.shape
    N = p_t.shape[1]
    out = torch.empty((), dtype=torch.float32, device=p_t.device)
    with torch.cuda.device(p_t.device):
        _lib.check(_lib.lib.moe_compute_loss(float(loss_fn.alpha), 0.0, N, k, 1, idx_t.data_ptr(), p_t.data_ptr(),
                                             None, 0, T, out.data_ptr(), torch.cuda.current_stream().cuda_stream))
    return out
