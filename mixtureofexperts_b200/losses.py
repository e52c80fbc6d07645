"""Load-balancing losses with the reference's names (src/balancing/)."""
from __future__ import annotations

from dataclasses import dataclass

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


class AuxiliaryFreeLoss(LoadBalancingLoss):
    """AuxiliaryFreeLoss(num_experts; ...) (src/balancing/auxiliary_free.jl:11-34).  The layer
    adds ``bias`` to the router logits before selecting experts (moe_layer.jl:137-140).

    Once a MoELayer holds this loss, ``bias``, ``bias_momentum`` and ``update_counter`` live in
    the layer's device handle, where every training forward updates them (update_bias!,
    auxiliary_free.jl:36-71) without a host round trip; reading an attribute here fetches the
    current device state, assigning ``bias`` pushes it.  Unattached (or attached to a layer whose
    configuration keeps the update on the host) the state is plain NumPy and ``update_bias`` applies
    the same update from per-expert counts."""

    def __init__(self, num_experts: int, bias_init: float = 0.0, learning_rate: float = 0.01, momentum: float = 0.9,
                 update_freq: int = 1, use_complementary_loss: bool = True, complementary_weight: float = 0.001,
                 bias=None, bias_momentum=None, update_counter: int = 0):
        self.num_experts = int(num_experts)
        self.bias_init = float(bias_init)
        self.learning_rate = float(learning_rate)
        self.momentum = float(momentum)
        self.update_freq = int(update_freq)
        self.use_complementary_loss = bool(use_complementary_loss)
        self.complementary_weight = float(complementary_weight)
        self._bias = (np.full(self.num_experts, self.bias_init, dtype=np.float32) if bias is None
                      else np.array(bias, dtype=np.float32))
        self._bias_momentum = (np.zeros(self.num_experts, dtype=np.float32) if bias_momentum is None
                               else np.array(bias_momentum, dtype=np.float32))
        self._update_counter = int(update_counter)
        self._device_state = None       # callable () -> (bias, momentum, counter) while a layer owns the state
        self._device_push = None        # callable () pushing the host copy to that layer

    def _pull(self) -> None:
        if self._device_state is not None:
            self._bias, self._bias_momentum, self._update_counter = self._device_state()

    @property
    def bias(self) -> np.ndarray:
        self._pull()
        return self._bias

    @bias.setter
    def bias(self, value) -> None:
        self._pull()
        self._bias = np.array(value, dtype=np.float32)
        if self._device_push is not None:
            self._device_push()

    @property
    def bias_momentum(self) -> np.ndarray:
        self._pull()
        return self._bias_momentum

    @property
    def update_counter(self) -> int:
        self._pull()
        return self._update_counter

    def update_bias(self, expert_counts) -> None:
        """update_bias! (src/balancing/auxiliary_free.jl:36-71) from per-expert counts, on the
        host.  Julia's promotion is kept: Int/Int target and the gradient are Float64, the
        momentum blend is rounded into the Float32 vector, the bias step and centring are Float32."""
        self._pull()
        self._update_counter += 1
        if self._update_counter % self.update_freq == 0:
            counts = np.asarray(expert_counts, dtype=np.float32)
            total = int(counts.sum(dtype=np.float64))
            if total != 0:
                f = np.float32
                grad = (counts.astype(np.float64) - total / self.num_experts) / total
                keep = (f(self.momentum) * self._bias_momentum).astype(np.float32)
                self._bias_momentum = (keep.astype(np.float64) + np.float64(f(1) - f(self.momentum)) * grad).astype(f)
                b = (self._bias - f(self.learning_rate) * self._bias_momentum).astype(f)
                mean = f(0)
                for v in b:
                    mean = f(mean + v)
                self._bias = (b - f(mean / f(self.num_experts))).astype(f)
        if self._device_push is not None:
            self._device_push()


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
