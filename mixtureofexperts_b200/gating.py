"""Gating mechanisms with the reference's names and semantics (src/gating/)."""
from __future__ import annotations

from dataclasses import dataclass

from . import _lib


class GatingMechanism:
    """abstract type GatingMechanism (src/gating/base.jl:7)."""


@dataclass
class TopKGating(GatingMechanism):
    """TopKGating(k) (src/gating/topk.jl:16-22): softmax, top-k of the probabilities
    (ties to the lowest index), gates renormalised over the selected k."""
    k: int
    use_softmax_renorm: bool = True
    use_raw_logits: bool = False


@dataclass
class SwitchGating(GatingMechanism):
    """SwitchGating() = TopKGating(1) (src/gating/switch.jl:7-11)."""

    @property
    def k(self) -> int:
        return 1


@dataclass
class SharedExpertGating(GatingMechanism):
    """SharedExpertGating(num_shared, base_gate, num_experts) (src/gating/advanced.jl:74-108):
    experts 1..num_shared are selected for every token with gate 1/k_tot, the base gate routes
    over the remaining experts and its gates are scaled by 1 - num_shared/k_tot."""
    num_shared: int
    base_gate: GatingMechanism
    num_experts: int


@dataclass
class JitterGating(GatingMechanism):
    """JitterGating(base_gate, ε) (src/gating/switch.jl:20-33): when ``compute_gates`` is called with
    ``training=True`` the logits are multiplied by uniform jitter in [1-ε, 1+ε) before the base
    gate.  The reference's Router calls ``compute_gates(gate, logits)`` without the keyword
    (src/core/router.jl:43), so inside a MoELayer this gate routes exactly like its base gate."""
    base_gate: GatingMechanism
    ε: float

    @property
    def eps(self) -> float:
        return float(self.ε)


def gate_kind_of(gate) -> tuple[int, int, int]:
    """(gate_kind, k, num_shared) of a gate object for the C ABI."""
    if isinstance(gate, JitterGating):
        return gate_kind_of(gate.base_gate)
    if isinstance(gate, TopKGating):
        return _lib.GATE_TOPK, int(gate.k), 0
    if isinstance(gate, SwitchGating):
        return _lib.GATE_SWITCH, 1, 0
    if isinstance(gate, SharedExpertGating):
        base = gate.base_gate
        if isinstance(base, (TopKGating, SwitchGating)):
            return _lib.GATE_SHARED_TOPK, int(base.k), int(gate.num_shared)
        raise _lib.MoEError(_lib.ERR_UNSUPPORTED, f"SharedExpertGating over {type(base).__name__} is not supported")
    raise _lib.MoEError(_lib.ERR_UNSUPPORTED,
                        f"gate {type(gate).__name__} is not accelerated (TopKGating, SwitchGating, SharedExpertGating are)")


def compute_gates(gate, router_logits, training: bool = False, jitter=None):
    """compute_gates(gate, router_logits[; training]) -> (expert_indices, expert_gates, router_probs)
    (src/gating/base.jl:22).  ``training`` only matters for JitterGating; ``jitter`` then optionally
    gives its uniform [0,1) draws, shaped like router_logits (drawn with torch when omitted).  router_logits: CUDA float32 tensor of shape (num_experts, T)
    whose memory is column-major like the reference's matrix, i.e. ``logits_TE.t()``.
    Returns tensors shaped (k, T), (k, T), (num_experts, T) with 1-based expert ids."""
    import torch

    kind, k, S = gate_kind_of(gate)
    lt = router_logits.t()
    if not lt.is_contiguous():
        lt = lt.contiguous()
    if lt.dtype != torch.float32 or not lt.is_cuda:
        raise _lib.MoEError(_lib.ERR_INVALID, "router_logits must be a CUDA float32 tensor")
    T, E = lt.shape
    k_tot = k + S
    idx = torch.empty((T, k_tot), dtype=torch.int32, device=lt.device)
    gates = torch.empty((T, k_tot), dtype=torch.float32, device=lt.device)
    probs = torch.empty((T, E), dtype=torch.float32, device=lt.device)
    shared = gate.base_gate if isinstance(gate, JitterGating) else gate
    if isinstance(shared, SharedExpertGating) and shared.num_experts != E:
        raise _lib.MoEError(_lib.ERR_INVALID, "SharedExpertGating.num_experts does not match the logits")
    with torch.cuda.device(lt.device):
        stream = torch.cuda.current_stream().cuda_stream
        if isinstance(gate, JitterGating) and training:
            if jitter is None:
                u = torch.rand((T, E), device=lt.device, dtype=torch.float32)
            else:
                u = jitter.to(device=lt.device, dtype=torch.float32).t().contiguous()
                if tuple(u.shape) != (T, E):
                    raise _lib.MoEError(_lib.ERR_INVALID, "jitter must be shaped like router_logits")
            _lib.check(_lib.lib.moe_compute_gates_jitter(kind, E, S, k, 1, lt.data_ptr(), u.data_ptr(), gate.eps, T,
                                                         idx.data_ptr(), gates.data_ptr(), probs.data_ptr(), stream))
            return idx.t(), gates.t(), probs.t()
        _lib.check(_lib.lib.moe_compute_gates(kind, E, S, k, 1, lt.data_ptr(), T, idx.data_ptr(),
                                              gates.data_ptr(), probs.data_ptr(), stream))
    return idx.t(), gates.t(), probs.t()
