"""Shared helpers of the parity tests: build a device layer from oracle weights and compare."""
from __future__ import annotations

import numpy as np

from oracle import moe_oracle as orc


def rel_inf(a, b) -> float:
    """||a-b||_inf / ||b||_inf, the per-tensor norm of the parity criteria."""
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    den = np.abs(b).max()
    return float(np.abs(a - b).max() / (den if den > 0 else 1.0))


def oracle_gate(kind, k, S=0, E=None):
    if kind == "topk":
        return orc.TopKGating(k)
    if kind == "switch":
        return orc.SwitchGating()
    return orc.SharedExpertGating(S, orc.TopKGating(k), E)


def device_gate(kind, k, S=0, E=None):
    import mixtureofexperts_b200 as m

    if kind == "topk":
        return m.TopKGating(k)
    if kind == "switch":
        return m.SwitchGating()
    return m.SharedExpertGating(S, m.TopKGating(k), E)


def make_device_layer(weights: orc.MoEWeights, *, D, H, O, gate, activation="silu", alpha=0.01, z=0.001,
                      compute_dtype="f32", num_shared_experts=0, balance_loss=None, router_bias=None, device=0,
                      **config_extra):
    """A MoELayer of the product package holding exactly the oracle's weights."""
    import mixtureofexperts_b200 as m

    act = {"silu": m.silu, "gelu": m.gelu, "relu": m.relu, "identity": m.identity}[activation]
    standard = isinstance(weights.experts[0], orc.StandardExpertWeights)
    cfg = m.create_moe_config(num_experts=len(weights.experts), expert_type="standard" if standard else "gated", input_dim=D, hidden_dim=H,
                              output_dim=O, activation=act, gate_type=gate,
                              balance_loss=balance_loss or m.SwitchTransformerLoss(alpha), z_loss_weight=z,
                              num_shared_experts=num_shared_experts, **config_extra)
    experts = []
    for e in weights.experts:
        if standard:
            ex = m.StandardExpert.__new__(m.StandardExpert)
            ex.input_dim, ex.hidden_dim, ex.output_dim, ex.activation = D, H, O, act
            ex.w1, ex.w2, ex.b1, ex.b2 = e.w1, e.w2, e.b1, e.b2
            experts.append(ex)
            continue
        ex = m.GatedExpert.__new__(m.GatedExpert)
        ex.input_dim, ex.hidden_dim, ex.output_dim, ex.activation = D, H, O, act
        ex.w1, ex.w2, ex.w3 = e.w1, e.w2, e.w3
        experts.append(ex)
    router = m.Router.__new__(m.Router)
    router.weight = weights.router
    router.noise_weight = None
    router.gate_type = gate
    router.noise_scale = 0.0
    router.use_fp32 = True
    if router_bias is not None:
        router.bias = router_bias
    return m.MoELayer(cfg, device=device, compute_dtype=compute_dtype, experts=experts, router=router)


def check_indices(dev_idx, ora_idx, logits64, k_routed, r0=0, tol=1e-6):
    """Expert ids must match exactly, except for tokens where the float64 logits of the
    k-th and (k+1)-th ranked routed experts differ by less than `tol` (a tie).
    dev_idx / ora_idx: (T, k_tot) 1-based.  Returns the number of tie-excused tokens."""
    dev_idx = np.asarray(dev_idx)
    ora_idx = np.asarray(ora_idx)
    assert dev_idx.shape == ora_idx.shape, (dev_idx.shape, ora_idx.shape)
    bad = np.where((dev_idx != ora_idx).any(axis=1))[0]
    excused = 0
    for t in bad:
        lg = np.sort(np.asarray(logits64[t, r0:], dtype=np.float64))[::-1]
        # any pair of neighbours in the ranking around the selected set may have swapped
        gaps = np.abs(np.diff(lg[:k_routed + 1]))
        assert gaps.min() < tol, f"token {t}: indices {dev_idx[t]} vs {ora_idx[t]} without a tie (min gap {gaps.min():.3e})"
        assert sorted(dev_idx[t]) == sorted(ora_idx[t]) or gaps[-1] < tol
        excused += 1
    return excused
