"""Independent float64 cross-check of oracle/moe_oracle.py (TEST INFRASTRUCTURE ONLY).

Written on purpose with a different structure from the NumPy oracle: every expert is evaluated
densely on every token and masked by the gate matrix (the shape of the reference's own GPU
path, src/cuda/experts.jl:28-57), top-k is an explicit k-pass arg-max with strict '>' so ties
go to the lowest index (src/cuda/kernels.jl:3-43), and everything runs in torch float64.
Agreement of the two restatements is what pins the oracle in the absence of a runnable
reference (no Julia runtime is available).
"""
from __future__ import annotations

import math

import torch


def _act(name, v):
    if name == "silu":
        return v * torch.sigmoid(v)
    if name == "gelu":
        return 0.5 * v * (1 + torch.tanh(math.sqrt(2 / math.pi) * (v + 0.044715 * v ** 3)))
    if name == "relu":
        return torch.clamp_min(v, 0)
    return v


def topk_passes(probs: torch.Tensor, k: int):
    """k passes of arg-max with 'previously selected' exclusion; strict '>' keeps the lowest
    index among equal values."""
    T, E = probs.shape
    taken = torch.zeros_like(probs, dtype=torch.bool)
    idx = torch.zeros((T, k), dtype=torch.int64)
    val = torch.zeros((T, k), dtype=probs.dtype)
    for s in range(k):
        masked = probs.masked_fill(taken, -1.0)
        best = torch.full((T,), -2.0, dtype=probs.dtype)
        arg = torch.zeros((T,), dtype=torch.int64)
        for e in range(E):
            better = masked[:, e] > best
            best = torch.where(better, masked[:, e], best)
            arg = torch.where(better, torch.full_like(arg, e), arg)
        idx[:, s] = arg
        val[:, s] = best
        taken[torch.arange(T), arg] = True
    return idx, val


def layer_forward64(x, router, experts, *, k, activation="silu", alpha=0.01, z_weight=0.001,
                    training=True, num_shared_gating=0, logit_bias=None, bias_gates_only=False):
    """x (T,D); router (E_r,D); experts list of (w1,w2,w3) with shapes (H,D),(O,H),(H,D),
    or of (w1,w2,b1,b2) for standard experts.
    num_shared_gating=S>0 reproduces SharedExpertGating(S, TopKGating(k), E)
    (src/gating/advanced.jl:80-108) inside forward_standard.
    Returns output (T,O), loss, 0-based indices (T,k_tot), gates, probs -- all float64."""
    x = torch.as_tensor(x, dtype=torch.float64)
    Wr = torch.as_tensor(router, dtype=torch.float64)
    T = x.shape[0]
    E = len(experts)
    S = num_shared_gating
    logits = x @ Wr.T
    sel_logits = logits
    if logit_bias is not None:
        b = torch.as_tensor(logit_bias, dtype=torch.float64)
        sel_logits = logits + b
        if not bias_gates_only:
            logits = sel_logits

    def gate_of(lg):
        r = lg[:, S:]
        p = torch.softmax(r, dim=-1)
        i, v = topk_passes(p, k)
        g = v / v.sum(-1, keepdim=True)
        return i, g, p

    r_idx, r_g, _ = gate_of(sel_logits)
    _, _, r_p = gate_of(logits)
    k_tot = S + k
    idx = torch.zeros((T, k_tot), dtype=torch.int64)
    g = torch.zeros((T, k_tot), dtype=torch.float64)
    probs = torch.zeros((T, E), dtype=torch.float64)
    if S:
        idx[:, :S] = torch.arange(S)
        g[:, :S] = 1.0 / k_tot
        probs[:, :S] = 1.0 / E
    idx[:, S:] = r_idx + S
    g[:, S:] = r_g * (1.0 - S / k_tot)
    probs[:, S:] = r_p * (1.0 - S / E)

    gate_matrix = torch.zeros((T, E), dtype=torch.float64)
    gate_matrix.scatter_add_(1, idx, g)
    O = experts[0][1].shape[0]
    out = torch.zeros((T, O), dtype=torch.float64)
    for e, ws in enumerate(experts):
        if not bool((gate_matrix[:, e] != 0).any()):
            continue
        f64 = lambda a: torch.as_tensor(a, dtype=torch.float64)
        if len(ws) == 4:      # StandardExpert (w1, w2, b1, b2): w2(act.(w1 x .+ b1)) .+ b2
            w1, w2, b1, b2 = (f64(a) for a in ws)
            y = _act(activation, x @ w1.T + b1) @ w2.T + b2
        else:
            w1, w2, w3 = (f64(a) for a in ws)
            y = (_act(activation, x @ w1.T) * (x @ w3.T)) @ w2.T
        out += gate_matrix[:, e:e + 1] * y

    loss = torch.zeros((), dtype=torch.float64)
    if training:
        counts = torch.bincount(idx.reshape(-1), minlength=E).to(torch.float64)
        f = counts / idx.numel()
        P = probs.mean(0)
        loss = alpha * E * (f * P).sum()
        if z_weight > 0:
            lse = torch.logsumexp(logits, dim=-1)
            loss = loss + z_weight * (lse ** 2).mean()
    return out, loss, idx, g, probs
