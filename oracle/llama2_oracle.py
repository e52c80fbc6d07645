"""CPU oracle of the Llama2 + MoE decode path (TEST INFRASTRUCTURE ONLY; see moe_oracle.py for
the status of parity: unpinned by the reference, pinned here by cross-checks).

Restates, one token at a time like the reference, moe_transformer! (src/llama2/inference.jl:14-50):
moe_attention! (src/llama2/attention.jl:15-48) with apply_rope_normal! (:69-88) and
compute_attention_output! (:137-168), dense_ffn_forward! (inference.jl:131-147), moe_ffn_forward!
(:58-121), final rmsnorm + classifier (:45-47), and convert_to_moe's expert construction
(src/llama2/conversion.jl:277-331, :358-367).  Llama2.jl itself is not vendored by the reference;
its two primitives are restated from llama2.c, which Llama2.jl ports: matmul!(o, W, x) = W^T x and
rmsnorm!(o, x, w) = w .* x ./ sqrt(mean(x.^2) + 1e-5).

Weight matrices are held as (out, in) C-order NumPy arrays, which is the memory of the reference's
(in x out) column-major arrays.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

import numpy as np

from . import moe_oracle as orc

RMS_EPS = np.float32(1e-5)


def rmsnorm(x: np.ndarray, w: np.ndarray) -> np.ndarray:
    ss = np.float32(np.dot(x, x) / np.float32(x.size)) + RMS_EPS
    return (w * (x * (np.float32(1.0) / np.sqrt(ss)))).astype(np.float32)


def rope_normal(v: np.ndarray, pos: int, n_heads: int, freq_base: float = 10000.0) -> np.ndarray:
    """apply_rope_normal! (attention.jl:69-88): adjacent pairs rotated as complex numbers by
    theta_i, theta_0 = pos-1 (pos is 1-based), theta_{i+1} = theta_i * freq_base^(-1/(head_size/2)),
    the recurrence evaluated in Float32 like the reference."""
    head = v.size // n_heads
    half = head // 2
    theta_scale = np.float32(np.float32(freq_base) ** np.float32(-1.0 / np.float32(half)))
    thetas = np.empty(half, dtype=np.float32)
    th = np.float32(pos - 1)
    for i in range(half):
        thetas[i] = th
        th = np.float32(th * theta_scale)
    c, s = np.cos(thetas), np.sin(thetas)
    out = v.reshape(n_heads, half, 2).copy()
    re, im = out[:, :, 0].copy(), out[:, :, 1].copy()
    out[:, :, 0] = re * c - im * s
    out[:, :, 1] = re * s + im * c
    return out.reshape(-1).astype(np.float32)


@dataclass
class LayerW:
    rms_att: np.ndarray
    rms_ffn: np.ndarray
    wq: np.ndarray
    wk: np.ndarray
    wv: np.ndarray
    wo: np.ndarray
    w1: np.ndarray            # (hidden, dim)
    w2: np.ndarray            # (dim, hidden)
    w3: np.ndarray            # (hidden, dim)
    use_moe: bool = False
    router: Optional[np.ndarray] = None                    # (E, dim)
    experts: List[orc.GatedExpertWeights] = field(default_factory=list)


@dataclass
class Model:
    dim: int
    hidden_dim: int
    n_heads: int
    n_kv_heads: int
    vocab_size: int
    seq_len: int
    embedding: np.ndarray     # (vocab, dim)
    layers: List[LayerW]
    rms_final: np.ndarray
    output: np.ndarray        # (vocab, dim)
    top_k: int = 2


def forward_tokens(m: Model, tokens) -> dict:
    """Runs moe_transformer! for positions 1..len(tokens) with a fresh KV cache.  Returns the
    logits of every position and, per MoE layer, the selected experts (1-based) of every position."""
    n = len(tokens)
    L = len(m.layers)
    head = m.dim // m.n_heads
    n_gqa = m.n_heads // m.n_kv_heads
    kc = np.zeros((L, n, m.n_kv_heads, head), dtype=np.float32)
    vc = np.zeros((L, n, m.n_kv_heads, head), dtype=np.float32)
    logits = np.zeros((n, m.vocab_size), dtype=np.float32)
    selected = {li: np.zeros((n, m.top_k), dtype=np.int64) for li, l in enumerate(m.layers) if l.use_moe}
    scale = np.float32(1.0) / np.sqrt(np.float32(head))
    for p in range(n):
        pos = p + 1
        x = m.embedding[tokens[p]].copy()
        for li, l in enumerate(m.layers):
            xb = rmsnorm(x, l.rms_att)
            q = rope_normal(l.wq @ xb, pos, m.n_heads)
            k = rope_normal(l.wk @ xb, pos, m.n_kv_heads)
            v = l.wv @ xb
            kc[li, p] = k.reshape(m.n_kv_heads, head)
            vc[li, p] = v.reshape(m.n_kv_heads, head)
            qh = q.reshape(m.n_heads, head)
            out = np.zeros((m.n_heads, head), dtype=np.float32)
            for h in range(m.n_heads):
                kvh = h // n_gqa
                att = (kc[li, :pos, kvh] @ qh[h]) * scale
                att = np.exp(att - att.max())
                att = att / att.sum(dtype=np.float32)
                out[h] = att @ vc[li, :pos, kvh]
            x = x + l.wo @ out.reshape(-1)
            xb = rmsnorm(x, l.rms_ffn)
            if l.use_moe:
                y, idx, _, _ = orc.moe_ffn_forward_token(l.router, l.experts, orc.TopKGating(m.top_k), m.top_k, xb)
                selected[li][p] = idx
            else:
                h1 = l.w1 @ xb
                y = l.w2 @ (orc.llama_silu(h1) * (l.w3 @ xb))
            x = x + y
        x = rmsnorm(x, m.rms_final)
        logits[p] = m.output @ x
    return {"logits": logits, "selected": selected}
