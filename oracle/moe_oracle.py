"""CPU oracle: a NumPy restatement of MixtureOfExperts.jl's MoE-layer forward pass.

TEST INFRASTRUCTURE ONLY.  Nothing under the product package may import this module; it is
the checker used by tests/, by __graft_entry__.smoke() and by bench.py's CPU-baseline legs.

PARITY UNPINNED: the reference is Julia and no Julia runtime is available to execute it, and
its own test script holds no golden vectors or known-answer fixtures for this path (only
property checks: gates sum to 1, indices in range, finite outputs, loss >= 0).  This file
therefore restates the reference line by line from its source, each function citing the
file:line it follows, and is cross-checked against an independently written float64
restatement (oracle/moe_oracle_torch64.py) and the reference's property checks.

Memory conventions: Julia is column-major, so the reference's (D x T) input is held here as
a C-order array of shape (T, D); (k x T) arrays are (T, k); (E x T) arrays are (T, E).
Weight matrices keep the reference's logical shape (out, in) as NumPy C-order arrays.
Expert ids are 1-based as in the reference; 0 marks a dropped slot.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Tuple

import numpy as np

# --------------------------------------------------------------------------------------
# activations (NNlib semantics; src/experts/gated.jl:36 for silu)
# --------------------------------------------------------------------------------------


def sigmoid(x):
    return 1 / (1 + np.exp(-x))


def silu(x):
    """x * sigmoid(x)  (src/experts/gated.jl:36; src/llama2/inference.jl:159-162)."""
    return x * sigmoid(x)


def gelu_tanh(x):
    """NNlib.gelu: 0.5x(1+tanh(sqrt(2/pi)(x+0.044715x^3))) (MoEConfig default activation,
    src/core/moe_layer.jl:10)."""
    c = x.dtype.type(math.sqrt(2.0 / math.pi))
    return x.dtype.type(0.5) * x * (1 + np.tanh(c * (x + x.dtype.type(0.044715) * x * x * x)))


def relu(x):
    return np.maximum(x, 0)


def identity(x):
    return x


ACTIVATIONS = {"silu": silu, "gelu": gelu_tanh, "relu": relu, "identity": identity}

# --------------------------------------------------------------------------------------
# gating
# --------------------------------------------------------------------------------------


def softmax_dim1(logits: np.ndarray) -> np.ndarray:
    """NNlib.softmax(logits; dims=1) on an (E x T) matrix = softmax over the last axis of
    our (T, E) array: subtract the column max, exponentiate, divide by the sum
    (src/gating/topk.jl:27)."""
    m = logits.max(axis=-1, keepdims=True)
    e = np.exp(logits - m)
    return e / e.sum(axis=-1, keepdims=True, dtype=logits.dtype)


def partialsortperm_rev(v: np.ndarray, k: int) -> np.ndarray:
    """Base.partialsortperm(v, 1:k, rev=true): indices of the k largest values, descending,
    equal values in ascending index order (src/gating/topk.jl:35; the reference's own GPU
    kernel breaks ties the same way, src/cuda/kernels.jl:24).  Returns 0-based indices."""
    order = np.argsort(-v, kind="stable")
    return order[:k]


@dataclass
class TopKGating:
    """src/gating/topk.jl:16-22"""
    k: int


@dataclass
class SwitchGating:
    """src/gating/switch.jl:7"""
    k: int = 1


@dataclass
class SharedExpertGating:
    """src/gating/advanced.jl:74-78 (positional: num_shared, base_gate, num_experts)"""
    num_shared: int
    base_gate: object
    num_experts: int


@dataclass
class JitterGating:
    """src/gating/switch.jl:20-23 (positional: base_gate, ε)"""
    base_gate: object
    eps: float


def compute_gates_topk(k: int, logits: np.ndarray):
    """compute_gates(::TopKGating, logits) (src/gating/topk.jl:24-44).
    logits (T, E) -> indices (T, k) int64 1-based, gates (T, k) float32, probs (T, E)."""
    probs = softmax_dim1(logits)
    T, _ = logits.shape
    indices = np.zeros((T, k), dtype=np.int64)
    gates = np.zeros((T, k), dtype=np.float32)
    # vectorised equivalent of the per-token loop at topk.jl:33-41
    order = np.argsort(-probs, axis=-1, kind="stable")[:, :k]
    sel = np.take_along_axis(probs, order, axis=-1)
    indices[:] = order + 1
    s = sel.sum(axis=-1, keepdims=True, dtype=probs.dtype)
    gates[:] = (sel / s).astype(np.float32)
    return indices, gates, probs


def compute_gates_shared(gate: SharedExpertGating, logits: np.ndarray):
    """compute_gates(::SharedExpertGating, logits) (src/gating/advanced.jl:80-108)."""
    T, E = logits.shape
    S = gate.num_shared
    routed_logits = logits[:, S:gate.num_experts]
    r_idx, r_gates, r_probs = compute_gates(gate.base_gate, routed_logits)
    r_idx = r_idx + S
    total_k = S + r_idx.shape[1]
    indices = np.zeros((T, total_k), dtype=np.int64)
    gates = np.zeros((T, total_k), dtype=np.float32)
    indices[:, :S] = np.arange(1, S + 1)
    gates[:, :S] = np.float32(1.0) / np.float32(total_k)
    indices[:, S:] = r_idx
    # 1.0f0 - num_shared/total_k: Int/Int is Float64 in Julia, Float32 - Float64 -> Float64,
    # the product is Float64 and is rounded on assignment into the Float32 gates array.
    gates[:, S:] = (r_gates.astype(np.float64) * (1.0 - S / total_k)).astype(np.float32)
    probs = np.zeros((T, E), dtype=np.float32)
    probs[:, :S] = np.float32(1.0) / np.float32(E)
    probs[:, S:gate.num_experts] = (r_probs.astype(np.float64) * (1.0 - S / E)).astype(np.float32)
    return indices, gates, probs


def compute_gates(gate, logits: np.ndarray, training: bool = False, jitter_u: Optional[np.ndarray] = None):
    """Dispatch of compute_gates (src/gating/base.jl:22).  `training` / `jitter_u` (the rand(Float32)
    draws) only reach JitterGating (src/gating/switch.jl:25-33), whose jitter is evaluated in Float32."""
    if isinstance(gate, JitterGating):
        if training:
            f = np.float32
            jit = f(1.0) + (f(2.0) * jitter_u.astype(f) - f(1.0)) * f(gate.eps)
            logits = logits * jit.astype(logits.dtype)
        return compute_gates(gate.base_gate, logits)
    if isinstance(gate, TopKGating):
        return compute_gates_topk(gate.k, logits)
    if isinstance(gate, SwitchGating):
        return compute_gates_topk(1, logits)           # src/gating/switch.jl:9-11
    if isinstance(gate, SharedExpertGating):
        return compute_gates_shared(gate, logits)
    raise TypeError(f"unsupported gate {gate!r}")


# --------------------------------------------------------------------------------------
# losses
# --------------------------------------------------------------------------------------


@dataclass
class AuxFreeState:
    """The mutable fields of AuxiliaryFreeLoss (src/balancing/auxiliary_free.jl:11-34)."""
    bias: np.ndarray
    bias_momentum: np.ndarray
    learning_rate: float = 0.01
    momentum: float = 0.9
    update_freq: int = 1
    update_counter: int = 0


def aux_free_update_bias(st: AuxFreeState, indices: np.ndarray) -> None:
    """update_bias! (src/balancing/auxiliary_free.jl:36-71), loop for loop, with Julia's promotion:
    target_count (Int/Int) and gradient are Float64; momentum*bias_momentum is Float32, the blend is
    Float64 and is rounded on assignment into the Float32 vector; bias -= lr*momentum and
    bias .-= mean(bias) are Float32."""
    f = np.float32
    st.update_counter += 1
    if st.update_counter % st.update_freq != 0:
        return
    n = st.bias.size
    counts = np.zeros(n, dtype=np.float32)
    total = 0
    for idx in indices.reshape(-1):
        if idx > 0:
            counts[idx - 1] += f(1)
            total += 1
    if total == 0:
        return
    target = total / n
    for i in range(n):
        grad = (float(counts[i]) - target) / total
        st.bias_momentum[i] = f(float(f(st.momentum) * st.bias_momentum[i]) + float(f(1) - f(st.momentum)) * grad)
        st.bias[i] = f(st.bias[i] - f(f(st.learning_rate) * st.bias_momentum[i]))
    mean = f(0)
    for v in st.bias:
        mean = f(mean + v)
    st.bias[:] = st.bias - f(mean / f(n))


def switch_transformer_loss(alpha: float, indices: np.ndarray, probs: np.ndarray) -> np.float32:
    """compute_loss(::SwitchTransformerLoss, indices, probs) (src/balancing/losses.jl:15-36)."""
    N = probs.shape[1]
    total = indices.size
    f = np.zeros(N, dtype=np.float32)
    flat = indices.reshape(-1)
    valid = flat[(flat > 0) & (flat <= N)]
    np.add.at(f, valid - 1, np.float32(1.0))
    if total > 0:
        f = f / np.float32(total)
    P = probs.mean(axis=0, dtype=np.float32)
    return np.float32(np.float32(alpha) * np.float32(N) * np.sum(f * P, dtype=np.float32))


def logsumexp_dim1(logits: np.ndarray) -> np.ndarray:
    """logsumexp(x; dims=1) (src/balancing/losses.jl:110-113)."""
    m = logits.max(axis=-1, keepdims=True)
    return m + np.log(np.exp(logits - m).sum(axis=-1, keepdims=True, dtype=logits.dtype))


def z_loss(beta: float, logits: np.ndarray) -> np.float32:
    """compute_loss(::ZLoss, logits) (src/balancing/losses.jl:103-108)."""
    lse = logsumexp_dim1(logits)
    return np.float32(np.float32(beta) * np.mean(lse * lse, dtype=np.float32))


def routing_entropy(probs: np.ndarray) -> np.float32:
    """update_stats!'s entropy (src/core/moe_layer.jl:262-263): the 1e-8 literal is Float64,
    so the logarithm and the sum run in Float64; the mean is pushed into a Float32 vector."""
    p = probs.astype(np.float64)
    ent = -(p * np.log(p + 1e-8)).sum(axis=-1)
    return np.float32(ent.mean())


def load_balance_score(counts) -> float:
    """load_balance_score (src/core/utils.jl:40-52)."""
    counts = np.asarray(counts, dtype=np.float64)
    n, total = counts.size, counts.sum()
    if total == 0:
        return 1.0
    ideal = total / n
    return float(1.0 - math.sqrt(((counts - ideal) ** 2).sum() / n) / ideal)


# --------------------------------------------------------------------------------------
# experts and the layer
# --------------------------------------------------------------------------------------


@dataclass
class GatedExpertWeights:
    """GatedExpert (src/experts/gated.jl:6-27): w1, w3 (H, D); w2 (O, H); no bias."""
    w1: np.ndarray
    w2: np.ndarray
    w3: np.ndarray


def gated_expert_forward(e: GatedExpertWeights, x: np.ndarray, act: Callable) -> np.ndarray:
    """(expert::GatedExpert)(x) (src/experts/gated.jl:29-34): w2(act.(w1 x) .* (w3 x)).
    x (n, D) -> (n, O)."""
    gate = act(x @ e.w1.T)
    up = x @ e.w3.T
    return (gate * up) @ e.w2.T


@dataclass
class StandardExpertWeights:
    """StandardExpert (src/experts/standard.jl:8-36): w1 (H, D), w2 (O, H), b1 (H,) / b2 (O,) or None."""
    w1: np.ndarray
    w2: np.ndarray
    b1: Optional[np.ndarray] = None
    b2: Optional[np.ndarray] = None


def standard_expert_forward(e: StandardExpertWeights, x: np.ndarray, act: Callable) -> np.ndarray:
    """(expert::StandardExpert)(x; training=false) (src/experts/standard.jl:38-55):
    w2(act.(w1 x .+ b1)) .+ b2; the Dropout branch only runs when training.  x (n, D) -> (n, O)."""
    h = x @ e.w1.T
    if e.b1 is not None:
        h = h + e.b1.astype(h.dtype)
    y = act(h) @ e.w2.T
    if e.b2 is not None:
        y = y + e.b2.astype(y.dtype)
    return y


def expert_forward(e, x: np.ndarray, act: Callable) -> np.ndarray:
    """Dispatch on the expert's type, like Julia's call overloads."""
    if isinstance(e, StandardExpertWeights):
        return standard_expert_forward(e, x, act)
    return gated_expert_forward(e, x, act)


@dataclass
class MoEConfig:
    """The MoEConfig fields the forward reads (src/core/moe_layer.jl:4-29)."""
    num_experts: int = 8
    input_dim: int = 768
    hidden_dim: int = 3072
    output_dim: int = 768
    activation: str = "gelu"
    gate_type: object = field(default_factory=lambda: TopKGating(2))
    balance_alpha: float = 0.01
    z_loss_weight: float = 0.001
    capacity_factor: float = 1.25
    drop_tokens: bool = False
    num_shared_experts: int = 0
    use_fp32_router: bool = True
    # AuxiliaryFreeLoss hook (src/core/moe_layer.jl:137-140): bias added to logits before a
    # second compute_gates; the probabilities used by the loss stay unbiased.
    aux_free_bias: Optional[np.ndarray] = None
    # the whole AuxiliaryFreeLoss: its bias selects like aux_free_bias and a training call updates it
    aux_free_state: Optional[AuxFreeState] = None
    # A bias that is part of the logits themselves (a router Dense with bias).
    router_bias: Optional[np.ndarray] = None
    # Router.noise_scale (src/core/router.jl:32-41): logits += noise_scale * randn when training; the
    # standard-normal draws are passed in (router_noise, shape (T, E_router)) so that a test can give
    # the device path the same draws.
    noise_scale: float = 0.0
    router_noise: Optional[np.ndarray] = None


@dataclass
class MoEWeights:
    router: np.ndarray                     # (E_router, D) float32  (Router.weight, router.jl:18)
    experts: List[GatedExpertWeights]
    noise_weight: Optional[np.ndarray] = None   # (E_router, D) float32  (Router.noise_weight, router.jl:20)


def softplus(x: np.ndarray) -> np.ndarray:
    """NNlib.softplus: log1p(exp(-|x|)) + relu(x)."""
    return np.log1p(np.exp(-np.abs(x))) + np.maximum(x, 0)


def router_forward(cfg: MoEConfig, w: MoEWeights, x: np.ndarray, dtype=np.float32, training: bool = False):
    """(router::Router)(x; training) (src/core/router.jl:25-46); cfg.router_noise holds the randn draws."""
    xr = x.astype(dtype) if cfg.use_fp32_router or x.dtype != dtype else x
    logits = xr @ w.router.astype(dtype).T
    if cfg.router_bias is not None:
        logits = logits + cfg.router_bias.astype(dtype)
    if training and cfg.noise_scale > 0:
        if w.noise_weight is not None:                                                  # router.jl:33-37
            noise = cfg.router_noise.astype(dtype) * softplus(xr @ w.noise_weight.astype(dtype).T)
            logits = logits + dtype(cfg.noise_scale) * noise
        else:
            logits = logits + (cfg.router_noise.astype(dtype) * dtype(cfg.noise_scale))     # router.jl:38-40
    indices, gates, probs = compute_gates(cfg.gate_type, logits)
    return indices, gates, probs, logits


def process_expert_forward(output: np.ndarray, experts: List[GatedExpertWeights], x: np.ndarray,
                           indices: np.ndarray, gates: np.ndarray, act: Callable):
    """process_expert_forward! (src/core/moe_layer.jl:187-219): bucket (token, slot) pairs per
    expert in ascending token order, run each non-empty expert on its gathered tokens, add
    gate * expert_output into the token's output (experts visited in ascending id)."""
    T, k = indices.shape
    E = len(experts)
    tok = np.repeat(np.arange(T), k)
    flat_e = indices.reshape(-1)
    flat_g = gates.reshape(-1)
    for eid in range(1, E + 1):
        sel = flat_e == eid
        if not sel.any():
            continue
        tokens = tok[sel]
        weights = flat_g[sel].astype(output.dtype)
        y = expert_forward(experts[eid - 1], x[tokens], act)
        # a token can list the same expert at most once per slot; np.add.at keeps duplicates right
        np.add.at(output, tokens, weights[:, None] * y.astype(output.dtype))


def apply_capacity_constraint(indices: np.ndarray, gates: np.ndarray, capacity_factor: float,
                              num_experts: int):
    """apply_capacity_constraint (src/core/moe_layer.jl:221-248): sequential first-come
    capacity ceil(cf*T/E); overflow slots get id 0 and gate 0, gates renormalised per token."""
    indices = indices.copy()
    gates = gates.copy()
    T, k = indices.shape
    # Float32 * Int / Int evaluates in Float32 in Julia
    capacity = math.ceil(float(np.float32(capacity_factor) * np.float32(T) / np.float32(num_experts)))
    counts = np.zeros(num_experts + 1, dtype=np.int64)
    for j in range(T):
        for s in range(k):
            e = indices[j, s]
            if e > 0:
                if counts[e] >= capacity:
                    indices[j, s] = 0
                    gates[j, s] = 0.0
                else:
                    counts[e] += 1
        gs = gates[j].sum(dtype=np.float32)
        if gs > 0:
            gates[j] = gates[j] / gs
    return indices, gates


def forward_standard(cfg: MoEConfig, w: MoEWeights, x: np.ndarray, training: bool, dtype=np.float32):
    """forward_standard (src/core/moe_layer.jl:130-156)."""
    T = x.shape[0]
    act = ACTIVATIONS[cfg.activation]
    output = np.zeros((T, cfg.output_dim), dtype=dtype)
    indices, gates, probs, logits = router_forward(cfg, w, x, dtype, training)
    aux_bias = cfg.aux_free_state.bias if cfg.aux_free_state is not None else cfg.aux_free_bias
    if aux_bias is not None:
        biased = logits + aux_bias.astype(logits.dtype)               # auxiliary_free.jl:90-92
        indices, gates, _ = compute_gates(cfg.gate_type, biased)
    if cfg.drop_tokens and training:
        indices, gates = apply_capacity_constraint(indices, gates, cfg.capacity_factor, cfg.num_experts)
    process_expert_forward(output, w.experts, x.astype(dtype), indices, gates, act)
    if training and cfg.aux_free_state is not None:
        aux_free_update_bias(cfg.aux_free_state, indices)            # compute_loss, auxiliary_free.jl:73-75
    loss = switch_transformer_loss(cfg.balance_alpha, indices, probs) if training else np.float32(0)
    stats = {
        "tokens_per_expert": np.bincount(indices.reshape(-1), minlength=cfg.num_experts + 1)[1:cfg.num_experts + 1],
        "routing_entropy": routing_entropy(probs),
    }
    return output, loss, dict(indices=indices, gates=gates, probs=probs, logits=logits, stats=stats)


def forward_with_shared_experts(cfg: MoEConfig, w: MoEWeights, x: np.ndarray, training: bool, dtype=np.float32):
    """forward_with_shared_experts (src/core/moe_layer.jl:158-185), quirks included: the loss
    sees indices shifted by +S against probs that only have E-S rows (losses.jl:16,23)."""
    T = x.shape[0]
    S = cfg.num_shared_experts
    act = ACTIVATIONS[cfg.activation]
    xd = x.astype(dtype)
    shared = np.zeros((T, cfg.output_dim), dtype=dtype)
    for i in range(S):
        shared += expert_forward(w.experts[i], xd, act) / dtype(S)
    indices, gates, probs, logits = router_forward(cfg, w, x, dtype)
    routed = np.zeros((T, cfg.output_dim), dtype=dtype)
    process_expert_forward(routed, w.experts[S:], xd, indices, gates, act)
    out = dtype(0.5) * shared + dtype(0.5) * routed
    shifted = indices + S
    loss = switch_transformer_loss(cfg.balance_alpha, shifted, probs) if training else np.float32(0)
    return out, loss, dict(indices=shifted, gates=gates, probs=probs, logits=logits, stats=None)


def moe_layer_forward(cfg: MoEConfig, w: MoEWeights, x: np.ndarray, training: bool = False, dtype=np.float32):
    """(moe::MoELayer)(x; training) (src/core/moe_layer.jl:107-128): returns
    (output (T, O), balance_loss, aux).  The z-loss is added when training and
    z_loss_weight > 0 (:117-121; the reference re-runs the router for the logits)."""
    if cfg.num_shared_experts > 0:
        out, loss, aux = forward_with_shared_experts(cfg, w, x, training, dtype)
    else:
        out, loss, aux = forward_standard(cfg, w, x, training, dtype)
    if training and cfg.z_loss_weight > 0:
        # the reference runs the router again with training=false: no noise in these logits
        clean = aux["logits"] if cfg.noise_scale <= 0 else router_forward(cfg, w, x, dtype, False)[3]
        loss = np.float32(loss + z_loss(cfg.z_loss_weight, clean))
    return out, np.float32(loss), aux


# --------------------------------------------------------------------------------------
# Llama2 glue (per-token restatement of the layer; src/llama2/inference.jl)
# --------------------------------------------------------------------------------------


def llama_silu(v):
    """silu as written in the Llama2 glue: v * (1/(1+exp(-v))) (src/llama2/inference.jl:159-162)."""
    return v * (v.dtype.type(1) / (v.dtype.type(1) + np.exp(-v)))


def gated_expert_forward_llama(e: GatedExpertWeights, xb: np.ndarray) -> np.ndarray:
    """gated_expert_forward! (src/llama2/inference.jl:154-167); weights held as (out, in)."""
    hb1 = e.w1 @ xb
    hb2 = e.w3 @ xb
    return e.w2 @ (llama_silu(hb1) * hb2)


def moe_ffn_forward_token(router_w: np.ndarray, experts: List[GatedExpertWeights], gate, top_k: int,
                          xb: np.ndarray):
    """moe_ffn_forward! after its rmsnorm (src/llama2/inference.jl:63-105): router matvec,
    compute_gates on a 1-column matrix, then the selected experts accumulated in slot order.
    router_w is (E, D) (= the reference's (D x E) array read as W^T x)."""
    logits = (router_w @ xb).reshape(1, -1)
    indices, gates, probs = compute_gates(gate, logits)
    n_sel = min(top_k, indices.shape[1])
    xb2 = np.zeros(experts[0].w2.shape[0], dtype=xb.dtype)
    for s in range(n_sel):
        eid = int(indices[0, s])
        if 0 < eid <= len(experts):
            xb2 = xb2 + gates[0, s] * gated_expert_forward_llama(experts[eid - 1], xb)
    return xb2, indices[0, :n_sel], gates[0, :n_sel], probs[0]


# --------------------------------------------------------------------------------------
# seeded synthetic inputs (stand-ins for the reference's checkpoint/prompts)
# --------------------------------------------------------------------------------------


def bf16_round(a: np.ndarray) -> np.ndarray:
    """Round float32 to the nearest-even bfloat16 and return it as float32."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return r.astype(np.uint32).view(np.float32).reshape(a.shape)


def glorot_uniform(rng, out_dim, in_dim):
    lim = math.sqrt(6.0 / (in_dim + out_dim))
    return rng.uniform(-lim, lim, size=(out_dim, in_dim)).astype(np.float32)


def make_layer_inputs(seed: int, T: int, D: int, H: int, O: int, E: int, *, e_router: Optional[int] = None,
                      init: str = "glorot", std: float = 0.02, bf16: bool = False, expert_kind: str = "gated"):
    """Seeded generator (NumPy PCG64): draws x, the router, then per expert w1, w3, w2
    (expert_kind='standard': w1, w2, then b1, b2 ~ N(0, 0.1^2), kept float32).
    init='glorot' -> Glorot-uniform; init='normal' -> N(0, std^2).  bf16=True rounds x and the
    expert weights to bfloat16-representable float32 values (the router stays float32)."""
    rng = np.random.Generator(np.random.PCG64(seed))
    x = rng.standard_normal((T, D), dtype=np.float32)
    er = E if e_router is None else e_router
    if init == "glorot":
        router = glorot_uniform(rng, er, D)
        mk = lambda o, i: glorot_uniform(rng, o, i)
    else:
        router = (rng.standard_normal((er, D), dtype=np.float32) * np.float32(std))
        mk = lambda o, i: (rng.standard_normal((o, i), dtype=np.float32) * np.float32(std))
    experts = []
    for _ in range(E):
        w1 = mk(H, D)
        if expert_kind == "standard":
            w2 = mk(O, H)
            b1 = rng.standard_normal(H, dtype=np.float32) * np.float32(0.1)
            b2 = rng.standard_normal(O, dtype=np.float32) * np.float32(0.1)
            experts.append(StandardExpertWeights(w1=w1, w2=w2, b1=b1, b2=b2))
            continue
        w3 = mk(H, D)
        w2 = mk(O, H)
        experts.append(GatedExpertWeights(w1=w1, w2=w2, w3=w3))
    if bf16:
        x = bf16_round(x)
        for e in experts:
            e.w1, e.w2 = bf16_round(e.w1), bf16_round(e.w2)
            if isinstance(e, GatedExpertWeights):
                e.w3 = bf16_round(e.w3)
    return x, MoEWeights(router=router, experts=experts)
