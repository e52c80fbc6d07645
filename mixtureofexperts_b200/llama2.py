"""Llama2 integration with the reference's entry points (src/llama2/): convert_to_moe,
sample_moe, moe_transformer -- the callers directly above the MoE-layer hot path.

The reference builds on Llama2.jl (not vendored, not pinned).  Its model container is mirrored
here by small dataclasses (ModelConfig, TransformerLayerWeights, TransformerWeights,
LanguageModel) holding float32 NumPy arrays.  A weight of the reference with Julia shape
(in x out) (column-major, used as W^T x by Llama2.matmul!) is held as an (out, in) C-order array:
the same bytes.

Only the MoE feed-forward step runs on the GPU (MoELayer -> libmoe_b200).  Attention, RoPE,
RMSNorm, the KV cache and sampling stay on the host like in the reference, which runs them on the
CPU one token at a time.  Unlike the reference, a prompt is pushed through each layer as ONE batch
of T = len(prompt) tokens (mathematically the same layer by layer), so the expert weights are read
once per layer instead of once per token; generation then proceeds token by token.
"""
from __future__ import annotations

import json
import math
import struct
import time
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np

from . import _lib
from .experts import silu
from .gating import GatingMechanism, TopKGating
from .layer import MoEConfig, MoELayer, Router
from .losses import LoadBalancingLoss, SwitchTransformerLoss

RMS_EPS = np.float32(1e-5)      # llama2.c / Llama2.jl rmsnorm epsilon


@dataclass
class ModelConfig:
    """Llama2.ModelConfig: the fields the MoE glue reads."""
    dim: int = 512
    hidden_dim: int = 1376
    n_layers: int = 8
    n_heads: int = 8
    n_kv_heads: int = 8
    vocab_size: int = 32000
    seq_len: int = 1024
    rope_freq_base: float = 10000.0
    rope_is_neox: bool = False


@dataclass
class TransformerLayerWeights:
    """Llama2.TransformerLayerWeights; matrices are (out, in)."""
    rms_att_weight: np.ndarray
    rms_ffn_weight: np.ndarray
    wq: np.ndarray
    wk: np.ndarray
    wv: np.ndarray
    wo: np.ndarray
    w1: np.ndarray      # (hidden, dim)   reference: (dim x hidden)
    w2: np.ndarray      # (dim, hidden)   reference: (hidden x dim)
    w3: np.ndarray      # (hidden, dim)


@dataclass
class TransformerWeights:
    token_embedding_table: np.ndarray   # (vocab, dim)  reference: (dim x vocab)
    layers: List[TransformerLayerWeights]
    rms_final_weight: np.ndarray
    output_weight: np.ndarray           # (vocab, dim)


class CharTokenizer:
    """Stand-in for Llama2.jl's tokenizer (cf. create_dummy_tokenizer,
    test_moeLlama2_integration.jl:552-569): ids 1 and 2 are BOS/EOS, then one id per byte."""

    def __init__(self, vocab_size: int):
        self.bos_token_id, self.eos_token_id = 1, 2
        self.id_to_token = ["<unk>", "<s>", "</s>"] + [chr(i) if 32 <= i < 127 else f"<{i}>" for i in range(256)]
        self.id_to_token += [f"<tok{i}>" for i in range(len(self.id_to_token), vocab_size)]
        self.id_to_token = self.id_to_token[:vocab_size]

    def encode(self, text: str) -> List[int]:
        return [3 + b for b in text.encode("utf-8") if 3 + b < len(self.id_to_token)]


@dataclass
class LanguageModel:
    """Llama2.LanguageModel."""
    config: ModelConfig
    tokenizer: CharTokenizer
    weights: TransformerWeights


def random_language_model(config: ModelConfig, seed: int = 0, std: float = 0.02) -> LanguageModel:
    """A random-init dense model of the given shape: every matrix N(0, std^2) (the scale of the
    reference's own fixtures, test_moeLlama2_integration.jl:734-758), norm weights 1."""
    rng = np.random.Generator(np.random.PCG64(seed))
    c = config
    head = c.dim // c.n_heads
    mk = lambda o, i: rng.standard_normal((o, i), dtype=np.float32) * np.float32(std)
    layers = []
    for _ in range(c.n_layers):
        layers.append(TransformerLayerWeights(
            rms_att_weight=np.ones(c.dim, np.float32), rms_ffn_weight=np.ones(c.dim, np.float32),
            wq=mk(c.dim, c.dim), wk=mk(c.n_kv_heads * head, c.dim), wv=mk(c.n_kv_heads * head, c.dim),
            wo=mk(c.dim, c.dim), w1=mk(c.hidden_dim, c.dim), w2=mk(c.dim, c.hidden_dim), w3=mk(c.hidden_dim, c.dim)))
    w = TransformerWeights(token_embedding_table=mk(c.vocab_size, c.dim), layers=layers,
                           rms_final_weight=np.ones(c.dim, np.float32), output_weight=mk(c.vocab_size, c.dim))
    return LanguageModel(config=c, tokenizer=CharTokenizer(c.vocab_size), weights=w)


# ---- MoE model types (src/llama2/types.jl) ---------------------------------------------------

@dataclass
class MoEExpertWeights:
    """MoEExpertWeights (src/llama2/types.jl:99-108): w1, w3 (hidden, dim); w2 (dim, hidden)."""
    w1: np.ndarray
    w2: np.ndarray
    w3: np.ndarray
    expert_type: str = "gated"


@dataclass
class MoETransformerLayerWeights:
    """MoETransformerLayerWeights: the dense layer plus, when use_moe, experts and router."""
    llama_layer: TransformerLayerWeights
    use_moe: bool = False
    moe_experts: Optional[List[MoEExpertWeights]] = None
    moe_router_weight: Optional[np.ndarray] = None     # (E, dim)   reference: (dim x E)
    moe_config: Optional[MoEConfig] = None
    _device_layer: Optional[MoELayer] = field(default=None, repr=False)
    # a loaded model holds the layer as a weight image (MoELayer.export_weights) until first use
    _weight_image: Optional[np.ndarray] = field(default=None, repr=False)


@dataclass
class MoELlamaConfig:
    """MoELlamaConfig (src/llama2/types.jl:14-48): the Llama2 config plus the MoE settings."""
    llama_config: ModelConfig
    moe_layers: List[int]
    moe_num_experts: int
    moe_top_k: int
    moe_expert_type: str
    moe_gate_type: GatingMechanism
    moe_balance_loss: LoadBalancingLoss
    expert_init_strategy: str
    expert_init_noise: float
    z_loss_weight: float = 0.001

    def __getattr__(self, name):        # getproperty delegation to the Llama2 config
        return getattr(object.__getattribute__(self, "llama_config"), name)


@dataclass
class MoELanguageModel:
    """MoELanguageModel (src/llama2/types.jl:159-169)."""
    config: MoELlamaConfig
    tokenizer: CharTokenizer
    token_embedding_table: np.ndarray
    rms_final_weight: np.ndarray
    output_weight: np.ndarray
    layers: List[MoETransformerLayerWeights]
    device: int = 0
    compute_dtype: str = "f32"
    routing_log: List[dict] = field(default_factory=list)


# ---- conversion (src/llama2/conversion.jl) ---------------------------------------------------

def _validate(model, moe_layers, num_experts, top_k, strategy):
    """validate_conversion_inputs (src/llama2/conversion.jl:393-420); ArgumentError -> ValueError."""
    n = model.config.n_layers
    for l in moe_layers:
        if l < 1 or l > n:
            raise ValueError(f"MoE layer index {l} out of range 1..{n}")
    if num_experts < 1:
        raise ValueError("num_experts must be positive")
    if top_k < 1 or top_k > num_experts:
        raise ValueError(f"top_k must be in 1..{num_experts}")
    if strategy not in ("copy", "perturb", "split", "random"):
        raise ValueError(f"Unknown expert initialization strategy: {strategy}")


def _create_single_expert(layer: TransformerLayerWeights, cfg: ModelConfig, strategy: str, idx: int,
                          num_experts: int, noise: float, rng) -> MoEExpertWeights:
    """create_single_expert (src/llama2/conversion.jl:277-331)."""
    dim, hid = cfg.dim, cfg.hidden_dim
    if strategy == "copy":
        w1, w2, w3 = layer.w1.copy(), layer.w2.copy(), layer.w3.copy()
    elif strategy == "perturb":
        ns = np.float32(noise)
        w1 = layer.w1 + rng.standard_normal(layer.w1.shape, dtype=np.float32) * ns
        w2 = layer.w2 + rng.standard_normal(layer.w2.shape, dtype=np.float32) * ns
        w3 = layer.w3 + rng.standard_normal(layer.w3.shape, dtype=np.float32) * ns
    elif strategy == "split":
        start = (idx * hid) // num_experts                      # 0-based form of :296-297
        end = min(((idx + 1) * hid) // num_experts, hid)
        w1, w2, w3 = np.zeros_like(layer.w1), np.zeros_like(layer.w2), np.zeros_like(layer.w3)
        w1[start:end, :] = layer.w1[start:end, :]
        w2[:, start:end] = layer.w2[:, start:end]
        w3[start:end, :] = layer.w3[start:end, :]
    else:
        s = np.float32(math.sqrt(2.0 / dim))
        w1 = rng.standard_normal((hid, dim), dtype=np.float32) * s
        w2 = rng.standard_normal((dim, hid), dtype=np.float32) * s
        w3 = rng.standard_normal((hid, dim), dtype=np.float32) * s
    return MoEExpertWeights(w1=w1.astype(np.float32), w2=w2.astype(np.float32), w3=w3.astype(np.float32))


def convert_to_moe(model: LanguageModel, moe_layers: Sequence[int], *, num_experts: int = 8, top_k: int = 2,
                   expert_init_strategy: str = "perturb", expert_init_noise: float = 0.01,
                   gate_type: Optional[GatingMechanism] = None, balance_loss: Optional[LoadBalancingLoss] = None,
                   expert_type: str = "gated", z_loss_weight: float = 0.001, seed=None, device: int = 0,
                   compute_dtype: str = "f32", verbose: bool = False, **unsupported) -> MoELanguageModel:
    """convert_to_moe(model, moe_layers; kwargs...) (src/llama2/conversion.jl:43-107): layers listed
    in ``moe_layers`` (1-based, like the reference) get ``num_experts`` gated experts built from the
    dense FFN by ``expert_init_strategy`` and a (num_experts x dim) router drawn randn*sqrt(2/dim)
    (:358-367); all other weights are copied.  ``seed`` (not in the reference, which never seeds)
    makes the draw reproducible.  Device handles are created on first use."""
    for k_, v in unsupported.items():
        if k_ in ("use_shared_experts", "use_cur", "drop_tokens") and v:
            raise _lib.MoEError(_lib.ERR_UNSUPPORTED, f"{k_} is not accelerated")
    strategy = str(expert_init_strategy).lstrip(":")
    moe_layers = [int(l) for l in moe_layers]
    _validate(model, moe_layers, num_experts, top_k, strategy)
    if expert_type not in ("gated", ":gated"):
        raise _lib.MoEError(_lib.ERR_UNSUPPORTED, "only expert_type='gated' is accelerated")
    rng = np.random.Generator(np.random.PCG64(seed)) if not isinstance(seed, np.random.Generator) else seed
    gate = gate_type if gate_type is not None else TopKGating(top_k)
    loss = balance_loss if balance_loss is not None else SwitchTransformerLoss(0.01)
    c = model.config
    if verbose:
        print(f"Converting Llama2 model to MoE...\n  Original layers: {c.n_layers}\n  MoE layers: {moe_layers}\n"
              f"  Experts per MoE layer: {num_experts}\n  Initialization strategy: {strategy}")
    layers = []
    for li, lw in enumerate(model.weights.layers, start=1):
        copy = TransformerLayerWeights(**{k_: np.array(v, copy=True) for k_, v in lw.__dict__.items()})
        if li not in moe_layers:
            layers.append(MoETransformerLayerWeights(llama_layer=copy, use_moe=False))
            continue
        experts = [_create_single_expert(lw, c, strategy, e, num_experts, expert_init_noise, rng)
                   for e in range(num_experts)]
        router = rng.standard_normal((num_experts, c.dim), dtype=np.float32) * np.float32(math.sqrt(2.0 / c.dim))
        layer_cfg = MoEConfig(num_experts=num_experts, expert_type="gated", input_dim=c.dim, hidden_dim=c.hidden_dim,
                              output_dim=c.dim, activation=silu, gate_type=gate, top_k=top_k, balance_loss=loss,
                              z_loss_weight=z_loss_weight)
        layers.append(MoETransformerLayerWeights(llama_layer=copy, use_moe=True, moe_experts=experts,
                                                 moe_router_weight=router, moe_config=layer_cfg))
    mcfg = MoELlamaConfig(llama_config=c, moe_layers=moe_layers, moe_num_experts=num_experts, moe_top_k=top_k,
                          moe_expert_type="gated", moe_gate_type=gate, moe_balance_loss=loss,
                          expert_init_strategy=strategy, expert_init_noise=expert_init_noise, z_loss_weight=z_loss_weight)
    return MoELanguageModel(config=mcfg, tokenizer=model.tokenizer,
                            token_embedding_table=model.weights.token_embedding_table.copy(),
                            rms_final_weight=model.weights.rms_final_weight.copy(),
                            output_weight=model.weights.output_weight.copy(), layers=layers, device=device,
                            compute_dtype=compute_dtype)


def count_parameters(model: MoELanguageModel) -> int:
    """count_parameters (src/llama2/conversion.jl:512-550): every weight, all experts included.  Like
    the reference, a MoE layer contributes its attention weights, router and experts but not its
    rms_ffn_weight (the reference's own run of stories42M with layers [2,4] x 4 experts prints
    70757888, which only comes out this way)."""
    n = model.token_embedding_table.size + model.rms_final_weight.size + model.output_weight.size
    c = model.config
    per = 3 * c.dim * c.hidden_dim
    for l in model.layers:
        ll = l.llama_layer
        n += sum(a.size for a in (ll.rms_att_weight, ll.wq, ll.wk, ll.wv, ll.wo))
        if l.use_moe:
            n += c.moe_num_experts * c.dim + c.moe_num_experts * per
        else:
            n += ll.rms_ffn_weight.size + ll.w1.size + ll.w2.size + ll.w3.size
    return int(n)


def count_active_parameters(model: MoELanguageModel) -> int:
    """count_active_parameters (src/llama2/conversion.jl:557-600): top_k of the experts of a MoE layer."""
    n = model.token_embedding_table.size + model.rms_final_weight.size + model.output_weight.size
    c = model.config
    per = 3 * c.dim * c.hidden_dim
    for l in model.layers:
        ll = l.llama_layer
        n += sum(a.size for a in (ll.rms_att_weight, ll.wq, ll.wk, ll.wv, ll.wo))
        if l.use_moe:
            n += c.moe_num_experts * c.dim + c.moe_top_k * per
        else:
            n += ll.rms_ffn_weight.size + ll.w1.size + ll.w2.size + ll.w3.size
    return int(n)


def usage_balance_score(usage_counts, num_experts: int) -> float:
    """The score print_expert_stats prints per MoE layer (src/llama2/generation.jl:318-324):
    1 - max|count - total/num_experts| / (total/num_experts)."""
    counts = np.asarray(usage_counts, dtype=np.float64)
    expected = counts.sum() / num_experts
    return float(1.0 - np.abs(counts - expected).max() / expected)


def expert_stats_lines(state: "MoERunState", model: MoELanguageModel, threshold: float = 0.0) -> List[str]:
    """The text of print_expert_stats (src/llama2/generation.jl:298-330) for the calls made with
    ``state`` so far, one list entry per line."""
    lines = ["", "--- Expert Usage Statistics ---"]
    for layer_idx in sorted(state.expert_usage):
        counts = state.expert_usage[layer_idx]
        total = int(counts.sum())
        lines += [f"Layer {layer_idx}:", f"  Total expert activations: {total}"]
        for e, cnt in enumerate(counts, start=1):
            if cnt > 0 and cnt / total * 100 >= threshold * 100:
                lines.append(f"    Expert {e:2d}: {int(cnt):4d} activations ({cnt / total * 100:.1f}%)")
        if total > 0:
            lines.append(f"  Load balance score: {usage_balance_score(counts, model.config.moe_num_experts):.3f} (1.0 = perfect)")
        lines.append("")
    return lines


# ---- inference (src/llama2/inference.jl, attention.jl) ---------------------------------------

def _device_layer(model: MoELanguageModel, l: MoETransformerLayerWeights) -> MoELayer:
    """The layer's libmoe_b200 handle, built on first use from the Llama2-layout weights (which
    are (out, in) C-order arrays, i.e. MOE_LAYOUT_IN_CONTIG: no transpose on the way in)."""
    if l._device_layer is None and l._weight_image is not None:
        l._device_layer = MoELayer(l.moe_config, device=model.device, compute_dtype=model.compute_dtype,
                                   weight_image=l._weight_image)
        l._weight_image = None
    if l._device_layer is None:
        cfg = l.moe_config
        experts = []
        for e in l.moe_experts:
            ex = type("ExpertView", (), {})()
            ex.w1, ex.w2, ex.w3 = e.w1, e.w2, e.w3
            experts.append(ex)
        router = Router.__new__(Router)
        router.weight, router.noise_weight, router.gate_type = l.moe_router_weight, None, cfg.gate_type
        router.noise_scale, router.use_fp32 = 0.0, True
        l._device_layer = MoELayer(cfg, device=model.device, compute_dtype=model.compute_dtype, experts=experts,
                                   router=router)
    return l._device_layer


def _rmsnorm_rows(x: np.ndarray, w: np.ndarray) -> np.ndarray:
    ss = (x * x).mean(axis=-1, keepdims=True, dtype=np.float32) + RMS_EPS
    return (w * (x / np.sqrt(ss))).astype(np.float32)


def _rope_rows(v: np.ndarray, pos0: int, n_heads: int, cfg) -> np.ndarray:
    """RoPE of rows at 0-based positions pos0.. (apply_rope_normal!/apply_rope_neox!,
    src/llama2/attention.jl:69-127): theta_i = pos * base^(-i/(head/2)) built by the reference's
    Float32 recurrence."""
    m = v.shape[0]
    head = v.shape[1] // n_heads
    half = head // 2
    scale = np.float32(np.float32(cfg.rope_freq_base) ** np.float32(-1.0 / np.float32(half)))
    th = np.arange(pos0, pos0 + m, dtype=np.float32)
    thetas = np.empty((m, half), dtype=np.float32)
    for i in range(half):
        thetas[:, i] = th
        th = (th * scale).astype(np.float32)
    c, s = np.cos(thetas)[:, None, :], np.sin(thetas)[:, None, :]
    if cfg.rope_is_neox:
        x = v.reshape(m, n_heads, 2, half)
        a, b = x[:, :, 0, :], x[:, :, 1, :]
        out = np.stack([a * c - b * s, a * s + b * c], axis=2)
    else:
        x = v.reshape(m, n_heads, half, 2)
        a, b = x[..., 0], x[..., 1]
        out = np.stack([a * c - b * s, a * s + b * c], axis=-1)
    return out.reshape(m, -1).astype(np.float32)


class MoERunState:
    """MoERunState / KV cache (src/llama2/types.jl): keys and values of every layer, plus the
    routing statistics the reference keeps in the state."""

    def __init__(self, model: MoELanguageModel, max_len: Optional[int] = None):
        c = model.config
        head = c.dim // c.n_heads
        self.max_len = int(max_len or c.seq_len)
        n = len(model.layers)
        self.key_cache = np.zeros((n, self.max_len, c.n_kv_heads, head), dtype=np.float32)
        self.value_cache = np.zeros((n, self.max_len, c.n_kv_heads, head), dtype=np.float32)
        self.pos = 0
        self.logits = None
        self.expert_load_counts = np.zeros(c.moe_num_experts, dtype=np.int64)
        self.selected_experts = {}          # layer index -> (T, k) 1-based ids of the last call
        self.expert_usage = {}              # 1-based layer number -> activations per expert (stats[:expert_usage])
        self.inference_stats = {"total_tokens": 0, "moe_layer_calls": 0, "expert_activations": 0}


def moe_transformer(tokens: Sequence[int], model: MoELanguageModel, state: MoERunState) -> np.ndarray:
    """moe_transformer! (src/llama2/inference.jl:14-50) for ``len(tokens)`` consecutive positions
    starting at ``state.pos``: returns the logits (len(tokens), vocab) and advances the state.
    One call with the whole prompt is the batched prefill; a call with one token is a decode step."""
    c = model.config
    tokens = np.asarray(tokens, dtype=np.int64)
    m, p0 = len(tokens), state.pos
    if p0 + m > state.max_len:
        raise _lib.MoEError(_lib.ERR_INVALID, "sequence longer than the KV cache")
    head = c.dim // c.n_heads
    n_gqa = c.n_heads // c.n_kv_heads
    x = model.token_embedding_table[tokens].astype(np.float32)
    att_scale = np.float32(1.0 / math.sqrt(head))
    causal = np.arange(p0 + m)[None, :] > (p0 + np.arange(m))[:, None]         # (m, p0+m)
    for li, l in enumerate(model.layers):
        ll = l.llama_layer
        xb = _rmsnorm_rows(x, ll.rms_att_weight)
        q = _rope_rows(xb @ ll.wq.T, p0, c.n_heads, c).reshape(m, c.n_heads, head)
        k = _rope_rows(xb @ ll.wk.T, p0, c.n_kv_heads, c).reshape(m, c.n_kv_heads, head)
        v = (xb @ ll.wv.T).reshape(m, c.n_kv_heads, head)
        state.key_cache[li, p0:p0 + m] = k
        state.value_cache[li, p0:p0 + m] = v
        keys = np.repeat(state.key_cache[li, :p0 + m], n_gqa, axis=1)             # (P, n_heads, head)
        vals = np.repeat(state.value_cache[li, :p0 + m], n_gqa, axis=1)
        att = np.einsum("mhd,phd->hmp", q, keys) * att_scale
        att = np.where(causal[None], -np.inf, att)
        att = np.exp(att - att.max(axis=-1, keepdims=True))
        att = att / att.sum(axis=-1, keepdims=True, dtype=np.float32)
        out = np.einsum("hmp,phd->mhd", att, vals).reshape(m, c.dim)
        x = x + out @ ll.wo.T
        xb = _rmsnorm_rows(x, ll.rms_ffn_weight)
        if l.use_moe:
            # moe_ffn_forward! (src/llama2/inference.jl:58-121) for all m positions at once
            layer = _device_layer(model, l)
            y, _, routing = layer(np.asfortranarray(xb.T), training=False, return_routing=True)
            y = np.ascontiguousarray(y.T)
            idx = np.ascontiguousarray(routing["indices"].T)
            state.selected_experts[li] = idx
            np.add.at(state.expert_load_counts, idx.ravel() - 1, 1)
            usage = state.expert_usage.setdefault(li + 1, np.zeros(c.moe_num_experts, dtype=np.int64))
            np.add.at(usage, idx.ravel() - 1, 1)
            state.inference_stats["moe_layer_calls"] += m
            state.inference_stats["expert_activations"] += idx.size
        else:
            # dense_ffn_forward! (src/llama2/inference.jl:131-147)
            h1 = xb @ ll.w1.T
            y = ((h1 * (np.float32(1.0) / (np.float32(1.0) + np.exp(-h1)))) * (xb @ ll.w3.T)) @ ll.w2.T
        x = x + y
    x = _rmsnorm_rows(x, model.rms_final_weight)
    logits = x @ model.output_weight.T
    state.pos += m
    state.logits = logits[-1]
    state.inference_stats["total_tokens"] += m
    return logits


def sample_next_token(logits: np.ndarray, temperature: float, rng) -> int:
    """sample_next_token (src/llama2/generation.jl:179-214): arg-max at temperature 0, else a draw
    from softmax(logits/temperature) by inverse CDF.  Returns a 0-based token id."""
    if temperature == 0.0:
        return int(np.argmax(logits))
    z = logits.astype(np.float32) / np.float32(temperature)
    z = np.exp(z - z.max())
    p = z / z.sum(dtype=np.float32)
    r = np.float32(rng.random())
    i = int(np.searchsorted(np.cumsum(p, dtype=np.float32), r, side="left"))
    return min(i, len(p) - 1)


def sample_moe(model: MoELanguageModel, prompt: str = "", *, temperature: float = 0.9,
               stop_on_special_token: bool = True, max_seq_len: Optional[int] = None, bos_token: bool = True,
               seed=None, verbose: bool = False) -> str:
    """sample_moe(model, prompt; kwargs...) (src/llama2/generation.jl:38-128): feeds the prompt,
    then generates until seq_len, max_seq_len or a BOS/EOS token; returns the generated text.
    Token ids are the tokenizer's (0-based list positions)."""
    if not bos_token and not prompt:
        raise ValueError("Prompt cannot be empty if bos_token = false")
    tok = model.tokenizer
    prompt_tokens = list(tok.encode(prompt))
    if bos_token:
        prompt_tokens.insert(0, tok.bos_token_id)
    limit = min(model.config.seq_len, max_seq_len or model.config.seq_len)
    rng = np.random.default_rng(seed)
    state = MoERunState(model, limit)
    n_prompt = min(len(prompt_tokens), limit)
    moe_transformer(prompt_tokens[:n_prompt], model, state)     # batched prefill
    pieces = []
    while state.pos < limit:
        nxt = sample_next_token(state.logits, float(temperature), rng)
        if stop_on_special_token and nxt in (tok.bos_token_id, tok.eos_token_id):
            break
        pieces.append(tok.id_to_token[nxt])
        if state.pos >= limit:
            break
        moe_transformer([nxt], model, state)
    text = "".join(pieces)
    if verbose:
        print(text)
    return text


# ---- save / load (src/llama2/utils.jl:22-113) -------------------------------------------------

MODEL_MAGIC = b"MOEB200M"
_LAYER_ARRAYS = ("rms_att_weight", "rms_ffn_weight", "wq", "wk", "wv", "wo")
_FFN_ARRAYS = ("w1", "w2", "w3")


def _gate_to_dict(g) -> dict:
    return {"name": type(g).__name__, "k": int(getattr(g, "k", 1))}


def _gate_from_dict(d: dict):
    """reconstruct_gate_type (src/llama2/utils.jl): by type name and top_k."""
    from .gating import SwitchGating

    if d["name"] == "TopKGating":
        return TopKGating(int(d["k"]))
    if d["name"] == "SwitchGating":
        return SwitchGating()
    raise _lib.MoEError(_lib.ERR_UNSUPPORTED, f"gate {d['name']} cannot be restored")


def serialize_config(config: MoELlamaConfig) -> dict:
    """serialize_config (src/llama2/utils.jl:119-153): the same keys for the fields this package has."""
    c = config.llama_config
    loss = config.moe_balance_loss
    return {
        "dim": c.dim, "hidden_dim": c.hidden_dim, "n_layers": c.n_layers, "n_heads": c.n_heads,
        "n_kv_heads": c.n_kv_heads, "vocab_size": c.vocab_size, "seq_len": c.seq_len,
        "rope_freq_base": float(getattr(c, "rope_freq_base", 10000.0)), "rope_is_neox": bool(getattr(c, "rope_is_neox", False)),
        "moe_layers": list(config.moe_layers), "moe_num_experts": config.moe_num_experts, "moe_top_k": config.moe_top_k,
        "moe_expert_type": config.moe_expert_type, "expert_init_strategy": config.expert_init_strategy,
        "expert_init_noise": float(config.expert_init_noise), "z_loss_weight": float(config.z_loss_weight),
        "gate_type_name": type(config.moe_gate_type).__name__, "gate": _gate_to_dict(config.moe_gate_type),
        "balance_loss_name": type(loss).__name__, "balance_loss_alpha": float(getattr(loss, "alpha", 0.01)),
    }


def deserialize_config(d: dict) -> MoELlamaConfig:
    """deserialize_config (src/llama2/utils.jl:160-206)."""
    fields_ = {k: d[k] for k in ("dim", "hidden_dim", "n_layers", "n_heads", "n_kv_heads", "vocab_size", "seq_len")}
    for opt in ("rope_freq_base", "rope_is_neox"):
        if opt in ModelConfig.__dataclass_fields__:
            fields_[opt] = d[opt]
    if d["balance_loss_name"] != "SwitchTransformerLoss":
        raise _lib.MoEError(_lib.ERR_UNSUPPORTED, f"balance loss {d['balance_loss_name']} cannot be restored")
    return MoELlamaConfig(llama_config=ModelConfig(**fields_), moe_layers=[int(v) for v in d["moe_layers"]],
                          moe_num_experts=int(d["moe_num_experts"]), moe_top_k=int(d["moe_top_k"]),
                          moe_expert_type=d["moe_expert_type"], moe_gate_type=_gate_from_dict(d["gate"]),
                          moe_balance_loss=SwitchTransformerLoss(float(d["balance_loss_alpha"])),
                          expert_init_strategy=d["expert_init_strategy"], expert_init_noise=float(d["expert_init_noise"]),
                          z_loss_weight=float(d["z_loss_weight"]))


def _write_container(filename: str, header: dict, arrays: dict) -> None:
    """File = MODEL_MAGIC, u32 version, u64 JSON length, JSON, then every array's raw bytes at the
    256-byte aligned offset its JSON entry names."""
    index, off = {}, 0
    for name, a in arrays.items():
        a = np.ascontiguousarray(a)
        arrays[name] = a
        index[name] = {"dtype": a.dtype.str, "shape": list(a.shape), "offset": off, "nbytes": int(a.nbytes)}
        off = (off + a.nbytes + 255) & ~255
    blob = json.dumps(dict(header, arrays=index)).encode("utf-8")
    head = MODEL_MAGIC + struct.pack("<IQ", 1, len(blob)) + blob
    base = (len(head) + 255) & ~255
    with open(filename, "wb") as f:
        f.write(head)
        f.write(b"\0" * (base - len(head)))
        for name, a in arrays.items():
            f.seek(base + index[name]["offset"])
            f.write(a.tobytes() if a.nbytes < (1 << 20) else memoryview(a).cast("B"))
        f.truncate(base + off)


def _read_container(filename: str):
    with open(filename, "rb") as f:
        magic = f.read(8)
        if magic != MODEL_MAGIC:
            raise ValueError(f"{filename} is not a saved MoE model (bad magic)")
        version, n = struct.unpack("<IQ", f.read(12))
        if version != 1:
            raise ValueError(f"saved model version {version} is not supported")
        header = json.loads(f.read(n).decode("utf-8"))
        base = (20 + n + 255) & ~255
        arrays = {}
        for name, e in header.pop("arrays").items():
            f.seek(base + e["offset"])
            buf = f.read(e["nbytes"])
            if len(buf) != e["nbytes"]:
                raise ValueError(f"{filename} is truncated at array {name}")
            arrays[name] = np.frombuffer(buf, dtype=np.dtype(e["dtype"])).reshape(e["shape"])
    return header, arrays


def save_moe_model(model: MoELanguageModel, filename: str, *, format: str = "device") -> None:
    """save_moe_model(model, filename) (src/llama2/utils.jl:22-36).  The reference writes Julia's
    Serialization format; here the file is a self-describing container whose MoE layers are stored
    as device weight images (``MoELayer.export_weights``: the library's own layout in the model's
    compute dtype), so ``load_moe_model`` brings a layer back with plain copies.  The dense
    weights are float32 arrays.  ``format="both"`` also writes ``<name>_metadata.json`` like the
    reference's ``:both``."""
    fmt = str(format).lstrip(":")
    if fmt not in ("device", "julia", "json", "both"):
        raise ValueError(f"unknown format {format!r}")
    header = {
        "config": serialize_config(model.config),
        "metadata": {"model_type": "MoELanguageModel", "save_timestamp": time.strftime("%Y-%m-%dT%H:%M:%S"),
                     "library_version": _lib.version(), "compute_dtype": model.compute_dtype},
        "statistics": {"total_parameters": count_parameters(model), "active_parameters": count_active_parameters(model)},
        "layers": [{"layer_index": i + 1, "use_moe": bool(l.use_moe)} for i, l in enumerate(model.layers)],
    }
    if fmt in ("json", "both"):
        stem = filename.rsplit(".", 1)[0] if "." in filename.rsplit("/", 1)[-1] else filename
        with open(stem + "_metadata.json", "w") as f:
            json.dump(header, f, indent=1)
        if fmt == "json":
            return
    arrays = {"token_embedding_table": model.token_embedding_table, "rms_final_weight": model.rms_final_weight,
              "output_weight": model.output_weight}
    for i, l in enumerate(model.layers):
        for name in _LAYER_ARRAYS:
            arrays[f"layers.{i}.{name}"] = getattr(l.llama_layer, name)
        if l.use_moe:
            arrays[f"layers.{i}.moe_image"] = (l._weight_image if l._device_layer is None and l._weight_image is not None
                                               else _device_layer(model, l).export_weights())
        else:
            for name in _FFN_ARRAYS:
                arrays[f"layers.{i}.{name}"] = getattr(l.llama_layer, name)
    _write_container(filename, header, arrays)


def load_moe_model(filename: str, *, device: int = 0) -> MoELanguageModel:
    """load_moe_model(filename) (src/llama2/utils.jl:73-113): the model comes back with its MoE
    layers as weight images; each becomes a device handle on first use, without the experts ever
    existing as host arrays (``moe_experts`` is None for such a layer)."""
    header, arrays = _read_container(filename)
    for key in ("config", "metadata", "layers"):               # validate_save_data
        if key not in header:
            raise ValueError(f"{filename}: missing section {key!r}")
    cfg = deserialize_config(header["config"])
    c = cfg.llama_config
    empty = np.zeros((0, 0), dtype=np.float32)
    layers = []
    for i, meta in enumerate(header["layers"]):
        dense = {name: np.array(arrays[f"layers.{i}.{name}"]) for name in _LAYER_ARRAYS}
        if not meta["use_moe"]:
            dense.update({name: np.array(arrays[f"layers.{i}.{name}"]) for name in _FFN_ARRAYS})
            layers.append(MoETransformerLayerWeights(llama_layer=TransformerLayerWeights(**dense), use_moe=False))
            continue
        dense.update({name: empty for name in _FFN_ARRAYS})
        layer_cfg = MoEConfig(num_experts=cfg.moe_num_experts, expert_type=cfg.moe_expert_type, input_dim=c.dim,
                              hidden_dim=c.hidden_dim, output_dim=c.dim, activation=silu, gate_type=cfg.moe_gate_type,
                              top_k=cfg.moe_top_k, balance_loss=cfg.moe_balance_loss, z_loss_weight=cfg.z_loss_weight)
        layers.append(MoETransformerLayerWeights(llama_layer=TransformerLayerWeights(**dense), use_moe=True,
                                                 moe_config=layer_cfg, _weight_image=np.array(arrays[f"layers.{i}.moe_image"])))
    return MoELanguageModel(config=cfg, tokenizer=CharTokenizer(c.vocab_size),
                            token_embedding_table=np.array(arrays["token_embedding_table"]),
                            rms_final_weight=np.array(arrays["rms_final_weight"]),
                            output_weight=np.array(arrays["output_weight"]), layers=layers, device=device,
                            compute_dtype=header["metadata"].get("compute_dtype", "f32"))
