"""CPU tests of the oracle itself: golden fixtures, the independent float64 restatement, and
the property checks the reference's own test script makes on this path
(test_moeLlama2_integration.jl:66-86, :114-130, :132-164, :459-479)."""
import os
import sys

import numpy as np
import pytest
import torch

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
import make_golden  # noqa: E402
from helpers import rel_inf  # noqa: E402
from oracle import moe_oracle as orc  # noqa: E402
from oracle.moe_oracle_torch64 import layer_forward64, topk_passes  # noqa: E402

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


@pytest.mark.parametrize("case", list(make_golden.CASES))
def test_oracle_reproduces_golden(case):
    got = make_golden.run_case(case)
    ref = np.load(os.path.join(GOLDEN, f"{case}.npz"))
    assert np.array_equal(got["indices"], ref["indices"])
    for key in ("out", "gates", "probs", "logits"):
        assert rel_inf(got[key], ref[key]) < 2e-6, key
    assert abs(float(got["loss"]) - float(ref["loss"])) <= 2e-6 * abs(float(ref["loss"]))


@pytest.mark.parametrize("case", ["c1", "c1_noz", "shared_gating", "switch_gelu"])
def test_oracle_agrees_with_float64_restatement(case):
    c, cfg, x, w = make_golden.build(case)
    out, loss, aux = orc.moe_layer_forward(cfg, w, x, training=True)
    g = c["gate"]
    S = g[2] if g[0] == "shared" else 0
    k = 1 if g[0] == "switch" else g[1]
    o64, l64, i64, g64, p64 = layer_forward64(
        x, w.router, [(e.w1, e.w2, e.w3) for e in w.experts], k=k, activation=c.get("activation", "silu"),
        alpha=0.01, z_weight=c["z"], training=True, num_shared_gating=S)
    assert np.array_equal(aux["indices"] - 1, i64.numpy())
    assert rel_inf(out, o64.numpy()) < 1e-5
    assert rel_inf(aux["gates"], g64.numpy()) < 1e-5
    assert rel_inf(aux["probs"], p64.numpy()) < 1e-5
    assert abs(float(loss) - float(l64)) < 1e-5 * abs(float(l64))


def test_reference_property_checks():
    """gates sum to 1 within 1e-6, indices in 1..E, at least 2 rows, finite output, loss >= 0."""
    rng = np.random.default_rng(0)
    logits = rng.standard_normal((17, 8)).astype(np.float32)
    idx, gates, probs = orc.compute_gates(orc.TopKGating(2), logits)
    assert idx.shape[1] >= 2
    assert ((idx >= 1) & (idx <= 8)).all()
    assert np.allclose(gates.sum(axis=1), 1.0, atol=1e-6)
    assert np.allclose(probs.sum(axis=1), 1.0, atol=1e-6)
    c, cfg, x, w = make_golden.build("c1")
    out, loss, _ = orc.moe_layer_forward(cfg, w, x[:1], training=False)
    assert out.shape == (1, 512) and np.isfinite(out).all() and loss >= 0


def test_gated_expert_matches_inline_matvecs():
    """gated_expert_forward! equals an inline restatement of the three matvecs to 1e-5."""
    x, w = orc.make_layer_inputs(5, 1, 64, 96, 64, 1, init="normal", std=0.02)
    e = w.experts[0]
    got = orc.gated_expert_forward_llama(e, x[0])
    h1 = e.w1 @ x[0]
    h3 = e.w3 @ x[0]
    want = e.w2 @ ((h1 * (1.0 / (1.0 + np.exp(-h1)))) * h3)
    assert np.abs(got - want).max() < 1e-5


@pytest.mark.parametrize("activation", ["gelu", "relu", "silu"])
def test_standard_expert_agrees_with_float64_restatement(activation):
    """StandardExpert (src/experts/standard.jl:38-55) through the whole layer against the
    independent float64 restatement, and its single-expert form against inline matvecs."""
    T, D, H, O, E = 64, 48, 80, 40, 6
    x, w = orc.make_layer_inputs(11, T, D, H, O, E, init="normal", std=0.2, expert_kind="standard")
    cfg = orc.MoEConfig(num_experts=E, input_dim=D, hidden_dim=H, output_dim=O, activation=activation,
                        gate_type=orc.TopKGating(2))
    out, loss, aux = orc.moe_layer_forward(cfg, w, x, training=True)
    o64, l64, i64, _, _ = layer_forward64(x, w.router, [(e.w1, e.w2, e.b1, e.b2) for e in w.experts], k=2,
                                          activation=activation, alpha=cfg.balance_alpha, z_weight=cfg.z_loss_weight,
                                          training=True)
    assert np.array_equal(aux["indices"] - 1, i64.numpy())
    assert rel_inf(out, o64.numpy()) < 1e-5
    assert abs(float(loss) - float(l64)) < 1e-5 * abs(float(l64))
    e = w.experts[0]
    h = e.w1 @ x[0] + e.b1
    want = e.w2 @ orc.ACTIVATIONS[activation](h) + e.b2
    assert np.abs(orc.standard_expert_forward(e, x[:1], orc.ACTIVATIONS[activation])[0] - want).max() < 1e-5
    e.b1 = e.b2 = None
    assert np.abs(orc.standard_expert_forward(e, x[:1], orc.ACTIVATIONS[activation])[0]
                  - e.w2 @ orc.ACTIVATIONS[activation](e.w1 @ x[0])).max() < 1e-5


def test_noise_network_softplus_scaling():
    """router.jl:33-37: logits + noise_scale * (randn .* softplus(noise_weight x)), softplus as NNlib's."""
    T, D, E = 20, 16, 4
    x, w = orc.make_layer_inputs(3, T, D, 8, 8, E, init="normal", std=0.25)
    rng = np.random.default_rng(0)
    w.noise_weight = rng.standard_normal((E, D)).astype(np.float32)
    noise = rng.standard_normal((T, E)).astype(np.float32)
    cfg = orc.MoEConfig(num_experts=E, input_dim=D, hidden_dim=8, output_dim=8, gate_type=orc.TopKGating(2),
                        noise_scale=0.3, router_noise=noise)
    lg = orc.router_forward(cfg, w, x, training=True)[3]
    want = x.astype(np.float64) @ w.router.T.astype(np.float64) + 0.3 * noise * np.log1p(
        np.exp(x.astype(np.float64) @ w.noise_weight.T.astype(np.float64)))
    assert rel_inf(lg, want) < 1e-5
    assert np.array_equal(orc.router_forward(cfg, w, x, training=False)[3], x @ w.router.T)
    assert abs(float(orc.softplus(np.float32(0))) - np.log(2)) < 1e-7 and orc.softplus(np.float32(100)) == 100


def test_jitter_gating_only_acts_when_training():
    rng = np.random.default_rng(1)
    logits = rng.standard_normal((50, 6)).astype(np.float32)
    u = rng.random((50, 6), dtype=np.float32)
    g = orc.JitterGating(orc.TopKGating(2), 0.5)
    base = orc.compute_gates(orc.TopKGating(2), logits)
    off = orc.compute_gates(g, logits)
    assert all(np.array_equal(a, b) for a, b in zip(base, off))
    on = orc.compute_gates(g, logits, training=True, jitter_u=u)
    want = orc.compute_gates(orc.TopKGating(2), logits * (1 + (2 * u - 1) * np.float32(0.5)))
    assert np.array_equal(on[0], want[0]) and rel_inf(on[2], want[2]) < 1e-6
    # jitter stays inside [1-eps, 1+eps)
    assert np.abs((1 + (2 * u - 1) * 0.5) - 1).max() <= 0.5


def test_aux_free_update_bias_restatement():
    """update_bias! (src/balancing/auxiliary_free.jl:36-71): overloaded experts get a falling bias, the
    bias stays mean-centred, update_freq skips calls, an all-dropped batch changes nothing."""
    st = orc.AuxFreeState(bias=np.zeros(4, dtype=np.float32), bias_momentum=np.zeros(4, dtype=np.float32),
                          learning_rate=0.01, momentum=0.9, update_freq=2)
    idx = np.array([[1, 2], [1, 3], [1, 4], [1, 2]])
    orc.aux_free_update_bias(st, idx)
    assert st.update_counter == 1 and not st.bias.any()              # skipped by update_freq
    orc.aux_free_update_bias(st, idx)
    # counts (4,2,1,1) of 8, target 2: gradient (0.25, 0, -0.125, -0.125); momentum = 0.1*gradient
    assert np.allclose(st.bias_momentum, [0.025, 0, -0.0125, -0.0125], atol=1e-7)
    raw = -0.01 * st.bias_momentum
    assert np.allclose(st.bias, raw - raw.mean(), atol=1e-8) and abs(float(st.bias.sum())) < 1e-7
    before = st.bias.copy()
    orc.aux_free_update_bias(st, np.zeros((4, 2), dtype=np.int64))
    orc.aux_free_update_bias(st, np.zeros((4, 2), dtype=np.int64))
    assert np.array_equal(st.bias, before)


def test_topk_ties_go_to_lowest_index():
    logits = np.array([[0.5, 2.0, 2.0, 2.0, -1.0]], dtype=np.float32)
    idx, gates, _ = orc.compute_gates(orc.TopKGating(2), logits)
    assert idx.tolist() == [[2, 3]]
    ti, _ = topk_passes(torch.softmax(torch.tensor(logits, dtype=torch.float64), -1), 2)
    assert ti.tolist() == [[1, 2]]


def test_determinism_three_runs():
    c, cfg, x, w = make_golden.build("shared_gating")
    outs = [orc.moe_layer_forward(cfg, w, x, training=True)[0] for _ in range(3)]
    assert np.abs(outs[0] - outs[1]).max() < 1e-6 and np.abs(outs[0] - outs[2]).max() < 1e-6


def test_layer_blend_loss_quirk():
    """forward_with_shared_experts computes the loss with ids shifted by +S against E-S
    probability rows: ids above E-S fall out of the count."""
    c, cfg, x, w = make_golden.build("layer_blend")
    _, loss, aux = orc.moe_layer_forward(cfg, w, x, training=True)
    S, Er = 2, 4
    idx0 = aux["indices"] - 1
    counts = np.bincount(idx0[idx0 < Er].ravel(), minlength=Er).astype(np.float32)
    f = counts / np.float32(idx0.size)
    want = np.float32(0.01) * Er * np.sum(f * aux["probs"].mean(axis=0)) + orc.z_loss(0.001, aux["logits"])
    assert abs(float(loss) - float(want)) < 1e-7


def test_capacity_constraint_sequential():
    idx = np.array([[1, 2], [1, 2], [1, 3], [1, 2]], dtype=np.int64)
    gates = np.full((4, 2), 0.5, dtype=np.float32)
    i2, g2 = orc.apply_capacity_constraint(idx, gates, capacity_factor=1.5, num_experts=3)  # capacity 2
    assert i2.tolist() == [[1, 2], [1, 2], [0, 3], [0, 0]]
    assert g2[2].tolist() == [0.0, 1.0] and g2[3].tolist() == [0.0, 0.0]


def test_bf16_round_matches_torch():
    a = np.random.default_rng(1).standard_normal(1000).astype(np.float32)
    want = torch.tensor(a).to(torch.bfloat16).to(torch.float32).numpy()
    assert np.array_equal(orc.bf16_round(a), want)


def test_llama_token_path_matches_layer():
    """moe_ffn_forward!'s per-token restatement equals the batched layer on the same weights."""
    x, w = orc.make_layer_inputs(9, 5, 32, 48, 32, 4, init="normal", std=0.2)
    cfg = orc.MoEConfig(num_experts=4, input_dim=32, hidden_dim=48, output_dim=32, activation="silu",
                        gate_type=orc.TopKGating(2), z_loss_weight=0.0)
    out, _, aux = orc.moe_layer_forward(cfg, w, x, training=False)
    for t in range(5):
        y, idx, gates, _ = orc.moe_ffn_forward_token(w.router, w.experts, orc.TopKGating(2), 2, x[t])
        assert np.array_equal(idx, aux["indices"][t])
        assert np.abs(y - out[t]).max() < 1e-5
