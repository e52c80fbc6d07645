"""GPU parity tests: the CUDA path, called through the C ABI (via the ctypes host mirror),
against the CPU oracle on the same seeded inputs.

Tolerances (from the task statement): expert indices bit-exact except gate-logit ties within
1e-6; FP32 outputs and loss within 1e-5 relative (||a-b||_inf/||b||_inf per tensor); the BF16
tensor-core path within 2e-2 relative, the oracle being evaluated in FP32 on the BF16-rounded
weights and activations."""
import os
import sys

import numpy as np
import pytest
import torch

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
import make_golden  # noqa: E402
from helpers import check_indices, device_gate, make_device_layer, oracle_gate, rel_inf  # noqa: E402
from oracle import moe_oracle as orc  # noqa: E402

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
F32_TOL = 1e-5
BF16_TOL = 2e-2


def logits64(x, w, bias=None):
    lg = x.astype(np.float64) @ w.router.astype(np.float64).T
    if bias is not None:
        lg = lg + bias.astype(np.float64)
    return lg


def run_case(T, D, H, O, E, gate_kind, k, S=0, *, seed=0, activation="silu", compute="f32", z=0.001,
             num_shared_experts=0, init="normal", std=0.25, host=False, training=True, tol=None, x_bf16=None, expert_kind="gated"):
    bf16 = compute == "bf16"
    e_router = E - num_shared_experts
    x, w = orc.make_layer_inputs(seed, T, D, H, O, E, e_router=e_router, init=init, std=std, bf16=bf16,
                                 expert_kind=expert_kind)
    ogate = oracle_gate(gate_kind, k, S, E)
    cfg = orc.MoEConfig(num_experts=E, input_dim=D, hidden_dim=H, output_dim=O, activation=activation,
                        gate_type=ogate, balance_alpha=0.01, z_loss_weight=z, num_shared_experts=num_shared_experts)
    o_out, o_loss, aux = orc.moe_layer_forward(cfg, w, x, training=training)
    layer = make_device_layer(w, D=D, H=H, O=O, gate=device_gate(gate_kind, k, S, E), activation=activation, z=z,
                              compute_dtype=compute, num_shared_experts=num_shared_experts)
    if host:
        xin = np.asfortranarray(x.T)
    else:
        xt = torch.from_numpy(x).cuda()
        if x_bf16 if x_bf16 is not None else bf16:
            xt = xt.to(torch.bfloat16)
        xin = xt.t()
    out, loss, stats, routing = layer(xin, training=training, return_stats=True, return_routing=True)
    if not host:
        torch.cuda.synchronize()
        out = out.cpu().numpy()
        loss = float(loss.item())
        routing = {k_: v.cpu().numpy() for k_, v in routing.items()}
    assert layer.device_status() == 0
    tol = tol or (BF16_TOL if bf16 else F32_TOL)
    r0 = S if gate_kind == "shared" else 0
    kk = 1 if gate_kind == "switch" else k
    excused = check_indices(routing["indices"].T, aux["indices"], logits64(x, w), kk, r0)
    assert rel_inf(routing["logits"].T, aux["logits"]) < F32_TOL
    if excused == 0:
        assert rel_inf(routing["gates"].T, aux["gates"]) < F32_TOL
        assert rel_inf(out.T, o_out) < tol, f"output rel err {rel_inf(out.T, o_out):.3e}"
    assert rel_inf(routing["probs"].T, aux["probs"]) < F32_TOL
    assert abs(float(loss) - float(o_loss)) <= F32_TOL * max(abs(float(o_loss)), 1e-30) + (1e-4 if excused else 0)
    if num_shared_experts == 0:
        assert np.array_equal(stats["tokens_per_expert"], aux["stats"]["tokens_per_expert"]) or excused
        assert abs(stats["routing_entropy"][-1] - float(aux["stats"]["routing_entropy"])) < 1e-5
    layer.close()
    return rel_inf(out.T, o_out)


# ---- golden fixtures (the 8-expert 512/2048/512 benchmark configuration and the small gate/shared-expert variants) -------------

@pytest.mark.parametrize("case", list(make_golden.CASES))
@pytest.mark.parametrize("host", [False, True])
def test_golden_fixture(case, host):
    c, cfg, x, w = make_golden.build(case)
    ref = np.load(os.path.join(GOLDEN, f"{case}.npz"))
    g = c["gate"]
    S = g[2] if g[0] == "shared" else 0
    k = 1 if g[0] == "switch" else g[1]
    nsh = c.get("num_shared_experts", 0)
    extra = {key: c[key] for key in ("drop_tokens", "capacity_factor", "noise_scale") if key in c}
    layer = make_device_layer(w, D=c["D"], H=c["H"], O=c["O"], gate=device_gate(g[0], k, S, c["E"]),
                              activation=c.get("activation", "silu"), z=c["z"], num_shared_experts=nsh, **extra)
    if cfg.noise_scale > 0:
        layer.router.noise_scale = cfg.noise_scale
        layer.router.noise_weight = w.noise_weight
        layer.sync_router()
    xin = np.asfortranarray(x.T) if host else torch.from_numpy(x).cuda().t()
    out, loss, routing = layer(xin, training=True, return_routing=True,
                               router_noise=None if cfg.router_noise is None else cfg.router_noise.T)
    if not host:
        out, loss = out.cpu().numpy(), float(loss.item())
        routing = {k_: v.cpu().numpy() for k_, v in routing.items()}
    assert np.array_equal(routing["indices"].T, ref["indices"])
    assert rel_inf(out.T, ref["out"]) < F32_TOL
    assert rel_inf(routing["gates"].T, ref["gates"]) < F32_TOL
    assert rel_inf(routing["probs"].T, ref["probs"]) < F32_TOL
    assert rel_inf(routing["logits"].T, ref["logits"]) < F32_TOL
    assert abs(float(loss) - float(ref["loss"])) < F32_TOL * abs(float(ref["loss"]))
    layer.close()


# ---- FP32 path: shape sweep with ragged sizes ---------------------------------------------------

@pytest.mark.parametrize("T", [1, 2, 31, 32, 33, 257])
@pytest.mark.parametrize("E,k", [(2, 1), (8, 2), (8, 8), (66, 6)])
def test_f32_shape_sweep(T, E, k):
    run_case(T, 72, 100, 52, E, "topk", k, seed=T * 100 + E)


@pytest.mark.parametrize("dims", [(512, 1376, 512), (36, 44, 20), (7, 9, 5), (128, 128, 128)])
def test_f32_odd_dims(dims):
    D, H, O = dims
    run_case(50, D, H, O, 8, "topk", 2, seed=D)


@pytest.mark.parametrize("activation", ["silu", "gelu", "relu", "identity"])
def test_f32_activations(activation):
    run_case(40, 64, 96, 64, 4, "topk", 2, activation=activation, seed=3)


def test_f32_switch_gate_and_inference_mode():
    run_case(100, 64, 96, 64, 8, "switch", 1, seed=5)
    run_case(100, 64, 96, 64, 8, "topk", 2, seed=6, training=False)


def test_f32_shared_expert_gating_and_layer_blend():
    run_case(130, 64, 96, 64, 10, "shared", 3, 2, seed=7)
    run_case(90, 64, 96, 48, 6, "topk", 2, seed=8, num_shared_experts=2)


def test_f32_bf16_input_is_cast_like_the_router():
    run_case(64, 64, 96, 64, 8, "topk", 2, seed=9, compute="f32", x_bf16=False)


def test_aux_free_bias_selects_but_does_not_change_probs():
    import mixtureofexperts_b200 as m

    T, D, H, O, E = 64, 64, 96, 64, 8
    x, w = orc.make_layer_inputs(11, T, D, H, O, E, init="normal", std=0.25)
    bias = np.random.default_rng(3).normal(0, 1.5, E).astype(np.float32)
    cfg = orc.MoEConfig(num_experts=E, input_dim=D, hidden_dim=H, output_dim=O, activation="silu",
                        gate_type=orc.TopKGating(2), balance_alpha=0.001, z_loss_weight=0.0, aux_free_bias=bias)
    o_out, _, aux = orc.moe_layer_forward(cfg, w, x, training=False)
    bl = m.AuxiliaryFreeLoss(E)
    bl.bias = bias.copy()
    layer = make_device_layer(w, D=D, H=H, O=O, gate=m.TopKGating(2), z=0.0, balance_loss=bl)
    out, _, routing = layer(torch.from_numpy(x).cuda().t(), training=False, return_routing=True)
    assert np.array_equal(routing["indices"].cpu().numpy().T, aux["indices"])
    assert rel_inf(routing["gates"].cpu().numpy().T, aux["gates"]) < F32_TOL
    assert rel_inf(routing["probs"].cpu().numpy().T, aux["probs"]) < F32_TOL
    assert rel_inf(out.cpu().numpy().T, o_out) < F32_TOL
    layer.close()


@pytest.mark.parametrize("update_freq,drop,host", [(1, False, False), (2, False, False), (1, True, False), (1, False, True)])
def test_aux_free_bias_update_runs_on_the_device(update_freq, drop, host):
    """AuxiliaryFreeLoss over several training steps: the bias the device handle updates after each
    call (update_bias!, src/balancing/auxiliary_free.jl:36-71) follows the oracle's, and so do
    the experts each later step selects with it.  A large learning rate makes the bias matter."""
    import mixtureofexperts_b200 as m

    T, D, H, O, E, steps = 96, 48, 64, 40, 8, 6
    _, w = orc.make_layer_inputs(21, T, D, H, O, E, init="normal", std=0.25)
    w.router[0] *= 3.0                                        # a popular expert to push against
    st = orc.AuxFreeState(bias=np.zeros(E, dtype=np.float32), bias_momentum=np.zeros(E, dtype=np.float32),
                          learning_rate=2.0, momentum=0.5, update_freq=update_freq)
    cfg = orc.MoEConfig(num_experts=E, input_dim=D, hidden_dim=H, output_dim=O, activation="silu",
                        gate_type=orc.TopKGating(2), balance_alpha=0.001, z_loss_weight=0.001, aux_free_state=st,
                        drop_tokens=drop, capacity_factor=2.5)
    bl = m.AuxiliaryFreeLoss(E, learning_rate=2.0, momentum=0.5, update_freq=update_freq)
    layer = make_device_layer(w, D=D, H=H, O=O, gate=m.TopKGating(2), balance_loss=bl, drop_tokens=drop,
                              capacity_factor=2.5)
    assert layer._aux_on_device
    first_idx = None
    for step in range(steps):
        x = np.random.default_rng(100 + step).standard_normal((T, D)).astype(np.float32)
        o_out, o_loss, aux = orc.moe_layer_forward(cfg, w, x, training=True)
        xin = np.asfortranarray(x.T) if host else torch.from_numpy(x).cuda().t()
        out, loss, routing = layer(xin, training=True, return_routing=True)
        idx = routing["indices"] if host else routing["indices"].cpu().numpy()
        assert np.array_equal(idx.T, aux["indices"]), f"step {step}"
        assert rel_inf(out if host else out.cpu().numpy(), o_out.T) < F32_TOL
        assert abs(float(loss) - float(o_loss)) < F32_TOL * abs(float(o_loss))
        assert rel_inf(bl.bias, st.bias) < F32_TOL and rel_inf(bl.bias_momentum, st.bias_momentum) < F32_TOL
        assert bl.update_counter == st.update_counter == step + 1
        assert abs(float(bl.bias.sum())) < 1e-5
        first_idx = aux["indices"] if first_idx is None else first_idx
    assert np.abs(st.bias).max() > 0.05 and st.bias[0] < 0            # the popular expert was pushed down
    # an inference call neither updates nor counts
    layer(torch.from_numpy(x).cuda().t(), training=False)
    assert bl.update_counter == steps
    # assigning the bias pushes it to the device; the momentum survives
    mom = bl.bias_momentum.copy()
    bl.bias = np.arange(E, dtype=np.float32)
    assert np.array_equal(bl.bias, np.arange(E, dtype=np.float32)) and np.array_equal(bl.bias_momentum, mom)
    layer.close()
    assert np.array_equal(bl.bias, np.arange(E, dtype=np.float32))    # the loss object keeps the final state


def test_aux_free_update_stays_on_the_host_with_layer_shared_experts():
    """forward_with_shared_experts (src/core/moe_layer.jl:158-185) never selects with the bias but
    still hands the shifted routed ids to compute_loss, which updates it."""
    import mixtureofexperts_b200 as m

    T, D, H, O, E, S = 64, 32, 48, 32, 6, 2
    x, w = orc.make_layer_inputs(4, T, D, H, O, E, e_router=E - S, init="normal", std=0.25)
    cfg = orc.MoEConfig(num_experts=E, input_dim=D, hidden_dim=H, output_dim=O, activation="silu",
                        gate_type=orc.TopKGating(2), balance_alpha=0.001, num_shared_experts=S)
    o_out, _, aux = orc.moe_layer_forward(cfg, w, x, training=True)
    start = np.array([3, -1, 2, -2, 1, -3], dtype=np.float32)
    st = orc.AuxFreeState(bias=start.copy(), bias_momentum=np.zeros(E, dtype=np.float32), learning_rate=1.0)
    orc.aux_free_update_bias(st, aux["indices"])
    bl = m.AuxiliaryFreeLoss(E, learning_rate=1.0, bias=start)
    layer = make_device_layer(w, D=D, H=H, O=O, gate=m.TopKGating(2), balance_loss=bl, num_shared_experts=S)
    assert not layer._aux_on_device
    out, _, routing = layer(torch.from_numpy(x).cuda().t(), training=True, return_routing=True)
    assert np.array_equal(routing["indices"].cpu().numpy().T, aux["indices"])       # the bias did not select
    assert rel_inf(out.cpu().numpy().T, o_out) < F32_TOL
    assert bl.update_counter == 1 and np.array_equal(bl.bias, st.bias)
    layer.close()
    with pytest.raises(m.MoEError):
        make_device_layer(w, D=D, H=H, O=O, gate=m.TopKGating(2), balance_loss=m.AuxiliaryFreeLoss(E - S),
                          num_shared_experts=S)


def test_router_bias_skews_routing_like_config4():
    """A per-expert logit bias N(0,1.5) that is part of the logits (the skew of the DeepSeek-style benchmark configuration)."""
    T, D, H, O, E, S, k = 300, 64, 96, 64, 18, 2, 6
    x, w = orc.make_layer_inputs(12, T, D, H, O, E, init="normal", std=0.25)
    bias = np.concatenate([np.zeros(S), np.random.default_rng(4).normal(0, 1.5, E - S)]).astype(np.float32)
    cfg = orc.MoEConfig(num_experts=E, input_dim=D, hidden_dim=H, output_dim=O, activation="silu",
                        gate_type=orc.SharedExpertGating(S, orc.TopKGating(k), E), z_loss_weight=0.001,
                        router_bias=bias)
    o_out, o_loss, aux = orc.moe_layer_forward(cfg, w, x, training=True)
    layer = make_device_layer(w, D=D, H=H, O=O, gate=device_gate("shared", k, S, E), router_bias=bias)
    out, loss, routing = layer(torch.from_numpy(x).cuda().t(), training=True, return_routing=True)
    check_indices(routing["indices"].cpu().numpy().T, aux["indices"], logits64(x, w, bias), k, S)
    assert rel_inf(out.cpu().numpy().T, o_out) < F32_TOL
    assert abs(float(loss.item()) - float(o_loss)) < F32_TOL * abs(float(o_loss))
    counts = np.bincount(aux["indices"].ravel() - 1, minlength=E)
    assert counts[S:].max() > 3 * max(counts[S:].min(), 1)  # routing is strongly skewed
    layer.close()


@pytest.mark.parametrize("T,E,k,cf,host", [(200, 8, 2, 1.25, False), (64, 4, 2, 0.5, True), (8300, 8, 2, 1.0, True),
                                             (333, 10, 3, 0.75, False)])
def test_capacity_constraint_drops_late_tokens(T, E, k, cf, host):
    """drop_tokens && training: apply_capacity_constraint (src/core/moe_layer.jl:221-248) - first come,
    first served in token order, dropped slots get id 0 / gate 0, gates renormalised per token."""
    D, H, O = 64, 96, 48
    x, w = orc.make_layer_inputs(400 + T, T, D, H, O, E, init="normal", std=0.25)
    cfg = orc.MoEConfig(num_experts=E, input_dim=D, hidden_dim=H, output_dim=O, activation="silu",
                        gate_type=orc.TopKGating(k), balance_alpha=0.01, z_loss_weight=0.001, drop_tokens=True,
                        capacity_factor=cf)
    o_out, o_loss, aux = orc.moe_layer_forward(cfg, w, x, training=True)
    assert (aux["indices"] == 0).any()                      # the case does drop something
    layer = make_device_layer(w, D=D, H=H, O=O, gate=device_gate("topk", k), drop_tokens=True, capacity_factor=cf)
    xin = np.asfortranarray(x.T) if host else torch.from_numpy(x).cuda().t()
    out, loss, stats, routing = layer(xin, training=True, return_stats=True, return_routing=True)
    if not host:
        out, loss = out.cpu().numpy(), float(loss.item())
        routing = {k_: v.cpu().numpy() for k_, v in routing.items()}
    assert np.array_equal(routing["indices"].T, aux["indices"])
    assert rel_inf(routing["gates"].T, aux["gates"]) < F32_TOL
    assert rel_inf(out.T, o_out) < F32_TOL
    assert abs(float(loss) - float(o_loss)) < F32_TOL * abs(float(o_loss))
    assert np.array_equal(stats["tokens_per_expert"], aux["stats"]["tokens_per_expert"])
    # inference mode ignores the constraint
    o2, _, aux2 = orc.moe_layer_forward(cfg, w, x, training=False)
    out2, _, rt2 = layer(xin, training=False, return_routing=True)
    out2 = out2 if host else out2.cpu().numpy()
    idx2 = rt2["indices"] if host else rt2["indices"].cpu().numpy()
    assert np.array_equal(idx2.T, aux2["indices"]) and rel_inf(out2.T, o2) < F32_TOL
    layer.close()


@pytest.mark.parametrize("host", [False, True])
def test_training_time_router_noise_with_given_draws(host):
    """noise_scale > 0 && training (src/core/router.jl:38-40): logits + noise_scale*randn feed the gate;
    the z-loss comes from the noise-free logits (the reference's second router pass).  The draws are
    passed in, so the comparison with the oracle is exact up to FP32 rounding."""
    T, D, H, O, E, k = 300, 64, 96, 48, 8, 2
    x, w = orc.make_layer_inputs(77, T, D, H, O, E, init="normal", std=0.25)
    noise = np.random.default_rng(9).standard_normal((T, E)).astype(np.float32)
    cfg = orc.MoEConfig(num_experts=E, input_dim=D, hidden_dim=H, output_dim=O, activation="silu",
                        gate_type=orc.TopKGating(k), balance_alpha=0.01, z_loss_weight=0.001, noise_scale=0.7,
                        router_noise=noise)
    o_out, o_loss, aux = orc.moe_layer_forward(cfg, w, x, training=True)
    clean_idx = orc.moe_layer_forward(cfg, w, x, training=False)[2]["indices"]
    assert (aux["indices"] != clean_idx).any()                   # the noise does change the routing
    layer = make_device_layer(w, D=D, H=H, O=O, gate=device_gate("topk", k), noise_scale=0.7)
    layer.router.noise_scale = 0.7
    xin = np.asfortranarray(x.T) if host else torch.from_numpy(x).cuda().t()
    out, loss, routing = layer(xin, training=True, return_routing=True, router_noise=noise.T)
    if not host:
        out, loss = out.cpu().numpy(), float(loss.item())
        routing = {k_: v.cpu().numpy() for k_, v in routing.items()}
    assert np.array_equal(routing["indices"].T, aux["indices"])
    assert rel_inf(routing["logits"].T, aux["logits"]) < F32_TOL
    assert rel_inf(routing["gates"].T, aux["gates"]) < F32_TOL
    assert rel_inf(out.T, o_out) < F32_TOL
    assert abs(float(loss) - float(o_loss)) < F32_TOL * abs(float(o_loss))
    # inference ignores the noise; a training call without given draws still runs (draws made on the device)
    out2, _, rt2 = layer(xin, training=False, return_routing=True)
    idx2 = rt2["indices"] if host else rt2["indices"].cpu().numpy()
    assert np.array_equal(idx2.T, clean_idx)
    out3, _ = layer(xin, training=True)
    assert np.isfinite(out3 if host else out3.cpu().numpy()).all()
    layer.close()


@pytest.mark.parametrize("E,k,host", [(8, 2, False), (8, 2, True), (33, 3, False), (64, 4, False)])
def test_router_noise_network(E, k, host):
    """use_noise_network (src/core/router.jl:33-37): logits + noise_scale * (randn .* softplus(noise_weight x)).
    The noise projection rides in the gate GEMM (2E columns); E = 33 and 64 cross its column buckets."""
    T, D, H, O = 260, 72, 64, 40
    x, w = orc.make_layer_inputs(31 + E, T, D, H, O, E, init="normal", std=0.25)
    rng = np.random.default_rng(E)
    w.noise_weight = (rng.standard_normal((E, D)) * 0.3).astype(np.float32)
    noise = rng.standard_normal((T, E)).astype(np.float32)
    cfg = orc.MoEConfig(num_experts=E, input_dim=D, hidden_dim=H, output_dim=O, activation="silu",
                        gate_type=orc.TopKGating(k), balance_alpha=0.01, z_loss_weight=0.001, noise_scale=0.5,
                        router_noise=noise)
    o_out, o_loss, aux = orc.moe_layer_forward(cfg, w, x, training=True)
    plain = orc.MoEWeights(router=w.router, experts=w.experts)
    assert (orc.moe_layer_forward(cfg, plain, x, training=True)[2]["indices"] != aux["indices"]).any()
    layer = make_device_layer(w, D=D, H=H, O=O, gate=device_gate("topk", k), noise_scale=0.5)
    layer.router.noise_scale = 0.5
    layer.router.noise_weight = w.noise_weight
    layer.sync_router()
    xin = np.asfortranarray(x.T) if host else torch.from_numpy(x).cuda().t()
    out, loss, routing = layer(xin, training=True, return_routing=True, router_noise=noise.T)
    if not host:
        out, loss = out.cpu().numpy(), float(loss.item())
        routing = {k_: v.cpu().numpy() for k_, v in routing.items()}
    lg64 = x.astype(np.float64) @ w.router.astype(np.float64).T + 0.5 * noise.astype(np.float64) * orc.softplus(
        x.astype(np.float64) @ w.noise_weight.astype(np.float64).T)
    excused = check_indices(routing["indices"].T, aux["indices"], lg64, k)
    assert rel_inf(routing["logits"].T, aux["logits"]) < F32_TOL
    if not excused:
        assert rel_inf(routing["gates"].T, aux["gates"]) < F32_TOL
        assert rel_inf(out.T, o_out) < F32_TOL
        assert abs(float(loss) - float(o_loss)) < F32_TOL * abs(float(o_loss))
    # inference reads neither the draws nor the network
    clean_idx = orc.moe_layer_forward(cfg, w, x, training=False)[2]["indices"]
    rt2 = layer(xin, training=False, return_routing=True)[2]
    idx2 = rt2["indices"] if host else rt2["indices"].cpu().numpy()
    assert np.array_equal(idx2.T, clean_idx)
    # removing the network falls back to plain Gaussian noise
    layer.router.noise_weight = None
    layer.sync_router()
    rt3 = layer(xin, training=True, return_routing=True, router_noise=noise.T)[2]
    idx3 = rt3["indices"] if host else rt3["indices"].cpu().numpy()
    assert np.array_equal(idx3.T, orc.moe_layer_forward(cfg, plain, x, training=True)[2]["indices"])
    layer.close()


def test_router_noise_network_is_refused_beyond_64_router_rows():
    import mixtureofexperts_b200 as m

    cfg = m.create_moe_config(num_experts=66, expert_type="gated", input_dim=16, hidden_dim=16, output_dim=16,
                              gate_type=m.TopKGating(2), noise_scale=0.1, use_noise_network=True)
    with pytest.raises(m.MoEError):
        m.MoELayer(cfg)


def test_empty_batch():
    x, w = orc.make_layer_inputs(1, 1, 64, 96, 64, 4, init="normal", std=0.25)
    layer = make_device_layer(w, D=64, H=96, O=64, gate=device_gate("topk", 2))
    out, loss = layer(torch.empty((64, 0), device="cuda"), training=True)
    assert tuple(out.shape) == (64, 0) and float(loss.item()) == 0.0
    out, loss = layer(np.zeros((64, 0), dtype=np.float32, order="F"), training=True)
    assert out.shape == (64, 0) and float(loss) == 0.0
    layer.close()


def test_two_runs_are_bit_identical_and_workspace_grows():
    x, w = orc.make_layer_inputs(2, 700, 64, 96, 64, 8, init="normal", std=0.25)
    layer = make_device_layer(w, D=64, H=96, O=64, gate=device_gate("topk", 2))
    xt = torch.from_numpy(x).cuda()
    small = layer(xt[:10].t(), training=True)[0].clone()
    a, la = layer(xt.t(), training=True)
    a = a.clone()
    b, lb = layer(xt.t(), training=True)
    assert torch.equal(a, b) and float(la.item()) == float(lb.item())
    # a 10-token call may take another kernel (weight streaming) than the 700-token call: same
    # values up to FP32 summation order
    assert (small - a[:, :10]).abs().max().item() <= 1e-5 * a.abs().max().item()
    layer.close()


@pytest.mark.parametrize("gate_kind,E,S,k", [("topk", 8, 0, 2), ("shared", 10, 2, 3)])
def test_chunked_host_call_equals_device_call(gate_kind, E, S, k):
    """Host calls with >= 8192 tokens are pipelined over token chunks (copy-in / compute / copy-out
    overlap); outputs must not change, and loss/entropy/counts finished from the summed chunk
    statistics must agree with the one-pass device call."""
    T, D, H, O = 8200 + 37, 64, 96, 48
    x, w = orc.make_layer_inputs(31, T, D, H, O, E, init="normal", std=0.25)
    layer = make_device_layer(w, D=D, H=H, O=O, gate=device_gate(gate_kind, k, S, E))
    out_d, loss_d, st_d, rt_d = layer(torch.from_numpy(x).cuda().t(), training=True, return_stats=True,
                                      return_routing=True)
    counts_d = st_d["tokens_per_expert"].copy()
    ent_d = st_d["routing_entropy"][-1]
    out_h, loss_h, st_h, rt_h = layer(np.asfortranarray(x.T), training=True, return_stats=True, return_routing=True)
    assert np.array_equal(out_h, out_d.cpu().numpy())
    assert np.array_equal(rt_h["indices"], rt_d["indices"].cpu().numpy())
    assert np.array_equal(rt_h["gates"], rt_d["gates"].cpu().numpy())
    assert np.array_equal(rt_h["probs"], rt_d["probs"].cpu().numpy())
    assert abs(float(loss_h) - float(loss_d.item())) < 1e-6 * abs(float(loss_d.item()))
    assert np.array_equal(st_h["tokens_per_expert"], 2 * counts_d)
    assert abs(st_h["routing_entropy"][-1] - ent_d) < 1e-6
    assert layer.device_status() == 0
    # repeated calls: same results, same number of kernels counted per call
    n0 = layer.launch_count()
    per_call = None
    for rep in range(3):
        out_r, loss_r, rt_r = layer(np.asfortranarray(x.T), training=True, return_routing=True)
        assert np.array_equal(out_r, out_h) and float(loss_r) == float(loss_h), rep
        assert np.array_equal(rt_r["indices"], rt_h["indices"]) and np.array_equal(rt_r["gates"], rt_h["gates"])
        n1 = layer.launch_count()
        assert per_call in (None, n1 - n0), (rep, per_call, n1 - n0)
        per_call, n0 = n1 - n0, n1
    # other arguments (no routing outputs, inference) and new input values on the same handle
    x2 = np.asfortranarray((x * 0.5).T)
    want2 = layer(torch.from_numpy(np.ascontiguousarray(x2.T)).cuda().t(), training=False)[0].cpu().numpy()
    for rep in range(3):
        assert np.array_equal(layer(x2, training=False)[0], want2), rep
    assert layer.device_status() == 0
    layer.close()


def test_device_resident_weights_still_being_produced():
    """Weights handed over as CUDA tensors right after the kernels that produce them were queued:
    the upload must wait for them (it runs on the handle's own stream)."""
    import mixtureofexperts_b200 as m

    T, D, H, O, E = 256, 1024, 2048, 1024, 4
    g = torch.Generator(device="cuda").manual_seed(5)
    big = torch.randn((64, 1024, 1024), device="cuda", generator=g)          # keeps the stream busy for a while
    for _ in range(4):
        big = big @ big.transpose(1, 2) * 1e-3
    ws = [[torch.randn(s, device="cuda", generator=g) * 0.05 for s in ((H, D), (O, H), (H, D))] for _ in range(E)]
    router = torch.randn((E, D), device="cuda", generator=g) * 0.05
    weights = orc.MoEWeights(router=router, experts=[orc.GatedExpertWeights(w1=a, w2=b, w3=c) for a, b, c in ws])
    layer = make_device_layer(weights, D=D, H=H, O=O, gate=m.TopKGating(2), z=0.0)   # uploads device tensors at once
    x = torch.randn((T, D), device="cuda", generator=g)
    out, _ = layer(x.t(), training=False)
    host = orc.MoEWeights(router=router.cpu().numpy(), experts=[
        orc.GatedExpertWeights(w1=a.cpu().numpy(), w2=b.cpu().numpy(), w3=c.cpu().numpy()) for a, b, c in ws])
    cfg = orc.MoEConfig(num_experts=E, input_dim=D, hidden_dim=H, output_dim=O, activation="silu",
                        gate_type=orc.TopKGating(2), z_loss_weight=0.0)
    o_out, _, _ = orc.moe_layer_forward(cfg, host, x.cpu().numpy(), training=False)
    assert torch.isfinite(out).all()
    assert rel_inf(out.cpu().numpy().T, o_out) < F32_TOL
    layer.close()


def test_token_permutation_equivariance():
    """Each token's output depends on that token only: permuting the batch permutes the output."""
    x, w = orc.make_layer_inputs(3, 500, 64, 96, 64, 8, init="normal", std=0.25)
    layer = make_device_layer(w, D=64, H=96, O=64, gate=device_gate("topk", 2))
    xt = torch.from_numpy(x).cuda()
    perm = torch.randperm(500, generator=torch.Generator().manual_seed(0)).cuda()
    a = layer(xt.t(), training=False)[0].clone()
    b = layer(xt[perm].t(), training=False)[0]
    assert torch.equal(a[:, perm], b)
    layer.close()


# ---- stand-alone operators ----------------------------------------------------------------------

def test_compute_gates_and_compute_loss_operators():
    import mixtureofexperts_b200 as m

    rng = np.random.default_rng(5)
    logits = rng.standard_normal((333, 16)).astype(np.float32)
    oi, og, op = orc.compute_gates(orc.TopKGating(4), logits)
    lt = torch.from_numpy(logits).cuda()
    di, dg, dp = m.compute_gates(m.TopKGating(4), lt.t())
    assert np.array_equal(di.cpu().numpy().T, oi)
    assert rel_inf(dg.cpu().numpy().T, og) < F32_TOL and rel_inf(dp.cpu().numpy().T, op) < F32_TOL
    # the reference's own property: gates of a token sum to 1 within 1e-6
    assert np.abs(dg.cpu().numpy().sum(axis=0) - 1).max() < 1e-6
    oi2, og2, op2 = orc.compute_gates(orc.SharedExpertGating(2, orc.TopKGating(3), 16), logits)
    di2, dg2, dp2 = m.compute_gates(m.SharedExpertGating(2, m.TopKGating(3), 16), lt.t())
    assert np.array_equal(di2.cpu().numpy().T, oi2)
    assert rel_inf(dg2.cpu().numpy().T, og2) < F32_TOL and rel_inf(dp2.cpu().numpy().T, op2) < F32_TOL
    want = orc.switch_transformer_loss(0.01, oi, op)
    got = m.compute_loss(m.SwitchTransformerLoss(0.01), di, dp)
    assert abs(float(got.item()) - float(want)) < F32_TOL * float(want)
    wz = orc.z_loss(0.001, logits)
    gz = m.compute_loss(m.ZLoss(0.001), lt.t())
    assert abs(float(gz.item()) - float(wz)) < F32_TOL * float(wz)


def test_jitter_gating_operator_and_layer():
    """JitterGating (src/gating/switch.jl:20-33): with training=true the base gate sees
    logits .* (1 .+ (2u .- 1) .* eps); inside a layer the router never passes the keyword, so
    the layer routes like the base gate."""
    import mixtureofexperts_b200 as m

    rng = np.random.default_rng(12)
    logits = (rng.standard_normal((500, 12)) * 2).astype(np.float32)
    u = rng.random((500, 12), dtype=np.float32)
    lt, ut = torch.from_numpy(logits).cuda(), torch.from_numpy(u).cuda()
    gate, ogate = m.JitterGating(m.TopKGating(2), 0.3), orc.JitterGating(orc.TopKGating(2), 0.3)
    oi, og, op = orc.compute_gates(ogate, logits, training=True, jitter_u=u)
    di, dg, dp = m.compute_gates(gate, lt.t(), training=True, jitter=ut.t())
    assert (oi != orc.compute_gates(ogate, logits)[0]).any()              # the jitter does move some choices
    assert np.array_equal(di.cpu().numpy().T, oi)
    assert rel_inf(dg.cpu().numpy().T, og) < F32_TOL and rel_inf(dp.cpu().numpy().T, op) < F32_TOL
    di0 = m.compute_gates(gate, lt.t())[0]                                 # training=false: the base gate
    assert np.array_equal(di0.cpu().numpy().T, orc.compute_gates(orc.TopKGating(2), logits)[0])
    di1 = m.compute_gates(gate, lt.t(), training=True)[0]                  # draws made on the device
    assert di1.shape == di.shape and int(di1.min()) >= 1 and int(di1.max()) <= 12
    # a layer configured with JitterGating equals the same layer with its base gate, training or not
    x, w = orc.make_layer_inputs(8, 120, 64, 96, 48, 8, init="normal", std=0.25)
    la = make_device_layer(w, D=64, H=96, O=48, gate=m.JitterGating(m.TopKGating(2), 0.3))
    lb = make_device_layer(w, D=64, H=96, O=48, gate=m.TopKGating(2))
    xin = torch.from_numpy(x).cuda().t()
    (oa, lossa), (ob, lossb) = la(xin, training=True), lb(xin, training=True)
    assert torch.equal(oa, ob) and float(lossa.item()) == float(lossb.item())
    la.close()
    lb.close()


def test_exact_ties_go_to_the_lowest_index():
    import mixtureofexperts_b200 as m

    logits = np.array([[0.5, 2.0, 2.0, 2.0, -1.0], [1.0, 1.0, 1.0, 1.0, 1.0]], dtype=np.float32)
    di, dg, _ = m.compute_gates(m.TopKGating(2), torch.from_numpy(logits).cuda().t())
    assert di.cpu().numpy().T.tolist() == [[2, 3], [1, 2]]


# ---- wide routers on the tensor cores (33..80 router rows, BF16 activations) ---------------------

@pytest.mark.parametrize("T,E,k,D,gate,S", [
    (1000, 66, 6, 2048, "shared", 2),     # the DeepSeek-style router: 64 routed + 2 shared rows, top-6
    (300, 64, 2, 4096, "topk", 0),        # the expert-parallel layer's router width and depth
    (129, 33, 3, 136, "topk", 0),         # narrowest width of the path, D not a multiple of the K block
    (1, 80, 8, 256, "topk", 0),           # widest width, a single token
    (2500, 48, 1, 512, "switch", 0),      # many tiles per CTA
])
def test_tensor_core_router_against_oracle(T, E, k, D, gate, S):
    """Indices by the tie rule, logits/gates/probs/loss at the FP32 tolerance: the split gate GEMM on the
    tensor cores plus the exact re-evaluation of close rankings must be indistinguishable from FP32."""
    run_case(T, D, 64, 64, E, gate, k, S, seed=T + E, compute="bf16", std=0.05)


def test_tensor_core_router_logit_error_and_rechecks(monkeypatch):
    """The tensor-core logits against float64, beside the FP32-FMA router kernel on the same inputs; and
    duplicated router rows (exact ties in every token) must be decided like the reference: lowest id."""
    import mixtureofexperts_b200 as m

    T, D, H, O, E, k = 4096, 4096, 64, 64, 64, 2
    x, w = orc.make_layer_inputs(11, T, D, H, O, E, init="normal", std=0.02, bf16=True)
    w.router[40] = w.router[7]                     # experts 8 and 41 always tie
    lg64 = logits64(x, w)
    cfg = orc.MoEConfig(num_experts=E, input_dim=D, hidden_dim=H, output_dim=O, activation="silu",
                        gate_type=orc.TopKGating(k), balance_alpha=0.01, z_loss_weight=0.001)
    o_idx, o_gates, o_probs, _ = orc.router_forward(cfg, w, x)
    xt = torch.from_numpy(x).cuda().to(torch.bfloat16)
    errs = {}
    for tc in ("1", "0"):
        monkeypatch.setenv("MOE_B200_ROUTER_TC", tc)
        layer = make_device_layer(w, D=D, H=H, O=O, gate=m.TopKGating(k), compute_dtype="bf16")
        _, _, routing = layer(xt.t(), training=True, return_routing=True)
        torch.cuda.synchronize()
        idx = routing["indices"].cpu().numpy().T
        check_indices(idx, o_idx, lg64, k)
        tied = (o_idx == 8).any(axis=1) | (o_idx == 41).any(axis=1)
        assert np.array_equal(idx[tied], o_idx[tied])          # 8 before 41, never 41 without 8
        assert rel_inf(routing["gates"].cpu().numpy().T, o_gates) < F32_TOL
        assert rel_inf(routing["probs"].cpu().numpy().T, o_probs) < F32_TOL
        errs[tc] = float(np.abs(routing["logits"].cpu().numpy().T.astype(np.float64) - lg64).max())
        rechecks = layer.router_rechecks()
        assert (rechecks >= int(tied.sum())) if tc == "1" else rechecks == 0
        layer.close()
    print(f"max |logit - float64|: tensor-core router {errs['1']:.3e}, FP32-FMA router {errs['0']:.3e}")
    assert errs["1"] < 5e-6 and errs["0"] < 5e-6          # |logits| are ~1.3 here: a few 1e-6 relative for both


# ---- StandardExpert: w2(act.(w1 x .+ b1)) .+ b2 -------------------------------------------------

@pytest.mark.parametrize("T,E,k,D,H,O,activation", [
    (257, 8, 2, 64, 96, 48, "gelu"),          # tiled FP32 kernel, MoEConfig's default activation
    (3, 8, 2, 36, 44, 20, "relu"),            # skinny FP32 kernel
    (500, 4, 1, 128, 130, 70, "silu"),
])
@pytest.mark.parametrize("host", [False, True])
def test_f32_standard_expert(T, E, k, D, H, O, activation, host):
    run_case(T, D, H, O, E, "topk", k, seed=T + 7, activation=activation, expert_kind="standard", host=host)


def test_f32_standard_expert_with_layer_blend_and_without_bias():
    run_case(130, 64, 96, 64, 6, "topk", 2, seed=5, activation="gelu", expert_kind="standard", num_shared_experts=2)
    import mixtureofexperts_b200 as m

    T, D, H, O, E = 100, 32, 48, 24, 4
    x, w = orc.make_layer_inputs(3, T, D, H, O, E, init="normal", std=0.25, expert_kind="standard")
    for e in w.experts:
        e.b1 = e.b2 = None
    cfg = orc.MoEConfig(num_experts=E, input_dim=D, hidden_dim=H, output_dim=O, activation="gelu",
                        gate_type=orc.TopKGating(2))
    o_out, _, _ = orc.moe_layer_forward(cfg, w, x, training=False)
    layer = make_device_layer(w, D=D, H=H, O=O, gate=m.TopKGating(2), activation="gelu")
    out, _ = layer(np.asfortranarray(x.T))
    assert rel_inf(out.T, o_out) < F32_TOL
    layer.close()


@pytest.mark.parametrize("pair", ["0", "1", "2"])
@pytest.mark.parametrize("T,E,k,D,H,O", [(1000, 8, 2, 512, 1024, 512), (300, 4, 1, 136, 200, 104), (3, 66, 2, 128, 256, 128)])
def test_bf16_standard_expert_on_both_tensor_core_kernels(pair, T, E, k, D, H, O, monkeypatch):
    monkeypatch.setenv("MOE_B200_PAIR", pair)
    err = run_case(T, D, H, O, E, "topk", k, seed=T + E, compute="bf16", std=0.05, activation="gelu",
                   expert_kind="standard")
    assert err < BF16_TOL


def test_standard_expert_setter_is_refused_on_a_gated_layer_and_dropout_is_rejected():
    import mixtureofexperts_b200 as m

    with pytest.raises(m.MoEError):
        m.MoELayer(m.create_moe_config(num_experts=2, expert_type="standard", input_dim=8, hidden_dim=8, output_dim=8,
                                       expert_dropout=0.1))
    layer = m.MoELayer(m.create_moe_config(num_experts=2, expert_type="gated", input_dim=8, hidden_dim=8, output_dim=8))
    w = np.zeros((8, 8), dtype=np.float32)
    from mixtureofexperts_b200 import _lib

    rc = _lib.lib.moe_layer_set_expert_standard(layer._handle, 0, w.ctypes.data, None, w.ctypes.data, None, 0, 0, 0)
    assert rc == _lib.ERR_STATE
    layer.close()


# ---- BF16 tensor-core path ----------------------------------------------------------------------

@pytest.mark.parametrize("T,E,k,D,H,O", [
    (1000, 8, 2, 512, 1024, 512),     # several m-tiles per expert, ragged last tiles
    (64, 8, 2, 256, 384, 256),        # fewer rows than one tile per expert
    (300, 4, 1, 136, 200, 104),       # D, H, O not multiples of the 64/128/256 tile edges
    (257, 66, 6, 128, 256, 128),      # many small experts, some empty
    (1, 8, 2, 128, 256, 128),         # a single token
    (4500, 2, 1, 128, 256, 128),      # many m-tiles per expert
])
def test_bf16_tensor_core_path(T, E, k, D, H, O):
    err = run_case(T, D, H, O, E, "topk", k, seed=T + E, compute="bf16", std=0.05)
    assert err < BF16_TOL


@pytest.mark.parametrize("pair", ["0", "1", "2"])
def test_bf16_both_tensor_core_kernels_on_ragged_experts(pair, monkeypatch):
    """MOE_B200_PAIR forces the single-CTA kernel (128-row tiles), the CTA-pair kernel or the two-accumulator
    kernel (256-row tiles) on shapes with empty experts, partial last tiles (with and without rows in
    their second half), widths off the tile edges, shared experts read in place, many tiles per expert."""
    monkeypatch.setenv("MOE_B200_PAIR", pair)
    assert run_case(777, 136, 200, 104, 10, "topk", 3, seed=91, compute="bf16", std=0.05) < BF16_TOL
    assert run_case(3, 128, 256, 128, 66, "topk", 2, seed=92, compute="bf16", std=0.05) < BF16_TOL
    assert run_case(4500, 128, 256, 128, 2, "topk", 1, seed=93, compute="bf16", std=0.05) < BF16_TOL
    assert run_case(1500, 256, 512, 264, 10, "shared", 3, 2, seed=94, compute="bf16", std=0.05) < BF16_TOL
    assert run_case(2048, 1024, 1536, 512, 4, "topk", 2, seed=95, compute="bf16", std=0.03) < BF16_TOL


def test_bf16_shared_gating_and_f32_input():
    run_case(400, 128, 256, 128, 10, "shared", 3, 2, seed=21, compute="bf16", std=0.05)
    run_case(200, 128, 256, 120, 8, "topk", 2, seed=22, compute="bf16", std=0.05, x_bf16=False)


def test_bf16_mixtral_shaped_slice_sampled_against_oracle():
    """Mixtral-shaped widths (d_model 4096, ffn 14336) at a reduced expert/token count; the
    oracle checks a sample of tokens (the dense oracle on all tokens would take minutes)."""
    import mixtureofexperts_b200 as m

    T, D, H, O, E = 2048, 4096, 14336, 4096, 2
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn((T, D), device="cuda", generator=g).to(torch.bfloat16)
    router = (torch.randn((E, D), device="cuda", generator=g) * 0.02)
    ws = [[(torch.randn(s, device="cuda", generator=g) * 0.02).to(torch.bfloat16) for s in ((H, D), (O, H), (H, D))]
          for _ in range(E)]
    weights = orc.MoEWeights(router=router.cpu().numpy(),
                             experts=[orc.GatedExpertWeights(w1=a, w2=b, w3=c) for a, b, c in ws])
    layer = make_device_layer(weights, D=D, H=H, O=O, gate=m.TopKGating(1), compute_dtype="bf16", z=0.0)
    out, loss, routing = layer(x.t(), training=True, return_routing=True)
    torch.cuda.synchronize()
    assert layer.device_status() == 0
    sample = np.arange(0, T, 97)
    xs = x[sample].float().cpu().numpy()
    cpu_w = orc.MoEWeights(router=weights.router, experts=[
        orc.GatedExpertWeights(w1=a.float().cpu().numpy(), w2=b.float().cpu().numpy(), w3=c.float().cpu().numpy())
        for a, b, c in ws])
    cfg = orc.MoEConfig(num_experts=E, input_dim=D, hidden_dim=H, output_dim=O, activation="silu",
                        gate_type=orc.TopKGating(1), z_loss_weight=0.0)
    o_out, _, aux = orc.moe_layer_forward(cfg, cpu_w, xs, training=False)
    assert np.array_equal(routing["indices"].cpu().numpy().T[sample], aux["indices"])
    err = rel_inf(out.cpu().numpy().T[sample], o_out)
    assert err < BF16_TOL, err
    layer.close()


# ---- seeded sweep over shapes nobody picked by hand ----------------------------------------------------------------

def _sweep_case(rng):
    compute = str(rng.choice(["f32", "bf16"]))
    kind = str(rng.choice(["topk", "switch", "shared"]))
    E = int(rng.choice([2, 3, 5, 8, 16, 31, 33, 48, 64, 66, 80, 96, 128]))
    S = int(rng.integers(1, 3)) if kind == "shared" else 0
    if kind == "shared" and E - S < 1:
        kind, S = "topk", 0
    k = 1 if kind == "switch" else int(rng.integers(1, max(1, min(E - S, 8 - S)) + 1))
    if compute == "bf16":      # the tensor-core path wants input and hidden widths in multiples of 8
        D, H = int(rng.integers(1, 65)) * 8, int(rng.integers(1, 97)) * 8
    else:
        D, H = int(rng.integers(3, 400)), int(rng.integers(3, 500))
    nse = 0
    if kind != "shared" and E >= 4 and rng.integers(0, 4) == 0:      # forward_with_shared_experts
        nse = int(rng.integers(1, 3))
        k = max(1, min(k, E - nse, 8 - nse))
    return dict(T=int(rng.choice([1, 2, 7, 33, 64, 100, 257, 1000, 2500])), D=D, H=H, O=int(rng.integers(1, 300)), E=E,
                gate_kind=kind, k=k, S=S, compute=compute, host=bool(rng.integers(0, 2)), training=bool(rng.integers(0, 2)),
                activation=str(rng.choice(["silu", "gelu", "relu"])), num_shared_experts=nse,
                expert_kind=str(rng.choice(["gated", "gated", "standard"])),
                x_bf16=bool(rng.integers(0, 2)) if compute == "bf16" else None)


@pytest.mark.parametrize("block", range(4))
def test_seeded_sweep_of_shapes_gates_and_dtypes(block):
    """Twelve drawn configurations per block: widths that are no multiple of any tile, 1 to 2500 tokens, every gate,
    both expert types and shared-expert mechanisms, device and host calls -- each against the oracle at the
    tolerances of its dtype (run_case)."""
    rng = np.random.default_rng(20240 + block)
    for i in range(12):
        c = _sweep_case(rng)
        T, D, H, O, E = c.pop("T"), c.pop("D"), c.pop("H"), c.pop("O"), c.pop("E")
        kind, k, S = c.pop("gate_kind"), c.pop("k"), c.pop("S")
        try:
            run_case(T, D, H, O, E, kind, k, S, seed=7000 + 100 * block + i, std=0.1, **c)
        except AssertionError as exc:
            raise AssertionError(f"case {i} of block {block}: T={T} D={D} H={H} O={O} E={E} {kind} k={k} S={S} {c}: {exc}") from exc


@pytest.mark.parametrize("expert_kind,activation", [("gated", "silu"), ("standard", "gelu")])
def test_the_three_tensor_core_kernels_give_the_same_bits(expert_kind, activation, monkeypatch):
    """Which kernel a batch gets depends on its size (rows per expert, K): the results must not.  The same layer
    and input through the single-CTA, the CTA-pair and the two-accumulator kernel: identical outputs, bit for bit."""
    T, D, H, O, E = 1500, 256, 512, 264, 4
    x, w = orc.make_layer_inputs(17, T, D, H, O, E, init="normal", std=0.05, bf16=True, expert_kind=expert_kind)
    xt = torch.from_numpy(x).cuda().to(torch.bfloat16)
    outs = []
    for kernel in ("0", "1", "2"):
        monkeypatch.setenv("MOE_B200_PAIR", kernel)
        layer = make_device_layer(w, D=D, H=H, O=O, gate=device_gate("topk", 2, 0, E), activation=activation, compute_dtype="bf16")
        assert layer.gemm_kernel(T) == int(kernel)
        out, _ = layer(xt.t(), training=False)
        torch.cuda.synchronize()
        outs.append(out.clone())
        layer.close()
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
