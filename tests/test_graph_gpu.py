"""Small batches replay a captured CUDA graph from the second call with the same buffers on.  The
replayed kernels are the launched ones, so every result must equal the plainly launched call bit
for bit, follow the buffers' current contents, agree with the CPU oracle, and survive whatever
drops the graphs (a larger batch, a setter, profiling)."""
import os
import sys

import numpy as np
import pytest
import torch

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
from helpers import device_gate, make_device_layer, oracle_gate, rel_inf  # noqa: E402
from oracle import moe_oracle as orc  # noqa: E402

pytestmark = pytest.mark.gpu


def _layer(compute, gate_kind="topk", k=2, S=0, E=8, D=256, H=512, O=256, seed=3):
    bf16 = compute == "bf16"
    x, w = orc.make_layer_inputs(seed, 64, D, H, O, E, init="normal", std=0.25, bf16=bf16)
    layer = make_device_layer(w, D=D, H=H, O=O, gate=device_gate(gate_kind, k, S, E), activation="silu", z=0.001,
                              compute_dtype=compute)
    cfg = orc.MoEConfig(num_experts=E, input_dim=D, hidden_dim=H, output_dim=O, activation="silu",
                        gate_type=oracle_gate(gate_kind, k, S, E), balance_alpha=0.01, z_loss_weight=0.001)
    return layer, cfg, w


def _inputs(T, D, seed, bf16):
    x = np.random.default_rng(seed).standard_normal((T, D)).astype(np.float32)
    xt = torch.from_numpy(x).cuda()
    if bf16:
        xt = xt.to(torch.bfloat16)
        x = xt.float().cpu().numpy()
    return x, xt


@pytest.mark.parametrize("compute,gate_kind,k,S", [("f32", "topk", 2, 0), ("bf16", "topk", 2, 0), ("f32", "switch", 1, 0),
                                                    ("bf16", "shared", 2, 1)])
def test_replays_equal_plain_launches_and_follow_the_buffers(compute, gate_kind, k, S):
    bf16 = compute == "bf16"
    layer, cfg, w = _layer(compute, gate_kind, k, S)
    T, D, O = 32, 256, 256
    buf = torch.empty((T, D), device="cuda", dtype=torch.bfloat16 if bf16 else torch.float32)
    out = torch.empty((T, O), device="cuda", dtype=torch.float32)
    # every call launched kernel by kernel (profiling keeps the graph path off)
    plain = []
    layer.set_profiling(1)
    for call in range(6):
        x, xt = _inputs(T, D, 100 + call, bf16)
        buf.copy_(xt)
        o, loss = layer(buf.t(), training=True, out=out)
        torch.cuda.synchronize()
        plain.append((o.t().cpu().numpy().copy(), float(loss.item())))
        assert layer.graph_replays() == 0
    counts_plain = layer.training_stats["tokens_per_expert"].copy()
    layer.set_profiling(0)
    seen = []
    for call in range(6):
        x, xt = _inputs(T, D, 100 + call, bf16)
        buf.copy_(xt)
        o, loss = layer(buf.t(), training=True, out=out)
        torch.cuda.synchronize()
        got, got_loss = o.t().cpu().numpy(), float(loss.item())
        assert np.array_equal(got, plain[call][0]) and got_loss == plain[call][1]
        ref_out, ref_loss, _ = orc.moe_layer_forward(cfg, w, x, training=True)
        assert rel_inf(got, ref_out) < (2e-2 if bf16 else 1e-5)
        assert abs(got_loss - float(ref_loss)) <= 1e-5 * abs(float(ref_loss))
        assert layer.device_status() == 0
        seen.append(layer.graph_replays())
    assert seen == [0, 1, 2, 3, 4, 5]      # first call plain, the second is captured and replayed
    assert np.array_equal(layer.training_stats["tokens_per_expert"], 2 * counts_plain)
    launches = layer.launch_count()
    layer(buf.t(), training=True, out=out)
    assert layer.launch_count() - launches >= 6     # the kernels inside the graph still count
    layer.close()


def test_growth_setters_and_other_keys_do_not_reuse_a_stale_graph():
    layer, cfg, w = _layer("f32")
    D, O = 256, 256
    out32 = torch.empty((32, O), device="cuda")
    x32, xt32 = _inputs(32, D, 7, False)
    for _ in range(3):
        layer(xt32.t(), training=True, out=out32)
    assert layer.graph_replays() == 2
    # a larger batch grows the workspace (the graphs held the old addresses)
    xbig, xtbig = _inputs(4096, D, 8, False)
    obig, _ = layer(xtbig.t(), training=False)
    torch.cuda.synchronize()
    ref_big, _, _ = orc.moe_layer_forward(cfg, w, xbig, training=False)
    assert rel_inf(obig.t().cpu().numpy(), ref_big) < 1e-5
    ref32, ref_loss, _ = orc.moe_layer_forward(cfg, w, x32, training=True)
    for _ in range(3):
        o, loss = layer(xt32.t(), training=True, out=out32)
        torch.cuda.synchronize()
        assert rel_inf(o.t().cpu().numpy(), ref32) < 1e-5
        assert abs(float(loss.item()) - float(ref_loss)) <= 1e-5 * abs(float(ref_loss))
    assert layer.graph_replays() == 4
    # inference on the same buffers is another key (no loss term), and so is another T
    o_inf, loss_inf = layer(xt32.t(), training=False, out=out32)
    torch.cuda.synchronize()
    assert float(loss_inf.item()) == 0.0 and layer.graph_replays() == 4
    # new router weights: the next calls must see them
    w2 = orc.make_layer_inputs(11, 64, D, 512, O, 8, init="normal", std=0.25)[1]
    layer.router.weight = w2.router.copy()
    layer.sync_router()
    w.router = w2.router
    ref_new, ref_loss_new, _ = orc.moe_layer_forward(cfg, w, x32, training=True)
    for _ in range(3):
        o, loss = layer(xt32.t(), training=True, out=out32)
        torch.cuda.synchronize()
        assert rel_inf(o.t().cpu().numpy(), ref_new) < 1e-5
        assert abs(float(loss.item()) - float(ref_loss_new)) <= 1e-5 * abs(float(ref_loss_new))
    layer.close()


@pytest.mark.parametrize("chain,graphs,replays", [("1", "1", 0), ("0", "1", 3), ("0", "0", 0), ("1", "0", 0)])
def test_small_host_calls_with_every_launch_mode(monkeypatch, chain, graphs, replays):
    """Per-position host calls: chained plain launches by default, a graph replay keyed on the staging
    buffers when chaining is switched off, plain launches when both are off -- same results each way."""
    monkeypatch.setenv("MOE_B200_CHAIN", chain)
    monkeypatch.setenv("MOE_B200_GRAPHS", graphs)
    layer, cfg, w = _layer("f32")
    D = 256
    for call in range(4):
        for T in (1, 7):
            x, _ = _inputs(T, D, 300 + 10 * call + T, False)
            out, loss, routing = layer(np.asfortranarray(x.T), training=True, return_routing=True)
            ref, ref_loss, aux = orc.moe_layer_forward(cfg, w, x, training=True)
            assert rel_inf(np.asarray(out).T, ref) < 1e-5
            assert abs(float(loss) - float(ref_loss)) <= 1e-5 * abs(float(ref_loss))
            assert np.array_equal(np.asarray(routing["indices"]).T, aux["indices"])
    # (the first calls of each batch size launch plainly; the staging block grows once in between)
    assert (layer.graph_replays() >= 4) if replays else (layer.graph_replays() == 0)
    assert layer.device_status() == 0
    layer.close()


@pytest.mark.parametrize("compute", ["f32", "bf16"])
def test_a_call_inside_the_callers_own_capture_joins_that_graph(compute):
    """A forward made while the caller's stream is being captured (here: torch.cuda.graph) must not start
    a capture of its own: its kernels become nodes of the caller's graph, and replaying that graph
    computes the layer on the buffers' current contents."""
    bf16 = compute == "bf16"
    layer, cfg, w = _layer(compute)
    T, D, O = 48, 256, 256
    buf = torch.empty((T, D), device="cuda", dtype=torch.bfloat16 if bf16 else torch.float32)
    out = torch.empty((T, O), device="cuda", dtype=torch.float32)
    call = layer.bind_forward(buf.t(), out, training=True)
    x, xt = _inputs(T, D, 41, bf16)
    buf.copy_(xt)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        call()                                  # plain launches: sizes the workspace outside any capture
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    replays_before = layer.graph_replays()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=side):
        call()
    assert layer.graph_replays() == replays_before          # no graph of the library's own was involved
    for seed in (42, 43):
        x, xt = _inputs(T, D, seed, bf16)
        buf.copy_(xt)
        out.zero_()
        g.replay()
        torch.cuda.synchronize()
        ref_out, ref_loss, _ = orc.moe_layer_forward(cfg, w, x, training=True)
        assert rel_inf(out.cpu().numpy(), ref_out) < (2e-2 if bf16 else 1e-5)
        assert abs(float(call.loss.item()) - float(ref_loss)) <= 1e-5 * abs(float(ref_loss))
    assert layer.device_status() == 0
    del g
    layer.close()
