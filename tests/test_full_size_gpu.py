"""Full-size checks on the benchmark workloads (c3: Mixtral-shaped, c4: DeepSeek-style), built by
bench.py's own workload builders: size-independent properties on every token, and parity with
the CPU oracle on a sample of tokens (the dense oracle on all tokens would take minutes)."""
import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import bench  # noqa: E402
from helpers import check_indices, rel_inf  # noqa: E402
from oracle import moe_oracle as orc  # noqa: E402

pytestmark = pytest.mark.gpu


def _oracle_weights(w, device):
    """The workload's weights, regenerated expert by expert (bench.make_expert_factory is a pure
    function of the expert id) and copied to the host as float32."""
    fac = bench.make_expert_factory(w, torch, device)
    experts = []
    for e in range(w["E"]):
        ex = fac(e)
        experts.append(orc.GatedExpertWeights(w1=ex.w1.float().cpu().numpy(), w2=ex.w2.float().cpu().numpy(),
                                              w3=ex.w3.float().cpu().numpy()))
    r = bench.make_router(w, torch, device)
    bias = r.bias.cpu().numpy() if getattr(r, "bias", None) is not None else None
    return orc.MoEWeights(router=r.weight.cpu().numpy(), experts=experts), bias


@pytest.mark.parametrize("name,n_sample", [("c3", 256), ("c4", 160)])
def test_benchmark_workload_full_size(name, n_sample):
    w = dict(bench.WORKLOADS[name])
    device = "cuda:0"
    layer = bench.build_layer(w, torch, 0)
    T, D, O, E, S, k = w["T"], w["D"], w["O"], w["E"], w["S"], w["k"]
    g = torch.Generator(device=device).manual_seed(99)
    x = torch.randn((T, D), device=device, generator=g).to(torch.bfloat16)
    out, loss, stats, routing = layer(x.t(), training=True, return_stats=True, return_routing=True)
    torch.cuda.synchronize()
    assert layer.device_status() == 0
    idx = routing["indices"].t()
    gates = routing["gates"].t()
    # properties that hold at any size (the reference's own checks among them)
    assert torch.isfinite(out).all() and float(loss.item()) >= 0
    assert int(idx.min()) >= 1 and int(idx.max()) <= E
    assert (gates.sum(dim=1) - 1).abs().max().item() < 1e-5            # gates of a token sum to 1
    assert (idx.sort(dim=1).values.diff(dim=1) > 0).all()              # a token never picks an expert twice
    counts = stats["tokens_per_expert"]
    assert counts.sum() == T * (k + S)
    assert np.array_equal(counts, torch.bincount(idx.reshape(-1) - 1, minlength=E).cpu().numpy())
    if S:
        assert (idx[:, :S] == torch.arange(1, S + 1, device=device)).all() and counts[:S].tolist() == [T] * S
        assert counts[S:].max() > 3 * max(int(counts[S:].min()), 1)   # the logit bias skews the routing
    # a second run is bit-identical; permuting the tokens permutes the output
    out2, loss2 = layer(x.t(), training=True)
    assert torch.equal(out, out2) and float(loss.item()) == float(loss2.item())
    perm = torch.randperm(T, generator=torch.Generator().manual_seed(1)).to(device)
    outp, _ = layer(x[perm].t(), training=True)
    assert torch.equal(out[:, perm], outp)
    # sampled parity with the oracle (FP32 on the BF16-rounded values), tolerance 2e-2
    weights, bias = _oracle_weights(w, device)
    sample = np.linspace(0, T - 1, n_sample).astype(np.int64)
    gate = orc.SharedExpertGating(S, orc.TopKGating(k), E) if S else orc.TopKGating(k)
    cfg = orc.MoEConfig(num_experts=E, input_dim=D, hidden_dim=w["H"], output_dim=O, activation="silu", gate_type=gate,
                        z_loss_weight=0.0, router_bias=bias)
    xs = x[sample].float().cpu().numpy()
    o_out, _, aux = orc.moe_layer_forward(cfg, weights, xs, training=False)
    got_idx = idx[sample].cpu().numpy()
    # expert ids: bit-exact, except where the float64 logits of neighbouring ranks around the
    # selected set differ by less than 1e-6 (the tie window of partialsortperm on FP32
    # probabilities, src/gating/topk.jl:35); check_indices fails on any other difference
    logits64 = xs.astype(np.float64) @ weights.router.astype(np.float64).T
    if bias is not None:
        logits64 = logits64 + bias.astype(np.float64)
    excused = check_indices(got_idx, aux["indices"], logits64, k, r0=S)
    same = (got_idx == aux["indices"]).all(axis=1)
    assert excused == int((~same).sum()) and excused <= max(1, n_sample // 50), excused
    # outputs of the tokens whose ids agree (a tie-excused token ran through other experts)
    err = rel_inf(out.t()[sample][same].cpu().numpy(), o_out[same])
    assert err < 2e-2, err
    g_err = rel_inf(gates[sample][same].cpu().numpy(), aux["gates"][same])
    assert g_err < 1e-5, g_err
    layer.close()
