"""Generates tests/golden/*.npz: outputs of the CPU oracle (oracle/moe_oracle.py) on seeded
synthetic inputs.  The reference itself cannot be executed (no Julia runtime is available), so
these fixtures pin the ORACLE; tests/test_oracle.py checks that the oracle still reproduces
them and that an independent float64 restatement agrees.

Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import moe_oracle as orc  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))

# name -> (seed, T, D, H, O, E, gate spec, extra config)
CASES = {
    # the CPU-runnable benchmark configuration: 8 GatedExperts (silu) 512/2048/512, TopKGating(2), SwitchTransformerLoss(0.01),
    # input 512x32 N(0,1), Glorot-uniform weights, training=true
    "c1": dict(seed=1235, T=32, D=512, H=2048, O=512, E=8, gate=("topk", 2), z=0.001, init="glorot"),
    "c1_noz": dict(seed=1235, T=32, D=512, H=2048, O=512, E=8, gate=("topk", 2), z=0.0, init="glorot"),
    # small DeepSeek-style layer: 2 always-on experts through SharedExpertGating over TopKGating(3)
    "shared_gating": dict(seed=77, T=40, D=64, H=96, O=64, E=10, gate=("shared", 3, 2), z=0.001, init="normal"),
    # MoEConfig.num_shared_experts path (forward_with_shared_experts)
    "layer_blend": dict(seed=78, T=24, D=64, H=96, O=48, E=6, gate=("topk", 2), z=0.001, init="normal",
                        num_shared_experts=2),
    # Switch (top-1) gating with gelu
    "switch_gelu": dict(seed=79, T=33, D=48, H=80, O=48, E=4, gate=("switch", 1), z=0.0, init="normal",
                        activation="gelu"),
    # StandardExpert (bias + gelu), the MoEConfig default expert type
    "standard_gelu": dict(seed=80, T=37, D=48, H=72, O=40, E=6, gate=("topk", 2), z=0.001, init="normal",
                          activation="gelu", expert_kind="standard"),
    # drop_tokens with capacity_factor 1.0: late pairs of popular experts are dropped, gates renormalised
    "capacity": dict(seed=81, T=90, D=32, H=48, O=32, E=4, gate=("topk", 2), z=0.001, init="normal",
                     drop_tokens=True, capacity_factor=1.0),
    # training-time router noise through the noise network: logits + 0.5 * (randn .* softplus(noise_weight x))
    "noise_net": dict(seed=82, T=50, D=40, H=48, O=32, E=8, gate=("topk", 2), z=0.001, init="normal",
                      noise_scale=0.5, noise_net=True),
}


def build(case):
    c = CASES[case]
    E = c["E"]
    nsh = c.get("num_shared_experts", 0)
    x, w = orc.make_layer_inputs(c["seed"], c["T"], c["D"], c["H"], c["O"], E, e_router=E - nsh,
                                 init=c["init"], std=0.3 if c["init"] == "normal" else 0.02,
                                 expert_kind=c.get("expert_kind", "gated"))
    noise = None
    if c.get("noise_scale", 0) > 0:
        rng = np.random.Generator(np.random.PCG64(c["seed"] + 1000))
        noise = rng.standard_normal((c["T"], E - nsh), dtype=np.float32)
        if c.get("noise_net"):
            w.noise_weight = rng.standard_normal((E - nsh, c["D"]), dtype=np.float32) * np.float32(0.3)
    g = c["gate"]
    if g[0] == "topk":
        gate = orc.TopKGating(g[1])
    elif g[0] == "switch":
        gate = orc.SwitchGating()
    else:
        gate = orc.SharedExpertGating(g[2], orc.TopKGating(g[1]), E)
    cfg = orc.MoEConfig(num_experts=E, input_dim=c["D"], hidden_dim=c["H"], output_dim=c["O"],
                        activation=c.get("activation", "silu"), gate_type=gate, balance_alpha=0.01,
                        z_loss_weight=c["z"], num_shared_experts=nsh, drop_tokens=c.get("drop_tokens", False),
                        capacity_factor=c.get("capacity_factor", 1.25), noise_scale=c.get("noise_scale", 0.0),
                        router_noise=noise)
    return c, cfg, x, w


def run_case(case):
    c, cfg, x, w = build(case)
    out, loss, aux = orc.moe_layer_forward(cfg, w, x, training=True)
    return dict(out=out, loss=np.float32(loss), indices=aux["indices"].astype(np.int32), gates=aux["gates"],
                probs=aux["probs"], logits=aux["logits"])


if __name__ == "__main__":
    for name in CASES:
        r = run_case(name)
        np.savez_compressed(os.path.join(HERE, f"{name}.npz"), **r)
        print(name, {k: getattr(v, "shape", v) for k, v in r.items()}, "loss", float(r["loss"]))
