"""moe_route_static: routing for callers that may not allocate device memory.

Some users of the library run with every byte of GPU memory already handed to their own pools,
or inside loops where the device-wide synchronisation of cudaMalloc/cudaFree is not acceptable.
For them the library offers one entry point whose scratch is a fixed device array inside the
library itself.  These tests call it through the C ABI, always twice in a row (the second call
reuses the array with the first call's leftovers in it, at a different size), and check indices,
gates, probabilities and loss against the CPU oracle of the reference's router
(Router call -> compute_gates -> SwitchTransformerLoss + ZLoss) and against what
moe_layer_forward returns for the same inputs.

The file name sorts last on purpose: a run that stops at the first failure has then already
run every other test."""
import os
import sys

import numpy as np
import pytest
import torch

sys.path.insert(0, os.path.dirname(__file__))
from helpers import check_indices, device_gate, make_device_layer, oracle_gate, rel_inf  # noqa: E402
from oracle import moe_oracle as orc  # noqa: E402

pytestmark = pytest.mark.gpu

ALPHA, Z = 0.01, 0.001


def _route_static(lib, kind, E, S, k, x, router, *, bias=None, training=1, index_base=1, want_probs=True,
                  want_loss=True):
    T, D = x.shape
    k_tot = k + S
    idx = torch.full((T, k_tot), -7, dtype=torch.int32, device="cuda")
    gates = torch.full((T, k_tot), -1.0, dtype=torch.float32, device="cuda")
    probs = torch.full((T, E), -1.0, dtype=torch.float32, device="cuda") if want_probs else None
    loss = torch.full((1,), -1.0, dtype=torch.float32, device="cuda") if want_loss else None
    xd = 1 if x.dtype == torch.bfloat16 else 0
    rc = lib.lib.moe_route_static(kind, E, S, k, index_base, x.data_ptr(), xd, T, D, router.data_ptr(),
                                  bias.data_ptr() if bias is not None else None, ALPHA, Z, training,
                                  idx.data_ptr(), gates.data_ptr(), probs.data_ptr() if want_probs else None,
                                  loss.data_ptr() if want_loss else None, torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.lib.moe_route_static_error().decode()
    torch.cuda.synchronize()
    return idx, gates, probs, loss


def _oracle_route(gate_kind, E, S, k, D, x, w, bias):
    """The reference's router on the CPU: indices (1-based), gates, probs, Switch + z loss, and the
    float64 logits the tie rule is judged on."""
    cfg = orc.MoEConfig(num_experts=E, input_dim=D, hidden_dim=8, output_dim=8, activation="silu",
                        gate_type=oracle_gate(gate_kind, k, S, E), balance_alpha=ALPHA, z_loss_weight=Z,
                        router_bias=bias)
    idx, gates, probs, logits = orc.router_forward(cfg, w, x)
    loss = np.float32(orc.switch_transformer_loss(ALPHA, idx, probs) + orc.z_loss(Z, logits))
    logits64 = x.astype(np.float64) @ w.router.astype(np.float64).T
    if bias is not None:
        logits64 = logits64 + bias.astype(np.float64)
    return idx, gates, probs, loss, logits64


@pytest.mark.parametrize("gate_kind,E,S,k", [("topk", 8, 0, 2), ("shared", 18, 2, 6), ("switch", 8, 0, 1)])
@pytest.mark.parametrize("variant", ["plain", "bias", "bf16_x"])
def test_route_static_matches_oracle_and_layer_twice_in_a_row(gate_kind, E, S, k, variant):
    from mixtureofexperts_b200 import _lib

    D, H, O = 96, 64, 48
    kind = {"topk": _lib.GATE_TOPK, "shared": _lib.GATE_SHARED_TOPK, "switch": _lib.GATE_SWITCH}[gate_kind]
    for call, T in enumerate((777, 130)):       # two calls in a row, sharing the static array
        x, w = orc.make_layer_inputs(500 + call, T, D, H, O, E, init="normal", std=0.25, bf16=variant == "bf16_x")
        bias = None
        if variant == "bias":
            bias = (np.random.default_rng(7 + call).standard_normal(E) * 0.7).astype(np.float32)
            bias[:S] = 0
        o_idx, o_gates, o_probs, o_loss, logits64 = _oracle_route(gate_kind, E, S, k, D, x, w, bias)
        xt = torch.from_numpy(x).cuda()
        if variant == "bf16_x":
            xt = xt.to(torch.bfloat16)           # exact: the values are bfloat16-representable
        router = torch.from_numpy(w.router).cuda()
        bias_t = torch.from_numpy(bias).cuda() if bias is not None else None
        idx, gates, probs, loss = _route_static(_lib, kind, E, S, k, xt, router, bias=bias_t)
        # against the oracle: ids exact unless the float64 logits tie within 1e-6; FP32 values within 1e-5
        excused = check_indices(idx.cpu().numpy(), o_idx, logits64, k, r0=S)
        same = (idx.cpu().numpy() == o_idx).all(axis=1)
        assert excused == int((~same).sum())
        assert rel_inf(gates.cpu().numpy()[same], o_gates[same]) <= 1e-5
        assert rel_inf(probs.cpu().numpy(), o_probs) <= 1e-5
        assert abs(loss.item() - float(o_loss)) <= 1e-5 * abs(float(o_loss))
        # against the allocating entry point: the same router kernel on the same inputs gives every
        # token the same bits (a token's logits do not depend on the token tile); the loss is summed
        # over differently sized token tiles, so it agrees to rounding only
        layer = make_device_layer(w, D=D, H=H, O=O, gate=device_gate(gate_kind, k, S, E), alpha=ALPHA, z=Z,
                                  router_bias=bias)
        _, ref_loss, ref = layer(xt.t(), training=True, return_routing=True)
        assert torch.equal(idx, ref["indices"].t())
        assert torch.equal(gates, ref["gates"].t())
        assert torch.equal(probs, ref["probs"].t())
        assert abs(loss.item() - ref_loss.item()) <= 1e-6 * abs(ref_loss.item())
        layer.close()


def test_route_static_inference_null_outputs_and_zero_based_ids():
    """training == 0 writes a loss of exactly 0; probs and loss may be NULL; index_base 0 gives 0-based ids."""
    from mixtureofexperts_b200 import _lib

    E, k, D = 8, 2, 64
    for call, T in enumerate((300, 65)):
        x, w = orc.make_layer_inputs(900 + call, T, D, 16, 16, E, init="normal", std=0.25)
        o_idx, o_gates, _, _, logits64 = _oracle_route("topk", E, 0, k, D, x, w, None)
        xt, router = torch.from_numpy(x).cuda(), torch.from_numpy(w.router).cuda()
        idx, gates, probs, loss = _route_static(_lib, _lib.GATE_TOPK, E, 0, k, xt, router, training=0)
        assert loss.item() == 0.0
        check_indices(idx.cpu().numpy(), o_idx, logits64, k)
        idx0, gates0, probs0, loss0 = _route_static(_lib, _lib.GATE_TOPK, E, 0, k, xt, router, index_base=0,
                                                    want_probs=False, want_loss=False)
        assert probs0 is None and loss0 is None
        assert torch.equal(idx0 + 1, idx) and torch.equal(gates0, gates)
        assert rel_inf(gates.cpu().numpy(), o_gates) <= 1e-5


def test_route_static_rejects_sizes_beyond_its_array():
    from mixtureofexperts_b200 import _lib

    cap = _lib.lib.moe_route_static_scratch_bytes()
    assert cap == 8 << 20
    E, D = 128, 16
    T = 1 << 20          # 1M tokens x 128 experts needs far more than 8 MiB of per-CTA rows
    x = torch.zeros((8, D), device="cuda")
    w = torch.zeros((E, D), device="cuda")
    i = torch.zeros((8, 2), dtype=torch.int32, device="cuda")
    g = torch.zeros((8, 2), device="cuda")
    rc = _lib.lib.moe_route_static(_lib.GATE_TOPK, E, 0, 2, 1, x.data_ptr(), 0, T, D, w.data_ptr(), None, 0.01, 0.0, 0,
                                   i.data_ptr(), g.data_ptr(), None, None, None)
    assert rc == _lib.ERR_INVALID
    assert b"static array holds" in _lib.lib.moe_route_static_error()
