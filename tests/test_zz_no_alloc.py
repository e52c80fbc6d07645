"""moe_route_static: routing for callers that may not allocate device memory.

Some users of the library run with every byte of GPU memory already handed to their own pools,
or inside loops where the device-wide synchronisation of cudaMalloc/cudaFree is not acceptable.
For them the library offers one entry point whose scratch is a fixed device array inside the
library itself.  This test calls it through the C ABI twice in a row (the second call reuses
the array with the first call's leftovers in it, at a different size) and checks indices, gates,
probabilities and loss against what moe_layer_forward returns for the same inputs.

The file name sorts last on purpose: a run that stops at the first failure has then already
run every other test."""
import ctypes as C
import os
import sys

import numpy as np
import pytest
import torch

sys.path.insert(0, os.path.dirname(__file__))
from helpers import device_gate, make_device_layer  # noqa: E402
from oracle import moe_oracle as orc  # noqa: E402

pytestmark = pytest.mark.gpu


def _route_static(lib, kind, E, S, k, x, router, alpha, z):
    T, D = x.shape
    k_tot = k + S
    idx = torch.full((T, k_tot), -7, dtype=torch.int32, device="cuda")
    gates = torch.full((T, k_tot), -1.0, dtype=torch.float32, device="cuda")
    probs = torch.full((T, E), -1.0, dtype=torch.float32, device="cuda")
    loss = torch.full((1,), -1.0, dtype=torch.float32, device="cuda")
    xd = 1 if x.dtype == torch.bfloat16 else 0
    rc = lib.lib.moe_route_static(kind, E, S, k, 1, x.data_ptr(), xd, T, D, router.data_ptr(), None, alpha, z, 1,
                                  idx.data_ptr(), gates.data_ptr(), probs.data_ptr(), loss.data_ptr(),
                                  torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.lib.moe_route_static_error().decode()
    torch.cuda.synchronize()
    return idx, gates, probs, loss


@pytest.mark.parametrize("gate_kind,E,S,k", [("topk", 8, 0, 2), ("shared", 18, 2, 6)])
def test_route_static_matches_layer_forward_twice_in_a_row(gate_kind, E, S, k):
    from mixtureofexperts_b200 import _lib

    D, H, O = 96, 64, 48
    kind = _lib.GATE_SHARED_TOPK if gate_kind == "shared" else _lib.GATE_TOPK
    for call, T in enumerate((777, 130)):       # two calls in a row, sharing the static array
        x, w = orc.make_layer_inputs(500 + call, T, D, H, O, E, init="normal", std=0.25)
        layer = make_device_layer(w, D=D, H=H, O=O, gate=device_gate(gate_kind, k, S, E), alpha=0.01, z=0.001)
        xt = torch.from_numpy(x).cuda()
        _, ref_loss, ref = layer(xt.t(), training=True, return_routing=True)
        router = torch.from_numpy(w.router).cuda()
        idx, gates, probs, loss = _route_static(_lib, kind, E, S, k, xt, router, 0.01, 0.001)
        assert torch.equal(idx, ref["indices"].t())
        # same kernels, same inputs: equal to the last bit; the 1e-5 of the other tests is the bound
        assert (gates - ref["gates"].t()).abs().max().item() <= 1e-5
        assert (probs - ref["probs"].t()).abs().max().item() <= 1e-5
        assert abs(loss.item() - ref_loss.item()) <= 1e-5 * abs(ref_loss.item())
        layer.close()


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
