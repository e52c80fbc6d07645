"""Failure handling in the forms that fault no GPU: bounded waits that are made to run out.

(1) The wait routine of the tensor-core kernels gives up after its limit and records a status
    code (a one-thread kernel waits on an mbarrier nobody arrives on).
(2) Expert parallel, 2+ GPUs: a rank that stays away from a forward call -- it leaves between
    steps, with nothing of its own in flight -- costs the other rank MOE_ERR_TIMEOUT after the
    configured deadline, the GPU stays usable, and the handle refuses further expert-parallel
    calls with MOE_ERR_STATE."""
import ctypes as C
import os
import sys
import time

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("limit_us", [1000, 20000])
def test_bounded_wait_gives_up_and_reports(limit_us):
    from mixtureofexperts_b200 import _lib

    st, waited = C.c_int32(-1), C.c_int32(-1)
    t0 = time.perf_counter()
    _lib.check(_lib.lib.moe_selftest_bounded_wait(0, limit_us, C.byref(st), C.byref(waited)))
    assert st.value == 1                                   # DEV_TIMEOUT_TMA_FULL
    assert limit_us <= waited.value < limit_us + 5000      # gave up right after the limit
    assert time.perf_counter() - t0 < 5.0
    # the context is still usable
    assert float(torch.ones(8, device="cuda").sum().item()) == 8.0
    assert _lib.lib.moe_selftest_bounded_wait(0, 0, C.byref(st), C.byref(waited)) == _lib.ERR_INVALID


def _absent_rank_main(rank, world, port, mode, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    os.environ["MOE_B200_EP_MODE"] = mode
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import mixtureofexperts_b200 as m
        from helpers import device_gate, make_device_layer, rel_inf
        from mixtureofexperts_b200 import _lib, parallel
        from oracle import moe_oracle as orc

        E, k, T, D, H, O = 8, 2, 64, 128, 256, 128
        x_all, w = orc.make_layer_inputs(77, T * world, D, H, O, E, init="normal", std=0.25)
        uid = parallel.broadcast_unique_id(dist, rank, None)
        cfg = m.create_moe_config(num_experts=E, expert_type="gated", input_dim=D, hidden_dim=H, output_dim=O,
                                  activation=m.silu, gate_type=m.TopKGating(k),
                                  balance_loss=m.SwitchTransformerLoss(0.01), z_loss_weight=0.001)
        experts = []
        for e in w.experts:
            ex = m.GatedExpert.__new__(m.GatedExpert)
            ex.input_dim, ex.hidden_dim, ex.output_dim, ex.activation = D, H, O, m.silu
            ex.w1, ex.w2, ex.w3 = e.w1, e.w2, e.w3
            experts.append(ex)
        router = m.Router.__new__(m.Router)
        router.weight, router.noise_weight, router.gate_type, router.noise_scale, router.use_fp32 = w.router, None, cfg.gate_type, 0.0, True
        layer = m.MoELayer(cfg, device=rank, compute_dtype="f32", experts=experts, router=router,
                           expert_parallel=(rank, world, uid))
        _lib.check(_lib.lib.moe_ep_set_timeout_ms(layer._handle, 1500))
        xt = torch.from_numpy(x_all[rank * T:(rank + 1) * T]).cuda()
        for _ in range(2):                      # everybody takes part: fine
            layer(xt.t(), training=True)
        torch.cuda.synchronize()
        assert layer.device_status() == 0
        dist.barrier()
        if rank == 0:
            t0 = time.perf_counter()
            code = None
            try:
                layer(xt.t(), training=True)    # the other ranks stay away from this call
                torch.cuda.synchronize()
            except m.MoEError as exc:
                code = exc.code
            waited = time.perf_counter() - t0
            # the GPU still answers and computes: a single-device layer against the oracle
            single = make_device_layer(w, D=D, H=H, O=O, gate=device_gate("topk", k))
            out, _ = single(xt.t(), training=False)
            cfg_o = orc.MoEConfig(num_experts=E, input_dim=D, hidden_dim=H, output_dim=O, activation="silu",
                                  gate_type=orc.TopKGating(k))
            ref, _, _ = orc.moe_layer_forward(cfg_o, w, x_all[:T], training=False)
            err = rel_inf(out.cpu().numpy().T, ref)
            single.close()
            code2 = None
            try:
                layer(xt.t(), training=True)    # the group is unusable from here on
            except m.MoEError as exc:
                code2 = exc.code
            q.put((rank, code, waited, err, code2))
        dist.barrier()                          # the absent ranks learn on the host that the call is over
        if rank != 0:
            q.put((rank, "absent", 0.0, 0.0, None))
        layer.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["peer", "nccl"])
def test_a_rank_that_stays_away_costs_a_timeout_and_leaves_the_gpu_usable(mode):
    from mixtureofexperts_b200 import _lib

    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29900 + (os.getpid() % 90) + (3 if mode == "nccl" else 0)
    procs = [ctx.Process(target=_absent_rank_main, args=(r, world, port, mode, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=240)
        assert p.exitcode == 0
    results = dict((r[0], r[1:]) for r in (q.get(timeout=5) for _ in range(world)))
    code, waited, err, code2 = results[0]
    assert code == _lib.ERR_TIMEOUT, code
    assert 1.0 < waited < 30.0, waited
    assert err < 1e-5
    assert code2 == _lib.ERR_STATE
