"""Expert-parallel layer on 2+ GPUs (skipped on a single-GPU box): every rank runs
moe_layer_forward with NCCL dispatch/combine on its own tokens; the result must equal the
single-device oracle on the concatenated batch."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

pytestmark = pytest.mark.gpu


def _rank_main(rank, world, port, compute, mode, E, k, T, D, H, O, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    os.environ["MOE_B200_EP_MODE"] = mode   # "peer": rows cross NVLink inside permute/combine; "nccl": send/recv
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import mixtureofexperts_b200 as m
        from helpers import rel_inf
        from mixtureofexperts_b200 import parallel
        from oracle import moe_oracle as orc

        bf16 = compute == "bf16"
        x_all, w = orc.make_layer_inputs(321, T * world, D, H, O, E, init="normal", std=0.05 if bf16 else 0.25, bf16=bf16)
        cfg_o = orc.MoEConfig(num_experts=E, input_dim=D, hidden_dim=H, output_dim=O, activation="silu",
                              gate_type=orc.TopKGating(k), balance_alpha=0.01, z_loss_weight=0.001)
        ref_out, ref_loss, aux = orc.moe_layer_forward(cfg_o, w, x_all, training=True)

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
        layer = m.MoELayer(cfg, device=rank, compute_dtype=compute, experts=experts, router=router,
                           expert_parallel=(rank, world, uid))
        xt = torch.from_numpy(x_all[rank * T:(rank + 1) * T]).cuda()
        if bf16:
            xt = xt.to(torch.bfloat16)
        # A small call first: it sizes the receive buffers for 40 tokens per rank, so the first full call
        # has to grow them (a collective re-exchange of the buffers' IPC handles); the second reuses them.
        layer(xt[:40].t(), training=True)
        torch.cuda.synchronize()
        errs = []
        for it in range(2):
            out, loss, routing = layer(xt.t(), training=True, return_routing=True)
            torch.cuda.synchronize()
            assert layer.device_status() == 0
            assert np.array_equal(routing["indices"].cpu().numpy().T, aux["indices"][rank * T:(rank + 1) * T])
            errs.append(rel_inf(out.cpu().numpy().T, ref_out[rank * T:(rank + 1) * T]))
            lerr = abs(float(loss.item()) - float(ref_loss)) / abs(float(ref_loss))
        q.put((rank, max(errs), lerr))
        layer.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["peer", "nccl"])
@pytest.mark.parametrize("compute,tol", [("f32", 1e-5), ("bf16", 2e-2)])
def test_expert_parallel_forward_matches_single_device_oracle(compute, tol, mode):
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    if world == 3:
        world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + (os.getpid() % 300) + (7 if mode == "peer" else 0) + (13 if compute == "bf16" else 0)
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, compute, mode, 8, 2, 333, 128, 256, 128, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
        assert p.exitcode == 0
    results = sorted(q.get(timeout=5) for _ in range(world))
    for _, err, lerr in results:
        assert err < tol, err
        assert lerr < 1e-5, lerr
