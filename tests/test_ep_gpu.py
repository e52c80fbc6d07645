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


def _rank_main(rank, world, port, compute, mode, E, k, T, D, H, O, q, host_call=False, std=None):
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
        x_all, w = orc.make_layer_inputs(321, T * world, D, H, O, E, init="normal",
                                         std=std if std is not None else (0.05 if bf16 else 0.25), bf16=bf16)
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
        xt = torch.from_numpy(x_all[rank * T:(rank + 1) * T])
        if bf16:
            xt = xt.to(torch.bfloat16)
        if host_call:
            xt = xt.pin_memory()        # host buffers: moe_layer_forward_host, chunked for large batches
        else:
            xt = xt.cuda()
        # A small call first: it sizes the receive buffers for 40 tokens per rank, so the first full call
        # has to grow them (a collective re-exchange of the buffers' IPC handles); the second reuses them.
        layer(xt[:40].t(), training=True)
        torch.cuda.synchronize()
        errs = []
        for it in range(2):
            out, loss, routing = layer(xt.t(), training=True, return_routing=True)
            torch.cuda.synchronize()
            assert layer.device_status() == 0
            assert np.array_equal(np.asarray(routing["indices"].cpu() if hasattr(routing["indices"], "cpu") else routing["indices"]).T,
                                  aux["indices"][rank * T:(rank + 1) * T])
            errs.append(rel_inf(np.asarray(out.cpu() if hasattr(out, "cpu") else out).T, ref_out[rank * T:(rank + 1) * T]))
            lerr = abs(float(loss) - float(ref_loss)) / abs(float(ref_loss))
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


def _run(world, args, timeout=600):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank_main, args=(r, world) + args[:9] + (q,) + args[9:]) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=timeout)
        assert p.exitcode == 0
    return sorted(q.get(timeout=5) for _ in range(world))


def test_expert_parallel_at_mixtral_widths():
    """d_model 4096 / ffn 14336 (the widths of the expert-parallel benchmark layer), 4 experts over 2 GPUs,
    a few hundred tokens per rank, BF16 tensor-core path, against the single-device oracle."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    port = 29700 + (os.getpid() % 200)
    for _, err, lerr in _run(2, (port, "bf16", "peer", 4, 2, 300, 4096, 14336, 4096, False, 0.02), timeout=900):
        assert err < 2e-2, err
        assert lerr < 1e-5, lerr


@pytest.mark.parametrize("compute,tol", [("f32", 1e-5), ("bf16", 2e-2)])
def test_expert_parallel_host_buffers_chunked(compute, tol):
    """moe_layer_forward_host under expert parallelism with a batch large enough to be cut into
    chunks: every chunk is a collective; outputs, ids and the loss over all ranks' tokens must
    not change."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    port = 29750 + (os.getpid() % 200) + (5 if compute == "bf16" else 0)
    for _, err, lerr in _run(2, (port, compute, "peer", 8, 2, 8300, 128, 256, 128, True)):
        assert err < tol, err
        assert lerr < 1e-5, lerr
