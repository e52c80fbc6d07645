#!/usr/bin/env python
"""MoE-layer forward benchmark: tokens/s of MoELayer(config)(x; training=true) on B200.

    python bench.py --gpus 1 --steps 20 --warmup 5              # Mixtral-shaped layer, 1 GPU
    torchrun --nproc-per-node N ... bench.py --gpus N ...       # expert-parallel layer, N GPUs
    python bench.py --impl reference ...                        # the CPU restatement of the
                                                                # reference path on the host cores

One step = one forward of the layer over one batch of synthetic tokens (router -> top-k ->
permute -> grouped GatedExpert GEMMs -> combine -> Switch loss + z-loss).  Rank 0 prints ONE
JSON line.  Workloads (synthetic stand-ins with the shapes and value distributions of the
benchmark configurations; weights N(0, 0.02^2), activations N(0, 1), seeded):
  c3  8 experts, d_model 4096, ffn 14336, top-2, BF16, 16384 tokens            (default at N=1)
  c5  64 experts over N GPUs, same widths, top-2, BF16, 8192 tokens per GPU    (default at N>1)
  c4  64 routed + 2 shared experts, d 2048, hidden 1408, top-6, 32768 tokens, skewed routing
  c1  8 experts 512/2048/512, top-2, FP32, 32 tokens
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    "c3": dict(E=8, S=0, k=2, D=4096, H=14336, O=4096, T=16384, dtype="bf16", std=0.02, bias_std=0.0,
               desc="Mixtral-shaped layer: 8 GatedExperts d_model=4096 ffn=14336 top-2 BF16, 16384 tokens"),
    "c5": dict(E=64, S=0, k=2, D=4096, H=14336, O=4096, T=8192, dtype="bf16", std=0.02, bias_std=0.0,
               desc="expert-parallel Mixtral-shaped layer: 64 experts over the GPUs, top-2 BF16, 8192 tokens per GPU"),
    "c4": dict(E=66, S=2, k=6, D=2048, H=1408, O=2048, T=32768, dtype="bf16", std=0.02, bias_std=1.5,
               desc="DeepSeek-style layer: 64 routed + 2 shared GatedExperts d=2048 hidden=1408 top-6 BF16, 32768 tokens, skewed"),
    "c1": dict(E=8, S=0, k=2, D=512, H=2048, O=512, T=32, dtype="f32", std=0.05, bias_std=0.0,
               desc="8 GatedExperts 512/2048/512 top-2 FP32, 32 tokens"),
}
SEED = 1234


def expert_flops(w, tokens):
    """Algorithmic FLOPs of the expert GEMMs: 2*H*(2D+O) per (token, expert) pair."""
    return 2.0 * w["H"] * (2 * w["D"] + w["O"]) * tokens * (w["k"] + w["S"])


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=p["hbm_gbs"], bf16_tflops=p["bf16_tflops"],
                    bf16_tflops_sustained=p.get("bf16_tflops_sustained", p["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clock, power and throttle reasons of one GPU through NVML from a thread while
    the timed region runs (the same quantities `nvidia-smi --query-gpu=clocks.sm,...` prints)."""

    def __init__(self, uuid: str):
        self.uuid = uuid
        self.samples = []
        self.stop_flag = threading.Event()
        self.thread = None
        self.err = None

    def start(self):
        try:
            import pynvml

            pynvml.nvmlInit()
            u = self.uuid if self.uuid.startswith("GPU-") else "GPU-" + self.uuid
            self.handle = pynvml.nvmlDeviceGetHandleByUUID(u.encode() if hasattr(u, "encode") else u)
            self.nv = pynvml
        except Exception as exc:  # noqa: BLE001
            self.err = f"NVML unavailable: {exc}"
            return
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.thread.start()

    def _run(self):
        nv = self.nv
        try:
            mx = nv.nvmlDeviceGetMaxClockInfo(self.handle, nv.NVML_CLOCK_SM)    # constant: asked once
        except Exception as exc:  # noqa: BLE001
            self.err = str(exc)
            return
        while not self.stop_flag.is_set():
            try:
                sm = nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM)
                pw = nv.nvmlDeviceGetPowerUsage(self.handle) / 1000.0
                rs = nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle) if hasattr(
                    nv, "nvmlDeviceGetCurrentClocksEventReasons") else nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                self.samples.append((time.perf_counter(), sm, mx, pw, rs))
            except Exception as exc:  # noqa: BLE001
                self.err = str(exc)
                return
            time.sleep(0.002)

    def mark(self):
        return time.perf_counter()

    def stop(self, t0=None, t1=None):
        self.stop_flag.set()
        if self.thread:
            self.thread.join(timeout=2)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [self.err or "no samples"]}
        sel = [s for s in self.samples if (t0 is None or s[0] >= t0) and (t1 is None or s[0] <= t1)] or self.samples
        sm = sorted(s[1] for s in sel)
        bits = 0
        for s in sel:
            bits |= int(s[4])
        # NVML clocks-event-reason bits
        names = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap",
                 0x80: "hw_power_brake_slowdown", 0x2: "applications_clocks_setting", 0x100: "display_clock_setting"}
        reasons = sorted(n for b, n in names.items() if bits & b)
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": max(s[2] for s in sel), "power_w_max": max(s[3] for s in sel),
                "samples": len(sel), "reasons": reasons}


def make_expert_factory(w, torch, device):
    """Expert e's weights are a pure function of (SEED, e), so every rank draws the same expert."""
    import mixtureofexperts_b200 as m

    dt = torch.bfloat16 if w["dtype"] == "bf16" else torch.float32

    def factory(e):
        g = torch.Generator(device=device).manual_seed(SEED * 1000 + e)
        ex = m.GatedExpert.__new__(m.GatedExpert)
        ex.input_dim, ex.hidden_dim, ex.output_dim, ex.activation = w["D"], w["H"], w["O"], m.silu
        mk = lambda o, i: (torch.randn((o, i), device=device, generator=g, dtype=torch.float32) * w["std"]).to(dt)
        ex.w1 = mk(w["H"], w["D"])
        ex.w3 = mk(w["H"], w["D"])
        ex.w2 = mk(w["O"], w["H"])
        return ex

    return factory


def make_router(w, torch, device):
    import mixtureofexperts_b200 as m

    g = torch.Generator(device=device).manual_seed(SEED)
    r = m.Router.__new__(m.Router)
    r.weight = torch.randn((w["E"], w["D"]), device=device, generator=g, dtype=torch.float32) * w["std"]
    r.noise_weight, r.noise_scale, r.use_fp32 = None, 0.0, True
    if w["bias_std"] > 0:
        b = torch.randn((w["E"],), device=device, generator=g, dtype=torch.float32) * w["bias_std"]
        b[: w["S"]] = 0
        r.bias = b
    return r


def build_layer(w, torch, device_index, ep=None):
    import mixtureofexperts_b200 as m

    device = f"cuda:{device_index}"
    gate = m.SharedExpertGating(w["S"], m.TopKGating(w["k"]), w["E"]) if w["S"] else m.TopKGating(w["k"])
    cfg = m.create_moe_config(num_experts=w["E"], expert_type="gated", input_dim=w["D"], hidden_dim=w["H"],
                              output_dim=w["O"], activation=m.silu, gate_type=gate,
                              balance_loss=m.SwitchTransformerLoss(0.01), z_loss_weight=0.001)
    router = make_router(w, torch, device)
    router.gate_type = gate
    return m.MoELayer(cfg, device=device_index, compute_dtype=w["dtype"], experts=make_expert_factory(w, torch, device),
                      router=router, expert_parallel=ep)


def cpu_forward_rate(w, tokens, steps, warmup, threads_note=True):
    """Times the CPU restatement of the reference path (the oracle) on `tokens` tokens of the
    workload.  Returns (tokens/s, cores used, seconds per step)."""
    import numpy as np

    from oracle import moe_oracle as orc

    rng = np.random.Generator(np.random.PCG64(SEED))
    E, D, H, O = w["E"], w["D"], w["H"], w["O"]
    x = rng.standard_normal((tokens, D), dtype=np.float32)
    router = rng.standard_normal((E, D), dtype=np.float32) * np.float32(w["std"])
    experts = []
    for _ in range(E):
        experts.append(orc.GatedExpertWeights(
            w1=rng.standard_normal((H, D), dtype=np.float32) * np.float32(w["std"]),
            w2=rng.standard_normal((O, H), dtype=np.float32) * np.float32(w["std"]),
            w3=rng.standard_normal((H, D), dtype=np.float32) * np.float32(w["std"])))
    gate = orc.SharedExpertGating(w["S"], orc.TopKGating(w["k"]), E) if w["S"] else orc.TopKGating(w["k"])
    bias = None
    if w["bias_std"] > 0:
        bias = (rng.standard_normal(E) * w["bias_std"]).astype(np.float32)
        bias[: w["S"]] = 0
    cfg = orc.MoEConfig(num_experts=E, input_dim=D, hidden_dim=H, output_dim=O, activation="silu", gate_type=gate,
                        balance_alpha=0.01, z_loss_weight=0.001, router_bias=bias)
    weights = orc.MoEWeights(router=router, experts=experts)
    for _ in range(warmup):
        orc.moe_layer_forward(cfg, weights, x, training=True)
    t0 = time.perf_counter()
    for _ in range(steps):
        orc.moe_layer_forward(cfg, weights, x, training=True)
    dt = (time.perf_counter() - t0) / max(steps, 1)
    return tokens / dt, os.cpu_count() or 1, dt


def run_reference_arm(args, w, name):
    """--impl reference: the reference's CPU path (its NumPy/OpenBLAS restatement; the Julia
    original cannot run without a Julia runtime) on all host cores, a bounded sample per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sample = min(w["T"], 1024 if w["dtype"] == "bf16" else w["T"])
    rate, cores, dt = cpu_forward_rate(w, sample, args.steps, max(args.warmup, 1))
    line = {
        "impl": "reference", "metric": "moe_layer_tokens_per_s", "value": rate, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{name}: {w['desc']}", "note": "CPU path, FP32 (OpenBLAS), host cores only"},
        "cpu_baseline": {"value": rate, "unit": "tokens/s", "cores": cores, "kind": "port",
                         "sample": f"{sample} tokens per step of the same layer (all {w['E']} experts, full widths)"},
        "e2e": {"value": rate, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="auto", choices=["auto"] + sorted(WORKLOADS))
    ap.add_argument("--tokens", type=int, default=0, help="override the tokens per GPU (profiling of small cases)")
    ap.add_argument("--experts", type=int, default=0, help="override the expert count (profiling of small cases)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3  # timing rule: at least 3 warm-up steps

    name = args.workload if args.workload != "auto" else ("c3" if args.gpus == 1 else "c5")
    w = dict(WORKLOADS[name])
    if args.tokens > 0:
        w["T"] = args.tokens
    if args.experts > 0:
        w["E"] = args.experts
        w["desc"] += f" [experts overridden to {args.experts}]"
    if args.impl == "reference":
        run_reference_arm(args, w, name)
        return

    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun --nproc-per-node {args.gpus}")
    torch.cuda.set_device(local_rank)
    device = f"cuda:{local_rank}"
    ep = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device(device))
        from mixtureofexperts_b200 import parallel

        uid = parallel.broadcast_unique_id(dist, rank, device)
        ep = (rank, world, uid)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()

    layer = build_layer(w, torch, local_rank, ep)
    T, D, O = w["T"], w["D"], w["O"]
    xdt = torch.bfloat16 if w["dtype"] == "bf16" else torch.float32
    gx = torch.Generator(device=device).manual_seed(SEED + 7 + rank)
    x = torch.randn((T, D), device=device, generator=gx, dtype=torch.float32).to(xdt)
    out = torch.empty((T, O), device=device, dtype=torch.float32)

    def step():
        return layer(x.t(), training=True, out=out)

    # ---- device-resident throughput ---------------------------------------------------------
    for _ in range(args.warmup):
        step()
    barrier()
    layer.set_profiling(min(args.steps, 1024))
    sampler = ClockSampler(str(torch.cuda.get_device_properties(local_rank).uuid))
    if rank == 0:
        sampler.start()
    launches0 = layer.launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t_mark0 = sampler.mark()
    ev0.record()
    for _ in range(args.steps):
        _, loss = step()
    ev1.record()
    barrier()
    t_mark1 = sampler.mark()
    ms_total = ev0.elapsed_time(ev1)
    clocks = sampler.stop(t_mark0, t_mark1) if rank == 0 else None
    launches = layer.launch_count() - launches0
    status = layer.device_status()
    if world > 1:
        t = torch.tensor([ms_total], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_step = ms_total / args.steps
    value = T * world / (ms_step * 1e-3)

    # per-stage device times of the timed steps (CUDA events on the launching stream)
    n_prof = min(args.steps, 1024)
    stages = {}
    for back in range(n_prof):
        for k_, v in layer.stage_ms(back).items():
            stages[k_] = stages.get(k_, 0.0) + v / n_prof
    layer.set_profiling(0)
    loss_value = float(loss.item())
    output_finite = bool(torch.isfinite(out).all().item())   # the timed steps produced real numbers

    # ---- end to end through the host entry point ---------------------------------------------
    e2e = None
    if not args.no_e2e:
        xh = torch.empty((T, D), dtype=xdt).pin_memory()
        xh.copy_(x)
        oh = torch.empty((T, O), dtype=torch.float32).pin_memory()
        for _ in range(2):
            layer(xh.t(), training=True, out=oh)
        barrier()
        n_e2e = max(3, min(args.steps, 10))
        t0 = time.perf_counter()
        for _ in range(n_e2e):
            layer(xh.t(), training=True, out=oh)   # synchronous: H2D x, forward, D2H output + loss
        torch.cuda.synchronize()
        dt = (time.perf_counter() - t0) / n_e2e
        if world > 1:
            t = torch.tensor([dt], device=device, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dt = float(t.item())
        e2e = {"value": T * world / dt, "unit": "tokens/s", "h2d_bytes_per_step": T * D * xh.element_size(),
               "d2h_bytes_per_step": T * O * 4 + 4, "ms_per_step": dt * 1e3,
               "timing": "host clock around synchronous moe_layer_forward_host calls (pinned buffers), max over ranks"}

    if rank == 0:
        peaks = measured_peaks()
        tokens_local_pairs = T  # per GPU
        f_g1 = 2.0 * w["H"] * 2 * w["D"] * tokens_local_pairs * (w["k"] + w["S"])
        f_g2 = 2.0 * w["H"] * w["O"] * tokens_local_pairs * (w["k"] + w["S"])
        roof = None
        # DRAM bytes of one group_gemm_tc_kernel<1> launch, from an ncu capture of this command at full
        # size (dram__bytes_read.sum + dram__bytes_write.sum, 1 pass; profiles/c3_dram_bytes.md).
        # Algorithmic bytes of the launch: weights 1.879 GB + rows 0.268 GB + h 0.940 GB = 3.087 GB.
        traffic, traffic_note = None, "no ncu capture for this workload size"
        if name == "c3" and args.tokens == 0 and args.experts == 0:
            traffic = 2889976576 + 925794304
            traffic_note = "ncu capture of this workload: 2.890 GB read + 0.926 GB written vs 3.087 GB algorithmic"
        if w["dtype"] == "bf16" and stages.get("gemm1", 0) > 0 and world == 1:
            ach = f_g1 / (stages["gemm1"] * 1e-3) / 1e12
            peak = peaks["bf16_tflops_sustained"]
            gemm_kernel = "group_gemm_tc2_kernel<1>, CTA pairs" if layer.tile_rows(T) == 256 else "group_gemm_tc_kernel<1>"
            roof = {"bound": "tensor", "kernel": gemm_kernel + " (x W1^T, x W3^T, act*up)",
                    "achieved": ach, "peak": peak, "unit": "TFLOP/s", "frac": ach / peak,
                    "peak_source": f"{peaks['source']} sustained cuBLAS bf16 (kernel timed inside a long step); burst {peaks['bf16_tflops']}",
                    "traffic": traffic, "traffic_unit": "bytes per launch",
                    "traffic_note": traffic_note,
                    "gemm2_achieved": f_g2 / (stages["gemm2"] * 1e-3) / 1e12 if stages.get("gemm2", 0) > 0 else None,
                    "layer_frac": expert_flops(w, T) / (ms_step * 1e-3) / 1e12 / peak}
        elif w["dtype"] == "bf16" and world > 1:
            ach = expert_flops(w, T) / (ms_step * 1e-3) / 1e12
            peak = peaks["bf16_tflops_sustained"]
            roof = {"bound": "tensor", "kernel": "whole layer per GPU (expert GEMM FLOPs / step time)",
                    "achieved": ach, "peak": peak, "unit": "TFLOP/s", "frac": ach / peak,
                    "peak_source": f"{peaks['source']} sustained cuBLAS bf16", "traffic": None}
        elif w["dtype"] == "f32":
            nbytes = 4.0 * w["E"] * w["H"] * (2 * w["D"] + w["O"])
            t_g = (stages.get("gemm1", 0) + stages.get("gemm2", 0)) * 1e-3
            if t_g > 0:
                ach = nbytes / t_g / 1e9
                roof = {"bound": "hbm", "kernel": "group_gemm_f32_kernel<1>+<2> (expert weights streamed once)",
                        "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": ach / peaks["hbm_gbs"],
                        "peak_source": peaks["source"], "traffic": None}
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            sample = min(T, 1024 if w["dtype"] == "bf16" else T)
            rate, cores, dt = cpu_forward_rate(w, sample, 2, 1)
            cpu = {"value": rate, "unit": "tokens/s", "cores": cores, "kind": "port",
                   "sample": f"{sample} tokens of the same layer (all {w['E']} experts, full widths), FP32 OpenBLAS, 2 timed passes"}
        line = {
            "metric": "moe_layer_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic",
            "config": {"workload": f"{name}: {w['desc']}", "tokens_per_gpu": T, "experts": w["E"],
                       "top_k": w["k"], "shared_experts": w["S"], "d_model": D, "ffn_hidden": w["H"],
                       "parallelism": "single GPU" if world == 1 else f"expert-parallel ep{world} (NCCL all-to-all)",
                       "training": True, "l2": "inputs (activations + expert weights) are larger than L2; no flush needed"},
            "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "roofline": roof, "cpu_baseline": cpu,
            "stage_ms": stages, "loss": loss_value, "output_finite": output_finite, "device_status": status,
        }
        print(json.dumps(line), flush=True)
        if not output_finite or status != 0:
            raise SystemExit("bench: the layer produced non-finite output or a device status")
    layer.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
