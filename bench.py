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

Keys of the line beyond the usual ones:
  roofline        the dominant kernel (expert GEMM 1): algorithmic FLOPs / mean CUDA-event time of
                  the timed steps, against the measured cuBLAS BF16 peaks (burst and sustained);
                  `library_same_gpu`: cuBLAS timed on this GPU on the same GEMM shapes and data
  e2e             the same metric through moe_layer_forward_host with pinned host buffers
  cpu_baseline    the CPU restatement of the reference path on the host cores, same token count
  parity          outside the timed region: every rank compares its tokens' expert ids (all local
                  tokens), a sample of outputs and the global loss with the CPU oracle
  other_workloads c1 and c4 measured after the timed region, and the per-position / per-prompt host
                  calls of the Llama2 MoE FFN (c2) (N=1 only)
"""
from __future__ import annotations

import argparse
import json
import os
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
    "c2": dict(E=8, S=0, k=2, D=512, H=1376, O=512, T=64, dtype="f32", std=0.02, bias_std=0.0,
               desc="MoE FFN of a converted Llama2 layer (dim 512, hidden 1376, 8 experts, top-2, FP32), 64 positions"),
}
SEED = 1234
ALPHA, ZW = 0.01, 0.001
CPU_BUDGET_S = 240.0        # the reference arm stops adding steps once it has used this much time


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


def recorded_dram_traffic(workload, kernel):
    """DRAM bytes per launch of `kernel` on `workload`, from the record the ncu capture step leaves in
    profiles/dram_traffic.txt (lines: workload kernel read_bytes write_bytes).  None if absent."""
    path = os.path.join(ROOT, "profiles", "dram_traffic.txt")
    try:
        with open(path) as f:
            for ln in f:
                parts = ln.split()
                if len(parts) >= 4 and not ln.startswith("#") and parts[0] == workload and parts[1] == kernel:
                    return int(parts[2]) + int(parts[3]), f"ncu capture recorded in profiles/dram_traffic.txt: {ln.strip()}"
    except OSError:
        pass
    return None, "no ncu capture recorded for this workload and kernel"


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
                              balance_loss=m.SwitchTransformerLoss(ALPHA), z_loss_weight=ZW)
    router = make_router(w, torch, device)
    router.gate_type = gate
    return m.MoELayer(cfg, device=device_index, compute_dtype=w["dtype"], experts=make_expert_factory(w, torch, device),
                      router=router, expert_parallel=ep)


def workload_config(name, w, world):
    """The `config` object of the JSON line: the same for the GPU arm and for the reference arm."""
    if world == 1:
        par = "single GPU"
    else:
        mode = os.environ.get("MOE_B200_EP_MODE", "peer")
        data = ("token rows cross NVLink by peer stores inside the permute kernel and the GEMM-2 epilogue; NCCL carries "
                "counts and the loss sums only") if mode != "nccl" else "token rows by grouped ncclSend/ncclRecv"
        par = f"expert-parallel ep{world}: {w['E'] // world} experts per GPU, tokens data-parallel; {data}"
    return {"workload": f"{name}: {w['desc']}", "tokens_per_gpu": w["T"], "experts": w["E"], "top_k": w["k"],
            "shared_experts": w["S"], "d_model": w["D"], "ffn_hidden": w["H"], "parallelism": par, "training": True,
            "l2": "inputs (activations + expert weights) are larger than L2; no flush needed"}


# --------------------------------------------------------------------------------------------------
# CPU leg: the restatement of the reference path (oracle/) timed on the host cores
# --------------------------------------------------------------------------------------------------

def cpu_forward_rate(w, world, steps, warmup, budget_s=CPU_BUDGET_S):
    """Times the CPU restatement of the reference path on the workload's own token count.

    world == 1: the whole layer (all experts, all T tokens).  world > 1: ONE rank's share of the
    expert-parallel layer -- its E/world local experts on T tokens' worth of pairs (T*k rows, what a
    rank receives on average) -- because all 64 experts in FP32 need 45 GB; the CPU doing the whole
    job would run `world` such shares one after the other, so whole-job tokens/s = T / (time of one
    share).  Weight values do not affect CPU time: one seeded N(0, std^2) draw per matrix shape is
    rotated to give every expert its own arrays.  Returns (tokens/s, cores, s/step, steps timed, note)."""
    import numpy as np

    from oracle import moe_oracle as orc

    rng = np.random.Generator(np.random.PCG64(SEED))
    E_all, D, H, O, T = w["E"], w["D"], w["H"], w["O"], w["T"]
    E = E_all if world == 1 else E_all // world
    S = w["S"] if world == 1 else 0
    x = rng.standard_normal((T, D), dtype=np.float32)
    router = rng.standard_normal((E, D), dtype=np.float32) * np.float32(w["std"])
    base = {"hd": rng.standard_normal((H, D), dtype=np.float32) * np.float32(w["std"]),
            "oh": rng.standard_normal((O, H), dtype=np.float32) * np.float32(w["std"])}
    experts = []
    for e in range(E):
        experts.append(orc.GatedExpertWeights(w1=np.roll(base["hd"], 7919 * (3 * e + 1)), w2=np.roll(base["oh"], 7919 * (3 * e + 2)),
                                              w3=np.roll(base["hd"], 7919 * (3 * e + 3))))
    gate = orc.SharedExpertGating(S, orc.TopKGating(w["k"]), E) if S else orc.TopKGating(w["k"])
    bias = None
    if w["bias_std"] > 0:
        bias = (rng.standard_normal(E) * w["bias_std"]).astype(np.float32)
        bias[:S] = 0
    cfg = orc.MoEConfig(num_experts=E, input_dim=D, hidden_dim=H, output_dim=O, activation="silu", gate_type=gate,
                        balance_alpha=ALPHA, z_loss_weight=ZW, router_bias=bias)
    weights = orc.MoEWeights(router=router, experts=experts)
    t_begin = time.perf_counter()
    for _ in range(warmup):
        orc.moe_layer_forward(cfg, weights, x, training=True)
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        orc.moe_layer_forward(cfg, weights, x, training=True)
        times.append(time.perf_counter() - t0)
        if time.perf_counter() - t_begin > budget_s:
            break
    dt = sum(times) / len(times)
    if world == 1:
        note = f"all {T} tokens of the same layer (all {E} experts, full widths), FP32 NumPy/OpenBLAS"
    else:
        note = (f"one rank's share of the {world}-GPU job: {E} local experts (full widths), {T} tokens top-{w['k']} = "
                f"{T * w['k']} rows, FP32 NumPy/OpenBLAS; whole-job tokens/s = {T} / share time")
    if len(times) < steps:
        note += f"; stopped after {len(times)} of {steps} steps (time budget {budget_s:.0f} s)"
    return T / dt, os.cpu_count() or 1, dt, len(times), note


def run_reference_arm(args, w, name):
    """--impl reference: the reference's CPU path (its NumPy/OpenBLAS restatement; the Julia
    original cannot run without a Julia runtime) on all host cores, on the GPU arm's workload."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = max(args.gpus, 1)
    rate, cores, dt, done, note = cpu_forward_rate(w, world, args.steps, args.warmup)
    line = {
        "impl": "reference", "metric": "moe_layer_tokens_per_s", "value": rate, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": done, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(name, w, world),
        "reference_note": "CPU path of the reference restated in NumPy (FP32, OpenBLAS on all host cores); no Julia runtime exists on the box",
        "cpu_baseline": {"value": rate, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": note},
        "e2e": {"value": rate, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------------------
# parity block (outside every timed region): the oracle as the checker of what was just timed
# --------------------------------------------------------------------------------------------------

def parity_block(w, layer, x, torch, rank, world, dist, device, n_sample=96):
    """Every rank checks its own tokens of the layer it just timed against the CPU oracle:
    expert ids of ALL local tokens (exact, except float64-logit ties below 1e-6), gates, the
    outputs of a sample of tokens (BF16: 2e-2, FP32: 1e-5, relative inf-norm) and the loss over all
    ranks' tokens (1e-5 relative; oracle sums all-reduced in float64).  Experts are regenerated one
    at a time from their seeds, so no rank ever holds more than one FP32 expert on the host.
    Returns the dict printed as `parity`; `ok` is False on any violation."""
    import numpy as np

    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from helpers import check_indices, rel_inf
    from oracle import moe_oracle as orc

    E, S, k, D, H, O, T = w["E"], w["S"], w["k"], w["D"], w["H"], w["O"], w["T"]
    out, loss, routing = layer(x.t(), training=True, return_routing=True)
    torch.cuda.synchronize()
    dev_idx = routing["indices"].t().cpu().numpy()
    dev_gates = routing["gates"].t().cpu().numpy()
    dev_out = out.t()
    router = make_router(w, torch, device)
    bias = router.bias.cpu().numpy() if getattr(router, "bias", None) is not None else None
    rw = router.weight.cpu().numpy()
    xs = x.float().cpu().numpy()
    gate = orc.SharedExpertGating(S, orc.TopKGating(k), E) if S else orc.TopKGating(k)
    cfg = orc.MoEConfig(num_experts=E, input_dim=D, hidden_dim=H, output_dim=O, activation="silu", gate_type=gate,
                        balance_alpha=ALPHA, z_loss_weight=ZW, router_bias=bias)
    o_idx, o_gates, o_probs, o_logits = orc.router_forward(cfg, orc.MoEWeights(router=rw, experts=[]), xs)
    logits64 = xs.astype(np.float64) @ rw.astype(np.float64).T
    if bias is not None:
        logits64 = logits64 + bias.astype(np.float64)
    res = {"tokens": int(T), "ok": True}
    try:
        res["idx_excused"] = int(check_indices(dev_idx, o_idx, logits64, k, r0=S))
    except AssertionError as exc:
        res.update(ok=False, idx_error=str(exc)[:200])
        res["idx_excused"] = -1
    same = (dev_idx == o_idx).all(axis=1)
    res["idx_mismatch_tokens"] = int((~same).sum())
    res["gates_rel_inf"] = rel_inf(dev_gates[same], o_gates[same])
    # global loss from the oracle's per-rank sums (Switch: f_i over all pairs, P_i mean prob; z: mean lse^2)
    sums = np.concatenate([np.bincount(o_idx.ravel() - 1, minlength=E).astype(np.float64),
                           o_probs.sum(axis=0, dtype=np.float64),
                           [float((orc.logsumexp_dim1(o_logits).astype(np.float64) ** 2).sum()), float(T)]])
    if world > 1:
        ts = torch.from_numpy(sums).to(device)
        dist.all_reduce(ts)
        sums = ts.cpu().numpy()
    Tg = sums[-1]
    n_probs = o_probs.shape[1]
    o_loss = ALPHA * n_probs * float(np.sum((sums[:E] / ((k + S) * Tg)) * (sums[E:E + n_probs] / Tg))) + ZW * sums[E + n_probs] / Tg
    res["loss_rel"] = abs(float(loss.item()) - o_loss) / abs(o_loss)
    # outputs: tokens whose oracle experts all lie in a small expert subset (spread over the ranks), so
    # that only those experts have to be regenerated on the host
    if 12.0 * E * H * D <= 8e9:
        subset = list(range(E))                            # the whole layer in FP32 is a few GB: every expert
    else:
        subset = sorted({(rank * 5 + j * (E // 8 + 1)) % E for j in range(8)})
    sub_mask = np.zeros(E + 1, dtype=bool)
    sub_mask[np.asarray(subset) + 1] = True
    cand = np.where(sub_mask[o_idx].all(axis=1) & same)[0]
    if len(cand) > n_sample:
        cand = cand[np.linspace(0, len(cand) - 1, n_sample).astype(np.int64)]
    res["out_tokens"] = int(len(cand))
    if len(cand):
        fac = make_expert_factory(w, torch, device)
        o_out = np.zeros((len(cand), O), dtype=np.float32)
        xc = xs[cand]
        for e in subset:                                   # ascending expert id, like the reference's expert loop
            rows, slots = np.where(o_idx[cand] == e + 1)
            if not len(rows):
                continue
            ex = fac(e)
            ew = orc.GatedExpertWeights(w1=ex.w1.float().cpu().numpy(), w2=ex.w2.float().cpu().numpy(),
                                        w3=ex.w3.float().cpu().numpy())
            y = orc.gated_expert_forward(ew, xc[rows], orc.silu)
            np.add.at(o_out, rows, o_gates[cand][rows, slots][:, None] * y)
            del ex, ew
        res["out_rel_inf"] = rel_inf(dev_out[torch.as_tensor(cand, device=device)].cpu().numpy(), o_out)
    else:
        res["out_rel_inf"] = None
    tol_out = 2e-2 if w["dtype"] == "bf16" else 1e-5
    if res["gates_rel_inf"] > 1e-5 or res["loss_rel"] > 1e-5 or not res["out_tokens"] or res["out_rel_inf"] > tol_out:
        res["ok"] = False
    res["tolerances"] = {"idx": "exact except float64-logit gaps < 1e-6", "gates": 1e-5, "loss_rel": 1e-5, "out_rel_inf": tol_out}
    if world > 1:                                           # one verdict for the job: every rank must pass
        agg = torch.tensor([0.0 if res["ok"] else 1.0, float(res["idx_mismatch_tokens"]), float(res["out_tokens"]),
                            float(T)], device=device, dtype=torch.float64)
        mx = torch.tensor([res["gates_rel_inf"], res["loss_rel"], res["out_rel_inf"] or 0.0], device=device, dtype=torch.float64)
        dist.all_reduce(agg)
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        res.update(ok=bool(agg[0].item() == 0), idx_mismatch_tokens=int(agg[1].item()),
                   idx_excused=int(agg[1].item()) if res["idx_excused"] >= 0 else -1, out_tokens=int(agg[2].item()),
                   tokens=int(agg[3].item()), gates_rel_inf=float(mx[0].item()), loss_rel=float(mx[1].item()),
                   out_rel_inf=float(mx[2].item()), ranks=world)
    return res


# --------------------------------------------------------------------------------------------------
# GPU measurement of one workload
# --------------------------------------------------------------------------------------------------

def measure_device(layer, x, out, steps, warmup, torch, barrier, sampler=None, stages_apart=False):
    """W untimed + K timed forwards with x resident in HBM; CUDA events on the launching stream.
    The per-stage events are recorded inside the timed steps, except with ``stages_apart`` (steps of a
    tenth of a millisecond, where seven event records per step would be a large part of what is timed
    and would keep the library from replaying its graph): then the K steps are timed bare, each step
    being the one C call moe_layer_forward with its arguments bound beforehand (MoELayer.bind_forward:
    the argument checks and allocations of the Python mirror's __call__ take longer than such a step),
    and the stage times come from K more steps after them."""
    step = (lambda: layer(x.t(), training=True, out=out)) if not stages_apart else layer.bind_forward(x.t(), out, training=True)
    for _ in range(warmup):
        step()
    barrier()
    if not stages_apart:
        layer.set_profiling(min(steps, 1024))
    launches0 = layer.launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t_mark0 = sampler.mark() if sampler else None
    ev0.record()
    loss = None
    for _ in range(steps):
        _, loss = step()
    ev1.record()
    barrier()
    t_mark1 = sampler.mark() if sampler else None
    ms_total = ev0.elapsed_time(ev1)
    launches = layer.launch_count() - launches0
    n_prof = min(steps, 1024)
    if stages_apart:
        layer.set_profiling(n_prof)
        for _ in range(n_prof):
            layer(x.t(), training=True, out=out)
        barrier()
    stages = {}
    for back in range(n_prof):
        for k_, v in layer.stage_ms(back).items():
            stages[k_] = stages.get(k_, 0.0) + v / n_prof
    layer.set_profiling(0)
    return ms_total, launches, stages, loss, (t_mark0, t_mark1)


def roofline_of(w, name, T, stages, ms_step, peaks, tile_rows, world, clocks, full_size):
    f_g1 = 2.0 * w["H"] * 2 * w["D"] * T * (w["k"] + w["S"])
    f_g2 = 2.0 * w["H"] * w["O"] * T * (w["k"] + w["S"])
    mhz = (clocks or {}).get("sm_mhz")
    if w["dtype"] == "bf16" and stages.get("gemm1", 0) > 0 and world == 1:
        ach = f_g1 / (stages["gemm1"] * 1e-3) / 1e12
        kernel = {0: "group_gemm_tc_kernel<1>", 1: "group_gemm_tc2_kernel<1>", 2: "group_gemm_tc_dual_kernel<1>"}[tile_rows]
        kind = {0: "", 1: " (CTA pairs)", 2: " (two accumulators per CTA)"}[tile_rows]
        traffic, note = recorded_dram_traffic(name, kernel) if full_size else (None, "not the recorded workload size")
        burst, sust = peaks["bf16_tflops"], peaks["bf16_tflops_sustained"]
        return {"bound": "tensor", "kernel": kernel + kind + ": x W1^T, x W3^T, act*up",
                "achieved": ach, "peak": burst, "unit": "TFLOP/s", "frac": ach / burst,
                "frac_burst": ach / burst, "frac_sustained": ach / sust, "peak_sustained": sust,
                "peak_source": f"{peaks['source']} cuBLAS bf16 8192^3: burst {burst} (best of 10), sustained {sust} (4 s loop under the "
                               "power cap); `frac` uses the burst figure, the timed region is a fraction of a second",
                "gemm1_ms": stages["gemm1"], "gemm1_ms_x_sm_mhz": stages["gemm1"] * mhz if mhz else None,
                "traffic": traffic, "traffic_unit": "bytes per launch", "traffic_note": note,
                "algorithmic_bytes": 2.0 * (2 * w["E"] * w["H"] * w["D"] + T * (w["k"] + w["S"]) * (w["D"] + w["H"])),
                "gemm2_achieved": f_g2 / (stages["gemm2"] * 1e-3) / 1e12 if stages.get("gemm2", 0) > 0 else None,
                "layer_achieved": expert_flops(w, T) / (ms_step * 1e-3) / 1e12,
                "layer_frac_burst": expert_flops(w, T) / (ms_step * 1e-3) / 1e12 / burst,
                "layer_frac_sustained": expert_flops(w, T) / (ms_step * 1e-3) / 1e12 / sust}
    if w["dtype"] == "bf16":
        ach = expert_flops(w, T) / (ms_step * 1e-3) / 1e12
        burst, sust = peaks["bf16_tflops"], peaks["bf16_tflops_sustained"]
        return {"bound": "tensor", "kernel": "whole layer per GPU (expert GEMM FLOPs / step time)",
                "achieved": ach, "peak": burst, "unit": "TFLOP/s", "frac": ach / burst, "frac_burst": ach / burst,
                "frac_sustained": ach / sust, "peak_sustained": sust,
                "peak_source": f"{peaks['source']} cuBLAS bf16: burst {burst}, sustained {sust}", "traffic": None}
    nbytes = 4.0 * w["E"] * w["H"] * (2 * w["D"] + w["O"])
    t_g = (stages.get("gemm1", 0) + stages.get("gemm2", 0)) * 1e-3
    if t_g <= 0:
        return None
    ach = nbytes / t_g / 1e9
    return {"bound": "hbm", "kernel": "FP32 expert GEMM pair (expert weights streamed once)",
            "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": ach / peaks["hbm_gbs"],
            "peak_source": f"{peaks['source']} STREAM-style copy", "traffic": None,
            "note": "the 100 MB of weights fit in L2 (126 MB): without an L2 flush between steps this is an L2-resident figure"}


def measure_other(name, torch, peaks, steps=10, warmup=3):
    """One more workload on cuda:0 after the headline's timed region: ms/step, stage times, roofline."""
    w = dict(WORKLOADS[name])
    layer = build_layer(w, torch, 0)
    T, D, O = w["T"], w["D"], w["O"]
    xdt = torch.bfloat16 if w["dtype"] == "bf16" else torch.float32
    if w["dtype"] == "f32":
        # a step of this workload is ~0.1 ms: a few warm-up steps do not bring the SM clock up from
        # idle, so warm up for a few tenths of a second and time more steps
        steps, warmup = max(steps, 200), max(warmup, 3000)
    gx = torch.Generator(device="cuda:0").manual_seed(SEED + 7)
    x = torch.randn((T, D), device="cuda:0", generator=gx, dtype=torch.float32).to(xdt)
    out = torch.empty((T, O), device="cuda:0", dtype=torch.float32)
    flush = torch.empty(160 << 20, dtype=torch.uint8, device="cuda:0") if w["dtype"] == "f32" else None

    def barrier():
        torch.cuda.synchronize()

    replays0 = layer.graph_replays()
    ms_total, launches, stages, loss, _ = measure_device(layer, x, out, steps, warmup, torch, barrier,
                                                         stages_apart=w["dtype"] == "f32")
    replays = layer.graph_replays() - replays0
    ms_step = ms_total / steps
    res = {"workload": f"{name}: {w['desc']}", "ms_per_step": ms_step, "tokens_per_s": T / (ms_step * 1e-3),
           "steps": steps, "warmup": warmup, "stage_ms": stages, "gpu_launches": launches,
           "roofline": roofline_of(w, name, T, stages, ms_step, peaks, layer.gemm_kernel(T), 1, None, True),
           "loss": float(loss.item()), "device_status": layer.device_status(), "graph_replays": replays}
    if w["dtype"] == "f32":
        res["timing_note"] = ("ms_per_step: bare moe_layer_forward calls with bound arguments (the library replays one captured "
                              "CUDA graph per step); stage_ms: the same steps launched kernel by kernel with an event after each")
    if flush is not None:
        # the FP32 workload's weights fit in L2: time it again with L2 flushed before every step
        layer.set_profiling(steps)
        for _ in range(steps):
            flush.fill_(1)
            layer(x.t(), training=True, out=out)
        torch.cuda.synchronize()
        cold = {}
        for back in range(steps):
            for k_, v in layer.stage_ms(back).items():
                cold[k_] = cold.get(k_, 0.0) + v / steps
        layer.set_profiling(0)
        res["stage_ms_l2_flushed"] = cold
        t_g = (cold.get("gemm1", 0) + cold.get("gemm2", 0)) * 1e-3
        if t_g > 0:
            nbytes = 4.0 * w["E"] * w["H"] * (2 * w["D"] + w["O"])
            res["roofline_l2_flushed"] = {"bound": "hbm", "achieved": nbytes / t_g / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                          "frac": nbytes / t_g / 1e9 / peaks["hbm_gbs"],
                                          "step_ms": sum(v for k_, v in cold.items() if k_ != "exchange")}
    layer.close()
    return res


def library_gemm_yardstick(w, T, stages, torch, steps=20, warmup=5):
    """cuBLAS (torch.matmul) on THIS GPU, on the expert GEMMs' shapes and value distributions, as a
    yardstick beside `roofline`: the pool's GPUs differ by several percent and every run sits at the
    power limit, so a figure from the same box says more about the kernels than the pool-wide peak.
    One GEMM per stage over all (token, expert) rows against ONE expert's weights -- no grouping,
    no gate * up epilogue, plain BF16 stores: the library's best case for the same FLOPs -- and the
    two alternated like a layer does.  Not on the product path."""
    rows, D, H, O = T * (w["k"] + w["S"]), w["D"], w["H"], w["O"]
    dev = "cuda:0"
    g = torch.Generator(device=dev).manual_seed(SEED + 99)
    mk = lambda r, c, std: (torch.randn((r, c), device=dev, generator=g, dtype=torch.float32) * std).to(torch.bfloat16)
    a1, w13 = mk(rows, D, 1.0), mk(2 * H, D, w["std"])
    h_in, w2 = mk(rows, H, 0.05), mk(O, H, w["std"])
    h_out = torch.empty((rows, 2 * H), device=dev, dtype=torch.bfloat16)
    y = torch.empty((rows, O), device=dev, dtype=torch.bfloat16)
    for _ in range(warmup):
        torch.matmul(a1, w13.t(), out=h_out)
        torch.matmul(h_in, w2.t(), out=y)
    torch.cuda.synchronize()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2 * steps + 1)]
    ev[0].record()
    for i in range(steps):
        torch.matmul(a1, w13.t(), out=h_out)
        ev[2 * i + 1].record()
        torch.matmul(h_in, w2.t(), out=y)
        ev[2 * i + 2].record()
    torch.cuda.synchronize()
    t1 = sum(ev[2 * i].elapsed_time(ev[2 * i + 1]) for i in range(steps)) / steps
    t2 = sum(ev[2 * i + 1].elapsed_time(ev[2 * i + 2]) for i in range(steps)) / steps
    f1, f2 = 2.0 * rows * 2 * H * D, 2.0 * rows * O * H
    ours = stages.get("gemm1", 0.0) + stages.get("gemm2", 0.0)
    return {"what": "torch.matmul (cuBLAS) BF16 on this GPU: all rows x one expert's [W1;W3], then x W2, alternated for "
                    f"{steps} steps after {warmup}; no grouping, no activation epilogue",
            "gemm1_ms": t1, "gemm2_ms": t2, "gemm1_tflops": f1 / t1 / 1e9, "gemm2_tflops": f2 / t2 / 1e9,
            "pair_ms": t1 + t2, "pair_tflops": (f1 + f2) / (t1 + t2) / 1e9,
            "ours_pair_ms": ours, "ours_vs_library": (t1 + t2) / ours if ours > 0 else None}


def measure_llama_ffn(torch, peaks, calls=1000, warmup=3000):
    """The MoE FFN of a converted Llama2 layer as the generation loop drives it: one host call of
    moe_layer_forward_host per position (decode, T = 1) and one call for a whole 64-token prompt
    (prefill), host buffers in and out, synchronous; per-call wall time with the library's default
    launch mode (chained plain launches) and with a graph replay instead.  Calls go straight to the
    C entry point with prebuilt arguments; a few tenths of a second of warm-up calls bring the SM
    clock up from idle first."""
    import ctypes as C

    import numpy as np

    from mixtureofexperts_b200 import _lib

    w = dict(WORKLOADS["c2"])
    res = {"workload": f"c2: {w['desc']}", "calls": calls, "warmup": warmup,
           "timing": "host clock around synchronous moe_layer_forward_host calls (pageable NumPy buffers), inference"}
    rng = np.random.default_rng(SEED + 2)
    for graphs in (0, 1):     # 1: MOE_B200_CHAIN=0 makes small host calls replay a captured graph instead
        old = os.environ.get("MOE_B200_CHAIN")
        if graphs:
            os.environ["MOE_B200_CHAIN"] = "0"
        try:
            layer = build_layer(w, torch, 0)
        finally:
            if graphs:
                if old is None:
                    del os.environ["MOE_B200_CHAIN"]
                else:
                    os.environ["MOE_B200_CHAIN"] = old
        for T, label in ((1, "decode_us_per_position"), (w["T"], "prefill_us_per_64_positions")):
            x = np.ascontiguousarray(rng.standard_normal((T, w["D"])).astype(np.float32))
            out = np.empty((T, w["O"]), dtype=np.float32)
            loss = np.zeros(1, dtype=np.float32)
            o = _lib.ForwardOutputs()
            o.loss = loss.ctypes.data
            args = (layer._handle, x.ctypes.data, _lib.DTYPE_F32, T, 0, out.ctypes.data, C.byref(o))
            for _ in range(warmup):
                _lib.check(_lib.lib.moe_layer_forward_host(*args))
            launches0, replays0 = layer.launch_count(), layer.graph_replays()
            t0 = time.perf_counter()
            for _ in range(calls):
                rc = _lib.lib.moe_layer_forward_host(*args)
            dt = time.perf_counter() - t0
            _lib.check(rc)
            key = label + ("_graph_replay" if graphs else "")
            res[key] = dt / calls * 1e6
            if graphs:
                res[label.split("_us_")[0] + "_graph_replays"] = layer.graph_replays() - replays0
            else:
                res[label.split("_us_")[0] + "_launches_per_call"] = (layer.launch_count() - launches0) / calls
                res[label.split("_us_")[0] + "_output_finite"] = bool(np.isfinite(out).all())
        res["device_status"] = layer.device_status()
        layer.close()
    # two experts' weights are touched per position: 2 * 4 * H * (2D + O) bytes
    nbytes = 2 * 4.0 * w["H"] * (2 * w["D"] + w["O"])
    res["decode_weight_stream_gbs"] = nbytes / (res["decode_us_per_position"] * 1e-6) / 1e9
    res["decode_note"] = (f"{nbytes / 1e6:.1f} MB of expert weights per position = {nbytes / peaks['hbm_gbs'] / 1e3:.1f} us at the "
                          "measured HBM rate: the call is bound by launches, copies and the synchronisation, not by the stream")
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="auto", choices=["auto"] + sorted(n for n in WORKLOADS if n != "c2"))
    ap.add_argument("--tokens", type=int, default=0, help="override the tokens per GPU (profiling of small cases)")
    ap.add_argument("--experts", type=int, default=0, help="override the expert count (profiling of small cases)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-parity", action="store_true")
    ap.add_argument("--no-others", action="store_true", help="skip the c1/c4 block measured after the timed region")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3  # timing rule: at least 3 warm-up steps

    name = args.workload if args.workload != "auto" else ("c3" if args.gpus == 1 else "c5")
    w = dict(WORKLOADS[name])
    full_size = args.tokens == 0 and args.experts == 0
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
    from mixtureofexperts_b200 import parallel

    # one process per GPU: run on the CPUs next to this GPU so the pinned buffers of the end-to-end leg
    # are allocated in the memory closest to it (MOE_B200_NUMA_BIND=0 leaves the affinity alone)
    numa = {"node": -1, "why": "MOE_B200_NUMA_BIND=0"}
    if os.environ.get("MOE_B200_NUMA_BIND", "1") != "0":
        props = torch.cuda.get_device_properties(local_rank)
        numa = parallel.bind_to_gpu_numa_node(f"{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0")
    ep = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device(device))

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

    # ---- device-resident throughput ---------------------------------------------------------
    sampler = ClockSampler(str(torch.cuda.get_device_properties(local_rank).uuid))
    if rank == 0:
        sampler.start()
    ms_total, launches, stages, loss, marks = measure_device(layer, x, out, args.steps, args.warmup, torch, barrier, sampler,
                                                             stages_apart=w["dtype"] == "f32")
    clocks = sampler.stop(*marks) if rank == 0 else None
    status = layer.device_status()
    if world > 1:
        t = torch.tensor([ms_total], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_step = ms_total / args.steps
    value = T * world / (ms_step * 1e-3)
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
               "timing": "host clock around synchronous moe_layer_forward_host calls (pinned buffers), max over ranks",
               "numa_rank0": numa}
        del xh, oh

    # ---- parity of what was just timed (outside the timed regions) --------------------------
    parity = None
    if not args.no_parity:
        parity = parity_block(w, layer, x, torch, rank, world, dist, device)

    tile_rows = layer.gemm_kernel(T)     # 0 / 1 / 2: which tensor-core kernel this batch gets
    layer.close()
    del layer
    fail = None
    if rank == 0:
        peaks = measured_peaks()
        roof = roofline_of(w, name, T, stages, ms_step, peaks, tile_rows, world, clocks, full_size)
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            rate, cores, dt_cpu, done, note = cpu_forward_rate(w, 1, 2, 0, budget_s=60.0)
            cpu = {"value": rate, "unit": "tokens/s", "cores": cores, "kind": "port", "s_per_step": dt_cpu,
                   "sample": note + f", {done} timed pass(es)"}
        others = None
        if world == 1 and not args.no_others and full_size:
            torch.cuda.empty_cache()
            others = {n: measure_other(n, torch, peaks) for n in ("c4", "c1") if n != name}
            others["c2"] = measure_llama_ffn(torch, peaks)
        if world == 1 and not args.no_others and full_size and w["dtype"] == "bf16":
            # last: two seconds of library GEMMs at the power limit would colour whatever is measured after them
            roof["library_same_gpu"] = library_gemm_yardstick(w, T, stages, torch, args.steps, args.warmup)
        line = {
            "metric": "moe_layer_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic",
            "config": workload_config(name, w, world),
            "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "roofline": roof, "cpu_baseline": cpu,
            "parity": parity, "stage_ms": stages, "loss": loss_value, "output_finite": output_finite,
            "device_status": status, "other_workloads": others,
        }
        print(json.dumps(line), flush=True)
        if not output_finite or status != 0:
            fail = "bench: the layer produced non-finite output or a device status"
        elif parity is not None and not parity["ok"]:
            fail = f"bench: parity against the CPU oracle failed: {parity}"
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if fail:
        raise SystemExit(fail)


if __name__ == "__main__":
    main()
