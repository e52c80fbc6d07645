"""bench.py's reference arm needs no GPU: it times the CPU restatement of the reference path.  These
tests run it the way the benchmark driver does (a plain process; with RANK/WORLD_SIZE for N > 1) on
the smallest workload and check the JSON line it has to print."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(args, env_extra=None):
    env = dict(os.environ)
    env.pop("RANK", None)
    env.pop("WORLD_SIZE", None)
    env.update(env_extra or {})
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py")] + args, cwd=ROOT, env=env, capture_output=True,
                          text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    return [json.loads(ln) for ln in proc.stdout.splitlines() if ln.startswith("{")]


def test_reference_arm_prints_one_line_with_the_contract_keys():
    lines = _run(["--impl", "reference", "--workload", "c1", "--steps", "2", "--warmup", "1"])
    assert len(lines) == 1
    d = lines[0]
    assert d["impl"] == "reference" and d["metric"] == "moe_layer_tokens_per_s" and d["unit"] == "tokens/s"
    assert d["higher_is_better"] is True and d["n_gpus"] == 1 and d["steps"] == 2 and d["warmup"] == 1
    assert d["value"] > 0 and abs(d["value"] - 32 / (d["ms_per_step"] * 1e-3)) <= 1e-6 * d["value"]
    assert d["config"]["workload"].startswith("c1:") and d["config"]["tokens_per_gpu"] == 32
    base = d["cpu_baseline"]
    assert base["kind"] == "port" and base["cores"] >= 1 and base["value"] == d["value"] and "32 tokens" in base["sample"]
    assert d["e2e"] == {"value": d["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert d["gpu_launches"] == 0 and d["vs_baseline"] is None


def test_reference_arm_under_a_multi_rank_launch():
    """Rank 0 alone runs and prints (one rank's share of the experts); the other ranks exit 0 silently."""
    args = ["--impl", "reference", "--workload", "c1", "--gpus", "2", "--steps", "1", "--warmup", "1"]
    assert _run(args, {"RANK": "1", "WORLD_SIZE": "2", "LOCAL_RANK": "1"}) == []
    lines = _run(args, {"RANK": "0", "WORLD_SIZE": "2", "LOCAL_RANK": "0"})
    assert len(lines) == 1 and lines[0]["n_gpus"] == 2
    assert "expert-parallel ep2" in lines[0]["config"]["parallelism"]
    assert lines[0]["value"] > 0
