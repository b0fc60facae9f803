"""bench.py prints one JSON line with the keys its consumers read (checked on the smallest workload)."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu


def _run(*extra):
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--steps", "3", "--warmup", "3", *extra],
                       capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert r.returncode == 0, r.stdout + r.stderr
    return json.loads(r.stdout.strip().splitlines()[-1])


def test_decode_line_has_the_contract_keys(cuda, lib):
    d = _run("--workload", "decode1", "--no-cpu-baseline")
    for k in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
              "vs_baseline", "dtype", "data", "config", "clocks", "e2e", "gpu_launches", "roofline"):
        assert k in d, k
    assert d["metric"] == "decode_attn_kv_bandwidth" and d["unit"] == "GB/s" and d["n_gpus"] == 1 and d["steps"] == 3
    assert d["config"]["workload"] == "decode1" and d["data"] == "synthetic" and d["vs_baseline"] is None
    assert d["value"] > 0 and d["gpu_launches"] >= 3 * 3          # prep + attention + merge per layer and step
    e = d["e2e"]
    assert e["value"] > 0 and e["h2d_bytes_per_step"] > 0 and e["d2h_bytes_per_step"] > 0
    assert e["value"] != d["value"]
    r = d["roofline"]
    assert r["bound"] == "hbm" and r["unit"] == "GB/s" and r["peak"] > 0 and r["traffic"] > 0
    assert abs(r["frac"] - r["achieved"] / r["peak"]) < 1e-9
    assert set(("sm_mhz", "sm_max_mhz", "reasons")) <= set(d["clocks"])
    assert len(d["out_fingerprint"]) == 64 and any(x != 0 for x in d["out_fingerprint"])


def test_fingerprint_is_a_function_of_the_seed_only(cuda, lib):
    a = _run("--workload", "verify8", "--no-cpu-baseline", "--chunk", "512")
    b = _run("--workload", "verify8", "--no-cpu-baseline", "--chunk", "2048")
    fa, fb = a["out_fingerprint"], b["out_fingerprint"]
    scale = max(abs(x) for x in fa)
    assert scale > 0 and max(abs(x - y) for x, y in zip(fa, fb)) <= 2e-3 * scale


def test_prefill_line(cuda, lib):
    d = _run("--workload", "prefill8k", "--no-cpu-baseline")
    assert d["metric"] == "prefill_attn_tflops" and d["unit"] == "TFLOP/s" and d["value"] > 0
    assert d["roofline"]["bound"] == "tensor" and 0 < d["roofline"]["frac"] < 1.5 and d["gpu_launches"] > 0
    assert d["e2e"]["h2d_bytes_per_step"] > 0 and d["e2e"]["value"] > 0 and d["config"]["workload"] == "prefill8k"
