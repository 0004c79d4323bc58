"""bench.py's output contract: one JSON line with the keys the driver reads, from both arms.  The CPU
reference arm runs anywhere; the GPU arm runs at 1/64 of every tensor so that the check takes seconds."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BASE_KEYS = {"metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling", "vs_baseline", "dtype",
             "data", "config", "e2e", "cpu_baseline"}


def _run(*args, timeout=600):
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True, timeout=timeout, cwd=ROOT)
    assert p.returncode == 0, p.stderr[-2000:]
    return json.loads(p.stdout.strip().splitlines()[-1])


def test_reference_arm_prints_the_contract_line():
    d = _run("--impl", "reference", "--steps", "1", "--warmup", "1")
    assert d["impl"] == "reference" and BASE_KEYS <= set(d)
    assert d["higher_is_better"] is True and d["unit"] == "GB/s" and d["value"] > 0
    assert d["e2e"] == {"value": d["value"], "unit": d["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert d["cpu_baseline"]["kind"] in ("port", "reference") and d["cpu_baseline"]["cores"] >= 1 and d["cpu_baseline"]["sample"]
    assert "workload" in d["config"] and "model" not in d["config"]


@pytest.mark.gpu
def test_gpu_arm_prints_the_contract_line_and_matches_the_reference_arm_config():
    d = _run("--scale-log2", "6", "--steps", "3", "--warmup", "3", "--no-ref-cuda")
    assert BASE_KEYS | {"roofline", "clocks", "gpu_launches", "verified"} <= set(d)
    assert d["verified"] is True and d["n_gpus"] == 1 and d["steps"] == 3 and d["warmup"] == 3
    assert d["gpu_launches"] >= 3 * 5                       # five kernels per step
    r = d["roofline"]
    assert r["bound"] == "hbm" and r["unit"] == "GB/s" and abs(r["frac"] - r["achieved"] / r["peak"]) < 1e-3
    e = d["e2e"]
    assert e["h2d_bytes_per_step"] > 0 and e["d2h_bytes_per_step"] > 0 and e["results_read_back"] is True and e["value"] != d["value"]
    assert {"sm_mhz", "sm_max_mhz", "reasons"} <= set(d["clocks"])
    assert d["cpu_baseline"]["value"] > 0
    ref = _run("--impl", "reference", "--steps", "1", "--warmup", "1")
    assert ref["metric"] == d["metric"] and ref["unit"] == d["unit"] and ref["higher_is_better"] == d["higher_is_better"]
