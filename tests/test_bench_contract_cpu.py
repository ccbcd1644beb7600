"""The bench's reference arm on CPU: one JSON line with the keys the contract names, for every workload that has a CPU arm;
and the product path refuses to run without a GPU instead of falling back."""
import json
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
KEYS = {"impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
        "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e", "gpu_launches"}


def run(*args):
    r = subprocess.run([sys.executable, str(ROOT / "bench.py"), *args], capture_output=True, text=True, timeout=600, cwd=ROOT)
    return r.returncode, r.stdout.strip().splitlines(), r.stderr


@pytest.mark.parametrize("wl", ["cfg2", "cfg4p8"])
def test_reference_arm_line(wl):
    rc, out, err = run("--impl", "reference", "--workload", wl, "--steps", "1", "--warmup", "0")
    assert rc == 0, err[-2000:]
    d = json.loads(out[-1])
    assert KEYS <= set(d), KEYS - set(d)
    assert d["impl"] == "reference" and d["gpu_launches"] == 0 and d["value"] > 0
    assert d["cpu_baseline"]["kind"] in ("reference", "port") and d["cpu_baseline"]["cores"] >= 1 and d["cpu_baseline"]["sample"]
    assert d["e2e"] == {"value": d["value"], "unit": d["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert d["steps"] == 1 and d["warmup"] == 0


def test_writers_have_no_cpu_arm():
    rc, out, _ = run("--impl", "reference", "--workload", "writers")
    assert rc == 0 and "unavailable" in json.loads(out[-1])


def test_product_arm_needs_a_gpu():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    rc, out, err = run("--steps", "1", "--warmup", "1", "--cpu-steps", "0")
    assert rc != 0                                       # no CPU fallback for the product path
