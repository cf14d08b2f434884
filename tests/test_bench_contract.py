"""bench.py's output contract, checked on the CPU through the reference arm (the only arm that
runs without a GPU): one JSON line with the agreed keys; our arm must refuse to run without CUDA."""
import json
import subprocess
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[1]


def _run(*args):
    return subprocess.run([sys.executable, str(ROOT / "bench.py"), *args], capture_output=True, text=True, timeout=600)


def test_reference_arm_prints_one_contract_line():
    r = _run("--impl", "reference", "--workload", "uniform", "--steps", "2", "--warmup", "1")
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    d = json.loads(lines[0])
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "impl", "cpu_baseline", "e2e", "gpu_launches"):
        assert key in d, key
    assert d["impl"] == "reference" and d["steps"] == 2 and d["warmup"] == 1 and d["n_gpus"] == 1
    assert d["config"]["workload"] == "uniform" and d["data"] == "synthetic"
    assert d["cpu_baseline"]["kind"] in ("port", "reference") and d["cpu_baseline"]["cores"] >= 1
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["d2h_bytes_per_step"] == 0
    assert d["e2e"]["value"] == d["value"] and d["value"] > 0


def test_our_arm_has_no_cpu_fallback():
    if torch.cuda.is_available():
        return
    r = _run("--workload", "uniform", "--steps", "1", "--warmup", "1")
    assert r.returncode != 0
    assert "CUDA" in (r.stderr + r.stdout)
