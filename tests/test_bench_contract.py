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


def test_kept_entry_mask_marks_exactly_the_dropped_entries():
    """The checker of `bench.py --op gcn` recomputes the layer over the entries the built format
    holds: its mask must zero exactly the entries the reference builder's 2-per-group rule drops
    (block_online.cpp:683-695), so that mask-weighted CSR x B equals the product of the format."""
    import importlib.util
    sys.path.insert(0, str(ROOT / "tr-spmm_zzx_b200"))
    sys.path.insert(0, str(ROOT))
    from oracle import oracle as O
    from trspmm import graphs
    from trspmm.format import Format
    spec = importlib.util.spec_from_file_location("bench_mod", ROOT / "bench.py")
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    rp, col, val = graphs.rmat_graph(10, 16, seed=2)
    arrays, info = O.build_format(rp, col, val)
    fmt = Format(arrays)
    n = rp.numel() - 1
    keep = bench.kept_entry_mask(rp, col, fmt, n)
    assert keep.numel() == col.numel()
    dropped = int((keep == 0).sum())
    assert dropped == info["dropped_nnz"] and dropped > 0
    # the product of the format (oracle forward over its three routes) equals the masked CSR product
    B = torch.randn(n, 32, generator=torch.Generator().manual_seed(1)).half().float()
    A = torch.sparse_csr_tensor(rp.long(), col.long(), val.half().float() * keep.float(), (n, n))
    want = torch.sparse.mm(A, B)
    got = O.spmm_from_format(arrays, B, n)
    assert torch.allclose(got, want, rtol=1e-4, atol=1e-4)
