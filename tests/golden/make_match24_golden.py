#!/usr/bin/env python3
"""Dicts returned by the reference's compiled CPU matchers (oracle/_ref, built unmodified from
TR-source/Block/block_matching_{window_para_dr,hash,bucket}.cpp) on seeded graphs ->
tests/golden/match24.json.  Run where the reference tree exists: python oracle/build_ref.py first."""
import json
import os
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT / "tr-spmm_zzx_b200"))
sys.path.insert(0, str(ROOT))
from oracle import oracle as O  # noqa: E402
from trspmm import graphs  # noqa: E402

GRAPHS = [
    ("uniform", dict(n=4096, per_row=16, seed=0)),
    ("clustered", dict(n=4096, community=128, intra=24, glob=4, seed=0)),
    ("rmat", dict(scale=12, edge_factor=16, seed=1)),
    ("uniform", dict(n=250, per_row=6, seed=1)),
]
CALLS = {
    "para_dr": ("matching_utils", "match_2to4", [dict(), dict(dense_threshold=4, t_max=2), dict(window_size=8)]),
    "hash": ("matching_utils_hash", "match_2to4_hash", [dict(), dict(window_size=12)]),
    "bucket": ("matching_utils_bucket", "match_2to4_bucket", [dict()]),
}


def quiet(fn, *a, **k):
    sys.stdout.flush()
    saved = os.dup(1); devnull = os.open(os.devnull, os.O_WRONLY); os.dup2(devnull, 1)
    try:
        return fn(*a, **k)
    finally:
        os.dup2(saved, 1); os.close(saved); os.close(devnull)


def main():
    cases = []
    for kind, kw in GRAPHS:
        rp, col, val = getattr(graphs, kind + "_graph")(**kw)
        case = {"graph": [kind, kw]}
        for variant, (mod, fn, calls) in CALLS.items():
            f = getattr(O.reference_module(mod), fn)
            case[variant] = [{"kwargs": c, "result": dict(quiet(f, rp.numpy(), col.numpy(), val.numpy(), **c))} for c in calls]
        cases.append(case)
    (Path(__file__).parent / "match24.json").write_text(json.dumps({"cases": cases}, indent=1, sort_keys=True))
    print("wrote", len(cases), "cases")


if __name__ == "__main__":
    main()
