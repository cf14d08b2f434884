#!/usr/bin/env python3
"""Generate the committed fixtures from the reference's own compiled builder.

Run in a container that has the reference tree (it cannot travel to a GPU box):

    python oracle/build_ref.py && python tests/golden/make_golden.py

For each seeded case the reference module Libra5BlockOnline.block_sptc_2to4_online
(TR-source/Block/block_online.cpp:545-871, compiled unmodified into oracle/_ref) is run and
its 29 array outputs are stored, together with the CSR input, in tests/golden/<case>.npz.
For the larger cases only SHA-256 digests of the arrays are stored (digests.json), the
inputs being regenerated from their seeds by the tests.
"""
import hashlib
import json
import os
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT / "tr-spmm_zzx_b200"))
sys.path.insert(0, str(ROOT))

from oracle import oracle as O  # noqa: E402
from trspmm import graphs  # noqa: E402

# name -> (generator, generator kwargs, builder kwargs, env)
SMALL_CASES = {
    "uniform_n256": ("uniform_graph", dict(n=256, per_row=8, seed=0), {}, {}),
    "uniform_n250_ragged": ("uniform_graph", dict(n=250, per_row=6, seed=1), {}, {}),
    "clustered_n512": ("clustered_graph", dict(n=512, community=64, intra=12, glob=2, seed=0), {}, {}),
    "clustered_n512_density4": ("clustered_graph", dict(n=512, community=64, intra=12, glob=2, seed=0),
                                dict(density=4), {}),
    "rmat_s9": ("rmat_graph", dict(scale=9, edge_factor=8, seed=0), {}, {}),
    "rmat_s9_parts": ("rmat_graph", dict(scale=9, edge_factor=8, seed=0),
                      dict(part_t=2, part_c=4, short_size=1, tc_min_util=0.55), {}),
    "rmat_s9_minnnz": ("rmat_graph", dict(scale=9, edge_factor=8, seed=2), dict(short_size=1),
                       {"LIBRA_SPTC_UNIT_MIN_NNZ": "40"}),
    "rmat_s9_skiptc": ("rmat_graph", dict(scale=9, edge_factor=8, seed=3), {}, {"LIBRA_SKIP_TC": "1"}),
}
DIGEST_CASES = {
    "config0_uniform_n4096": ("uniform_graph", dict(n=4096, per_row=16, seed=0), {}, {}),
    "clustered_n4096": ("clustered_graph", dict(n=4096, community=128, intra=24, glob=4, seed=0), {}, {}),
    "rmat_s13": ("rmat_graph", dict(scale=13, edge_factor=16, seed=0), {}, {}),
}


def run_reference(gen, gkw, bkw, env):
    rp, col, val = getattr(graphs, gen)(**gkw)
    saved = {k: os.environ.get(k) for k in env}
    os.environ.update(env)
    try:
        out = O.reference_builder(rp, col, val, **bkw)
    finally:
        for k, v in saved.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v
    if out is None:
        raise SystemExit("oracle/_ref is not built: run python oracle/build_ref.py first")
    return (rp, col, val), out[:29]


def digest(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().numpy().tobytes()).hexdigest()


def main():
    here = Path(__file__).resolve().parent
    for name, (gen, gkw, bkw, env) in SMALL_CASES.items():
        (rp, col, val), arrs = run_reference(gen, gkw, bkw, env)
        payload = {"in_rowptr": rp.numpy(), "in_col": col.numpy(), "in_val": val.numpy()}
        payload.update({n: a.numpy() for n, a in zip(O.FORMAT_NAMES, arrs)})
        np.savez_compressed(here / f"{name}.npz", **payload)
        print(name, "nnz", col.numel(), "groups", arrs[17].shape[0], "tc blocks", arrs[2].numel() // 8,
              "long parts", arrs[8].numel(), "short parts", arrs[13].numel())
    digests = {}
    for name, (gen, gkw, bkw, env) in DIGEST_CASES.items():
        (rp, col, val), arrs = run_reference(gen, gkw, bkw, env)
        digests[name] = {"input": {"rowptr": digest(rp), "col": digest(col), "val": digest(val)},
                         "shapes": {n: list(a.shape) for n, a in zip(O.FORMAT_NAMES, arrs)},
                         "sha256": {n: digest(a) for n, a in zip(O.FORMAT_NAMES, arrs)}}
        print(name, "nnz", col.numel())
    meta = {"small": {k: [v[0], v[1], v[2], v[3]] for k, v in SMALL_CASES.items()},
            "digest": {k: [v[0], v[1], v[2], v[3]] for k, v in DIGEST_CASES.items()}}
    (here / "cases.json").write_text(json.dumps(meta, indent=1, sort_keys=True))
    (here / "digests.json").write_text(json.dumps(digests, indent=1, sort_keys=True))


if __name__ == "__main__":
    main()
