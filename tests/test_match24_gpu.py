"""GPU matching statistics against the reference's own compiled CPU matchers (oracle/_ref) and
against committed dicts those modules produced (tests/golden/match24.json).  The three CPU
matchers are deterministic, so the bar is exact equality of every dict entry."""
import json
import math
import os
from pathlib import Path

import numpy as np
import pytest

from oracle import oracle as O
from trspmm import graphs

pytestmark = pytest.mark.gpu
GOLD = Path(__file__).parent / "golden" / "match24.json"

MODULES = {
    "para_dr": ("matching_utils", "match_2to4"),
    "hash": ("matching_utils_hash", "match_2to4_hash"),
    "bucket": ("matching_utils_bucket", "match_2to4_bucket"),
}


def _graph(spec):
    kind, kw = spec
    rp, col, val = getattr(graphs, kind + "_graph")(**kw)
    return rp.numpy(), col.numpy(), val.numpy()


def _same(got, want):
    assert set(got) == set(want), (sorted(got), sorted(want))
    for k, v in want.items():
        if isinstance(v, float):
            assert math.isclose(got[k], v, rel_tol=1e-12), k
        else:
            assert got[k] == v, (k, got[k], v)


@pytest.mark.parametrize("variant", sorted(MODULES))
def test_matches_committed_reference_dicts(variant):
    import importlib
    gold = json.loads(GOLD.read_text())
    mod = importlib.import_module(MODULES[variant][0])
    fn = getattr(mod, MODULES[variant][1])
    for case in gold["cases"]:
        rp, col, val = _graph(case["graph"])
        for call in case[variant]:
            _same(fn(rp, col, val, **call["kwargs"]), call["result"])


@pytest.mark.parametrize("variant", sorted(MODULES))
def test_matches_live_reference(variant):
    import importlib
    ref = O.reference_module(MODULES[variant][0])
    if ref is None:
        pytest.skip("oracle/_ref not built")
    mine = getattr(importlib.import_module(MODULES[variant][0]), MODULES[variant][1])
    theirs = getattr(ref, MODULES[variant][1])
    specs = [("rmat", dict(scale=13, edge_factor=16, seed=31)), ("clustered", dict(n=8192, community=128, intra=24, glob=4, seed=3)),
             ("uniform", dict(n=3001, per_row=9, seed=5))]
    for spec in specs:
        rp, col, val = _graph(spec)
        # the reference prints a table from C: silence fd 1 around it
        saved = os.dup(1); devnull = os.open(os.devnull, os.O_WRONLY); os.dup2(devnull, 1)
        try:
            want = dict(theirs(rp, col, val))
        finally:
            os.dup2(saved, 1); os.close(saved); os.close(devnull)
        _same(mine(rp, col, val), want)


def test_argument_errors():
    import matching_utils
    rp, col, val = _graph(("uniform", dict(n=64, per_row=3, seed=1)))
    with pytest.raises(RuntimeError):
        matching_utils.match_2to4(rp, col, val, window_size=0)
    with pytest.raises(RuntimeError):
        matching_utils.match_2to4(np.zeros(5, dtype=np.int32), np.zeros(0, dtype=np.int32), np.zeros(0, dtype=np.float32))


def test_cuda_and_online_entry_points_keep_the_invariants():
    """matching_utils_cuda / matching_utils_online: the reference versions are race-dependent, so the
    contract is the set of keys and the invariants its driver checks (test_24_matching.py:170-199,
    317-344)."""
    import torch
    import matching_utils_cuda
    import matching_utils_online
    rp, col, val = graphs.rmat_graph(12, 16, seed=8)
    nnz = col.numel()
    d = matching_utils_cuda.match_2to4(rp.cuda(), col.cuda(), val.cuda())
    assert set(d) == {"total_rows", "total_cols", "total_nnz", "sparsity", "num_row_panels", "num_groups",
                      "num_16x16_blocks", "block_padding_groups", "fine_fallback", "coarse_fallback", "fake_zeros"}
    assert d["total_nnz"] == nnz and d["num_row_panels"] == 256
    assert d["block_padding_groups"] == d["num_16x16_blocks"] * 4 - d["num_groups"]
    assert d["total_nnz"] + d["fake_zeros"] <= d["num_groups"] * 32       # capacity (test_24_matching.py:188-199)
    assert d == matching_utils_cuda.match_2to4(rp.cuda(), col.cuda(), val.cuda())   # deterministic
    with pytest.raises(RuntimeError):
        matching_utils_cuda.match_2to4(rp, col.cuda(), val.cuda())
    with pytest.raises(RuntimeError):
        matching_utils_cuda.match_2to4(rp.cuda(), col.cuda(), val.cuda(), window_size=17)
    o = matching_utils_online.match_2to4_online(rp.numpy(), col.numpy(), val.numpy())
    assert o == matching_utils_online.match_2to4_online(rp.numpy(), col.numpy(), val.numpy())   # deterministic
    assert set(o) == {"total_rows", "total_cols", "total_nnz", "num_sptc_groups", "num_tc_blocks", "dense_to_tc_cols",
                      "dense_to_sptc_cols", "fine_fb", "coarse_fb_cols", "num_16x16_blocks", "block_padding_groups",
                      "fake_zeros"}
    assert o["block_padding_groups"] == o["num_16x16_blocks"] * 4 - o["num_sptc_groups"]
    assert o["dense_to_tc_cols"] == o["num_tc_blocks"] * 8 and o["dense_to_sptc_cols"] >= 0
    assert o["total_nnz"] == nnz


def _wide_window_graph(n_rows=48, distinct=2600, seed=4):
    """A few windows, one of which touches more distinct columns than the 2048 slots of the
    reference's per-window table (the columns beyond are lost, block_matching_online.cu:163-176),
    with column ids that collide modulo 2048."""
    rng = np.random.default_rng(seed)
    rows = []
    for r in range(n_rows):
        if r < 16:
            cols = rng.choice(6000, size=distinct // 8, replace=False)
        else:
            cols = rng.choice(6000, size=int(rng.integers(0, 40)), replace=False)
        rows.append(np.sort(cols))
    rp = np.zeros(n_rows + 1, dtype=np.int32)
    rp[1:] = np.cumsum([len(c) for c in rows])
    col = np.concatenate(rows).astype(np.int32)
    return rp, col, np.ones(col.size, dtype=np.float32)


@pytest.mark.parametrize("case", ["rmat", "clustered", "uniform_ragged", "wide", "threshold"])
def test_online_variant_matches_its_cpu_replay(case):
    """trs_match24_stats variant 3 against oracle.match_online_emulation: the same rules
    (block_matching_online.cu:85-431) replayed in plain Python for the row-sequential schedule."""
    import matching_utils_online
    kw = {}
    if case == "rmat":
        rp, col, val = (t.numpy() for t in graphs.rmat_graph(9, 12, seed=3))
    elif case == "clustered":
        rp, col, val = (t.numpy() for t in graphs.clustered_graph(n=600, community=64, intra=20, glob=3, seed=2))
    elif case == "uniform_ragged":
        rp, col, val = (t.numpy() for t in graphs.uniform_graph(n=333, per_row=7, seed=9))
    elif case == "wide":
        rp, col, val = _wide_window_graph()
    else:
        rp, col, val = (t.numpy() for t in graphs.rmat_graph(9, 12, seed=5))
        kw = dict(dense_threshold=4, t_max=2)
    got = matching_utils_online.match_2to4_online(rp, col, val, **kw)
    want = O.match_online_emulation(rp, col, **kw)
    want["fake_zeros"] = ((want["fake_zeros"] + 2 ** 31) % 2 ** 32) - 2 ** 31
    assert got == want
    if case == "wide":
        assert got["total_nnz"] == col.size      # the input count, lost columns included


def _heavy_window_graph(seed=6):
    """48 rows: a window of ~1400 non-zeros (above the 512 of the reference's light class, so its
    table is compacted with the 1024-thread stride), a light one, and a ragged last window."""
    rng = np.random.default_rng(seed)
    rows = []
    for r in range(44):
        k = int(rng.integers(60, 120)) if r < 16 else int(rng.integers(0, 12))
        rows.append(np.sort(rng.choice(3000, size=k, replace=False)))
    rp = np.zeros(len(rows) + 1, dtype=np.int32)
    rp[1:] = np.cumsum([len(c) for c in rows])
    col = np.concatenate(rows).astype(np.int32)
    return rp, col, np.ones(col.size, dtype=np.float32)


@pytest.mark.parametrize("case", ["rmat", "clustered", "uniform_ragged", "heavy", "window8"])
def test_cuda_variant_matches_its_cpu_replay(case):
    """trs_match24_stats variant 4 against oracle.match_cuda_emulation: the rules of
    block_match_cuda.cu:822-1201 replayed in plain Python for the same schedule."""
    import torch
    import matching_utils_cuda
    kw = {}
    if case == "rmat":
        rp, col, val = (t.numpy() for t in graphs.rmat_graph(9, 12, seed=3))
    elif case == "clustered":
        rp, col, val = (t.numpy() for t in graphs.clustered_graph(n=600, community=64, intra=20, glob=3, seed=2))
    elif case == "uniform_ragged":
        rp, col, val = (t.numpy() for t in graphs.uniform_graph(n=333, per_row=7, seed=9))
    elif case == "heavy":
        rp, col, val = _heavy_window_graph()
    else:
        rp, col, val = (t.numpy() for t in graphs.rmat_graph(8, 10, seed=5))
        kw = dict(window_size=8)
    got = matching_utils_cuda.match_2to4(torch.from_numpy(rp).cuda(), torch.from_numpy(col).cuda(),
                                         torch.from_numpy(val).cuda(), **kw)
    _same(got, O.match_cuda_emulation(rp, col, **kw))
