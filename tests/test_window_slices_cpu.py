"""Window independence of the builder, on the CPU: every window's segment of a full build equals
the build of that window's 16 rows alone (block_online.cpp:584-734 processes windows one by
one).  This is the property the full-size GPU test rests on; here the pinned restatement plays
both roles and, where the reference's compiled builder is present, the reference builds the slices."""
import pytest
import torch

from oracle import oracle as O
from trspmm import graphs
from window_slices import compare_window, pick_windows, slice_window, window_segment


@pytest.mark.parametrize("case", [
    ("rmat", dict(scale=11, edge_factor=16, seed=2), {}),
    ("clustered", dict(n=2048, community=128, intra=24, glob=4, seed=3), {}),
    ("uniform", dict(n=1000, per_row=9, seed=4), dict(short_size=1, part_c=2)),
])
def test_segments_equal_single_window_builds(case):
    kind, gkw, bkw = case
    rp, col, val = getattr(graphs, kind + "_graph")(**gkw)
    full, _ = O.build_format(rp, col, val, **bkw)
    named = dict(zip(O.FORMAT_NAMES, full))
    groups = named["s_offset"][1:] - named["s_offset"][:-1]
    have_ref = O.reference_module("Libra5BlockOnline") is not None
    last = (rp.numel() - 2) // 16
    for w in pick_windows(groups, n_heavy=4, thresholds=(48,), per_threshold=2, n_random=10, seed=1) + [last]:
        sub = slice_window(rp, col, val, w)
        seg = window_segment(named, w)
        compare_window(seg, O.build_format(*sub, **bkw)[0], f"{kind} window {w} (restatement)")
        if have_ref:
            compare_window(seg, O.reference_builder(*sub, **bkw)[:29], f"{kind} window {w} (compiled reference)")
