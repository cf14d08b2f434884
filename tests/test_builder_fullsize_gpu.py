"""The GPU builder pinned at the benchmark sizes, window by window.

BASELINE configs 1, 2 and 4 (clustered N = 262 144, R-MAT scale 21, R-MAT scale 20) are built whole
on the GPU; the reference's CPU builder cannot do that (its matching is quadratic in the columns
of a window in time and memory, block_online.cpp:340-352).  Windows are independent
(block_online.cpp:584-734), so for >= 64 sampled windows per matrix - the 8 heaviest, 8 whose unit
counts sit next to the builder's tier thresholds (one thread / one warp / one block per window),
the rest random - the window's segment of all 29 arrays is compared bit for bit with the pinned
restatement run on the window's 16 rows alone and, where the compiled reference finishes within a
few seconds, with the reference itself.  The windows the reference is not run on are reported."""
import time

import pytest
import torch

from oracle import oracle as O
from trspmm import build_format, graphs
from window_slices import compare_window, pick_windows, slice_window, window_segment

pytestmark = pytest.mark.gpu

REFERENCE_MAX_GROUPS = 6000   # ~ 12 000 units: about 4 s and 0.6 GB in the reference's O(U^2) matching


@pytest.mark.parametrize("workload", ["rmat21", "rmat20", "clustered"])
def test_sampled_windows_equal_cpu_builders(workload, record_property):
    dev = torch.device("cuda")
    if workload == "rmat21":
        rp, col, val = graphs.rmat_graph(21, 32, seed=0, device=dev)
    elif workload == "rmat20":
        rp, col, val = graphs.rmat_graph(20, 16, seed=0, device=dev)
    else:
        rp, col, val = graphs.clustered_graph(262144, 128, 24, 4, seed=0, device=dev)
    fmt, _ = build_format(rp, col, val)
    named = dict(zip(O.FORMAT_NAMES, fmt.arrays()))
    groups = (named["s_offset"][1:] - named["s_offset"][:-1]).cpu()
    windows = pick_windows(groups, n_heavy=8, thresholds=(48, 1024), per_threshold=4, n_random=52, seed=7)
    assert len(windows) >= 64
    rp_c = rp.cpu()
    have_ref = O.reference_module("Libra5BlockOnline") is not None
    excluded, ref_checked, slowest = [], 0, 0.0
    for w in windows:
        sub = slice_window(rp_c, col, val, w)
        seg = window_segment(named, w)
        compare_window(seg, O.build_format(*sub)[0], f"{workload} window {w} (restatement)")
        if have_ref and int(groups[w]) <= REFERENCE_MAX_GROUPS:
            t0 = time.perf_counter()
            compare_window(seg, O.reference_builder(*sub)[:29], f"{workload} window {w} (compiled reference)")
            slowest = max(slowest, time.perf_counter() - t0)
            ref_checked += 1
        else:
            excluded.append((w, int(groups[w])))
    record_property("windows_checked", len(windows))
    record_property("windows_checked_against_compiled_reference", ref_checked)
    record_property("windows_not_run_through_the_reference(window, groups)", excluded)
    print(f"{workload}: {len(windows)} windows vs restatement, {ref_checked} vs compiled reference "
          f"(slowest {slowest:.1f} s); reference not run on (window, groups): {excluded}")
    if have_ref:
        assert ref_checked >= 48
