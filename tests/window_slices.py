"""Window-by-window comparison of format arrays (test infrastructure).

Every 16-row window of the reference's builder is processed independently
(TR-source/Block/block_online.cpp:584-734), so the segment a window contributes to each of the 29
output arrays equals, after subtracting the prefix offsets, the whole output of the builder run on
those 16 rows alone (row pointers rebased, column ids kept global).  `window_segment` cuts that
segment out of a full format; `slice_window` makes the 16-row CSR; `compare_window` checks them
array by array.  This is how builds too large for the CPU builder are pinned: sampled windows of
the GPU-built format against the restatement and the compiled reference run on the slices.
"""
from __future__ import annotations

import torch

from oracle import oracle as O


def slice_window(rp, col, val, w, window=16):
    """CSR of rows [w * window, (w + 1) * window) as CPU tensors (17 row pointers starting at 0)."""
    n = rp.numel() - 1
    r0, r1 = w * window, min((w + 1) * window, n)
    e0, e1 = int(rp[r0]), int(rp[r1])
    sub = (rp[r0:r1 + 1] - e0).to(torch.int32).cpu()
    if r1 - r0 < window:  # ragged last window: pad with empty rows, as the reference's caller does
        sub = torch.cat([sub, sub[-1:].expand(window - (r1 - r0))])
    return sub.contiguous(), col[e0:e1].cpu().contiguous(), val[e0:e1].cpu().contiguous()


def _range_of(sorted_keys, lo, hi):
    a = int(torch.searchsorted(sorted_keys, torch.tensor(lo, device=sorted_keys.device, dtype=sorted_keys.dtype)))
    b = int(torch.searchsorted(sorted_keys, torch.tensor(hi, device=sorted_keys.device, dtype=sorted_keys.dtype)))
    return a, b


def window_segment(named, w, window=16):
    """The part of every array that window w produced, rebased as if w were the only window.
    `named`: dict name -> tensor of a full format (any device).  Returns dict name -> CPU tensor."""
    out = {}
    row_lo, row_hi = w * window, (w + 1) * window
    # ---- TC parts (t_window_row holds w * 16 per part, ascending)
    twr = named["t_window_row"]
    p0, p1 = _range_of(twr, row_lo, row_lo + 1) if twr.numel() else (0, 0)
    tro = named["t_row_offset"]
    if p1 > p0:
        b0, b1 = int(tro[p0]), int(tro[p1])
        tbo = named["t_block_offset"]
        v0, v1 = int(tbo[b0]), int(tbo[b1])
        out["t_row_offset"] = tro[p0:p1 + 1] - b0
        out["t_block_offset"] = tbo[b0:b1 + 1] - v0
        out["t_column"] = named["t_column"][8 * b0:8 * b1]
        out["t_value"] = named["t_value"][v0:v1]
        out["t_window_row"] = twr[p0:p1] - row_lo
        out["t_atomic"] = named["t_atomic"][p0:p1]
        out["t_binary"] = named["t_binary"][2 * b0:2 * b1]
    else:
        for k in ("t_row_offset", "t_block_offset", "t_column", "t_value", "t_window_row", "t_atomic", "t_binary"):
            out[k] = named[k][:0]
    # ---- CSR parts (c_row / cs_row hold global rows, ascending)
    for k in ("c", "cs"):
        rows = named[f"{k}_row"]
        q0, q1 = _range_of(rows, row_lo, row_hi) if rows.numel() else (0, 0)
        if q1 > q0:
            off = named[f"{k}_row_offset"]
            e0, e1 = int(off[q0]), int(off[q1])
            out[f"{k}_row_offset"] = off[q0:q1 + 1] - e0
            out[f"{k}_row"] = rows[q0:q1] - row_lo
            out[f"{k}_atomic"] = named[f"{k}_atomic"][q0:q1]
            out[f"{k}_column"] = named[f"{k}_column"][e0:e1]
            out[f"{k}_value"] = named[f"{k}_value"][e0:e1]
        else:
            for s in ("row_offset", "row", "atomic", "column", "value"):
                out[f"{k}_{s}"] = named[f"{k}_{s}"][:0]
    # ---- SPTC groups and tiles
    so, wto = named["s_offset"], named["s_window_tile_offset"]
    g0, g1 = int(so[w]), int(so[w + 1])
    t0, t1 = int(wto[w]), int(wto[w + 1])
    for k in ("s_column", "s_mask", "s_value", "s_pos"):
        out[k] = named[k][g0:g1]
    out["s_window"] = named["s_window"][g0:g1] - w
    out["s_offset"] = torch.tensor([0, g1 - g0], dtype=torch.int32)
    out["s_tile_window"] = named["s_tile_window"][t0:t1] - w
    out["s_tile_group"] = named["s_tile_group"][t0:t1] - g0
    for k in ("s_tile_column", "s_packed_a", "s_packed_meta"):
        out[k] = named[k][t0:t1]
    out["s_window_tile_offset"] = torch.tensor([0, t1 - t0], dtype=torch.int32)
    return {k: v.cpu() for k, v in out.items()}


def _flat_or_empty(t):
    return t.reshape(-1)


def compare_window(segment, single, what=""):
    """`single`: the 29 arrays of a builder run on the window's 16 rows alone.  A prefix array of a
    route the window does not use may come back as [0] or as empty; both mean "no parts"."""
    single = dict(zip(O.FORMAT_NAMES, single))
    for name in O.FORMAT_NAMES:
        a, b = segment[name], single[name].cpu()
        if name in ("t_row_offset", "t_block_offset", "c_row_offset", "cs_row_offset") and a.numel() <= 1 and b.numel() <= 1:
            continue
        assert a.dtype == b.dtype, (what, name, a.dtype, b.dtype)
        assert a.numel() == b.numel(), (what, name, tuple(a.shape), tuple(b.shape))
        assert torch.equal(_flat_or_empty(a), _flat_or_empty(b)), (what, name)


def pick_windows(groups_per_window, n_heavy=8, thresholds=(48, 1024), per_threshold=4, n_random=48, seed=0):
    """Window ids to pin: the heaviest ones, the ones whose unit count sits next to the builder's
    tier thresholds (a window with G matched groups has about 2 G units), and a seeded random rest."""
    g = groups_per_window.to(torch.int64).cpu()
    W = g.numel()
    chosen = []
    order = torch.argsort(g, descending=True, stable=True)
    chosen += order[:min(n_heavy, W)].tolist()
    for thr in thresholds:
        dist = (g - thr).abs()
        below = torch.where(g <= thr, dist, torch.full_like(dist, 1 << 40))
        above = torch.where(g > thr, dist, torch.full_like(dist, 1 << 40))
        half = per_threshold // 2
        chosen += torch.argsort(below, stable=True)[:half].tolist()
        chosen += torch.argsort(above, stable=True)[:per_threshold - half].tolist()
    gen = torch.Generator().manual_seed(seed)
    chosen += torch.randint(0, W, (n_random,), generator=gen).tolist()
    seen, out = set(), []
    for w in chosen:
        if w not in seen:
            seen.add(w)
            out.append(int(w))
    return out
