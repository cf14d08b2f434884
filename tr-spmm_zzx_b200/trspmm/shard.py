"""Row-window sharding for one multi-GPU box.

Every 16-row window is an independent unit of both the builder and the SpMM
(TR-source/Block/block_online.cpp:584 loops over windows; the SPTC kernel's grid x is the
window, TR-source/SpMM/mGCNkernel_online.cu:830), so the matrix is cut into contiguous window
ranges of about equal nnz, one per rank.  Each rank builds and multiplies its own rows against
a full replica of B; no collective is needed for a single SpMM.
"""
from __future__ import annotations

import torch


def balanced_window_cuts(rowptr: torch.Tensor, parts: int, window: int = 16):
    """Row boundaries [r_0=0, r_1, ..., r_parts=n_rows], every inner boundary a multiple of
    `window`, chosen so that each range holds about nnz/parts entries."""
    n = rowptr.numel() - 1
    W = (n + window - 1) // window
    idx = torch.arange(0, W + 1, device=rowptr.device) * window
    idx[-1] = n
    prefix = rowptr[idx.clamp_max(n)].long()  # nnz before each window boundary
    total = int(prefix[-1])
    cuts = [0]
    for k in range(1, parts):
        target = total * k // parts
        w = int(torch.searchsorted(prefix, torch.tensor(target, device=prefix.device), right=False))
        # choose the boundary closest to the target among w-1, w
        if w > 0 and abs(int(prefix[w - 1]) - target) <= abs(int(prefix[min(w, W)]) - target):
            w -= 1
        w = max(w, cuts[-1] // window if cuts[-1] % window == 0 else 0)
        cuts.append(min(w, W) * window if w < W else n)
    cuts.append(n)
    for i in range(1, len(cuts)):  # monotone
        cuts[i] = max(cuts[i], cuts[i - 1])
    return cuts


def cuts_from_window_costs(cost: torch.Tensor, parts: int, n_rows: int, window: int = 16):
    """Row boundaries from a per-window cost vector (e.g. k-steps of the built format + a fixed
    per-window overhead): contiguous window ranges of about equal total cost."""
    W = cost.numel()
    prefix = torch.zeros(W + 1, dtype=torch.float64, device=cost.device)
    prefix[1:] = torch.cumsum(cost.double(), 0)
    total = float(prefix[-1])
    cuts = [0]
    for k in range(1, parts):
        w = int(torch.searchsorted(prefix, torch.tensor(total * k / parts, dtype=torch.float64, device=cost.device)))
        w = min(max(w, cuts[-1] // window), W)
        cuts.append(min(w * window, n_rows))
    cuts.append(n_rows)
    for i in range(1, len(cuts)):
        cuts[i] = max(cuts[i], cuts[i - 1])
    return cuts


def window_steps(fmt, n_windows: int):
    """k-steps per window of a built format: packed tiles + pairs of TC blocks."""
    off = fmt.s_window_tile_offset
    steps = (off[1:] - off[:-1]).to(torch.float32)
    if steps.numel() < n_windows:
        steps = torch.cat([steps, torch.zeros(n_windows - steps.numel(), device=steps.device)])
    if fmt.t_window_row.numel():
        blocks_per_part = (fmt.t_row_offset[1:] - fmt.t_row_offset[:-1]).to(torch.float32)
        win = (fmt.t_window_row // 16).long()
        blocks = torch.zeros(n_windows, device=steps.device).index_add_(0, win, blocks_per_part)
        steps = steps + torch.ceil(blocks / 2)
    return steps


def slice_csr(rowptr: torch.Tensor, col: torch.Tensor, val: torch.Tensor, r0: int, r1: int):
    """Rows [r0, r1) as their own CSR (row pointers rebased, global column ids kept)."""
    b, e = int(rowptr[r0]), int(rowptr[r1])
    return (rowptr[r0:r1 + 1] - rowptr[r0]).to(torch.int32).contiguous(), col[b:e].contiguous(), val[b:e].contiguous()


def shard_for_rank(rowptr, col, val, rank: int, world: int, window: int = 16):
    cuts = balanced_window_cuts(rowptr, world, window)
    r0, r1 = cuts[rank], cuts[rank + 1]
    return (r0, r1), slice_csr(rowptr, col, val, r0, r1)
