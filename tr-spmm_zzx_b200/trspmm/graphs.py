"""Seeded synthetic sparse matrices standing in for the SuiteSparse / DGL graphs the reference
benchmarks on (TR-source/README.md:200-211, spmm/tr_csr_fp16/tr_paths.py:22-30), which are
not redistributable here.

Every generator returns canonical CSR — int32 row pointers, int32 column ids ascending and
duplicate-free per row, fp32 values — which is what scipy's ``tocsr()`` hands the reference
builder (spmm/tr_csr_fp16/mdataset2_online.py:62-98).  All work is vectorised torch on the
requested device; a (seed, device type) pair fixes the output.
"""
from __future__ import annotations

import torch


def _gen(seed: int, device) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return g


def coo_to_csr(rows: torch.Tensor, cols: torch.Tensor, n_rows: int, n_cols: int):
    """Sort + deduplicate COO coordinates; returns (rowptr int32, col int32, row int64)."""
    key = torch.unique(rows.long() * n_cols + cols.long())  # sorted, unique
    r = torch.div(key, n_cols, rounding_mode="floor")
    c = (key - r * n_cols).to(torch.int32)
    counts = torch.bincount(r, minlength=n_rows)
    rowptr = torch.zeros(n_rows + 1, dtype=torch.int64, device=key.device)
    rowptr[1:] = torch.cumsum(counts, 0)
    if rowptr[-1] >= 2 ** 31:
        raise ValueError("nnz does not fit the reference's int32 row pointers")
    return rowptr.to(torch.int32), c, r


def _gcn_values(rowptr, col, row):
    deg = (rowptr[1:] - rowptr[:-1]).float().clamp_min(1.0)
    return (deg[row].rsqrt() * deg[col.long()].rsqrt()).float()


def uniform_graph(n: int = 4096, per_row: int = 16, seed: int = 0, device="cpu"):
    """`per_row` distinct uniform columns per row plus the diagonal; values 1/deg(row)."""
    g = _gen(seed, device)
    if n <= 8192:
        pick = torch.rand(n, n, generator=g, device=device).argsort(dim=1)[:, :per_row]
    else:  # with replacement, duplicates removed below
        pick = torch.randint(n, (n, per_row), generator=g, device=device)
    rows = torch.arange(n, device=device).repeat_interleave(per_row + 1)
    cols = torch.cat([pick, torch.arange(n, device=device)[:, None]], dim=1).reshape(-1)
    rowptr, col, row = coo_to_csr(rows, cols, n, n)
    deg = (rowptr[1:] - rowptr[:-1]).float()
    return rowptr, col, (1.0 / deg)[row].float()


def clustered_graph(n: int = 262144, community: int = 128, intra: int = 24, glob: int = 4,
                    seed: int = 0, device="cpu"):
    """Stochastic-block graph: per row `intra` uniform edges inside its community, `glob` uniform
    global edges and a self loop; symmetrised, deduplicated; values 1/sqrt(deg_i deg_j)."""
    g = _gen(seed, device)
    base = (torch.arange(n, device=device) // community) * community
    ci = base[:, None] + torch.randint(community, (n, intra), generator=g, device=device)
    cg = torch.randint(n, (n, glob), generator=g, device=device)
    cols = torch.cat([ci, cg], dim=1).clamp_max(n - 1).reshape(-1)
    rows = torch.arange(n, device=device).repeat_interleave(intra + glob)
    diag = torch.arange(n, device=device)
    rowptr, col, row = coo_to_csr(torch.cat([rows, cols, diag]), torch.cat([cols, rows, diag]), n, n)
    return rowptr, col, _gcn_values(rowptr, col, row)


def rmat_graph(scale: int, edge_factor: int, a=0.57, b=0.19, c=0.19, d=0.05, seed: int = 0,
               device="cpu", chunk: int = 1 << 24):
    """Power-law R-MAT graph, symmetrised, deduplicated, self loops added, GCN-normalised values."""
    g = _gen(seed, device)
    n = 1 << scale
    m = n * edge_factor
    keys = []
    for s in range(0, m, chunk):
        k = min(chunk, m - s)
        src = torch.zeros(k, dtype=torch.int64, device=device)
        dst = torch.zeros(k, dtype=torch.int64, device=device)
        for _ in range(scale):
            u = torch.rand(k, generator=g, device=device)
            sbit = (u >= a + b).long()                       # quadrants c, d -> lower half
            dbit = (((u >= a) & (u < a + b)) | (u >= a + b + c)).long()  # quadrants b, d -> right half
            src = (src << 1) | sbit
            dst = (dst << 1) | dbit
        keys.append(torch.unique(torch.cat([src * n + dst, dst * n + src])))
    diag = torch.arange(n, device=device, dtype=torch.int64)
    key = torch.unique(torch.cat(keys + [diag * n + diag]))
    del keys
    row = torch.div(key, n, rounding_mode="floor")
    col = (key - row * n).to(torch.int32)
    del key
    counts = torch.bincount(row, minlength=n)
    rowptr = torch.zeros(n + 1, dtype=torch.int64, device=device)
    rowptr[1:] = torch.cumsum(counts, 0)
    if rowptr[-1] >= 2 ** 31:
        raise ValueError("nnz does not fit the reference's int32 row pointers")
    rowptr = rowptr.to(torch.int32)
    return rowptr, col, _gcn_values(rowptr, col, row)


def pad_rows(rowptr: torch.Tensor, window: int = 16):
    """Pad the row count to a multiple of `window` with empty rows (mdataset2_online.py:60-63)."""
    n = rowptr.numel() - 1
    extra = (-n) % window
    if extra == 0:
        return rowptr
    return torch.cat([rowptr, rowptr[-1:].expand(extra)])
