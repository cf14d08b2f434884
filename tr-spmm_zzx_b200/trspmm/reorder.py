"""Deterministic row reordering on the device: the slot the reference fills with
apply_tca_reorder (spmm/tr_csr_fp16/tr_tca_reorder.py:44-357, called from
mdataset2_online.py:73-94 when LIBRA_TCA_REORDER=1).

The reference clusters rows with similar column sets (MinHash LSH from the third-party
`datasketch` package, Jaccard similarity, a priority queue and union-find, clusters of at most 16
rows, then clusters of clusters) in pure Python; columns keep their ids, only rows move, and the
function returns the permuted CSR plus `reorder_id` (new row -> old row).  Here the same
contract is served by sort-based orders that run as a handful of torch kernels on the GPU and do
not depend on hash-table iteration order:

  "minhash"  rows sorted lexicographically by `num_hashes` min-hash values of their column sets:
             two rows share a min-hash with probability equal to their Jaccard similarity, so
             similar rows become neighbours and land in the same 16-row window;
  "hub"      rows sorted by their most popular column (highest column degree), then by degree:
             rows hanging off the same hub share at least that column;
  "degree"   rows sorted by descending degree (dense windows first, TC blocks more likely).

The permutation differs from the reference's (its result depends on datasketch's random
permutations and on Python set order; datasketch is not available here), so this is a labelled
configuration of its own, never a parity case: what is tested is that it is a permutation, that
the permuted CSR is exactly the row-gathered matrix, and that it lowers the number of distinct
(window, column) pairs on graphs with hidden structure.
"""
from __future__ import annotations

import numpy as np
import torch

METHODS = ("minhash", "hub", "degree")
_MERSENNE = (1 << 31) - 1


def _rows_of(rowptr: torch.Tensor) -> torch.Tensor:
    n = rowptr.numel() - 1
    deg = (rowptr[1:] - rowptr[:-1]).long()
    return torch.repeat_interleave(torch.arange(n, device=rowptr.device), deg), deg


def _lexsort(keys) -> torch.Tensor:
    """Stable lexicographic argsort; keys[0] is the most significant."""
    perm = torch.arange(keys[0].numel(), device=keys[0].device)
    for k in reversed(keys):
        perm = perm[torch.sort(k[perm], stable=True).indices]
    return perm


def row_order(rowptr: torch.Tensor, col: torch.Tensor, method: str = "minhash", num_hashes: int = 4,
              seed: int = 2022, n_cols: int | None = None) -> torch.Tensor:
    """reorder_id (int64, new row -> old row) for the CSR pattern, on the pattern's device."""
    if method not in METHODS:
        raise ValueError(f"method must be one of {METHODS}")
    n = rowptr.numel() - 1
    dev = rowptr.device
    rows, deg = _rows_of(rowptr)
    c = col.long()
    if method == "degree":
        return torch.sort(-deg, stable=True).indices
    if method == "hub":
        if n_cols is None:
            n_cols = int(c.max()) + 1 if c.numel() else 1
        pop = torch.bincount(c, minlength=n_cols)
        # rank 0 = most popular column; ties by column id
        order = torch.sort(-pop, stable=True).indices
        rank = torch.empty_like(order)
        rank[order] = torch.arange(n_cols, device=dev)
        hub = torch.full((n,), n_cols, dtype=torch.long, device=dev)
        hub.scatter_reduce_(0, rows, rank[c], reduce="amin", include_self=True)
        return _lexsort([hub, -deg])
    gen = np.random.default_rng(seed)
    keys = []
    for _ in range(num_hashes):
        a = int(gen.integers(1, _MERSENNE))
        b = int(gen.integers(0, _MERSENNE))
        h = (c * a + b) % _MERSENNE
        sig = torch.full((n,), _MERSENNE, dtype=torch.long, device=dev)  # empty rows sort last
        sig.scatter_reduce_(0, rows, h, reduce="amin", include_self=True)
        keys.append(sig)
    return _lexsort(keys)


def permute_rows(rowptr: torch.Tensor, col: torch.Tensor, val: torch.Tensor | None, reorder_id: torch.Tensor):
    """CSR whose row i is row reorder_id[i] of the input (columns and the order inside a row kept)."""
    rid = reorder_id.long()
    n = rowptr.numel() - 1
    if rid.numel() != n:
        raise ValueError("reorder_id must have one entry per row")
    rp = rowptr.long()
    deg = (rp[1:] - rp[:-1])[rid]
    new_rp = torch.zeros(n + 1, dtype=torch.long, device=rowptr.device)
    new_rp[1:] = torch.cumsum(deg, 0)
    shift = torch.repeat_interleave(rp[:-1][rid] - new_rp[:-1], deg)
    src = torch.arange(col.numel(), device=col.device) + shift
    new_val = val[src] if val is not None else None
    return new_rp.to(rowptr.dtype), col[src], new_val


def window_column_pairs(rowptr: torch.Tensor, col: torch.Tensor, window: int = 16) -> int:
    """Number of distinct (row window, column) pairs: the B rows a window-wise SpMM gathers."""
    rows, _ = _rows_of(rowptr)
    n_cols = int(col.max()) + 1 if col.numel() else 1
    return int(torch.unique(torch.div(rows, window, rounding_mode="floor") * n_cols + col.long()).numel())


def apply_tca_reorder(row_ptr, col_ind, num_nodes, thres=16, verbose=True, method="minhash"):
    """Call-compatible with the reference function (numpy in, numpy out):
    returns (new_row_ptr int32, new_col_ind int32, reorder_id int32 new -> old).
    `thres` (the reference's maximal cluster size) has no role in a sort-based order."""
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    rp = torch.as_tensor(np.asarray(row_ptr), device=dev)[: num_nodes + 1]
    ci = torch.as_tensor(np.asarray(col_ind), device=dev)
    before = window_column_pairs(rp, ci) if verbose else 0
    rid = row_order(rp, ci, method)
    nrp, nci, _ = permute_rows(rp, ci, None, rid)
    if verbose:
        print(f"TCA ({method}): (window, column) pairs {before} -> {window_column_pairs(nrp, nci)}")
    return (nrp.cpu().numpy().astype(np.int32), nci.cpu().numpy().astype(np.int32),
            rid.cpu().numpy().astype(np.int32))
