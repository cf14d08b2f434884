"""Matrix ingestion compatible with the reference's loaders: MatrixMarket files and the two .npz
layouts its drivers read (TR-source/test_24_matching.py:80-146, spmm/tr_csr_fp16/tr_paths.py:22-30).
Returns canonical CSR as torch tensors (int32 row pointers and columns, float32 values)."""
from __future__ import annotations

import os

import numpy as np
import torch


def load_matrix(path: str, device="cpu"):
    """`.mtx` (coordinate or array; real / integer / pattern; general / symmetric) or `.npz`
    (scipy.sparse.save_npz layout, or the edge-list layout with src_li / dst_li [/ data] and either
    `shape` or num_nodes_src / num_nodes_dst).  Duplicate entries are summed, columns sorted."""
    import scipy.sparse as sp
    ext = os.path.splitext(path)[1].lower()
    if ext == ".npz":
        raw = np.load(path)
        keys = set(raw.keys())
        if "format" in keys or "indices" in keys:
            mat = sp.load_npz(path)
        else:
            src, dst = raw["src_li"], raw["dst_li"]
            val = raw["data"].astype(np.float32) if "data" in keys else np.ones(len(src), dtype=np.float32)
            if "shape" in keys:
                shape = tuple(int(x) for x in raw["shape"].tolist())
            else:
                shape = (int(raw["num_nodes_src"]), int(raw["num_nodes_dst"]))
            mat = sp.coo_matrix((val, (src, dst)), shape=shape)
    elif ext == ".mtx":
        from scipy.io import mminfo, mmread
        field = mminfo(path)[4]
        mat = mmread(path)
        if isinstance(mat, np.ndarray):
            mat = sp.csr_matrix(mat)
        elif field == "pattern":
            mat.data = np.ones(mat.nnz, dtype=np.float32)
    else:
        raise ValueError(f"unsupported matrix file type: {ext}")
    mat = mat.tocsr()
    mat.sum_duplicates()
    mat.sort_indices()
    if mat.indptr[-1] >= 2 ** 31:
        raise ValueError("nnz does not fit int32 row pointers")
    rowptr = torch.from_numpy(mat.indptr.astype(np.int32)).to(device)
    col = torch.from_numpy(mat.indices.astype(np.int32)).to(device)
    val = torch.from_numpy(mat.data.astype(np.float32)).to(device)
    return rowptr, col, val, mat.shape
