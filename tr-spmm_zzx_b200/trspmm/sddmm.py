"""SDDMM on a CSR pattern (trs_sddmm).  The reference has no such operator; the definition is
out[e] = fp16(sum_k fp32(X[row(e),k]) * fp32(Y[col(e),k])) in CSR entry order."""
from __future__ import annotations

import torch

from . import _lib


def sddmm(rowptr: torch.Tensor, col: torch.Tensor, X: torch.Tensor, Y: torch.Tensor,
          out: torch.Tensor | None = None) -> torch.Tensor:
    lib = _lib.load()
    dev = X.device
    if dev.type != "cuda":
        raise ValueError("sddmm needs CUDA tensors (there is no CPU fallback)")
    for t, dt in ((rowptr, torch.int32), (col, torch.int32), (X, torch.float16), (Y, torch.float16)):
        if t.dtype != dt or t.device != dev or not t.is_contiguous():
            raise ValueError("rowptr/col must be int32, X/Y fp16, all contiguous on one CUDA device")
    if X.dim() != 2 or Y.dim() != 2 or X.shape[1] != Y.shape[1] or rowptr.numel() - 1 != X.shape[0]:
        raise ValueError("X must be [n_rows, K], Y [n_cols, K]")
    if out is None:
        out = torch.empty(col.numel(), dtype=torch.float16, device=dev)
    with torch.cuda.device(dev):
        _lib.check(lib.trs_sddmm(rowptr.data_ptr(), col.data_ptr(), X.data_ptr(), Y.data_ptr(), out.data_ptr(),
                                 X.shape[0], Y.shape[0], X.shape[1], _lib.current_stream_ptr(dev)))
    return out
