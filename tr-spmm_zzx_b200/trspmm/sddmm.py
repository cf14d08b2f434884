"""SDDMM on a CSR pattern (trs_sddmm).  The reference has no such operator; the definition is
out[e] = fp16(sum_k fp32(X[row(e),k]) * fp32(Y[col(e),k])) in CSR entry order."""
from __future__ import annotations

import ctypes as C

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


class SddmmPlan:
    """trs_sddmm_plan_*: a CSR pattern prepared once for many SDDMMs.  The plan groups the entries
    by (16-row window, column) so that every distinct Y row of a window is gathered once and the
    dot products run on the tensor cores (K = 32, 64, 128); other K fall back to the entry-parallel
    kernel.  `rowptr` / `col` (canonical CSR, int32, CUDA) are kept alive by the plan."""

    def __init__(self, rowptr: torch.Tensor, col: torch.Tensor, n_cols: int):
        self.lib = _lib.load()
        dev = rowptr.device
        if dev.type != "cuda":
            raise ValueError("SddmmPlan needs CUDA tensors (there is no CPU fallback)")
        for t in (rowptr, col):
            if t.dtype != torch.int32 or t.device != dev or not t.is_contiguous():
                raise ValueError("rowptr/col must be contiguous int32 tensors on one CUDA device")
        self.rowptr, self.col, self.device = rowptr, col, dev
        self.n_rows, self.n_cols = rowptr.numel() - 1, int(n_cols)
        self._handle = C.c_void_p()
        with torch.cuda.device(dev):
            _lib.check(self.lib.trs_sddmm_plan_create(rowptr.data_ptr(), col.data_ptr(), self.n_rows, self.n_cols,
                                                      _lib.current_stream_ptr(dev), C.byref(self._handle)))
        pairs, blocks = C.c_longlong(), C.c_longlong()
        _lib.check(self.lib.trs_sddmm_plan_info(self._handle, C.byref(pairs), C.byref(blocks)))
        self.n_pairs, self.n_blocks = pairs.value, blocks.value

    def run(self, X: torch.Tensor, Y: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        for t in (X, Y):
            if t.dtype != torch.float16 or t.device != self.device or not t.is_contiguous() or t.dim() != 2:
                raise ValueError("X/Y must be contiguous fp16 matrices on the plan's device")
        if X.shape[0] != self.n_rows or Y.shape[0] != self.n_cols or X.shape[1] != Y.shape[1]:
            raise ValueError("X must be [n_rows, K], Y [n_cols, K]")
        if out is None:
            out = torch.empty(self.col.numel(), dtype=torch.float16, device=self.device)
        elif out.dtype != torch.float16 or out.numel() != self.col.numel() or not out.is_contiguous():
            raise ValueError("out must be a contiguous fp16 vector with one element per entry")
        with torch.cuda.device(self.device):
            _lib.check(self.lib.trs_sddmm_plan_run(self._handle, X.data_ptr(), Y.data_ptr(), out.data_ptr(),
                                                   X.shape[1], _lib.current_stream_ptr(self.device)))
        return out

    def close(self):
        if getattr(self, "_handle", None) is not None and self._handle:
            self.lib.trs_sddmm_plan_destroy(self._handle)
            self._handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
