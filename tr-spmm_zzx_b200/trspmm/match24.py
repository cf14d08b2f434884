"""2:4 matching statistics (trs_match24_stats): GPU versions of the reference's statistic-only
matchers.  The dict keys and the integer wrap of `fake_zeros` (a C `int` in the reference) follow
the reference modules."""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from . import _lib

VARIANTS = {"para_dr": 0, "hash": 1, "bucket": 2, "online": 3, "cuda": 4}


class TrsMatchStats(C.Structure):
    _fields_ = [("total_rows", C.c_int32), ("total_cols", C.c_int32), ("total_nnz", C.c_longlong),
                ("sparsity", C.c_double), ("num_row_panels", C.c_int32), ("num_groups", C.c_longlong),
                ("num_tc_blocks", C.c_longlong), ("num_16x16_blocks", C.c_longlong),
                ("block_padding_groups", C.c_longlong), ("fine_fallback", C.c_longlong),
                ("coarse_fallback", C.c_longlong), ("fake_zeros", C.c_longlong), ("tc_total_nnz", C.c_longlong),
                ("tc_block_count", C.c_longlong), ("tc_block_max_nnz", C.c_int32), ("tc_block_min_nnz", C.c_int32),
                ("fake_zeros_exact", C.c_longlong), ("dense_to_tc_cols", C.c_longlong),
                ("dense_to_sptc_cols", C.c_longlong)]


def _as_int32(x: int) -> int:
    return ((int(x) + 2 ** 31) % 2 ** 32) - 2 ** 31


def _device_csr(row_ptr, col_ind):
    if isinstance(row_ptr, torch.Tensor):
        rp, ci = row_ptr, col_ind
    else:  # numpy with forcecast, like the pybind signatures of the reference
        rp = torch.from_numpy(np.ascontiguousarray(np.asarray(row_ptr).astype(np.int32, copy=False)))
        ci = torch.from_numpy(np.ascontiguousarray(np.asarray(col_ind).astype(np.int32, copy=False)))
    if not torch.cuda.is_available():
        raise RuntimeError("the matching statistics run on a CUDA device (there is no CPU fallback)")
    dev = rp.device if rp.is_cuda else torch.device("cuda", torch.cuda.current_device())
    return rp.to(dev, torch.int32).contiguous(), ci.to(dev, torch.int32).contiguous()


def match_stats(variant: str, row_ptr, col_ind, window_size: int = 16, dense_threshold: int = 8, t_max: int = 8):
    lib = _lib.load()
    if not hasattr(lib.trs_match24_stats, "_bound"):
        lib.trs_match24_stats.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
                                          C.c_void_p, C.POINTER(TrsMatchStats)]
        lib.trs_match24_stats.restype = C.c_int
        lib.trs_match24_stats._bound = True
    rp, ci = _device_csr(row_ptr, col_ind)
    rows = rp.numel() - 1
    if window_size < 1 or window_size > 64:
        raise RuntimeError("window_size must be in [1, 64]")
    if window_size > 16:
        raise RuntimeError("window_size above 16 is not supported: the row masks are 16 bits wide")
    if rows <= 0 or ci.numel() == 0:
        raise RuntimeError("invalid matrix dimensions")
    st = TrsMatchStats()
    with torch.cuda.device(rp.device):
        _lib.check(lib.trs_match24_stats(VARIANTS[variant], rp.data_ptr(), ci.data_ptr(), rows, window_size,
                                         dense_threshold, t_max, _lib.current_stream_ptr(rp.device), C.byref(st)))
    return st


def common_fields(st):
    return {"total_rows": st.total_rows, "total_cols": st.total_cols, "total_nnz": st.total_nnz,
            "sparsity": st.sparsity, "num_row_panels": st.num_row_panels}
