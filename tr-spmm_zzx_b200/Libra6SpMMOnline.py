"""Drop-in for the reference's `Libra6SpMMOnline` torch extension
(TR-source/SpMM/mGCN_online.cpp:1142-1152): same function names, positional signatures,
argument checks and return tuples, executed by libtrspmm.so (hand-written sm_100a CUDA).

As in the reference every tensor argument must be a CPU tensor; device memory is allocated,
filled and released inside each call and the result comes back as an fp32 CPU tensor.  Argument
errors raise RuntimeError like TORCH_CHECK does.  The three routes run fused in one kernel, so
the per-route millisecond slots of the 6-tuple are returned as 0 and `ms` carries the total.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

from trspmm import _lib
from trspmm.format import FORMAT_NAMES, Format

__all__ = [
    "forward_fp16_tcu_cuda_sptc_mma_parallel_online", "forward_fp16_sptc_online",
    "forward_fp16_sptc_mma_online", "forward_fp16_sptc_mma_packed_online",
]


def _check(cond, msg):
    if not cond:
        raise RuntimeError(msg)


def _cpu(x, name, dtype):
    _check(isinstance(x, torch.Tensor), f"{name} must be a tensor")
    _check(not x.is_cuda, f"{name} must be a CPU tensor")
    _check(x.dtype == dtype, f"{name} has an unexpected dtype")
    return x.contiguous()


def _scalars(window, dimN, mOri, kOri, epoches, limit16=True):
    if limit16:
        _check(0 < window <= 16, "parallel mma path requires 0 < window <= 16")
    else:
        _check(window > 0, "window must be positive")
    _check(dimN > 0, "dimN must be positive")
    _check(mOri > 0, "mOri must be positive")
    _check(kOri > 0, "kOri must be positive")
    _check(epoches > 0, "epoches must be positive")


def _ms(x):
    return torch.tensor(float(x))


def _empty(dtype, *shape):
    return torch.empty(shape or (0,), dtype=dtype)


def forward_fp16_tcu_cuda_sptc_mma_parallel_online(
        t_row_offset, t_blockNew_offset, t_column, t_value, t_window_row, t_atomic, t_binary,
        c_row_offsets, c_row, c_atomic, c_column, c_value,
        c_row_offsets_short, c_row_short, c_atomic_short, c_column_short, c_value_short,
        s_column, s_value, s_pos, s_offsets, s_tile_window, s_tile_column, s_packed_a, s_packed_meta,
        s_window_tile_offset, rhs_matrix,
        parts_t, parts_c, partsize_c, parts_c_short, window, dimN, mOri, kOri, epoches):
    """mGCN_online.cpp:760-1138.  Returns [C fp32 [mOri, dimN], ms, ms_tc, ms_cuda_long,
    ms_cuda_short, ms_sptc]."""
    i32, f16 = torch.int32, torch.float16
    t_row_offset = _cpu(t_row_offset, "t_row_offset", i32)
    t_blockNew_offset = _cpu(t_blockNew_offset, "t_blockNew_offset", i32)
    t_column = _cpu(t_column, "t_column", i32)
    t_value = _cpu(t_value, "t_value", f16)
    t_window_row = _cpu(t_window_row, "t_window_row", i32)
    t_atomic = _cpu(t_atomic, "t_atomic", i32)
    t_binary = _cpu(t_binary, "t_binary", torch.int64)
    c_row_offsets = _cpu(c_row_offsets, "c_row_offsets", i32)
    c_row = _cpu(c_row, "c_row", i32)
    c_atomic = _cpu(c_atomic, "c_atomic", i32)
    c_column = _cpu(c_column, "c_column", i32)
    c_value = _cpu(c_value, "c_value", f16)
    c_row_offsets_short = _cpu(c_row_offsets_short, "c_row_offsets_short", i32)
    c_row_short = _cpu(c_row_short, "c_row_short", i32)
    c_atomic_short = _cpu(c_atomic_short, "c_atomic_short", i32)
    c_column_short = _cpu(c_column_short, "c_column_short", i32)
    c_value_short = _cpu(c_value_short, "c_value_short", f16)
    s_column = _cpu(s_column, "s_column", i32)
    s_value = _cpu(s_value, "s_value", torch.float32)
    s_pos = _cpu(s_pos, "s_pos", torch.int8)
    s_offsets = _cpu(s_offsets, "s_offsets", i32)
    s_tile_window = _cpu(s_tile_window, "s_tile_window", i32)
    s_tile_column = _cpu(s_tile_column, "s_tile_column", i32)
    s_packed_a = _cpu(s_packed_a, "s_packed_a", i32)
    s_packed_meta = _cpu(s_packed_meta, "s_packed_meta", i32)
    s_window_tile_offset = _cpu(s_window_tile_offset, "s_window_tile_offset", i32)
    rhs_matrix = _cpu(rhs_matrix, "rhs_matrix", f16)

    _scalars(window, dimN, mOri, kOri, epoches)
    _check(rhs_matrix.numel() == kOri * dimN, "rhs_matrix must have kOri * dimN elements")
    _check(s_column.dim() == 2 and s_column.size(1) == 4, "s_column must have shape [groups, 4]")
    _check(s_value.dim() == 3 and s_value.size(1) == window and s_value.size(2) == 2,
           "s_value must have shape [groups, window, 2]")
    _check(s_pos.dim() == 3 and s_pos.size(1) == window and s_pos.size(2) == 2,
           "s_pos must have shape [groups, window, 2]")
    _check(s_offsets.dim() == 1 and s_offsets.size(0) >= 1, "s_offsets must be 1-D with at least one item")
    _check(s_tile_window.dim() == 1, "s_tile_window must be 1-D")
    _check(s_tile_column.dim() == 2 and s_tile_column.size(1) == 16, "s_tile_column must have shape [tiles, 16]")
    _check(s_packed_a.dim() == 4 and tuple(s_packed_a.shape[1:]) == (8, 4, 2),
           "s_packed_a must have shape [tiles, 8, 4, 2]")
    _check(s_packed_meta.dim() == 2 and s_packed_meta.size(1) == 8, "s_packed_meta must have shape [tiles, 8]")
    groups = s_column.size(0)
    _check(s_value.size(0) == groups, "s_value group count mismatch")
    _check(s_pos.size(0) == groups, "s_pos group count mismatch")
    _check(int(s_offsets[0]) == 0, "s_offsets must start with 0")
    _check(int(s_offsets[-1]) == groups, "s_offsets end must equal group count")
    per_window = s_offsets[1:] - s_offsets[:-1]
    _check(bool((per_window >= 0).all()), "s_offsets must be non-decreasing")
    num_tiles = int(((per_window + 3) // 4).sum())
    packed = s_tile_window.size(0)
    _check(s_tile_column.size(0) == packed, "s_tile_column tile count mismatch")
    _check(s_packed_a.size(0) == packed, "s_packed_a tile count mismatch")
    _check(s_packed_meta.size(0) == packed, "s_packed_meta tile count mismatch")
    _check(packed == num_tiles, "packed tile count must match offsets-derived tile count")
    _check(t_atomic.numel() == parts_t and c_atomic.numel() == parts_c and c_atomic_short.numel() == parts_c_short,
           "parts_t / parts_c / parts_c_short must match the part arrays")

    skip_tc = os.environ.get("LIBRA_SKIP_TC_KERNEL", "") not in ("", "0")  # mGCNkernel_online.cu:1398
    e32 = _empty(i32)
    arrays = {
        "t_row_offset": e32 if skip_tc else t_row_offset, "t_block_offset": e32 if skip_tc else t_blockNew_offset,
        "t_column": e32 if skip_tc else t_column, "t_value": _empty(f16) if skip_tc else t_value,
        "t_window_row": e32 if skip_tc else t_window_row, "t_atomic": e32 if skip_tc else t_atomic,
        "t_binary": _empty(torch.int64) if skip_tc else t_binary,
        "c_row_offset": c_row_offsets, "c_row": c_row, "c_atomic": c_atomic, "c_column": c_column, "c_value": c_value,
        "cs_row_offset": c_row_offsets_short, "cs_row": c_row_short, "cs_atomic": c_atomic_short,
        "cs_column": c_column_short, "cs_value": c_value_short,
        "s_column": s_column, "s_mask": _empty(torch.uint8), "s_value": s_value, "s_pos": s_pos,
        "s_window": e32, "s_offset": s_offsets, "s_tile_window": s_tile_window, "s_tile_group": e32,
        "s_tile_column": s_tile_column, "s_packed_a": s_packed_a, "s_packed_meta": s_packed_meta,
        "s_window_tile_offset": s_window_tile_offset,
    }
    return _run_host(Format(arrays, window), rhs_matrix, dimN, mOri, kOri, window, epoches, six=True)


def _run_host(fmt, rhs, dimN, mOri, kOri, window, epoches, six):
    lib = _lib.load()
    out = torch.empty((mOri, dimN), dtype=torch.float32)
    timing = _lib.TrsTiming()
    cf = fmt.c_struct()
    _lib.check(lib.trs_spmm_forward_host(C.byref(cf), rhs.data_ptr(), out.data_ptr(), dimN, mOri, kOri, window,
                                         epoches, C.byref(timing)))
    if six:
        return [out, _ms(timing.total_ms), _ms(0.0), _ms(0.0), _ms(0.0), _ms(0.0)]
    return [out, _ms(timing.total_ms)]


def forward_fp16_sptc_mma_packed_online(s_tile_column, s_packed_a, s_packed_meta, s_window_tile_offset, rhs_matrix,
                                        window, dimN, mOri, kOri, epoches):
    """mGCN_online.cpp:654-757: SPTC route alone, from the packed tiles.  Returns [C, ms]."""
    i32 = torch.int32
    s_tile_column = _cpu(s_tile_column, "s_tile_column", i32)
    s_packed_a = _cpu(s_packed_a, "s_packed_a", i32)
    s_packed_meta = _cpu(s_packed_meta, "s_packed_meta", i32)
    s_window_tile_offset = _cpu(s_window_tile_offset, "s_window_tile_offset", i32)
    rhs_matrix = _cpu(rhs_matrix, "rhs_matrix", torch.float16)
    _check(0 < window <= 16, "packed mma path requires 0 < window <= 16")
    _scalars(window, dimN, mOri, kOri, epoches)
    _check(s_tile_column.dim() == 2 and s_tile_column.size(1) == 16, "s_tile_column must have shape [tiles, 16]")
    _check(s_packed_a.dim() == 4 and tuple(s_packed_a.shape[1:]) == (8, 4, 2),
           "s_packed_a must have shape [tiles, 8, 4, 2]")
    _check(s_packed_meta.dim() == 2 and s_packed_meta.size(1) == 8, "s_packed_meta must have shape [tiles, 8]")
    _check(s_window_tile_offset.dim() == 1 and s_window_tile_offset.size(0) >= 2,
           "s_window_tile_offset must be 1-D with at least 2 elements")
    _check(rhs_matrix.numel() == kOri * dimN, "rhs_matrix must have kOri * dimN elements")
    tiles = s_tile_column.size(0)
    _check(s_packed_a.size(0) == tiles, "s_packed_a tile count mismatch")
    _check(s_packed_meta.size(0) == tiles, "s_packed_meta tile count mismatch")
    e32 = _empty(i32)
    arrays = {n: e32 for n in FORMAT_NAMES}
    arrays.update({"t_value": _empty(torch.float16), "c_value": _empty(torch.float16),
                   "cs_value": _empty(torch.float16), "t_binary": _empty(torch.int64),
                   "s_tile_column": s_tile_column, "s_packed_a": s_packed_a, "s_packed_meta": s_packed_meta,
                   "s_window_tile_offset": s_window_tile_offset})
    return _run_host(Format(arrays, window), rhs_matrix, dimN, mOri, kOri, window, epoches, six=False)


def _unpacked(s_column, s_value, s_pos, s_window, s_offsets, rhs_matrix, window, dimN, mOri, kOri, epoches):
    lib = _lib.load()
    i32 = torch.int32
    s_column = _cpu(s_column, "s_column", i32)
    s_value = _cpu(s_value, "s_value", torch.float32)
    s_pos = _cpu(s_pos, "s_pos", torch.int8)
    rhs_matrix = _cpu(rhs_matrix, "rhs_matrix", torch.float16)
    _scalars(window, dimN, mOri, kOri, epoches, limit16=False)
    _check(window <= 16, "window must not exceed 16")
    _check(rhs_matrix.numel() == kOri * dimN, "rhs_matrix must have kOri * dimN elements")
    _check(s_column.dim() == 2 and s_column.size(1) == 4, "s_column must have shape [groups, 4]")
    groups = s_column.size(0)
    _check(s_value.numel() == groups * window * 2, "s_value must have shape [groups, window, 2]")
    _check(s_pos.numel() == groups * window * 2, "s_pos must have shape [groups, window, 2]")
    out = torch.empty((mOri, dimN), dtype=torch.float32)
    timing = _lib.TrsTiming()
    nw = 0
    if s_offsets is not None:
        s_offsets = _cpu(s_offsets, "s_offsets", i32)
        nw = s_offsets.numel() - 1
    if s_window is not None:
        s_window = _cpu(s_window, "s_window", i32)
        _check(s_window.numel() == groups, "s_window must have one entry per group")
    _lib.check(lib.trs_sptc_unpacked_forward_host(
        s_column.data_ptr() if groups else None, s_value.data_ptr() if groups else None,
        s_pos.data_ptr() if groups else None,
        s_window.data_ptr() if s_window is not None and groups else None,
        s_offsets.data_ptr() if s_offsets is not None else None,
        groups, nw, rhs_matrix.data_ptr(), out.data_ptr(), window, dimN, mOri, kOri, epoches, C.byref(timing)))
    return [out, _ms(timing.total_ms)]


def forward_fp16_sptc_online(s_column, s_value, s_pos, s_window, rhs_matrix, window, dimN, mOri, kOri, epoches):
    """mGCN_online.cpp:202-400: SPTC route alone from the un-packed arrays, one window id per group."""
    return _unpacked(s_column, s_value, s_pos, s_window, None, rhs_matrix, window, dimN, mOri, kOri, epoches)


def forward_fp16_sptc_mma_online(s_column, s_value, s_pos, s_offsets, rhs_matrix, window, dimN, mOri, kOri, epoches):
    """mGCN_online.cpp:404-652: SPTC route alone from the un-packed arrays and per-window offsets."""
    return _unpacked(s_column, s_value, s_pos, None, s_offsets, rhs_matrix, window, dimN, mOri, kOri, epoches)
