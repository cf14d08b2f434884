"""GPU format builder (trs_build_*): CSR on the device -> the reference's 29 format arrays,
bit-exact with Libra5BlockOnline.block_sptc_2to4_online (TR-source/Block/block_online.cpp:545-871)."""
from __future__ import annotations

import ctypes as C
import os

import torch

from . import _lib
from .format import FORMAT_NAMES, Format

_DTYPES = {
    "t_value": torch.float32, "c_value": torch.float32, "cs_value": torch.float32,
    "s_value": torch.float32, "t_binary": torch.int64, "s_mask": torch.uint8, "s_pos": torch.int8,
    "s_packed_a": torch.int32, "s_packed_meta": torch.int32,
}


def _shape(name: str, n: int, window: int):
    if name == "s_column":
        return (n // 4, 4)
    if name == "s_mask":
        return (n // window, window)
    if name in ("s_value", "s_pos"):
        return (n // (2 * window), window, 2)
    if name == "s_tile_column":
        return (n // 16, 16)
    if name == "s_packed_a":
        return (n // 64, 8, 4, 2)
    if name == "s_packed_meta":
        return (n // 8, 8)
    return (n,)


def env_switches():
    """The two environment switches the reference's builder reads at call time
    (block_online.cpp:564-567)."""
    skip = os.environ.get("LIBRA_SKIP_TC")
    skip_tc = skip in ("1", "true", "TRUE")
    v = os.environ.get("LIBRA_SPTC_UNIT_MIN_NNZ")
    try:
        unit_min = int(v) if v is not None else 2
    except ValueError:
        unit_min = 0  # atoi of a non-number
    return skip_tc, unit_min


def arena_bytes(n_rows: int, nnz: int, window: int = 16, strict: bool = False) -> int:
    """trs_build_query: upper bound of the device memory one build of a matrix of this size needs."""
    cfg = _lib.TrsBuildConfig(32, 32, 3, 8, window, 0.0, 0, 2, int(bool(strict)))
    n = C.c_size_t()
    _lib.check(_lib.load().trs_build_query(int(n_rows), int(nnz), C.byref(cfg), C.byref(n)))
    return n.value


def build_format(rowptr: torch.Tensor, col: torch.Tensor, val: torch.Tensor, part_t: int = 32, part_c: int = 32,
                 short_size: int = 3, density: int = 8, window: int = 16, tc_min_util: float = 0.0,
                 skip_tc: bool | None = None, unit_min_nnz: int | None = None, strict: bool = False,
                 arena: torch.Tensor | None = None):
    """Build on the GPU.  Inputs: CUDA int32 row pointers / columns (canonical CSR) and fp32 values.
    Returns (Format on the same device, stats dict).  strict=True builds a lossless format: the
    entries the reference drops (third / fourth non-zero of a row inside a 4-column group) go to the
    row's CUDA-core part; those arrays are then no longer bit-identical to the reference's.
    With `arena` (a uint8 CUDA tensor, see arena_bytes) the library allocates nothing
    (trs_build_fill): outputs and temporaries are cut out of the arena and the returned arrays are
    views of it, valid until the caller reuses that memory; stats["arena_used"] is the high-water mark."""
    dev = rowptr.device
    if dev.type != "cuda":
        raise ValueError("build_format needs CUDA tensors (there is no CPU fallback)")
    if rowptr.dtype != torch.int32 or col.dtype != torch.int32 or val.dtype != torch.float32:
        raise TypeError("rowptr/col must be int32 and values float32")
    if col.device != dev or val.device != dev:
        raise ValueError("all inputs must live on one device")
    rowptr, col, val = rowptr.contiguous(), col.contiguous(), val.contiguous()
    e_skip, e_min = env_switches()
    cfg = _lib.TrsBuildConfig(part_t, part_c, short_size, density, window, float(tc_min_util),
                              int(e_skip if skip_tc is None else skip_tc),
                              int(e_min if unit_min_nnz is None else unit_min_nnz), int(bool(strict)))
    lib = _lib.load()
    handle = C.c_void_p()
    if arena is not None:
        if arena.device != dev or arena.dtype != torch.uint8 or not arena.is_contiguous():
            raise ValueError("arena must be a contiguous uint8 tensor on the inputs' device")
        base = arena.data_ptr()
        skip = (-base) % 256                      # the library wants a 256-byte aligned start
        if arena.numel() <= skip:
            raise ValueError("arena too small")
    arena_used = 0
    with torch.cuda.device(dev):
        stream = _lib.current_stream_ptr(dev)
        args = (rowptr.data_ptr(), col.data_ptr() if col.numel() else None, val.data_ptr() if val.numel() else None,
                rowptr.numel() - 1, C.byref(cfg))
        if arena is None:
            _lib.check(lib.trs_build_create(*args, stream, C.byref(handle)))
        else:
            _lib.check(lib.trs_build_fill(*args, base + skip, arena.numel() - skip, stream, C.byref(handle)))
        try:
            sizes = (C.c_longlong * len(FORMAT_NAMES))()
            _lib.check(lib.trs_build_sizes(handle, sizes))
            stats = _lib.TrsBuildStats()
            _lib.check(lib.trs_build_stats(handle, C.byref(stats)))
            arrays = []
            for i, name in enumerate(FORMAT_NAMES):
                dt = _DTYPES.get(name, torch.int32)
                n_el = int(sizes[i])
                if arena is None:
                    t = torch.empty(n_el, dtype=dt, device=dev)
                    if n_el:
                        _lib.check(lib.trs_build_copy(handle, i, t.data_ptr(), 0, stream))
                elif n_el:
                    off = int(lib.trs_build_array(handle, i)) - base
                    t = arena[off:off + n_el * torch.empty(0, dtype=dt).element_size()].view(dt)
                else:
                    t = torch.empty(0, dtype=dt, device=dev)
                arrays.append(t.view(_shape(name, n_el, window)))
            if arena is not None:
                used = C.c_size_t()
                _lib.check(lib.trs_build_arena_used(handle, C.byref(used)))
                arena_used = used.value + skip
            torch.cuda.current_stream(dev).synchronize()
        finally:
            lib.trs_build_destroy(handle)
    info = {n: getattr(stats, n) for n, _ in stats._fields_}
    info["arena_used"] = arena_used
    return Format(arrays, window), info


def stdsort_order(keys):
    """The builder's emulation of libstdc++ std::sort (descending unit nnz, identity start),
    run on the host by the library; returns (permutation, number of heap-sort fallbacks)."""
    import numpy as np
    keys = np.ascontiguousarray(keys, dtype=np.uint8)
    out = np.empty(len(keys), dtype=np.int32)
    heaps = C.c_int()
    _lib.check(_lib.load().trs_debug_stdsort_order(keys.ctypes.data, len(keys), out.ctypes.data, C.byref(heaps)))
    return out, heaps.value
