"""ctypes binding of libtrspmm.so (C ABI declared in include/trspmm.h)."""
from __future__ import annotations

import ctypes as C
from pathlib import Path

PKG_ROOT = Path(__file__).resolve().parents[1]


def lib_path() -> Path:
    return PKG_ROOT / "libtrspmm.so"


class TrsError(RuntimeError):
    """An error code returned across the C ABI (negative: argument error, positive: CUDA error)."""

    def __init__(self, code: int, what: str):
        super().__init__(f"{what} (trspmm error {code})")
        self.code = code


class TrsFormat(C.Structure):
    """struct trs_format of include/trspmm.h (field order is ABI)."""
    _fields_ = [
        ("t_row_offset", C.c_void_p), ("t_block_offset", C.c_void_p), ("t_column", C.c_void_p),
        ("t_value", C.c_void_p), ("t_window_row", C.c_void_p), ("t_binary", C.c_void_p),
        ("parts_t", C.c_int32), ("blocks", C.c_int32),
        ("c_row_offset", C.c_void_p), ("c_row", C.c_void_p), ("c_column", C.c_void_p), ("c_value", C.c_void_p),
        ("parts_c", C.c_int32),
        ("cs_row_offset", C.c_void_p), ("cs_row", C.c_void_p), ("cs_column", C.c_void_p), ("cs_value", C.c_void_p),
        ("parts_c_short", C.c_int32),
        ("s_window_tile_offset", C.c_void_p), ("s_tile_column", C.c_void_p), ("s_packed_a", C.c_void_p),
        ("s_packed_meta", C.c_void_p),
        ("num_windows", C.c_int32), ("tiles", C.c_int32),
    ]


class TrsBuildConfig(C.Structure):
    _fields_ = [("part_t", C.c_int32), ("part_c", C.c_int32), ("short_size", C.c_int32), ("density", C.c_int32),
                ("window", C.c_int32), ("tc_min_util", C.c_float), ("skip_tc", C.c_int32), ("unit_min_nnz", C.c_int32),
                ("strict", C.c_int32)]


class TrsBuildStats(C.Structure):
    _fields_ = [(n, C.c_longlong) for n in ("nnz", "dropped_nnz", "distinct_window_columns", "units", "tc_nnz",
                                            "csr_nnz", "groups", "tiles", "tc_blocks")] + [("build_ms", C.c_float)]


class TrsTiming(C.Structure):
    _fields_ = [(n, C.c_float) for n in
                ("total_ms", "tc_ms", "cuda_long_ms", "cuda_short_ms", "sptc_ms", "h2d_ms", "d2h_ms")]


_LIB = None


def load():
    """Load the library; fails loudly when it has not been built."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = lib_path()
    if not path.exists():
        raise RuntimeError(
            f"{path} is missing: build it with `python {PKG_ROOT / 'build.py'}` "
            "(there is no CPU fallback for the CUDA operators)")
    lib = C.CDLL(str(path))
    vp, i32, sz = C.c_void_p, C.c_int, C.c_size_t
    lib.trs_strerror.restype = C.c_char_p
    lib.trs_strerror.argtypes = [i32]
    lib.trs_version.restype = i32
    lib.trs_device_count.restype = i32
    lib.trs_spmm_plan_create.argtypes = [C.POINTER(TrsFormat), i32, i32, i32, i32, vp, C.POINTER(vp)]
    lib.trs_spmm_plan_destroy.argtypes = [vp]
    lib.trs_spmm_workspace_bytes.argtypes = [vp, i32, C.POINTER(sz)]
    lib.trs_spmm_run.argtypes = [vp, vp, vp, i32, i32, vp, sz, vp]
    lib.trs_spmm_launches.argtypes = [vp]
    lib.trs_spmm_run_ex.argtypes = [vp, vp, vp, i32, i32, i32, vp, sz, vp]
    lib.trs_spmm_run_ex.restype = i32
    lib.trs_spmm_run_bcast.argtypes = [vp, vp, C.POINTER(vp), i32, C.c_longlong, i32, i32, vp, sz, vp]
    lib.trs_spmm_run_bcast.restype = i32
    lib.trs_rows_gemm_bcast.argtypes = [vp, vp, C.POINTER(vp), i32, C.c_longlong, i32, i32, i32, vp]
    lib.trs_rows_gemm_bcast.restype = i32
    lib.trs_rows_gemm_mcast.argtypes = [vp, vp, vp, C.c_longlong, i32, i32, i32, vp]
    lib.trs_rows_gemm_mcast.restype = i32
    lib.trs_spmm_run_static.argtypes = [vp, vp, vp, i32, i32, vp]
    lib.trs_spmm_run_static.restype = i32
    lib.trs_spmm_static_scratch_bytes.argtypes = [vp, i32, C.POINTER(sz)]
    lib.trs_spmm_static_scratch_bytes.restype = i32
    lib.trs_spmm_forward_host.argtypes = [C.POINTER(TrsFormat), vp, vp, i32, i32, i32, i32, i32, C.POINTER(TrsTiming)]
    lib.trs_resident_create.argtypes = [C.POINTER(TrsFormat), i32, i32, i32, i32, C.POINTER(vp)]
    lib.trs_resident_create_device.argtypes = [C.POINTER(TrsFormat), i32, i32, i32, i32, C.POINTER(vp)]
    lib.trs_resident_create_device.restype = i32
    lib.trs_resident_forward.argtypes = [vp, vp, vp, i32, i32, C.POINTER(TrsTiming)]
    lib.trs_resident_destroy.argtypes = [vp]
    lib.trs_resident_submit.argtypes = [vp, vp, vp, i32, i32]
    lib.trs_resident_submit.restype = i32
    lib.trs_resident_wait.argtypes = [vp]
    lib.trs_resident_wait.restype = i32
    lib.trs_spmm_run_windows.argtypes = [vp, vp, vp, i32, i32, i32, vp, sz, vp, i32, i32]
    lib.trs_spmm_run_windows.restype = i32
    lib.trs_spmm_num_windows.argtypes = [vp]
    lib.trs_spmm_num_windows.restype = i32
    lib.trs_sptc_unpacked_forward_host.argtypes = [vp, vp, vp, vp, vp, i32, i32, vp, vp, i32, i32, i32, i32, i32,
                                                   C.POINTER(TrsTiming)]
    lib.trs_sddmm.argtypes = [vp, vp, vp, vp, vp, i32, i32, i32, vp]
    lib.trs_spmm_status.argtypes = [vp, C.POINTER(i32)]
    lib.trs_sddmm_plan_create.argtypes = [vp, vp, i32, i32, vp, C.POINTER(vp)]
    lib.trs_sddmm_plan_run.argtypes = [vp, vp, vp, vp, i32, vp]
    lib.trs_sddmm_plan_info.argtypes = [vp, C.POINTER(C.c_longlong), C.POINTER(C.c_longlong)]
    lib.trs_sddmm_plan_destroy.argtypes = [vp]
    for name in ("trs_sddmm_plan_create", "trs_sddmm_plan_run", "trs_sddmm_plan_info", "trs_sddmm_plan_destroy"):
        getattr(lib, name).restype = i32
    lib.trs_build_create.argtypes = [vp, vp, vp, i32, C.POINTER(TrsBuildConfig), vp, C.POINTER(vp)]
    lib.trs_build_fill.argtypes = [vp, vp, vp, i32, C.POINTER(TrsBuildConfig), vp, sz, vp, C.POINTER(vp)]
    lib.trs_build_fill.restype = i32
    lib.trs_build_query.argtypes = [i32, C.c_longlong, C.POINTER(TrsBuildConfig), C.POINTER(sz)]
    lib.trs_build_query.restype = i32
    lib.trs_build_arena_used.argtypes = [vp, C.POINTER(sz)]
    lib.trs_build_arena_used.restype = i32
    lib.trs_build_destroy.argtypes = [vp]
    lib.trs_build_sizes.argtypes = [vp, C.POINTER(C.c_longlong)]
    lib.trs_build_stats.argtypes = [vp, C.POINTER(TrsBuildStats)]
    lib.trs_build_array.argtypes = [vp, i32]
    lib.trs_build_array.restype = vp
    lib.trs_build_copy.argtypes = [vp, i32, vp, i32, vp]
    lib.trs_build_format.argtypes = [vp, C.POINTER(TrsFormat), vp]
    lib.trs_debug_stdsort_order.argtypes = [vp, i32, vp, C.POINTER(i32)]
    for name in ("trs_spmm_plan_create", "trs_spmm_plan_destroy", "trs_spmm_workspace_bytes", "trs_spmm_run",
                 "trs_spmm_launches", "trs_spmm_forward_host", "trs_resident_create", "trs_resident_forward",
                 "trs_resident_destroy", "trs_sptc_unpacked_forward_host", "trs_sddmm", "trs_spmm_status",
                 "trs_build_create", "trs_build_destroy", "trs_build_sizes", "trs_build_stats", "trs_build_copy",
                 "trs_build_format", "trs_debug_stdsort_order"):
        getattr(lib, name).restype = i32
    _LIB = lib
    return lib


def check(code: int):
    if code != 0:
        raise TrsError(code, load().trs_strerror(code).decode())


def current_stream_ptr(device) -> int:
    import torch
    return torch.cuda.current_stream(device).cuda_stream
