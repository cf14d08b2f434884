"""No GPU needed: the C-ABI library loads, exports every symbol include/trspmm.h declares, and
the entry points refuse bad arguments / a missing device with error codes instead of crashing."""
import ctypes
import re
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]


def _declared():
    text = (ROOT / "include" / "trspmm.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(trs_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from trspmm import _lib
    lib = ctypes.CDLL(str(_lib.lib_path()))
    names = _declared()
    assert len(names) >= 25
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_error_strings_and_version():
    from trspmm import load
    lib = load()
    assert lib.trs_version() >= 100
    for code in range(-10, 1):
        assert lib.trs_strerror(code)
    assert b"window" in lib.trs_strerror(-2)
    assert b"canonical" in lib.trs_strerror(-8)


def test_entry_points_reject_bad_arguments_without_a_device():
    from trspmm import _lib
    lib = _lib.load()
    plan = ctypes.c_void_p()
    fmt = _lib.TrsFormat()
    assert lib.trs_spmm_plan_create(None, 16, 16, 16, 1, None, ctypes.byref(plan)) == -1
    assert lib.trs_spmm_plan_create(ctypes.byref(fmt), 0, 16, 16, 1, None, ctypes.byref(plan)) == -1
    assert lib.trs_spmm_plan_create(ctypes.byref(fmt), 16, 16, 17, 1, None, ctypes.byref(plan)) == -2
    assert lib.trs_spmm_run(None, None, None, 8, 0, None, 0, None) == -1
    assert lib.trs_sddmm(None, None, None, None, None, 4, 4, 8, None) == -1
    # entries added beside the reference's surface: same convention (negative code, nothing launched)
    assert lib.trs_spmm_run_windows(None, None, None, 8, 0, 0, None, 0, None, 0, 1) == -1
    assert lib.trs_spmm_num_windows(None) == -1
    assert lib.trs_resident_submit(None, None, None, 8, 0) == -1
    assert lib.trs_resident_wait(None) == -1
    sp = ctypes.c_void_p()
    assert lib.trs_sddmm_plan_create(None, None, 4, 4, None, ctypes.byref(sp)) == -1
    assert lib.trs_sddmm_plan_create(rp0 := (ctypes.c_int * 2)(0, 0), None, 0, 4, None, ctypes.byref(sp)) == -1
    assert lib.trs_sddmm_plan_run(None, None, None, None, 64, None) == -1
    assert lib.trs_sddmm_plan_destroy(None) == 0
    cfg = _lib.TrsBuildConfig(32, 32, 3, 8, 99, 0.0, 0, 2, 0)
    b = ctypes.c_void_p()
    rp = (ctypes.c_int * 2)(0, 0)
    assert lib.trs_build_create(rp, None, None, 1, ctypes.byref(cfg), None, ctypes.byref(b)) == -2
    if not torch.cuda.is_available():
        assert lib.trs_device_count() == 0
        # valid arguments, no device: a clean error code, never a CPU fallback
        assert lib.trs_spmm_plan_create(ctypes.byref(fmt), 16, 16, 16, 1, None, ctypes.byref(plan)) == -9
        cfg.window = 16
        assert lib.trs_build_create(rp, None, None, 1, ctypes.byref(cfg), None, ctypes.byref(b)) == -9


def test_python_operators_fail_loudly_without_cuda():
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    from trspmm import Format, SpmmPlan, build_format, sddmm
    rp = torch.tensor([0, 1], dtype=torch.int32)
    col = torch.tensor([0], dtype=torch.int32)
    with pytest.raises(ValueError):
        build_format(rp, col, torch.ones(1))
    with pytest.raises(ValueError):
        sddmm(rp, col, torch.ones(1, 8).half(), torch.ones(1, 8).half())
    from oracle import oracle as O
    arrays, _ = O.build_format(rp, col, torch.ones(1))
    with pytest.raises(ValueError):
        SpmmPlan(Format(arrays), 1, 1)
