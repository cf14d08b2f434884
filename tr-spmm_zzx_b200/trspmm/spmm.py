"""SpMM over the hybrid format: plan/run on device tensors, and the host-buffer entries."""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from .format import Format

OUT_F32, OUT_F16 = 0, 1


def _out_code(dtype) -> int:
    if dtype == torch.float32:
        return OUT_F32
    if dtype == torch.float16:
        return OUT_F16
    raise TypeError("output dtype must be torch.float32 or torch.float16")


class SpmmPlan:
    """Device-resident plan (trs_spmm_plan_create): replaces the device half of
    Libra6SpMMOnline.forward_fp16_tcu_cuda_sptc_mma_parallel_online
    (TR-source/SpMM/mGCN_online.cpp:760-1138).  The format tensors must be CUDA tensors and
    stay alive as long as the plan."""

    def __init__(self, fmt: Format, m_rows: int, k_cols: int, window: int = 16, validate: bool = True):
        if fmt.device.type != "cuda":
            raise ValueError("SpmmPlan needs the format on a CUDA device (use spmm_forward_host for CPU tensors)")
        self.lib = _lib.load()
        self.fmt = fmt.half_values().contiguous()
        self.m_rows, self.k_cols, self.window = int(m_rows), int(k_cols), int(window)
        self.device = self.fmt.device
        self._handle = C.c_void_p()
        self._ws = {}
        with torch.cuda.device(self.device):
            cf = self.fmt.c_struct()
            _lib.check(self.lib.trs_spmm_plan_create(C.byref(cf), self.m_rows, self.k_cols, self.window,
                                                     int(validate), _lib.current_stream_ptr(self.device),
                                                     C.byref(self._handle)))

    def workspace_bytes(self, F: int) -> int:
        n = C.c_size_t()
        _lib.check(self.lib.trs_spmm_workspace_bytes(self._handle, int(F), C.byref(n)))
        return n.value

    def static_scratch_bytes(self, F: int) -> int:
        """Bytes of the library's fixed scratch array run_static would use for feature width F."""
        n = C.c_size_t()
        _lib.check(self.lib.trs_spmm_static_scratch_bytes(self._handle, int(F), C.byref(n)))
        return n.value

    def status(self) -> int:
        """Health word of the plan's kernels (trs_spmm_status): always 0 - no kernel of the library waits on
        a flag another warp or kernel sets, so no wait can give up.  Kept for callers of earlier versions."""
        v = C.c_int()
        _lib.check(self.lib.trs_spmm_status(self._handle, C.byref(v)))
        return v.value

    @property
    def launches(self) -> int:
        return self.lib.trs_spmm_launches(self._handle)

    def _check_B(self, B: torch.Tensor) -> int:
        """Every entry that hands B to a kernel goes through this: a short or strided B would become
        an out-of-range gather on the device."""
        if B.device != self.device or B.dtype != torch.float16 or B.dim() != 2 or not B.is_contiguous():
            raise ValueError("B must be a contiguous fp16 [k_cols, F] tensor on the plan's device")
        if B.shape[0] != self.k_cols:
            raise ValueError(f"B has {B.shape[0]} rows, the plan expects {self.k_cols}")
        if B.shape[1] <= 0:
            raise ValueError("B needs at least one feature column")
        return B.shape[1]

    def _check_out(self, out: torch.Tensor, F: int):
        if out.shape != (self.m_rows, F) or not out.is_contiguous() or out.device != self.device:
            raise ValueError("out must be a contiguous [m_rows, F] tensor on the plan's device")
        _out_code(out.dtype)

    def _workspace(self, F: int) -> torch.Tensor:
        ws = self._ws.get(F)
        if ws is None:
            ws = torch.empty(max(self.workspace_bytes(F), 16), dtype=torch.uint8, device=self.device)
            self._ws[F] = ws
        return ws

    def run(self, B: torch.Tensor, out: torch.Tensor | None = None, out_dtype=torch.float16,
            relu: bool = False) -> torch.Tensor:
        F = self._check_B(B)
        if out is None:
            out = torch.empty((self.m_rows, F), dtype=out_dtype, device=self.device)
        else:
            self._check_out(out, F)
        ws = self._workspace(F)
        with torch.cuda.device(self.device):
            _lib.check(self.lib.trs_spmm_run_ex(self._handle, B.data_ptr(), out.data_ptr(), F, _out_code(out.dtype),
                                                1 if relu else 0, ws.data_ptr(), ws.numel(),
                                                _lib.current_stream_ptr(self.device)))
        return out

    @property
    def num_windows(self) -> int:
        return self.lib.trs_spmm_num_windows(self._handle)

    def run_windows(self, B: torch.Tensor, out: torch.Tensor, window_begin: int, window_end: int,
                    relu: bool = False) -> torch.Tensor:
        """trs_spmm_run_windows: the product restricted to the row windows [window_begin, window_end);
        only those rows of `out` are written."""
        F = self._check_B(B)
        self._check_out(out, F)
        ws = self._workspace(F)
        with torch.cuda.device(self.device):
            _lib.check(self.lib.trs_spmm_run_windows(self._handle, B.data_ptr(), out.data_ptr(), F, _out_code(out.dtype),
                                                     1 if relu else 0, ws.data_ptr(), ws.numel(),
                                                     _lib.current_stream_ptr(self.device), int(window_begin),
                                                     int(window_end)))
        return out

    def run_bcast(self, B: torch.Tensor, dst_ptrs, row0: int, relu: bool = False):
        """trs_spmm_run_bcast: the fp16 result rows go straight from the kernel's epilogue into every
        buffer of `dst_ptrs` (device pointers of [N_total, F] fp16 matrices: this GPU's and its
        NVLink peers') at rows row0 + local row.  Asynchronous on the current stream."""
        F = self._check_B(B)
        if not 1 <= len(dst_ptrs) <= 8 or row0 < 0:
            raise ValueError("1 to 8 destination buffers and a non-negative row offset")
        ws = self._workspace(F)
        arr = (C.c_void_p * len(dst_ptrs))(*[int(p) for p in dst_ptrs])
        with torch.cuda.device(self.device):
            _lib.check(self.lib.trs_spmm_run_bcast(self._handle, B.data_ptr(), arr, len(dst_ptrs), int(row0), F,
                                                   1 if relu else 0, ws.data_ptr(), ws.numel(),
                                                   _lib.current_stream_ptr(self.device)))

    def run_static(self, B: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """trs_spmm_run_static: the same product with the partial sums of split windows kept in
        the library's fixed device array, for callers that may not allocate device memory (the
        whole device belongs to their own pool, or an allocation would stall their streams).
        `out` must be given: this path allocates nothing, here or in the library.  Raises
        TrsError(-10) when the plan needs more scratch than the fixed array holds.  Calls on one
        device share the array, so do not let two of them overlap on the GPU."""
        self._check_out(out, self._check_B(B))
        with torch.cuda.device(self.device):
            _lib.check(self.lib.trs_spmm_run_static(self._handle, B.data_ptr(), out.data_ptr(), B.shape[1],
                                                    _out_code(out.dtype), _lib.current_stream_ptr(self.device)))
        return out

    def close(self):
        if getattr(self, "_handle", None) is not None and self._handle:
            self.lib.trs_spmm_plan_destroy(self._handle)
            self._handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def _cpu_format(fmt: Format) -> Format:
    if fmt.device.type != "cpu":
        raise ValueError("the host-buffer entry takes CPU tensors")
    return fmt.half_values().contiguous()


def spmm_forward_host(fmt: Format, rhs: torch.Tensor, dimN: int, mOri: int, kOri: int, window: int = 16,
                      epoches: int = 1):
    """trs_spmm_forward_host: CPU tensors in, fp32 CPU result out; everything is uploaded, run
    `epoches` times and released inside the call, like the reference entry it mirrors."""
    lib = _lib.load()
    f = _cpu_format(fmt)
    rhs = rhs.contiguous()
    out = torch.empty((mOri, dimN), dtype=torch.float32)
    timing = _lib.TrsTiming()
    cf = f.c_struct()
    _lib.check(lib.trs_spmm_forward_host(C.byref(cf), rhs.data_ptr(), out.data_ptr(), dimN, mOri, kOri, window,
                                         epoches, C.byref(timing)))
    return out, timing


class ResidentSpmm:
    """trs_resident_*: the format is uploaded once; each forward copies B host->device, runs,
    and copies C device->host.  For host-resident callers that reuse one matrix."""

    def __init__(self, fmt: Format, mOri: int, kOri: int, window: int = 16, max_dimN: int = 256):
        self.lib = _lib.load()
        self._handle = C.c_void_p()
        self.mOri, self.kOri, self.max_dimN = mOri, kOri, max_dimN
        self._inflight = []  # host tensors of submitted calls, kept alive until wait()
        if fmt.device.type == "cuda":  # e.g. straight from the GPU builder: no host round trip
            self._keep = fmt.half_values().contiguous()
            cf = self._keep.c_struct()
            with torch.cuda.device(fmt.device):
                _lib.check(self.lib.trs_resident_create_device(C.byref(cf), mOri, kOri, window, max_dimN,
                                                               C.byref(self._handle)))
        else:
            self._keep = _cpu_format(fmt)
            cf = self._keep.c_struct()
            _lib.check(self.lib.trs_resident_create(C.byref(cf), mOri, kOri, window, max_dimN, C.byref(self._handle)))

    def _check_host(self, rhs: torch.Tensor, out: torch.Tensor):
        """Shared by forward and submit: the library copies kOri * F and mOri * F elements, so a
        short or strided host tensor would be read or written past its end."""
        if rhs.device.type != "cpu" or out.device.type != "cpu":
            raise ValueError("ResidentSpmm takes host tensors")
        if rhs.dim() != 2 or not rhs.is_contiguous() or not out.is_contiguous() or rhs.dtype != torch.float16:
            raise ValueError("rhs must be a contiguous fp16 [kOri, F] tensor, out contiguous")
        if rhs.shape[0] != self.kOri or out.shape != (self.mOri, rhs.shape[1]):
            raise ValueError(f"rhs must be [{self.kOri}, F] and out [{self.mOri}, F]")
        if not 0 < rhs.shape[1] <= self.max_dimN:
            raise ValueError(f"F must be in 1..{self.max_dimN} (the width this object was created for)")
        _out_code(out.dtype)

    def forward(self, rhs: torch.Tensor, out: torch.Tensor):
        self._check_host(rhs, out)
        timing = _lib.TrsTiming()
        _lib.check(self.lib.trs_resident_forward(self._handle, rhs.data_ptr(), out.data_ptr(), rhs.shape[1],
                                                 _out_code(out.dtype), C.byref(timing)))
        return out, timing

    def submit(self, rhs: torch.Tensor, out: torch.Tensor):
        """trs_resident_submit: enqueue one call and return at once.  Consecutive submits overlap
        (input copy of the next call beside the kernels and the output copy of this one); `rhs`
        and `out` must be pinned host tensors that stay untouched until wait() returns."""
        self._check_host(rhs, out)
        self._inflight.append((rhs, out))
        _lib.check(self.lib.trs_resident_submit(self._handle, rhs.data_ptr(), out.data_ptr(), rhs.shape[1],
                                                _out_code(out.dtype)))

    def wait(self):
        """trs_resident_wait: block until every submitted call is complete."""
        try:
            _lib.check(self.lib.trs_resident_wait(self._handle))
        finally:
            self._inflight.clear()

    def close(self):
        if self._handle:
            self.lib.trs_resident_destroy(self._handle)
            self._handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
