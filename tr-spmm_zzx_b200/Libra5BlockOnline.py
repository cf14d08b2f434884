"""Drop-in for the reference's `Libra5BlockOnline` torch extension
(TR-source/Block/block_online.cpp:873-876): same function name, positional signature and return
list, with the build done by GPU kernels of libtrspmm.so.

As in the reference the inputs are CPU tensors (int32 / int32 / float32) and 30 CPU tensors come
back, the last one a 0-d float32 with the build time in seconds.  CUDA inputs are accepted as an
extension and then the arrays are returned on that device.  `wide`, `sptc_min_util` and
`sptc_threshold` are accepted and unused, exactly like the reference (block_online.cpp:548-553).
"""
from __future__ import annotations

import time

import torch

from trspmm.builder import build_format

__all__ = ["block_sptc_2to4_online"]


def block_sptc_2to4_online(row1, column1, values1, partSize_t, partSize_c, shortSize, density, window, wide,
                           tc_min_util, sptc_min_util, sptc_threshold):
    if not (row1.dtype == torch.int32 and column1.dtype == torch.int32):
        raise RuntimeError("Expected row1.dtype() == torch::kInt32 && column1.dtype() == torch::kInt32 to be true")
    if values1.dtype != torch.float32:
        raise RuntimeError("Expected values1.dtype() == torch::kFloat32 to be true")
    if not (0 < window <= 32 and 0 < wide <= 32):
        raise RuntimeError("Expected window > 0 && window <= 32 && wide > 0 && wide <= 32 to be true")
    if window > 16:
        raise RuntimeError("window must be <= 16: the 2-bit-per-row column vectors of the format hold 16 rows")
    t0 = time.perf_counter()
    on_cpu = not row1.is_cuda
    dev = torch.device("cuda", torch.cuda.current_device()) if on_cpu else row1.device
    fmt, _ = build_format(row1.to(dev), column1.to(dev), values1.to(dev), int(partSize_t), int(partSize_c),
                          int(shortSize), int(density), int(window), float(tc_min_util))
    arrays = fmt.arrays()
    if on_cpu:
        arrays = [a.cpu() for a in arrays]
    return arrays + [torch.tensor(time.perf_counter() - t0, dtype=torch.float32)]
