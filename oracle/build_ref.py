#!/usr/bin/env python3
"""Compile the reference's own CPU sources, where they lie, into oracle/_ref/.

TEST INFRASTRUCTURE ONLY.  Nothing the product ships imports this directory.

What gets built (each straight from the read-only reference tree, unmodified,
with the system g++; no reference source is copied into this repository):

  Libra5BlockOnline      TR-source/Block/block_online.cpp            (torch C++ extension)
  matching_utils         TR-source/Block/block_matching_window_para_dr.cpp   (pybind11)
  matching_utils_hash    TR-source/Block/block_matching_hash.cpp             (pybind11)
  matching_utils_bucket  TR-source/Block/block_matching_bucket.cpp           (pybind11)

The resulting modules are used (a) to pin the restatement in oracle/ against the
real reference, (b) to generate the committed fixtures in tests/golden/ and
(c) optionally as a timed CPU baseline.  When the reference tree is absent
(e.g. on a GPU box) the script does nothing and reports that.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"
CXX = "/usr/bin/g++"  # the image's default g++ wrapper produces a module that crashes in iostream


def _ref_root() -> Path:
    return Path(os.environ.get("TRS_REFERENCE_ROOT", "/root/reference"))


def _ext_suffix() -> str:
    return sysconfig.get_config_var("EXT_SUFFIX")


def _up_to_date(dst: Path, src: Path) -> bool:
    return dst.exists() and dst.stat().st_mtime >= src.stat().st_mtime


def build_torch_ext(name: str, src: Path, verbose: bool = True) -> Path | None:
    from torch.utils import cpp_extension as ce  # heavy import, keep local
    import torch

    dst = OUT / f"{name}{_ext_suffix()}"
    if _up_to_date(dst, src):
        return dst
    inc = [f"-I{p}" for p in ce.include_paths()] + [f"-I{sysconfig.get_paths()['include']}"]
    libdir = ce.library_paths()[0]
    cmd = [
        CXX, "-O3", "-fopenmp", "-mcx16", "-std=c++17", "-shared", "-fPIC",
        f"-DTORCH_EXTENSION_NAME={name}", "-DTORCH_API_INCLUDE_EXTENSION_H",
        f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
        *inc, str(src), "-o", str(dst),
        f"-L{libdir}", f"-Wl,-rpath,{libdir}",
        "-lc10", "-ltorch_cpu", "-ltorch", "-ltorch_python",
    ]
    if verbose:
        print("[oracle/_ref]", " ".join(cmd), flush=True)
    subprocess.run(cmd, check=True)
    return dst


def build_pybind_ext(name: str, src: Path, verbose: bool = True) -> Path | None:
    import pybind11

    dst = OUT / f"{name}{_ext_suffix()}"
    if _up_to_date(dst, src):
        return dst
    cmd = [
        CXX, "-O3", "-fopenmp", "-std=c++17", "-shared", "-fPIC",
        f"-I{pybind11.get_include()}", f"-I{sysconfig.get_paths()['include']}",
        str(src), "-o", str(dst),
    ]
    if verbose:
        print("[oracle/_ref]", " ".join(cmd), flush=True)
    subprocess.run(cmd, check=True)
    return dst


def build_all(verbose: bool = True) -> dict:
    """Build whatever can be built; returns {module: path or reason}."""
    root = _ref_root()
    report: dict = {}
    if not root.exists():
        return {"skipped": f"reference tree {root} not present"}
    OUT.mkdir(exist_ok=True)
    block = root / "TR-source" / "Block"
    jobs = [
        ("Libra5BlockOnline", block / "block_online.cpp", build_torch_ext),
        ("matching_utils", block / "block_matching_window_para_dr.cpp", build_pybind_ext),
        ("matching_utils_hash", block / "block_matching_hash.cpp", build_pybind_ext),
        ("matching_utils_bucket", block / "block_matching_bucket.cpp", build_pybind_ext),
    ]
    for name, src, fn in jobs:
        try:
            report[name] = str(fn(name, src, verbose))
        except Exception as exc:  # report, never hide
            report[name] = f"FAILED: {exc}"
    return report


if __name__ == "__main__":
    rep = build_all()
    for k, v in rep.items():
        print(f"{k}: {v}")
    sys.exit(1 if any(str(v).startswith("FAILED") for v in rep.values()) else 0)
