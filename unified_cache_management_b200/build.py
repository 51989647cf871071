"""Builds ``libucmr_b200.so`` (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

``python -m unified_cache_management_b200.build`` or ``build_library()``.
"""
from __future__ import annotations

import os
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
INCLUDE = os.path.join(os.path.dirname(PKG_DIR), "include")
LIB_PATH = os.path.join(PKG_DIR, "libucmr_b200.so")
SOURCES = ["api.cu", "scan.cu", "scan_ring.cu", "scan_rows.cu", "topk.cu", "gather.cu", "encode.cu", "noalloc.cu", "float_retrieval.cu"]


def _sources():
    return [os.path.join(CSRC, s) for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]


def _deps():
    deps = _sources() + [os.path.join(CSRC, "common.cuh"), os.path.join(INCLUDE, "ucmr.h")]
    return [d for d in deps if os.path.exists(d)]


TRACE_LIB_PATH = os.path.join(PKG_DIR, "libucmr_b200_trace.so")


def up_to_date(path: str = LIB_PATH) -> bool:
    if not os.path.exists(path):
        return False
    t = os.path.getmtime(path)
    return all(os.path.getmtime(d) <= t for d in _deps())


def build_library(force: bool = False, verbose: bool = False, trace: bool = False) -> str:
    """Builds the library; ``trace`` builds the step-timeline variant (-DUCMR_TRACE, see ucmr_trace_read in ucmr.h)
    next to it as ``libucmr_b200_trace.so`` (load it through the UCMR_LIBRARY environment variable)."""
    out = TRACE_LIB_PATH if trace else LIB_PATH
    if not force and up_to_date(out):
        return out
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
           "-shared", "-Xcompiler", "-fPIC", "-I" + INCLUDE, "-I" + CSRC, "--threads", "4"]
    if trace:
        cmd += ["-DUCMR_TRACE"]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += _sources() + ["-o", out]
    subprocess.check_call(cmd)
    return out


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv, trace="--trace" in sys.argv))
