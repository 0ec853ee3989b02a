"""Builds libggr_attn.so (CUDA kernels + C ABI) in-tree for sm_100a with nvcc.

Usage: python -m gguf_runner_b200.build [--force] [-v] [--trace]
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_PATH = os.path.join(PKG_DIR, "libggr_attn.so")
# diagnostic build: the kernels additionally write phase time stamps (see `bench.py --case decode_stamps`)
TRACE_LIB_PATH = os.path.join(PKG_DIR, "libggr_attn_trace.so")
SOURCES = ["ggr_attn.cu", "host_plan.cpp"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the attention library can only be built with the CUDA toolkit")


def _stale(path: str = LIB_PATH) -> bool:
    if not os.path.exists(path):
        return True
    built = os.path.getmtime(path)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    deps.append(os.path.join(PKG_DIR, "..", "include", "ggr_attn.h"))
    return any(os.path.getmtime(d) > built for d in deps if os.path.exists(d))


def build_library(force: bool = False, verbose: bool = False, trace: bool = False) -> str:
    """Compiles the library if it is missing or older than its sources; returns its path.
    trace=True builds the diagnostic variant (-DGGR_TC_TRACE) next to it."""
    out = TRACE_LIB_PATH if trace else LIB_PATH
    if not force and not _stale(out):
        return out
    cmd = [
        _nvcc(),
        "-gencode", "arch=compute_100a,code=sm_100a",
        "-lineinfo", "-O3", "-std=c++17",
        "-Xcompiler", "-fPIC", "-shared",
        "-o", out,
    ]
    if trace:
        cmd += ["-DGGR_TC_TRACE"]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += [os.path.join(CSRC, s) for s in SOURCES]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + proc.stdout + proc.stderr)
    if verbose:
        sys.stderr.write(proc.stderr)
    return out


if __name__ == "__main__":
    path = build_library(force="--force" in sys.argv, verbose="-v" in sys.argv, trace="--trace" in sys.argv)
    print(path)
