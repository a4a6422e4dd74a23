"""Compile libfeather_b200.so in-tree with nvcc for sm_100a.

    python -m feather_b200.csrc.build [--force] [--verbose] [--debug-bounds]

The library is plain CUDA runtime code behind a C ABI (include/feather_b200.h):
no torch headers, no pybind; Python reaches it with ctypes.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
LIB = os.path.join(PKG, "libfeather_b200.so")
LIB_DEBUG = os.path.join(PKG, "libfeather_b200_debug.so")  # -DFEATHER_DEBUG_BOUNDS
SOURCES = ["feather_b200.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-shared", "-cudart", "shared"]


def dependencies() -> list:
    """Every file the library is built from: all kernel sources and headers in
    this directory plus the public C header."""
    import glob
    deps = sorted(glob.glob(os.path.join(HERE, "*.cu")) + glob.glob(os.path.join(HERE, "*.cuh")))
    deps.append(os.path.join(os.path.dirname(PKG), "include", "feather_b200.h"))
    return deps


def _nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: cannot build libfeather_b200.so")
    return nvcc


def is_stale(lib: str = LIB) -> bool:
    if not os.path.exists(lib):
        return True
    t = os.path.getmtime(lib)
    return any(os.path.getmtime(d) > t for d in dependencies() if os.path.exists(d))


def build(force: bool = False, verbose: bool = False, extra_flags=(), debug_bounds: bool = False) -> str:
    """Build the library; ``debug_bounds`` builds the bounds-checking variant
    beside it (loaded when FEATHER_DEBUG_BOUNDS=1 is in the environment)."""
    lib = LIB_DEBUG if debug_bounds else LIB
    if debug_bounds:
        extra_flags = (*extra_flags, "-DFEATHER_DEBUG_BOUNDS")
    if not force and not is_stale(lib):
        return lib
    cmd = [_nvcc(), *NVCC_FLAGS, *extra_flags, *(["-Xptxas", "-v"] if verbose else []), "-o", lib,
           *[os.path.join(HERE, s) for s in SOURCES]]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode:
        raise RuntimeError("nvcc failed building " + os.path.basename(lib))
    return lib


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv,
                debug_bounds="--debug-bounds" in sys.argv))
