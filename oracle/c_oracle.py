"""Build + ctypes binding of the C oracle (TEST INFRASTRUCTURE ONLY).

``feather_oracle.c`` is the multi-threaded restatement used for full-size
parity checks and as the timed CPU baseline.  Only tests, the smoke check and
the benchmark's CPU legs may import this module.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SRC = os.path.join(_HERE, "feather_oracle.c")
_LIB = os.path.join(_HERE, "libfeather_oracle.so")
_MODE = {"E5M2": 0, "E4M3": 1}
_lib = None


def build(force: bool = False) -> str:
    """gcc -O3 -fopenmp the C restatement into oracle/libfeather_oracle.so."""
    if not force and os.path.exists(_LIB) and os.path.getmtime(_LIB) >= os.path.getmtime(_SRC):
        return _LIB
    cmd = ["gcc", "-O3", "-march=x86-64-v2", "-ffp-contract=off", "-fopenmp", "-fPIC",
           "-shared", "-o", _LIB, _SRC, "-lm"]
    subprocess.run(cmd, check=True)
    return _LIB


def load():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB):
            build()
        lib = ctypes.CDLL(_LIB)
        vp, i32, i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64
        lib.fo_num_threads.restype = i32
        lib.fo_set_num_threads.argtypes = [i32]
        lib.fo_encode.argtypes = [vp, i32, vp, i64, i32]
        lib.fo_pack.argtypes = [vp, i32, vp, i64, i32]
        lib.fo_decode_table.argtypes = [vp, i32, i32]
        lib.fo_unpack.argtypes = [vp, vp, i64, i32, i32]
        lib.fo_gemv.argtypes = [vp, vp, vp, i64, i64, i32, i32]
        lib.fo_gemv_f64.argtypes = [vp, vp, vp, i64, i64, i32]
        lib.fo_dot.argtypes = [vp, vp, i64, i32, i32]
        lib.fo_dot.restype = ctypes.c_double
        _lib = lib
    return _lib


def _mode(mode: str) -> int:
    if mode not in _MODE:
        raise NotImplementedError(f"Mode {mode} not supported")
    return _MODE[mode]


def _ptr(a: np.ndarray) -> ctypes.c_void_p:
    return ctypes.c_void_p(a.ctypes.data)


def num_threads() -> int:
    return int(load().fo_num_threads())


def use_all_cores() -> int:
    """Run on every core this process may use, whatever OMP_NUM_THREADS says."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    load().fo_set_num_threads(n)
    return num_threads()


def pack(x: np.ndarray, mode: str = "E5M2") -> np.ndarray:
    x = np.ascontiguousarray(np.asarray(x).reshape(-1))
    if x.dtype not in (np.float16, np.float32):
        raise TypeError(x.dtype)
    out = np.zeros((x.size + 3) // 4, dtype=np.uint32)
    load().fo_pack(_ptr(x), 0 if x.dtype == np.float16 else 1, _ptr(out), x.size, _mode(mode))
    return out


def decode_table(mode: str, semantics: str = "kernel") -> np.ndarray:
    tab = np.empty(256, dtype=np.float32)
    load().fo_decode_table(_ptr(tab), _mode(mode), {"kernel": 0, "ieee": 1}[semantics])
    return tab


def unpack(words: np.ndarray, mode: str = "E5M2", semantics: str = "kernel",
           n_elems: int | None = None) -> np.ndarray:
    w = np.ascontiguousarray(np.asarray(words).view(np.uint32).reshape(-1))
    n = w.size * 4 if n_elems is None else int(n_elems)
    out = np.empty(n, dtype=np.float32)
    load().fo_unpack(_ptr(w), _ptr(out), n, _mode(mode), {"kernel": 0, "ieee": 1}[semantics])
    return out


def gemv(m_words: np.ndarray, v_words: np.ndarray, m_shape, mode: str = "E5M2",
         acc: str = "f32") -> np.ndarray:
    M, N = int(m_shape[0]), int(m_shape[1])
    if N % 4:
        raise ValueError("N must be a multiple of 4")
    m = np.ascontiguousarray(np.asarray(m_words).view(np.uint32).reshape(-1))
    v = np.ascontiguousarray(np.asarray(v_words).view(np.uint32).reshape(-1))
    assert m.size >= M * (N // 4) and v.size >= N // 4
    if acc == "f64":
        out = np.empty(M, dtype=np.float64)
        load().fo_gemv_f64(_ptr(m), _ptr(v), _ptr(out), M, N, _mode(mode))
        return out
    out = np.empty(M, dtype=np.float32)
    load().fo_gemv(_ptr(m), _ptr(v), _ptr(out), M, N, _mode(mode), 0)
    return out


def dot(x1_words: np.ndarray, x2_words: np.ndarray, mode: str = "E5M2", acc: str = "f32"):
    a = np.ascontiguousarray(np.asarray(x1_words).view(np.uint32).reshape(-1))
    b = np.ascontiguousarray(np.asarray(x2_words).view(np.uint32).reshape(-1))
    if a.size != b.size:
        raise ValueError("operands differ in length")
    r = load().fo_dot(_ptr(a), _ptr(b), a.size, _mode(mode), 1 if acc == "f64" else 0)
    return np.float64(r) if acc == "f64" else np.float32(r)


if __name__ == "__main__":
    print(build(force=True))
