"""Seeded input generators shared by the fixture generator's consumers.

These restate ``tests/golden/make_golden.py``'s generators without importing
the reference, so the tests can rebuild the inputs whose reference outputs are
stored in ``tests/golden/*.npz``.
"""
import numpy as np

GEMV_CASES = {"n01_33x2052": ((33, 2052), 21), "n01_16x8192": ((16, 8192), 22),
              "n01_7x12": ((7, 12), 23), "int_16x4096": ((16, 4096), 24),
              "c3_24x4100": ((24, 4100), 25)}
DOT_CASES = ((10_000, 31), (500_000, 32), (1027, 33), (1_500_000, 34))  # bench_dot.py:15 + a ragged length


def sample_f32(kind: str, n: int, seed: int) -> np.ndarray:
    rng = np.random.default_rng(seed)
    if kind == "bits":
        return rng.integers(0, 2 ** 32, size=n, dtype=np.uint64).astype(np.uint32).view(np.float32)
    if kind == "lognormal":
        return (rng.standard_normal(n) * np.exp(rng.uniform(-20, 12, n))).astype(np.float32)
    raise ValueError(kind)


def c3_matrix(shape, seed: int) -> np.ndarray:
    """90 % 4*N(0,1), 5 % magnitudes in [2^-9, 2^-6] (E4M3 subnormal range),
    5 % in [448, 1000] (beyond E4M3 saturation), random signs; fp32."""
    rng = np.random.default_rng(seed)
    n = int(np.prod(shape))
    x = (4.0 * rng.standard_normal(n)).astype(np.float32)
    u = rng.random(n)
    sign = np.where(rng.random(n) < 0.5, -1.0, 1.0).astype(np.float32)
    small = (sign * rng.uniform(2.0 ** -9, 2.0 ** -6, n)).astype(np.float32)
    big = (sign * rng.uniform(448.0, 1000.0, n)).astype(np.float32)
    x = np.where(u < 0.05, small, np.where(u < 0.10, big, x))
    return x.reshape(shape).astype(np.float32)


def gemv_case(name: str):
    shape, seed = GEMV_CASES[name]
    rng = np.random.default_rng(seed)
    if name.startswith("n01"):
        A = rng.standard_normal(shape).astype(np.float16)
        v = rng.standard_normal(shape[1]).astype(np.float16)
    elif name.startswith("int"):
        A = rng.integers(-3, 3, size=shape).astype(np.float16)
        v = rng.integers(-3, 3, size=shape[1]).astype(np.float16)
    else:
        A = c3_matrix(shape, seed)
        v = rng.standard_normal(shape[1]).astype(np.float32)
    return A, v


def dot_case(n: int, seed: int):
    rng = np.random.default_rng(seed)
    return rng.standard_normal(n).astype(np.float16), rng.standard_normal(n).astype(np.float16)
