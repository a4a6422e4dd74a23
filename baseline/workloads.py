"""Seeded synthetic workloads of the benchmark configurations, generated with a
torch Generator on a given device.  The reference worker (its own process) and
the tests / the benchmark call the same function with the same seed on the same
GPU model and get the same tensors, so only results travel between the two
processes, never the inputs.
"""
from __future__ import annotations

import torch

#: name -> (kind, shape or length, seed, mode)
CASES = {
    "c1_e5m2_4096": ("n01", (4096, 4096), 0, "E5M2"),
    "c1_e4m3_4096": ("n01", (4096, 4096), 0, "E4M3"),
    "c2_e5m2_16384": ("n01", (16384, 16384), 1, "E5M2"),
    "c3_e4m3_8192x8192": ("c3", (8192, 8192), 2, "E4M3"),
    "c3_e4m3_16384x8192": ("c3", (16384, 8192), 3, "E4M3"),
    "c3_e4m3_16384x16384": ("c3", (16384, 16384), 4, "E4M3"),
    # feather/benchmark/bench_gemv.py:14-15, 48-58: integers in [-3, 2], every (M, N) combination
    **{f"int_{m}x{n}": ("int", (m, n), 40 + i, "E5M2")
       for i, (m, n) in enumerate((m, n) for m in (4096, 8192, 16384) for n in (4096, 8192, 16384))},
    "dot_e5m2_2pow26": ("dot", 1 << 26, 1, "E5M2"),
    # feather/benchmark/bench_dot.py:15
    "dot_e5m2_1500000": ("dot", 1_500_000, 33, "E5M2"),
    "dot_e5m2_10000": ("dot", 10_000, 34, "E5M2"),
    # feather/benchmark/bench_attention.py:14-15: sequence lengths up to 8192, widths 64, 256, 512
    # (plus 128, and a length that leaves the last key tile ragged)
    "attn_s4096_d128": ("attn", (4096, 128), 60, "E5M2"),
    "attn_s8192_d64": ("attn", (8192, 64), 61, "E5M2"),
    "attn_s4096_d256": ("attn", (4096, 256), 62, "E5M2"),
    "attn_s2500_d64": ("attn", (2500, 64), 63, "E5M2"),
    "attn_s1024_d512": ("attn", (1024, 512), 64, "E5M2"),
}


def c3_matrix(shape, gen: torch.Generator, device) -> torch.Tensor:
    """fp32: 90 % 4*N(0,1), 5 % magnitudes uniform in [2^-9, 2^-6] (the E4M3
    subnormal range), 5 % uniform in [448, 1000] (beyond E4M3 saturation),
    random signs."""
    M, N = shape
    x = 4.0 * torch.randn(M, N, device=device, generator=gen)
    u = torch.rand(M, N, device=device, generator=gen)
    sign = torch.where(torch.rand(M, N, device=device, generator=gen) < 0.5, -1.0, 1.0)
    r = torch.rand(M, N, device=device, generator=gen)
    small = sign * (2.0 ** -9 + r * (2.0 ** -6 - 2.0 ** -9))
    big = sign * (448.0 + r * (1000.0 - 448.0))
    return torch.where(u < 0.05, small, torch.where(u < 0.10, big, x))


def make(name: str, device="cuda"):
    """Returns (A, v, mode) for a GEMV case, (x1, x2, mode) for a dot case, ((q, k, v), None,
    mode) for an attention case."""
    kind, shape, seed, mode = CASES[name]
    gen = torch.Generator(device=device).manual_seed(seed)
    if kind == "attn":
        return (tuple(torch.randn(*shape, device=device, generator=gen, dtype=torch.float16) for _ in range(3)),
                None, mode)
    if kind == "n01":
        M, N = shape
        return (torch.randn(M, N, device=device, generator=gen, dtype=torch.float16),
                torch.randn(N, device=device, generator=gen, dtype=torch.float16), mode)
    if kind == "c3":
        A = c3_matrix(shape, gen, device)
        return A, torch.randn(shape[1], device=device, generator=gen), mode
    if kind == "int":
        M, N = shape
        return (torch.randint(-3, 3, (M, N), device=device, generator=gen).to(torch.float16),
                torch.randint(-3, 3, (N,), device=device, generator=gen).to(torch.float16), mode)
    if kind == "dot":
        return (torch.randn(shape, device=device, generator=gen).half(),
                torch.randn(shape, device=device, generator=gen).half(), mode)
    raise KeyError(name)


def is_dot(name: str) -> bool:
    return CASES[name][0] == "dot"


def is_attention(name: str) -> bool:
    return CASES[name][0] == "attn"
