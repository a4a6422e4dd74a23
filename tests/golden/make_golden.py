"""Generate the golden fixtures in this directory from the REFERENCE itself.

Run where the reference checkout is available (it is not needed afterwards;
the ``.npz`` files are committed):

    TRITON_INTERPRET=1 PYTHONDONTWRITEBYTECODE=1 \
        PYTHONPATH=<reference checkout> python tests/golden/make_golden.py

What is executed is the reference's own code only: its packer
(``feather/packers/fp8.py``: numpy + ml_dtypes), its CPU unpacker, and its
Triton GEMV / dot kernels run on CPU tensors through Triton's interpreter (the
reference launch wrappers hard-code the "cuda" device, so the jitted kernel
objects are launched directly with the same arguments the wrappers pass).
Inputs are seeded; tests regenerate them from the seeds stored here and never
need the reference.
"""
import logging
import os
import sys
import warnings

os.environ.setdefault("TRITON_INTERPRET", "1")
import numpy as np
import torch

logging.disable(logging.WARNING)  # the packer logs whole arrays for fp32 input
warnings.simplefilter("ignore")

import feather.routines.activations as ref_act
import feather.routines.attention as ref_attn
import feather.routines.dot as ref_dot
import feather.routines.gemv as ref_gemv
from feather.packers.fp8 import pack_fp8_ndarray, pack_fp8_tensor, unpack_into_fp8_ndarray

HERE = os.path.dirname(os.path.abspath(__file__))
MODES = ("E5M2", "E4M3")
GEMV_KERNEL = {"E5M2": ref_gemv._gemv_fp8_e5m2_acc_fp32_kernel,
               "E4M3": ref_gemv._gemv_fp8_e4m3_acc_fp32_kernel}

# fp32 edge inputs: zeros, E4M3/E5M2 subnormal range and ties, saturation
# boundaries, infinities and NaNs with payloads.
EDGE_F32 = np.concatenate([
    np.array([0.0, -0.0, 2.0 ** -17, 2.0 ** -16, 2.0 ** -15, 2.0 ** -14, 2.0 ** -10,
              2.0 ** -10 * (1 + 2.0 ** -20), 2.0 ** -10 * (1 - 2.0 ** -20), 2.0 ** -9,
              3 * 2.0 ** -10, 2.0 ** -6, 2.0 ** -6 * (1 - 2.0 ** -5), 448.0, 463.99997, 464.0,
              464.00003, 464.25, 480.0, 1000.0, 57344.0, 61439.996, 61440.0, 65504.0, 65520.0,
              1e30, 1e-30, np.inf], dtype=np.float32),
    -np.array([2.0 ** -10, 464.0, 464.25, 61440.0, np.inf, 1e-30], dtype=np.float32),
    np.array([0x7F800001, 0xFF800001, 0x7FC00000, 0xFFC00000, 0x7FFFFFFF, 0xFFFFFFFF,
              0x00000001, 0x807FFFFF], dtype=np.uint32).view(np.float32),
])


def sample_f32(kind: str, n: int, seed: int) -> np.ndarray:
    """Seeded fp32 inputs; tests call this too (imported from here)."""
    rng = np.random.default_rng(seed)
    if kind == "bits":  # uniform random bit patterns
        return rng.integers(0, 2 ** 32, size=n, dtype=np.uint64).astype(np.uint32).view(np.float32)
    if kind == "lognormal":  # magnitudes across every binade both formats cover
        return (rng.standard_normal(n) * np.exp(rng.uniform(-20, 12, n))).astype(np.float32)
    raise ValueError(kind)


def c3_matrix(shape, seed: int) -> np.ndarray:
    """fp32 matrix with 90 % 4*N(0,1), 5 % in the E4M3 subnormal range
    [2^-9, 2^-6], 5 % beyond saturation [448, 1000], random signs."""
    rng = np.random.default_rng(seed)
    n = int(np.prod(shape))
    x = (4.0 * rng.standard_normal(n)).astype(np.float32)
    u = rng.random(n)
    sign = np.where(rng.random(n) < 0.5, -1.0, 1.0).astype(np.float32)
    small = (sign * rng.uniform(2.0 ** -9, 2.0 ** -6, n)).astype(np.float32)
    big = (sign * rng.uniform(448.0, 1000.0, n)).astype(np.float32)
    x = np.where(u < 0.05, small, np.where(u < 0.10, big, x))
    return x.reshape(shape).astype(np.float32)


def ref_pack(x: np.ndarray, mode: str) -> np.ndarray:
    return np.ascontiguousarray(pack_fp8_ndarray(x, mode=mode)).view(np.uint32).copy()


def run_gemv(mw: np.ndarray, vw: np.ndarray, shape, mode: str) -> np.ndarray:
    M, N = shape
    m = torch.from_numpy(mw.view(np.int32).copy())
    v = torch.from_numpy(vw.view(np.int32).copy())
    out = torch.empty((M,), dtype=torch.float32)
    GEMV_KERNEL[mode][(M,)](m, v, out, N // 4, BLOCK_SIZE=1024)  # gemv.py:178-183
    return out.numpy().copy()


def run_dot(aw: np.ndarray, bw: np.ndarray) -> np.float32:
    a = torch.from_numpy(aw.view(np.int32).copy())
    b = torch.from_numpy(bw.view(np.int32).copy())
    out = torch.tensor(0.0, dtype=torch.float32)
    n = a.numel()
    grid = ((n + 1023) // 1024,)
    ref_dot._dot_fp8_e5m2_acc_fp32_kernel[grid](a, b, out, n, BLOCK_SIZE=1024)  # dot.py:253-259
    return np.float32(out.item())


def run_relu(xw: np.ndarray) -> np.ndarray:
    x = torch.from_numpy(xw.view(np.int32).copy())
    out = torch.empty((4 * x.numel(),), dtype=torch.float32)
    grid = ((x.numel() + 8191) // 8192,)
    ref_act._relu_1d_fp8_ret_fp32_kernel[grid](x, out, x.numel(), 8192)  # activations.py:36-40
    return out.numpy().copy()


def make_relu() -> None:
    """ReLU of packed E5M2 through the reference kernel: every code (as a byte
    stream, so every lane), and a seeded N(0, 1) vector that spans two blocks."""
    r = {}
    r["all_codes_out"] = run_relu(np.arange(256, dtype=np.uint8).view(np.uint32))
    rng = np.random.default_rng(41)
    x = rng.standard_normal(4 * 9000 + 4).astype(np.float16)
    r["n36004_out"] = run_relu(ref_pack(x, "E5M2"))
    r["n36004_seed"] = np.array(41, dtype=np.int64)
    np.savez_compressed(os.path.join(HERE, "relu.npz"), **r)
    print("relu", os.path.getsize(os.path.join(HERE, "relu.npz")), "bytes")


def make_attention() -> None:
    """Flash attention on packed E5M2 through the reference kernel (its jitted
    function under the autotuner, launched as the wrapper does, attention.py:172-178):
    N(0, 1) inputs at sequence lengths that do and do not fill the last key tile."""
    a = {}
    for seq, d, seed in ((128, 64, 51), (100, 32, 52), (200, 128, 53), (64, 16, 54), (130, 256, 55),
                         (64, 512, 56)):
        rng = np.random.default_rng(seed)
        q, k, v = (ref_pack(rng.standard_normal((seq, d)).astype(np.float16), "E5M2") for _ in range(3))
        tq, tk, tv = (torch.from_numpy(x.view(np.int32).copy()) for x in (q, k, v))
        out = torch.empty((seq, d), dtype=torch.float32)
        kern = ref_attn._flash_attention_fp8_e5m2_acc_fp32_kernel
        kern = getattr(kern, "fn", kern)                       # the jitted function under the autotuner
        kern[((seq + 63) // 64,)](tq, tk, tv, out, seq, d // 4, _tile_sz=64)
        a[f"s{seq}_d{d}_out"] = out.numpy().copy()
        a[f"s{seq}_d{d}_seed"] = np.array(seed, dtype=np.int64)
    np.savez_compressed(os.path.join(HERE, "attention.npz"), **a)
    print("attention", os.path.getsize(os.path.join(HERE, "attention.npz")), "bytes")


def make_dot() -> None:
    """dot through the reference kernel (E5M2 is the only FP8 dot it has)."""
    d = {}
    d["doc"] = run_dot(ref_pack(np.array([2, 0, -3, 1], dtype=np.float16), "E5M2"),
                       ref_pack(np.array([-1, 0, -3, 1], dtype=np.float16), "E5M2"))  # dot.py:244-251
    # bench_dot.py:15 has n = 10 000, 500 000 and 1 500 000; 1027 adds a ragged length
    for n, seed in ((10_000, 31), (500_000, 32), (1027, 33), (1_500_000, 34)):
        rng = np.random.default_rng(seed)
        x1 = rng.standard_normal(n).astype(np.float16)
        x2 = rng.standard_normal(n).astype(np.float16)
        a, bb = ref_pack(x1, "E5M2"), ref_pack(x2, "E5M2")
        if n <= 20_000:  # larger inputs are regenerated from the seed by the tests
            d[f"n{n}_a"], d[f"n{n}_b"] = a, bb
        d[f"n{n}_wordsum"] = np.array([a.astype(np.uint64).sum(), bb.astype(np.uint64).sum()],
                                      dtype=np.uint64)
        d[f"n{n}_out"] = run_dot(a, bb)
        d[f"n{n}_seed"] = np.array(seed, dtype=np.int64)
    np.savez_compressed(os.path.join(HERE, "dot.npz"), **d)


def main() -> None:
    if sys.argv[1:] == ["dot"]:  # only the dot fixture (the others are unchanged)
        return make_dot()
    if sys.argv[1:] == ["relu"]:  # only the ReLU fixture (the others are unchanged)
        return make_relu()
    if sys.argv[1:] == ["attention"]:
        return make_attention()
    make_relu()
    make_attention()
    # 1. encode: every fp16 bit pattern, seeded fp32 samples, fp32 edge list
    enc = {}
    h = np.arange(65536, dtype=np.uint16).view(np.float16)
    for mode in MODES:
        enc[f"fp16_all_{mode}"] = ref_pack(h, mode).view(np.uint8)
        for kind, seed in (("bits", 11), ("lognormal", 12)):
            enc[f"fp32_{kind}_{mode}"] = ref_pack(sample_f32(kind, 131072, seed), mode).view(np.uint8)
        enc[f"fp32_edge_{mode}"] = ref_pack(EDGE_F32, mode).view(np.uint8)[: EDGE_F32.size]
    enc["fp32_edge_input_bits"] = EDGE_F32.view(np.uint32)
    # pack_fp8_tensor layout: ragged tail (numel % 4 != 0) and 2-D input
    t = torch.from_numpy(sample_f32("lognormal", 4 * 7 + 3, 13).astype(np.float16))
    for mode in MODES:
        w = pack_fp8_tensor(t, mode=mode)
        assert w.dtype == torch.uint32 and w.ndim == 1
        enc[f"ragged31_{mode}"] = w.view(torch.int32).numpy().view(np.uint32)
        w2 = pack_fp8_tensor(t[:28].reshape(7, 4), mode=mode)
        enc[f"matrix7x4_{mode}"] = w2.view(torch.int32).numpy().view(np.uint32)
    np.savez_compressed(os.path.join(HERE, "encode.npz"), **enc)

    # 2. decode tables.  kernel semantics: each code alone in byte lane k of a
    # one-word row, times 1.0 in the same lane of the vector (also pins the
    # lane pairing).  ieee semantics: the reference CPU unpacker.
    dec = {}
    one = {"E5M2": 0x3C, "E4M3": 0x38}
    codes = np.arange(256, dtype=np.uint32)
    for mode in MODES:
        for lane in range(4):
            mw = codes << (8 * lane)
            vw = np.array([one[mode] << (8 * lane)], dtype=np.uint32)
            dec[f"kernel_{mode}_lane{lane}"] = run_gemv(mw, vw, (256, 4), mode)
        allcodes = np.arange(256, dtype=np.uint8).view(np.uint32).view(np.float32)
        dec[f"ieee_{mode}"] = unpack_into_fp8_ndarray(allcodes, mode=mode).astype(np.float32)
    np.savez_compressed(os.path.join(HERE, "decode.npz"), **dec)

    # 3. GEMV through the reference kernels
    g = {}
    a = np.array([[1, 1, -2, 0], [-3, -3, -2, -3], [0, 1, 1, -2], [2, 0, -1, 2]], dtype=np.float16)
    b = np.array([2, 2, -1, 2], dtype=np.float16)
    for mode in MODES:  # the docstring example, gemv.py:163-174
        g[f"doc_{mode}"] = run_gemv(ref_pack(a, mode), ref_pack(b, mode), (4, 4), mode)
    cases = {"n01_33x2052": ((33, 2052), 21), "n01_16x8192": ((16, 8192), 22),
             "n01_7x12": ((7, 12), 23), "int_16x4096": ((16, 4096), 24),
             "c3_24x4100": ((24, 4100), 25)}
    for name, (shape, seed) in cases.items():
        rng = np.random.default_rng(seed)
        if name.startswith("n01"):
            A = rng.standard_normal(shape).astype(np.float16)
            v = rng.standard_normal(shape[1]).astype(np.float16)
        elif name.startswith("int"):  # bench_gemv.py:52-57: integers in [-3, 2]
            A = rng.integers(-3, 3, size=shape).astype(np.float16)
            v = rng.integers(-3, 3, size=shape[1]).astype(np.float16)
        else:
            A = c3_matrix(shape, seed)
            v = rng.standard_normal(shape[1]).astype(np.float32)
        for mode in MODES:
            mw, vw = ref_pack(A, mode), ref_pack(v, mode)
            g[f"{name}_{mode}_m"] = mw
            g[f"{name}_{mode}_v"] = vw
            g[f"{name}_{mode}_out"] = run_gemv(mw, vw, shape, mode)
        g[f"{name}_shape"] = np.array(shape, dtype=np.int64)
        g[f"{name}_seed"] = np.array(seed, dtype=np.int64)
    # raw random words: every code (inf/NaN included) meets every code
    rng = np.random.default_rng(26)
    mw = rng.integers(0, 2 ** 32, size=8 * 512, dtype=np.uint64).astype(np.uint32)
    vw = rng.integers(0, 2 ** 32, size=512, dtype=np.uint64).astype(np.uint32)
    for mode in MODES:
        g[f"rawbits_{mode}_out"] = run_gemv(mw, vw, (8, 2048), mode)
    g["rawbits_m"], g["rawbits_v"] = mw, vw
    np.savez_compressed(os.path.join(HERE, "gemv.npz"), **g)

    make_dot()
    for f in ("encode", "decode", "gemv", "dot"):
        print(f, os.path.getsize(os.path.join(HERE, f + ".npz")), "bytes")


if __name__ == "__main__":
    sys.exit(main())
