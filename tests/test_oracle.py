"""Pin the CPU oracles (numpy and C) to vectors produced by the reference.

The ``.npz`` files under tests/golden were written by running the reference's
own packer, CPU unpacker and (through Triton's interpreter) GEMV / dot
kernels; see tests/golden/make_golden.py.
"""
import numpy as np
import pytest

from oracle import feather_oracle as O
from tests.golden_inputs import DOT_CASES, GEMV_CASES, dot_case, gemv_case, sample_f32

MODES = ("E5M2", "E4M3")
IMPLS = ("numpy", "c")


def _pack(impl, c_oracle, x, mode):
    return O.pack_fp8_ndarray(x, mode) if impl == "numpy" else c_oracle.pack(x, mode)


def _same_floats(a, b):
    a, b = np.asarray(a, np.float32), np.asarray(b, np.float32)
    nan = np.isnan(a)
    return np.array_equal(nan, np.isnan(b)) and np.array_equal(
        a.view(np.uint32)[~nan], b.view(np.uint32)[~nan])


@pytest.mark.parametrize("impl", IMPLS)
@pytest.mark.parametrize("mode", MODES)
def test_encode_every_fp16_pattern(golden, c_oracle, impl, mode):
    h = np.arange(65536, dtype=np.uint16).view(np.float16)
    got = _pack(impl, c_oracle, h, mode).view(np.uint8)
    assert np.array_equal(got, golden("encode")[f"fp16_all_{mode}"])


@pytest.mark.parametrize("mode", MODES)
def test_e5m2_closed_form_agrees(golden, mode):
    if mode != "E5M2":
        pytest.skip("closed form exists for E5M2 only")
    got = O.encode_e5m2_from_fp16_bits(np.arange(65536, dtype=np.uint16))
    assert np.array_equal(got, golden("encode")["fp16_all_E5M2"])


@pytest.mark.parametrize("impl", IMPLS)
@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("kind,seed", [("bits", 11), ("lognormal", 12)])
def test_encode_fp32_samples(golden, c_oracle, impl, mode, kind, seed):
    x = sample_f32(kind, 131072, seed)
    got = _pack(impl, c_oracle, x, mode).view(np.uint8)
    assert np.array_equal(got, golden("encode")[f"fp32_{kind}_{mode}"])


@pytest.mark.parametrize("impl", IMPLS)
@pytest.mark.parametrize("mode", MODES)
def test_encode_fp32_edges(golden, c_oracle, impl, mode):
    g = golden("encode")
    x = g["fp32_edge_input_bits"].view(np.float32)
    got = _pack(impl, c_oracle, x, mode).view(np.uint8)[: x.size]
    assert np.array_equal(got, g[f"fp32_edge_{mode}"])


@pytest.mark.parametrize("impl", IMPLS)
@pytest.mark.parametrize("mode", MODES)
def test_pack_layout_ragged_and_2d(golden, c_oracle, impl, mode):
    g = golden("encode")
    t = sample_f32("lognormal", 31, 13).astype(np.float16)
    assert np.array_equal(_pack(impl, c_oracle, t, mode), g[f"ragged31_{mode}"])
    assert np.array_equal(_pack(impl, c_oracle, t[:28].reshape(7, 4), mode), g[f"matrix7x4_{mode}"])


@pytest.mark.parametrize("impl", IMPLS)
@pytest.mark.parametrize("mode", MODES)
def test_decode_tables(golden, c_oracle, impl, mode):
    g = golden("decode")
    tab = (O if impl == "numpy" else c_oracle).decode_table
    # The vector lane holds the code of 1.0 and the other lanes are zero, so the
    # reference kernel returned decode(code) * 1 + 0 + 0 + 0 (which maps -0 to +0).
    with np.errstate(invalid="ignore"):
        expect = tab(mode, "kernel") * np.float32(1.0) + np.float32(0.0)
    for lane in range(4):
        assert _same_floats(expect, g[f"kernel_{mode}_lane{lane}"])
    assert _same_floats(tab(mode, "ieee"), g[f"ieee_{mode}"])


def test_e4m3_kernel_decode_differs_from_ieee_on_16_codes():
    k, i = O.decode_table("E4M3", "kernel"), O.decode_table("E4M3", "ieee")
    differ = [c for c in range(256) if not _same_floats(k[c:c + 1], i[c:c + 1])]
    assert differ == list(range(1, 8)) + [0x7F] + list(range(0x81, 0x88)) + [0xFF]
    assert k[0x7F] == 480.0 and k[0xFF] == -480.0 and k[0x01] == 2.0 ** -17


@pytest.mark.parametrize("impl", IMPLS)
@pytest.mark.parametrize("mode", MODES)
def test_gemv_docstring_example(golden, c_oracle, impl, mode):
    a = np.array([[1, 1, -2, 0], [-3, -3, -2, -3], [0, 1, 1, -2], [2, 0, -1, 2]], dtype=np.float16)
    b = np.array([2, 2, -1, 2], dtype=np.float16)
    gemv = O.gemv if impl == "numpy" else c_oracle.gemv
    y = gemv(_pack(impl, c_oracle, a, mode), _pack(impl, c_oracle, b, mode), (4, 4), mode)
    assert np.array_equal(y, np.array([6, -16, -3, 9], dtype=np.float32))
    assert np.array_equal(y, golden("gemv")[f"doc_{mode}"])


@pytest.mark.parametrize("impl", IMPLS)
@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("case", sorted(GEMV_CASES))
def test_gemv_matches_reference_kernel(golden, c_oracle, impl, mode, case):
    g = golden("gemv")
    A, v = gemv_case(case)
    mw, vw = _pack(impl, c_oracle, A, mode), _pack(impl, c_oracle, v, mode)
    assert np.array_equal(mw, g[f"{case}_{mode}_m"])  # packed bytes bit-exact
    assert np.array_equal(vw, g[f"{case}_{mode}_v"])
    gemv = O.gemv if impl == "numpy" else c_oracle.gemv
    y = gemv(mw, vw, A.shape, mode)
    ref = g[f"{case}_{mode}_out"]
    if case.startswith("int"):
        assert np.array_equal(y, ref)  # integer data: every order is exact
        assert np.array_equal(y, A.astype(np.float32) @ v.astype(np.float32))
    else:
        # tolerance from the north star: max relative (scale-normalised) 1e-5
        assert O.normalised_error(y, ref) < 1e-5
        assert O.normalised_error(gemv(mw, vw, A.shape, mode, acc="f64"), ref) < 1e-5


@pytest.mark.parametrize("impl", IMPLS)
@pytest.mark.parametrize("mode", MODES)
def test_gemv_raw_bits_nonfinite_pattern(golden, c_oracle, impl, mode):
    """Random words: inf/NaN codes meet every code.  Non-finite outputs must
    agree in class; finite ones within tolerance."""
    g = golden("gemv")
    gemv = O.gemv if impl == "numpy" else c_oracle.gemv
    y = gemv(g["rawbits_m"], g["rawbits_v"], (8, 2048), mode)
    ref = g[f"rawbits_{mode}_out"]
    assert np.array_equal(np.isnan(y), np.isnan(ref))
    assert np.array_equal(np.isinf(y), np.isinf(ref))
    fin = np.isfinite(ref)
    if fin.any():
        assert O.normalised_error(y[fin], ref[fin]) < 1e-5


@pytest.mark.parametrize("impl", IMPLS)
def test_dot_matches_reference_kernel(golden, c_oracle, impl):
    g = golden("dot")
    dot = O.dot if impl == "numpy" else c_oracle.dot
    a = _pack(impl, c_oracle, np.array([2, 0, -3, 1], dtype=np.float16), "E5M2")
    b = _pack(impl, c_oracle, np.array([-1, 0, -3, 1], dtype=np.float16), "E5M2")
    assert dot(a, b) == 8.0 == g["doc"]
    for n, seed in DOT_CASES:
        x1, x2 = dot_case(n, seed)
        a, b = _pack(impl, c_oracle, x1, "E5M2"), _pack(impl, c_oracle, x2, "E5M2")
        sums = np.array([a.astype(np.uint64).sum(), b.astype(np.uint64).sum()], dtype=np.uint64)
        assert np.array_equal(sums, g[f"n{n}_wordsum"])
        if f"n{n}_a" in g:
            assert np.array_equal(a, g[f"n{n}_a"]) and np.array_equal(b, g[f"n{n}_b"])
        ref = float(g[f"n{n}_out"])
        # scale for a dot product: sum of |products|
        scale = float(np.abs(O.unpack(a) * O.unpack(b)).sum())
        assert abs(float(dot(a, b)) - ref) / scale < 1e-5
        assert abs(float(dot(a, b, acc="f64")) - ref) / scale < 1e-5


@pytest.mark.parametrize("mode", MODES)
def test_numpy_and_c_oracles_agree_bitwise(c_oracle, mode):
    rng = np.random.default_rng(5)
    A = rng.standard_normal((19, 4104)).astype(np.float16)
    v = rng.standard_normal(4104).astype(np.float16)
    mw, vw = O.pack_fp8_ndarray(A, mode), O.pack_fp8_ndarray(v, mode)
    assert np.array_equal(O.gemv(mw, vw, A.shape, mode), c_oracle.gemv(mw, vw, A.shape, mode))
    assert O.dot(mw[:5000], mw[5000:10000], mode) == c_oracle.dot(mw[:5000], mw[5000:10000], mode)
    assert np.array_equal(O.unpack(mw, mode), c_oracle.unpack(mw, mode))


def test_unknown_mode_raises():
    with pytest.raises(NotImplementedError):
        O.pack_fp8_ndarray(np.zeros(4, np.float16), "E3M4")


# ------------------------------------------------------------ ReLU on unpack --
def test_relu_matches_reference_kernel(golden):
    """The restated ReLU (activations.py:8-29) against the reference kernel run
    through Triton's interpreter.  All codes: equal where the value is not NaN;
    on the six NaN codes the interpreter (numpy maximum) keeps NaN while the
    compiled kernel's maximum -- which the restatement follows -- returns 0."""
    g = golden("relu")
    want = g["all_codes_out"]
    got = O.relu(np.arange(256, dtype=np.uint8).view(np.uint32))
    nan = np.isnan(want)
    assert sorted(np.flatnonzero(nan)) == [0x7D, 0x7E, 0x7F, 0xFD, 0xFE, 0xFF]
    assert np.array_equal(got[~nan], want[~nan]) and np.all(got[nan] == 0)
    assert not np.signbit(got).any()            # -0 and negative codes give +0
    assert got[0x7C] == np.inf and got[0xFC] == 0
    rng = np.random.default_rng(int(g["n36004_seed"]))
    x = rng.standard_normal(4 * 9000 + 4).astype(np.float16)
    assert np.array_equal(O.relu(O.pack_fp8_ndarray(x, "E5M2").view(np.uint32)), g["n36004_out"])
    # ragged length and the E4M3 extension (kernel decode: 0x7F is 480, 0x01 is 2^-17)
    assert O.relu(np.array([0x3C3CBC3C], dtype=np.uint32), 3).tolist() == [1.0, 0.0, 1.0]
    e4 = O.relu(np.array([0x8101FF7F], dtype=np.uint32), mode="E4M3")
    assert e4.tolist() == [480.0, 0.0, 2.0 ** -17, 0.0]


# ------------------------------------------------------------------ attention --
@pytest.mark.parametrize("seq,d", [(128, 64), (100, 32), (200, 128), (64, 16), (130, 256), (64, 512)])
def test_attention_matches_reference_kernel(golden, seq, d):
    """The restated attention (attention.py:14-108) against the reference kernel run
    through Triton's interpreter, including sequence lengths that leave the last key
    tile partly empty (the reference does not mask those keys)."""
    g = golden("attention")
    rng = np.random.default_rng(int(g[f"s{seq}_d{d}_seed"]))
    q, k, v = (O.pack_fp8_ndarray(rng.standard_normal((seq, d)).astype(np.float16), "E5M2").view(np.uint32)
               for _ in range(3))
    got = O.flash_attention(q, k, v, seq, d // 4)
    assert got.shape == (seq, d) and O.normalised_error(got, g[f"s{seq}_d{d}_out"]) < 1e-6
    if seq % 64 == 0:  # full tiles: the textbook softmax(Q K^T / sqrt(d)) V up to the FP16 probabilities
        dec = lambda w: O.unpack(w, "E5M2")[: seq * d].reshape(seq, d).astype(np.float64)
        s = dec(q) @ dec(k).T / np.sqrt(d)
        p = np.exp(s - s.max(axis=1, keepdims=True))
        assert O.normalised_error(got, (p / p.sum(axis=1, keepdims=True)) @ dec(v)) < 1e-3


def test_reference_cpu_path_worker_agrees_with_the_oracle(c_oracle):
    """The reference's CPU leg that the benchmark times (its packer + a torch
    decode with the GPU kernels' bit semantics + torch.mv, run by
    baseline/reference_worker.py) computes what the oracle computes."""
    import json
    import os
    import subprocess
    import sys
    import torch
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    if not os.path.isdir(os.path.join(root, "baseline", "_ref", "feather", "routines")):
        pytest.skip("baseline/_ref is not installed (baseline/install_reference.sh)")
    res = subprocess.run([sys.executable, os.path.join(root, "baseline", "reference_worker.py"), "cpu",
                          "--M", "256", "--N", "512"], capture_output=True, text=True, timeout=600)
    line = [l for l in res.stdout.splitlines() if l.startswith("REFERENCE_WORKER ")][0]
    got = json.loads(line[len("REFERENCE_WORKER "):])
    assert "unavailable" not in got, got
    torch.manual_seed(0)
    A = torch.randn(256, 512).half().numpy()
    v = torch.randn(512).half().numpy()
    for mode in ("E5M2", "E4M3"):
        y = c_oracle.gemv(c_oracle.pack(A, mode), c_oracle.pack(v, mode), (256, 512), mode, acc="f64")
        assert abs(got[mode]["checksum"] - float(np.abs(y).sum())) < 1e-4 * float(np.abs(y).sum())
