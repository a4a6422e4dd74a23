"""GPU parity tests: the CUDA path, called through the C ABI (ctypes), against
the oracle and the golden vectors produced by the reference.

Bars: packed bytes and decoded values bit-exact; GEMV / dot within max relative
error 1e-5, where "relative" is normalised by the largest reference output
(GEMV) or by the sum of |products| (dot) -- FP32 accumulation is
order-dependent and the reference's own order is unspecified.
"""
import ctypes

import numpy as np
import pytest
import torch

from oracle import feather_oracle as O
from tests.golden_inputs import DOT_CASES, GEMV_CASES, c3_matrix, dot_case, gemv_case, sample_f32

pytestmark = pytest.mark.gpu
MODES = ("E5M2", "E4M3")
TOL = 1e-5  # max relative error stated by the north star


@pytest.fixture(scope="module")
def fb():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import feather_b200
    feather_b200._lib.load()
    return feather_b200


def dev(a: np.ndarray) -> torch.Tensor:
    if a.dtype == np.uint32:
        return torch.from_numpy(a.view(np.int32)).cuda().view(torch.uint32)
    return torch.from_numpy(a).cuda()


def host_words(t: torch.Tensor) -> np.ndarray:
    return t.view(torch.int32).cpu().numpy().view(np.uint32)


def same_floats(a, b) -> bool:
    a, b = np.asarray(a, np.float32), np.asarray(b, np.float32)
    nan = np.isnan(a)
    return bool(np.array_equal(nan, np.isnan(b)) and
                np.array_equal(a.view(np.uint32)[~nan], b.view(np.uint32)[~nan]))


# ------------------------------------------------------------------ encode --
@pytest.mark.parametrize("mode", MODES)
def test_encode_every_fp16_pattern(fb, golden, mode):
    h = torch.arange(65536, dtype=torch.int32).to(torch.int16).view(torch.float16).cuda()
    got = host_words(fb.pack_fp8_tensor(h, mode)).view(np.uint8)
    assert np.array_equal(got, golden("encode")[f"fp16_all_{mode}"])


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("kind,seed", [("bits", 11), ("lognormal", 12)])
def test_encode_fp32_samples(fb, golden, mode, kind, seed):
    x = dev(sample_f32(kind, 131072, seed))
    got = host_words(fb.pack_fp8_tensor(x, mode)).view(np.uint8)
    assert np.array_equal(got, golden("encode")[f"fp32_{kind}_{mode}"])


@pytest.mark.parametrize("mode", MODES)
def test_encode_fp32_edges(fb, golden, mode):
    g = golden("encode")
    x = dev(g["fp32_edge_input_bits"].view(np.float32).copy())
    got = host_words(fb.pack_fp8_tensor(x, mode)).view(np.uint8)[: x.numel()]
    assert np.array_equal(got, g[f"fp32_edge_{mode}"])


@pytest.mark.parametrize("mode", MODES)
def test_encode_layout_ragged_2d_and_cpu_input(fb, golden, mode):
    g = golden("encode")
    t = torch.from_numpy(sample_f32("lognormal", 31, 13).astype(np.float16))
    w = fb.pack_fp8_tensor(t.cuda(), mode)
    assert w.dtype == torch.uint32 and w.ndim == 1 and w.is_cuda
    assert np.array_equal(host_words(w), g[f"ragged31_{mode}"])
    assert np.array_equal(host_words(fb.pack_fp8_tensor(t[:28].reshape(7, 4).cuda(), mode)),
                          g[f"matrix7x4_{mode}"])
    w_cpu = fb.pack_fp8_tensor(t, mode)  # CPU in -> CPU out, as the reference returns
    assert not w_cpu.is_cuda and np.array_equal(w_cpu.view(torch.int32).numpy().view(np.uint32),
                                                g[f"ragged31_{mode}"])


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("dtype", [np.float16, np.float32])
def test_encode_large_random_and_ragged_lengths_vs_oracle(fb, c_oracle, mode, dtype):
    rng = np.random.default_rng(7)
    bits = rng.integers(0, 2 ** 32, size=(1 << 22) + 77, dtype=np.uint64).astype(np.uint32)
    x = bits.view(np.float32) if dtype == np.float32 else bits.view(np.float16)
    xd = dev(x.copy())
    assert np.array_equal(host_words(fb.pack_fp8_tensor(xd, mode)), c_oracle.pack(x, mode))
    for n in (0, 1, 2, 3, 4, 5, 15, 16, 17, 63, 4099):
        assert np.array_equal(host_words(fb.pack_fp8_tensor(xd[:n], mode)), c_oracle.pack(x[:n], mode))
    # source not 16-byte aligned: takes the word-granular kernel
    assert np.array_equal(host_words(fb.pack_fp8_tensor(xd[1:5001], mode)), c_oracle.pack(x[1:5001], mode))


def test_encode_rejects(fb):
    with pytest.raises(NotImplementedError):
        fb.pack_fp8_tensor(torch.zeros(4, dtype=torch.float16, device="cuda"), "E3M4")
    with pytest.raises(TypeError):
        fb.pack_fp8_tensor(torch.zeros(4, dtype=torch.bfloat16, device="cuda"))


# ------------------------------------------------------------------ decode --
@pytest.mark.parametrize("mode", MODES)
def test_decode_all_codes_all_lanes(fb, golden, mode):
    g = golden("decode")
    words = np.arange(256, dtype=np.uint8).view(np.uint32)  # every code, every byte lane
    for sem in ("kernel", "ieee"):
        got = fb.unpack_fp8_tensor(dev(words.copy()), mode, sem).cpu().numpy()
        assert same_floats(got, O.decode_table(mode, sem))  # signed zeros included
    assert same_floats(fb.unpack_fp8_tensor(dev(words.copy()), mode, "ieee").cpu().numpy(),
                       g[f"ieee_{mode}"])
    got = fb.unpack_fp8_tensor(dev(words.copy()), mode, "kernel").cpu().numpy()
    with np.errstate(invalid="ignore"):
        assert same_floats(got * np.float32(1) + np.float32(0), g[f"kernel_{mode}_lane0"])
    # ragged element count and a large random buffer
    rng = np.random.default_rng(8)
    w = rng.integers(0, 2 ** 32, size=100003, dtype=np.uint64).astype(np.uint32)
    for n in (1, 2, 3, 5, 400009):
        got = fb.unpack_fp8_tensor(dev(w), mode, "kernel", n_elems=n).cpu().numpy()
        assert same_floats(got, O.unpack(w, mode, "kernel", n))


@pytest.mark.parametrize("mode", MODES)
def test_gemv_uses_kernel_decode_for_every_code_and_lane(fb, golden, mode):
    """The GEMV kernels themselves (fast and general path) multiply with the
    reference kernel's decode: one code per row times 1.0, every byte lane."""
    g = golden("decode")
    one = {"E5M2": 0x3C, "E4M3": 0x38}[mode]
    for lane in range(4):
        ref = g[f"kernel_{mode}_lane{lane}"]
        # general path: one word per row
        mw = (np.arange(256, dtype=np.uint32) << (8 * lane))
        vw = np.array([one << (8 * lane)], dtype=np.uint32)
        got = fb.gemv_fp8_acc_fp32_gpu(dev(mw), dev(vw), (256, 4), mode).cpu().numpy()
        assert same_floats(got, ref)
        # streaming path: 256 rows x 1024 columns, the code at column 16*r + 4*j + lane
        M, N = 256, 1024
        m = np.zeros((M, N), dtype=np.uint8)
        v = np.zeros(N, dtype=np.uint8)
        cols = (np.arange(M) * 4 + lane) % N
        m[np.arange(M), cols] = np.arange(256)
        v[:] = one  # other columns hold code 0 -> +0 * 1.0
        got = fb.gemv_fp8_acc_fp32_gpu(dev(m.reshape(-1).view(np.uint32)), dev(v.view(np.uint32)),
                                       (M, N), mode).cpu().numpy()
        assert same_floats(got, ref)


# -------------------------------------------------------------------- gemv --
@pytest.mark.parametrize("mode", MODES)
def test_gemv_docstring_example(fb, golden, mode):
    a = torch.tensor([[1, 1, -2, 0], [-3, -3, -2, -3], [0, 1, 1, -2], [2, 0, -1, 2]],
                     dtype=torch.float16, device="cuda")
    b = torch.tensor([2, 2, -1, 2], dtype=torch.float16, device="cuda")
    fn = fb.gemv_fp8_e5m2_acc_fp32_gpu if mode == "E5M2" else fb.gemv_fp8_e4m3_acc_fp32_gpu
    y = fn(fb.pack_fp8_tensor(a, mode), fb.pack_fp8_tensor(b, mode), a.shape)
    assert y.dtype == torch.float32 and y.shape == (4,) and y.is_cuda
    assert y.cpu().tolist() == [6.0, -16.0, -3.0, 9.0] == golden("gemv")[f"doc_{mode}"].tolist()


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("case", sorted(GEMV_CASES))
def test_gemv_matches_reference_kernel_outputs(fb, golden, mode, case):
    g = golden("gemv")
    A, v = gemv_case(case)
    mw, vw = fb.pack_fp8_tensor(dev(A), mode), fb.pack_fp8_tensor(dev(v), mode)
    assert np.array_equal(host_words(mw), g[f"{case}_{mode}_m"])  # packed bytes bit-exact
    assert np.array_equal(host_words(vw), g[f"{case}_{mode}_v"])
    y = fb.gemv_fp8_acc_fp32_gpu(mw, vw, A.shape, mode).cpu().numpy()
    ref = g[f"{case}_{mode}_out"]
    if case.startswith("int"):
        assert np.array_equal(y, ref)
    else:
        assert O.normalised_error(y, ref) < TOL


@pytest.mark.parametrize("mode", MODES)
def test_gemv_raw_bits_nonfinite_classes(fb, golden, mode):
    g = golden("gemv")
    y = fb.gemv_fp8_acc_fp32_gpu(dev(g["rawbits_m"]), dev(g["rawbits_v"]), (8, 2048), mode).cpu().numpy()
    ref = g[f"rawbits_{mode}_out"]
    assert np.array_equal(np.isnan(y), np.isnan(ref)) and np.array_equal(np.isinf(y), np.isinf(ref))
    fin = np.isfinite(ref)
    if fin.any():
        assert O.normalised_error(y[fin], ref[fin]) < TOL


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("shape", [(1, 4), (3, 8), (17, 20), (5, 4100), (1, 16384), (2, 16),
                                   (300, 2048), (1031, 4096), (40, 16400), (9, 32784), (64, 65536),
                                   (7, 2080), (295, 1056), (297, 528), (3000, 5632), (600, 32768),
                                   (4097, 1040), (20000, 48), (513, 8208)])
def test_gemv_edge_shapes_vs_oracle(fb, c_oracle, mode, shape):
    rng = np.random.default_rng(shape[0] * 131 + shape[1])
    A = rng.standard_normal(shape).astype(np.float16)
    v = rng.standard_normal(shape[1]).astype(np.float16)
    mw, vw = c_oracle.pack(A, mode), c_oracle.pack(v, mode)
    y = fb.gemv_fp8_acc_fp32_gpu(dev(mw), dev(vw), shape, mode).cpu().numpy()
    ref = c_oracle.gemv(mw, vw, shape, mode, acc="f64")
    assert O.normalised_error(y, ref) < TOL
    # matrix base not 16-byte aligned (a view one word into a larger buffer)
    buf = dev(np.concatenate([np.zeros(1, np.uint32), mw]))
    y2 = fb.gemv_fp8_acc_fp32_gpu(buf[1:], dev(vw), shape, mode).cpu().numpy()
    assert O.normalised_error(y2, ref) < TOL


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("shape", [(4737, 4096), (5000, 16400), (4800, 32784), (4736, 65536),
                                   (6001, 4112), (9999, 8192)])
def test_gemv_ring_path_ragged_shapes_vs_oracle(fb, c_oracle, mode, shape):
    """Shapes that take the bulk-copy ring kernel: row counts that leave partial
    row blocks, rows that end inside a 4 KiB segment, several column tiles."""
    M, N = shape
    gen = torch.Generator(device="cuda").manual_seed(M + N)
    A = torch.randn(M, N, device="cuda", generator=gen, dtype=torch.float16)
    v = torch.randn(N, device="cuda", generator=gen, dtype=torch.float16)
    mw, vw = fb.pack_fp8_tensor(A, mode), fb.pack_fp8_tensor(v, mode)
    y = fb.gemv_fp8_acc_fp32_gpu(mw, vw, shape, mode).cpu().numpy()
    ref = c_oracle.gemv(host_words(mw), host_words(vw), shape, mode, acc="f64")
    assert O.normalised_error(y, ref) < TOL
    fb.device_status()  # no bounded wait gave up


@pytest.mark.parametrize("mode", MODES)
def test_gemv_static_matrix_option_same_bits(fb, mode):
    """FEATHER_GEMV_STATIC_MATRIX only changes when the matrix bytes start to
    stream; repeated back-to-back calls give the bits of the default path."""
    M, N = 6000, 8192
    gen = torch.Generator(device="cuda").manual_seed(21)
    mats = [fb.pack_fp8_tensor(torch.randn(M, N, device="cuda", generator=gen, dtype=torch.float16), mode)
            for _ in range(2)]
    vs = [fb.pack_fp8_tensor(torch.randn(N, device="cuda", generator=gen, dtype=torch.float16), mode)
          for _ in range(3)]
    torch.cuda.synchronize()  # the promise: nothing in flight writes the matrices
    ref = [fb.gemv_fp8_acc_fp32_gpu(mats[i % 2], vs[i % 3], (M, N), mode) for i in range(6)]
    torch.cuda.synchronize()
    outs = [torch.empty(M, dtype=torch.float32, device="cuda") for _ in range(6)]
    for i in range(6):  # back to back: each kernel starts streaming under its predecessor's tail
        fb.gemv(mats[i % 2], vs[i % 3], original_shape=(M, N), mode=mode, out=outs[i], static_matrix=True)
    torch.cuda.synchronize()
    for i in range(6):
        assert torch.equal(outs[i], ref[i])
    lib = fb._lib.load()
    assert lib.feather_gemv_fp8_ex(mats[0].data_ptr(), vs[0].data_ptr(), outs[0].data_ptr(), M, N, 0, 8, None) == -1


def test_gemv_empty_and_rejects(fb):
    z = torch.zeros(8, dtype=torch.int32, device="cuda")
    assert fb.gemv_fp8_acc_fp32_gpu(z, z, (0, 8)).shape == (0,)
    assert fb.gemv_fp8_acc_fp32_gpu(z, z, (5, 0)).tolist() == [0.0] * 5
    with pytest.raises(ValueError):
        fb.gemv_fp8_acc_fp32_gpu(z, z, (2, 6))          # N % 4 != 0
    with pytest.raises(ValueError):
        fb.gemv_fp8_acc_fp32_gpu(z, z[:1], (2, 16))     # vector too short
    with pytest.raises(ValueError):
        fb.gemv_fp8_acc_fp32_gpu(z.cpu(), z, (2, 16))   # no CPU path
    with pytest.raises(NotImplementedError):
        fb.gemv_fp8_acc_fp32_gpu(z, z, (2, 16), "E3M4")
    with pytest.raises(TypeError):
        fb.gemv(z, z)                                   # original_shape is required


def test_readme_surface_and_mode_tag(fb):
    import feather
    torch.manual_seed(3)
    a = torch.randn(64, 256, dtype=torch.float16, device="cuda")
    b = torch.randn(256, dtype=torch.float16, device="cuda")
    for mode in MODES:
        mp = feather.pack_fp8_tensor(a, mode=mode).cuda()
        vp = feather.pack_fp8_tensor(b, mode=mode).cuda()
        assert mp.feather_mode == mode and mp.view(torch.uint32).feather_mode == mode
        y = feather.gemv(mp, vp, original_shape=a.shape)  # mode comes from the packed operand
        y2 = fb.gemv_fp8_acc_fp32_gpu(mp, vp, a.shape, mode)
        assert torch.equal(y, y2)
        d = feather.dot(vp, vp)
        assert torch.equal(d, fb.dot_fp8_acc_fp32_gpu(vp, vp, mode))
    from feather.packers.fp8 import pack_fp8_tensor
    from feather.routines.dot import dot_fp8_e5m2_acc_fp32_gpu
    from feather.routines.gemv import gemv_fp8_e4m3_acc_fp32_gpu, gemv_fp8_e5m2_acc_fp32_gpu
    mp = pack_fp8_tensor(a, mode="E5M2").view(torch.uint32).to("cuda")  # as bench_gemv.py does
    vp = pack_fp8_tensor(b, mode="E5M2").view(torch.uint32).to("cuda")
    assert gemv_fp8_e5m2_acc_fp32_gpu(mp, vp, a.shape).shape == (64,)
    assert gemv_fp8_e4m3_acc_fp32_gpu(mp.view(torch.int32), vp.view(torch.float32), a.shape).shape == (64,)
    assert dot_fp8_e5m2_acc_fp32_gpu(vp, vp).ndim == 0


@pytest.mark.parametrize("mode", MODES)
def test_gemv_bench_gemv_integer_inputs_exact(fb, mode):
    """feather/benchmark/bench_gemv.py:14-15, 48-93: integer-valued inputs in
    [-3, 2] are exact in both formats, so the result equals torch.mv exactly;
    every (M, N) combination of the reference's grid."""
    torch.manual_seed(4)
    for M, N in ((m, n) for m in (4096, 8192, 16384) for n in (4096, 8192, 16384)):
        a = torch.randint(-3, 3, (M, N), device="cuda").to(torch.float16)
        b = torch.randint(-3, 3, (N,), device="cuda").to(torch.float16)
        y = fb.gemv_fp8_acc_fp32_gpu(fb.pack_fp8_tensor(a, mode), fb.pack_fp8_tensor(b, mode),
                                     a.shape, mode)
        assert torch.equal(y, torch.mv(a.float(), b.float()))


@pytest.mark.parametrize("mode", MODES)
def test_gemv_config1_4096(fb, c_oracle, mode):
    """seed 0, 4096 x 4096 fp16 N(0,1): packed bytes, decode round trip, GEMV."""
    torch.manual_seed(0)
    A = torch.randn(4096, 4096).half()
    v = torch.randn(4096).half()
    mw, vw = fb.pack_fp8_tensor(A.cuda(), mode), fb.pack_fp8_tensor(v.cuda(), mode)
    mw_ref = c_oracle.pack(A.numpy(), mode)
    assert np.array_equal(host_words(mw), mw_ref)
    assert same_floats(fb.unpack_fp8_tensor(mw, mode).cpu().numpy(), c_oracle.unpack(mw_ref, mode))
    y = fb.gemv_fp8_acc_fp32_gpu(mw, vw, A.shape, mode).cpu().numpy()
    assert O.normalised_error(y, c_oracle.gemv(mw_ref, host_words(vw), A.shape, mode, acc="f64")) < TOL
    assert O.normalised_error(y, c_oracle.gemv(mw_ref, host_words(vw), A.shape, mode)) < TOL


def test_gemv_config2_e5m2_16384_full_size(fb, c_oracle):
    torch.manual_seed(1)
    M = N = 16384
    A = torch.randn(M, N, dtype=torch.float16, device="cuda")
    v = torch.randn(N, dtype=torch.float16, device="cuda")
    mw, vw = fb.pack_fp8_tensor(A, "E5M2"), fb.pack_fp8_tensor(v, "E5M2")
    mh, vh = host_words(mw), host_words(vw)
    assert np.array_equal(mh[: 1 << 20], c_oracle.pack(A[:256].cpu().numpy(), "E5M2"))
    y = fb.gemv_fp8_acc_fp32_gpu(mw, vw, (M, N), "E5M2").cpu().numpy()
    assert O.normalised_error(y, c_oracle.gemv(mh, vh, (M, N), "E5M2", acc="f64")) < TOL
    # linearity in the vector: scaling v by 2 (exact in FP8) doubles the result exactly
    y2 = fb.gemv_fp8_acc_fp32_gpu(mw, fb.pack_fp8_tensor(v * 2, "E5M2"), (M, N), "E5M2").cpu().numpy()
    assert np.array_equal(y2, 2 * y)


@pytest.mark.parametrize("shape,seed", [((8192, 8192), 2), ((16384, 8192), 3), ((16384, 16384), 4)])
def test_gemv_config3_e4m3_shape_sweep(fb, c_oracle, shape, seed):
    """fp32 matrices: 90 % 4*N(0,1), 5 % E4M3-subnormal magnitudes, 5 % beyond
    saturation; E4M3 packed.  Generated on the device (same recipe as
    c3_matrix) because the full-size host generator is slow."""
    M, N = shape
    gen = torch.Generator(device="cuda").manual_seed(seed)
    x = 4.0 * torch.randn(M, N, device="cuda", generator=gen)
    u = torch.rand(M, N, device="cuda", generator=gen)
    sign = torch.where(torch.rand(M, N, device="cuda", generator=gen) < 0.5, -1.0, 1.0)
    r = torch.rand(M, N, device="cuda", generator=gen)
    small = sign * (2.0 ** -9 + r * (2.0 ** -6 - 2.0 ** -9))
    big = sign * (448.0 + r * (1000.0 - 448.0))
    x = torch.where(u < 0.05, small, torch.where(u < 0.10, big, x))
    del u, sign, r, small, big
    v = torch.randn(N, device="cuda", generator=gen)
    mw, vw = fb.pack_fp8_tensor(x, "E4M3"), fb.pack_fp8_tensor(v, "E4M3")
    mh, vh = host_words(mw), host_words(vw)
    assert np.array_equal(mh[: 1 << 18], c_oracle.pack(x.reshape(-1)[: 1 << 20].cpu().numpy(), "E4M3"))
    codes = mh[: 1 << 20].view(np.uint8)
    assert ((codes & 0x7F) == 0x7F).mean() > 0.02 and ((codes & 0x78) == 0).mean() > 0.03
    y = fb.gemv_fp8_acc_fp32_gpu(mw, vw, shape, "E4M3").cpu().numpy()
    assert O.normalised_error(y, c_oracle.gemv(mh, vh, shape, "E4M3", acc="f64")) < TOL


def test_gemv_65536_sampled_rows(fb, c_oracle):
    """4 GiB packed matrix (the row-sharded configuration on one GPU): rows are
    generated and packed block by block on the device; 2048 sampled rows are
    checked against the oracle."""
    M = N = 65536
    gen = torch.Generator(device="cuda").manual_seed(5)
    v = torch.randn(N, device="cuda", generator=gen).half()
    vw = fb.pack_fp8_tensor(v, "E5M2")
    mw = torch.empty(M * (N // 4), dtype=torch.int32, device="cuda").view(torch.uint32)
    blk = 4096
    for r0 in range(0, M, blk):
        a = torch.randn(blk, N, device="cuda", generator=gen, dtype=torch.float16)
        mw[r0 * (N // 4):(r0 + blk) * (N // 4)] = fb.pack_fp8_tensor(a, "E5M2")
    del a
    y = fb.gemv_fp8_acc_fp32_gpu(mw, vw, (M, N), "E5M2")
    rows = torch.from_numpy(np.random.default_rng(5).choice(M, 2048, replace=False)).cuda()
    sub = mw.view(torch.int32).view(M, N // 4)[rows].contiguous()
    ref = c_oracle.gemv(sub.cpu().numpy().view(np.uint32), host_words(vw), (2048, N), "E5M2", acc="f64")
    assert O.normalised_error(y[rows].cpu().numpy(), ref) < TOL
    # a contiguous row block computed alone (what one rank of a sharded run does)
    # gives bit-identical values: rows never interact
    y_blk = fb.gemv_fp8_acc_fp32_gpu(mw[8192 * (N // 4): 2 * 8192 * (N // 4)], vw, (8192, N), "E5M2")
    assert torch.equal(y_blk, y[8192:16384])


@pytest.mark.parametrize("shape", [(2048, 2048), (256, 2048), (5632, 2048), (2048, 5632), (32000, 2048)])
def test_gemv_config5_tinyllama_shapes_e4m3_small_weights(fb, c_oracle, shape):
    """The GEMV shapes of a TinyLlama-1.1B layer and its lm_head with N(0, 0.02)
    weights in E4M3: more than half of the codes have exponent field 0, which
    the reference kernel decodes as m * 2^-17 (not the IEEE m * 2^-9).  Parity
    means reproducing that."""
    M, N = shape
    gen = torch.Generator(device="cuda").manual_seed(6)
    W = (0.02 * torch.randn(M, N, device="cuda", generator=gen)).half()
    x = torch.randn(N, device="cuda", generator=gen).half()
    mw, vw = fb.pack_fp8_tensor(W, "E4M3"), fb.pack_fp8_tensor(x, "E4M3")
    mh, vh = host_words(mw), host_words(vw)
    codes = mh.view(np.uint8)
    assert ((codes & 0x78) == 0).mean() > 0.5
    assert np.array_equal(mh, c_oracle.pack(W.cpu().numpy(), "E4M3"))
    y = fb.gemv_fp8_acc_fp32_gpu(mw, vw, shape, "E4M3").cpu().numpy()
    ref = c_oracle.gemv(mh, vh, shape, "E4M3", acc="f64")
    assert O.normalised_error(y, ref) < TOL
    # the IEEE reading of the same codes gives a visibly different answer
    ieee = O.decode_table("E4M3", "ieee")[codes].reshape(M, N).astype(np.float64) @ \
        np.nan_to_num(O.decode_table("E4M3", "ieee")[vh.view(np.uint8)].astype(np.float64))
    assert O.normalised_error(ieee, ref) > 1e-3


def test_gemv_chain_driver_runs(fb):
    from feather_b200 import chain
    assert chain.weight_bytes() == 1034420224  # 22 layers + lm_head, one byte per weight
    c = chain.GemvChain(layers=1)
    c.token()
    torch.cuda.synchronize()
    assert len(c.ops) == 8 and all(torch.isfinite(o).all() for _, _, _, o in c.ops)


# ------------------------------------------------- one launch for a table of GEMVs --
def _chain_operands(fb, shapes, seed):
    gen = torch.Generator(device="cuda").manual_seed(seed)
    ops = []
    for (M, N), mode in shapes:
        A = torch.randn(M, N, device="cuda", generator=gen) * (1.0 if mode == "E5M2" else 0.05)
        v = torch.randn(N, device="cuda", generator=gen)
        ops.append({"m": fb.pack_fp8_tensor(A, mode), "v": fb.pack_fp8_tensor(v, mode),
                    "shape": (M, N), "mode": mode})
    return ops


def test_gemv_chain_kernel_each_op_has_the_bits_of_the_single_call(fb):
    """Independent ops of mixed shape and format (ragged N, M below the SM
    count, M not a multiple of 4, shared vectors), FP32 and packed outputs."""
    from feather_b200.chain import PersistentGemvChain
    shapes = [((37, 2064), "E4M3"), ((2048, 2048), "E4M3"), ((256, 2048), "E5M2"), ((100, 5632), "E4M3"),
              ((5632, 2048), "E5M2"), ((3, 16), "E4M3"), ((2046, 8192), "E5M2"), ((1, 4096), "E4M3"),
              ((4737, 1040), "E4M3")]
    ops = _chain_operands(fb, shapes, 50)
    ops[2]["v"], ops[2]["mode"] = ops[1]["v"], "E4M3"      # two consecutive ops share a vector
    ops[2]["m"] = fb.pack_fp8_tensor(torch.randn(256, 2048, device="cuda") * 0.05, "E4M3")
    for i in (1, 3, 4, 8):
        ops[i]["out_mode"] = "E4M3" if i != 4 else "E5M2"
    chain = PersistentGemvChain(ops, static_matrix=False)
    for rep in range(3):                                    # the plan is reusable
        for o in chain.outs:
            o.view(torch.int32).fill_(-1) if o.dtype != torch.float32 else o.fill_(float("nan"))
        chain.token()
        fb.device_status()
        for op, got in zip(ops, chain.outs):
            if op.get("out_mode") is None:
                want = fb.gemv_fp8_acc_fp32_gpu(op["m"], op["v"], op["shape"], op["mode"])
            else:
                want = fb.gemv_fp8_ret_packed_gpu(op["m"], op["v"], op["shape"], op["mode"],
                                                  out_mode=op["out_mode"])
            assert torch.equal(got.view(torch.int32), want.view(torch.int32)), op["shape"]


@pytest.mark.parametrize("static_matrix", [False, True])
def test_gemv_chain_kernel_dependent_ops_and_graph_replay(fb, static_matrix):
    """A real dependency chain: every op's vector is the packed output of the op
    before it.  Equal, bit for bit, to the same GEMVs issued one by one."""
    from feather_b200.chain import PersistentGemvChain
    dims = [2048, 5632, 2048, 256, 2048, 8192, 1040, 2048]
    gen = torch.Generator(device="cuda").manual_seed(51)
    x = fb.pack_fp8_tensor(torch.randn(dims[0], device="cuda", generator=gen), "E4M3")
    ops, v = [], x
    for i in range(len(dims) - 1):
        W = torch.randn(dims[i + 1], dims[i], device="cuda", generator=gen) / dims[i] ** 0.5
        out = torch.zeros((dims[i + 1] + 3) // 4, dtype=torch.int32, device="cuda").view(torch.uint32)
        ops.append({"m": fb.pack_fp8_tensor(W, "E4M3"), "v": v, "shape": (dims[i + 1], dims[i]),
                    "out": out, "out_mode": "E4M3", "wait_op": i - 1})
        v = out
    ops.append({"m": ops[-1]["m"], "v": ops[-2]["out"], "shape": ops[-1]["shape"], "wait_op": len(ops) - 2})
    chain = PersistentGemvChain(ops, "E4M3", static_matrix=static_matrix)
    want, v = [], x
    for op in ops[:-1]:
        v = fb.gemv_fp8_ret_packed_gpu(op["m"], v, op["shape"], "E4M3")
        want.append(v.clone())
    want.append(fb.gemv_fp8_acc_fp32_gpu(ops[-1]["m"], want[-2], ops[-1]["shape"], "E4M3"))

    def check():
        fb.device_status()
        for got, w in zip(chain.outs, want):
            assert torch.equal(got.view(torch.int32), w.view(torch.int32))
            got.view(torch.int32).zero_()
    for _ in range(3):
        chain.token()
        check()
    stream, graph = torch.cuda.Stream(), torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        chain.token()
        torch.cuda.synchronize()
        with torch.cuda.graph(graph, stream=stream):
            chain.token()
            chain.token()                                    # two launches back to back in one graph
    check()
    for _ in range(3):
        graph.replay()
        check()


def test_gemv_chain_kernel_config5_token_equals_the_155_launches(fb):
    from feather_b200 import chain
    c = chain.GemvChain(layers=2)
    c.token()
    p = chain.PersistentGemvChain.from_chain(c)
    want = [o.clone() for _, _, _, o in c.ops]
    for _, _, _, o in c.ops:
        o.fill_(float("nan"))
    p.token()
    fb.device_status()
    assert len(p.outs) == 15
    for got, w in zip(p.outs, want):
        assert torch.equal(got, w)
    # the model's data flow (q/k/v read the previous down output and wait for the same op, o
    # reads q's output ...) and the fully serial one: after the launch every op's output equals
    # the single-op call on the inputs the launch left behind (its writers' final outputs)
    for flow, merged in (("model", False), ("model", True), ("serial", False)):
        d = chain.PersistentGemvChain.from_chain(chain.GemvChain(layers=2, merge_projections=merged),
                                                 dependent=flow)
        for _ in range(2):
            d.token()
        fb.device_status()
        for (m, v, shape, mode, out_mode), got in zip(d.specs, d.outs):
            want = fb.gemv_fp8_ret_packed_gpu(m, v, shape, mode, out_mode=out_mode)
            assert torch.equal(got.view(torch.int32), want.view(torch.int32)), (flow, merged, shape)


def test_gemv_chain_kernel_rejects(fb):
    from feather_b200.chain import PersistentGemvChain
    ok = _chain_operands(fb, [((64, 2048), "E4M3")], 52)[0]
    with pytest.raises(ValueError):      # rows longer than the kernel's vector buffers
        PersistentGemvChain(_chain_operands(fb, [((8, 8208), "E4M3")], 53))
    with pytest.raises(ValueError):      # rows that are not whole 16-byte chunks
        PersistentGemvChain(_chain_operands(fb, [((8, 2052), "E4M3")], 54))
    with pytest.raises(ValueError):      # an op may only wait for an earlier op
        PersistentGemvChain([dict(ok, wait_op=0)])
    with pytest.raises(ValueError):
        PersistentGemvChain([])
    with pytest.raises(NotImplementedError):
        PersistentGemvChain([dict(ok, mode="E3M4")])
    lib = fb._lib.load()
    assert lib.feather_gemv_chain_plan_bytes(0) == 0
    assert lib.feather_gemv_chain_fp8(None, 1, 0, None) == -1


# --------------------------------------------------------------------- dot --
def test_dot_golden_and_docstring(fb, golden):
    g = golden("dot")
    a = fb.pack_fp8_tensor(torch.tensor([2, 0, -3, 1], dtype=torch.float16, device="cuda"))
    b = fb.pack_fp8_tensor(torch.tensor([-1, 0, -3, 1], dtype=torch.float16, device="cuda"))
    d = fb.dot_fp8_e5m2_acc_fp32_gpu(a, b)
    assert d.ndim == 0 and d.dtype == torch.float32 and d.item() == 8.0 == float(g["doc"])
    for n, seed in DOT_CASES:
        x1, x2 = dot_case(n, seed)
        aw, bw = fb.pack_fp8_tensor(dev(x1)), fb.pack_fp8_tensor(dev(x2))
        ah, bh = host_words(aw), host_words(bw)
        sums = np.array([ah.astype(np.uint64).sum(), bh.astype(np.uint64).sum()], dtype=np.uint64)
        assert np.array_equal(sums, g[f"n{n}_wordsum"])
        scale = float(np.abs(O.unpack(ah) * O.unpack(bh)).sum())
        assert abs(fb.dot_fp8_e5m2_acc_fp32_gpu(aw, bw).item() - float(g[f"n{n}_out"])) / scale < TOL


@pytest.mark.parametrize("mode", MODES)
def test_dot_sizes_alignment_determinism(fb, c_oracle, mode):
    rng = np.random.default_rng(9)
    for n_words in (0, 1, 3, 4, 5, 1023, 1024, 4097, (1 << 20) + 3):
        a = rng.integers(0, 2 ** 32, size=n_words + 1, dtype=np.uint64).astype(np.uint32)
        b = rng.integers(0, 2 ** 32, size=n_words + 1, dtype=np.uint64).astype(np.uint32)
        # keep values finite: clear the top exponent bit of every code
        a &= 0xBFBFBFBF
        b &= 0xBFBFBFBF
        ad, bd = dev(a), dev(b)
        for off in (0, 1):  # off=1: operands are not 16-byte aligned
            aw, bw = ad[off:off + n_words], bd[off:off + n_words]
            got = fb.dot_fp8_acc_fp32_gpu(aw, bw, mode).item()
            ref = float(c_oracle.dot(a[off:off + n_words], b[off:off + n_words], mode, acc="f64"))
            scale = float(np.abs(O.unpack(a[off:off + n_words], mode).astype(np.float64) *
                                 O.unpack(b[off:off + n_words], mode)).sum()) or 1.0
            assert abs(got - ref) / scale < TOL
            assert fb.dot_fp8_acc_fp32_gpu(aw, bw, mode).item() == got  # same bits every run


def test_dot_config2_two_pow_26(fb, c_oracle):
    gen = torch.Generator(device="cuda").manual_seed(1)
    n = 1 << 26
    x1 = torch.randn(n, device="cuda", generator=gen).half()
    x2 = torch.randn(n, device="cuda", generator=gen).half()
    aw, bw = fb.pack_fp8_tensor(x1), fb.pack_fp8_tensor(x2)
    ah, bh = host_words(aw), host_words(bw)
    got = fb.dot_fp8_e5m2_acc_fp32_gpu(aw, bw).item()
    ref = float(c_oracle.dot(ah, bh, "E5M2", acc="f64"))
    scale = float((x1.float().abs() * x2.float().abs()).sum().item())
    assert abs(got - ref) / scale < TOL
    assert fb.dot_fp8_e5m2_acc_fp32_gpu(aw, bw).item() == got


# ------------------------------------------------------------------- C ABI --
def test_c_abi_status_codes_on_device(fb):
    lib = fb._lib.load()
    z = torch.zeros(64, dtype=torch.int32, device="cuda")
    o = torch.zeros(8, dtype=torch.float32, device="cuda")
    p, po = z.data_ptr(), o.data_ptr()
    assert lib.feather_gemv_fp8(p, p, po, 2, 16, 0, None) == 0
    assert lib.feather_gemv_fp8(p, p, po, 2, 18, 0, None) == -1
    assert lib.feather_gemv_fp8(p, p, po, 2, 16, 7, None) == -3
    assert lib.feather_gemv_fp8(p + 2, p, po, 2, 16, 0, None) == -2
    assert lib.feather_gemv_fp8(None, p, po, 2, 16, 0, None) == -1
    assert lib.feather_dot_fp8(p, p, po, None, 4, 0, None) == -6
    assert lib.feather_encode_fp8(po, 5, p, 4, 0, None) == -3
    assert lib.feather_decode_fp8(p, po, 4, 0, 9, None) == -3
    assert lib.feather_device_status(None) == 0
    torch.cuda.synchronize()


# ------------------------------------------------------- bounded device waits --
def test_sharded_wait_gives_up_and_reports_instead_of_hanging(fb):
    """A rank whose peer never delivers must not hang: the fused sharded kernel
    waits a bounded time for the peer's epoch flag, raises the device status
    word and returns; the host reads FEATHER_ERR_TIMEOUT and the context stays
    usable.  The "peer" here is a second flag block on the same GPU that nothing
    ever writes (no second process, no fault)."""
    lib = fb._lib.load()
    rows, N = 4736, 4096
    assert lib.feather_gemv_fp8_sharded_supported(rows, N) == 1
    gen = torch.Generator(device="cuda").manual_seed(11)
    A = torch.randn(rows, N, device="cuda", generator=gen, dtype=torch.float16)
    v = torch.randn(N, device="cuda", generator=gen, dtype=torch.float16)
    mw, vw = fb.pack_fp8_tensor(A, "E5M2"), fb.pack_fp8_tensor(v, "E5M2")
    out = [torch.zeros(2 * rows, dtype=torch.float32, device="cuda") for _ in range(2)]
    flags = [torch.zeros(32, dtype=torch.int32, device="cuda") for _ in range(2)]
    arr = ctypes.c_void_p * 2
    outs, flgs = arr(*[t.data_ptr() for t in out]), arr(*[t.data_ptr() for t in flags])
    assert lib.feather_device_status(None) == 0
    assert lib.feather_set_wait_limit_ms(100) == 0
    try:
        st = lib.feather_gemv_fp8_sharded(mw.data_ptr(), vw.data_ptr(), rows, N, 0, outs, flgs,
                                          0, 2, 1, None)
        assert st == 0
        assert lib.feather_device_status(None) == -7          # the wait gave up, no hang
        assert lib.feather_device_status(None) == 0           # sticky word was cleared
        with pytest.raises(fb._lib.FeatherError):
            fb._lib.check(-7)
        # rank 0's own rows were still computed and delivered to both buffers
        ref = fb.gemv_fp8_acc_fp32_gpu(mw, vw, (rows, N), "E5M2")
        assert torch.equal(out[0][:rows], ref) and torch.equal(out[1][:rows], ref)
        # with the missing flag supplied by hand the next call completes cleanly
        flags[0][1] = 2
        st = lib.feather_gemv_fp8_sharded(mw.data_ptr(), vw.data_ptr(), rows, N, 0, outs, flgs,
                                          0, 2, 2, None)
        assert st == 0 and lib.feather_device_status(None) == 0
    finally:
        assert lib.feather_set_wait_limit_ms(2000) == 0


# ------------------------------------------- column-sharded GEMV + all-reduce --
def _tagged(values: torch.Tensor, tag: int) -> torch.Tensor:
    """(value, tag) pairs as the all-reduce kernel exchanges them, viewed as floats."""
    pairs = torch.empty(values.numel(), 2, dtype=torch.int32, device=values.device)
    pairs[:, 0] = values.view(torch.int32)
    pairs[:, 1] = tag
    return pairs.reshape(-1).view(torch.float32)


@pytest.mark.parametrize("mode", MODES)
def test_allreduce_gemv_with_hand_fed_peer(fb, mode):
    """feather_gemv_fp8_allreduce as rank 0 of 2, the "peer" being a second inbox
    on the same GPU that the test fills by hand (no second process): the result
    is own partial + peer partial, the own partial lands tagged in the peer's
    inbox, the call counter advances on the device, halves alternate, and M may
    change between calls."""
    lib = fb._lib.load()
    max_rows, world = 2048, 2
    slot_max = 2 * max_rows
    inbox_floats = 2 * world * slot_max
    half = inbox_floats // 2
    inbox = [torch.zeros(inbox_floats, dtype=torch.float32, device="cuda") for _ in range(world)]
    flags = [torch.zeros(32, dtype=torch.int32, device="cuda") for _ in range(world)]
    arr = ctypes.c_void_p * world
    inb, flg = arr(*[t.data_ptr() for t in inbox]), arr(*[t.data_ptr() for t in flags])
    gen = torch.Generator(device="cuda").manual_seed(23)
    assert lib.feather_device_status(None) == 0
    for call, (M, n_local) in enumerate([(2048, 256), (2048, 704), (1000, 48), (37, 2064), (2048, 256)],
                                        start=1):
        A = torch.randn(M, n_local, device="cuda", generator=gen, dtype=torch.float16)
        v = torch.randn(n_local, device="cuda", generator=gen, dtype=torch.float16)
        mw, vw = fb.pack_fp8_tensor(A, mode), fb.pack_fp8_tensor(v, mode)
        own = fb.gemv_fp8_acc_fp32_gpu(mw, vw, (M, n_local), mode)
        peer = torch.randn(M, device="cuda", generator=gen, dtype=torch.float32)
        padded = (M + 15) // 16 * 16
        slot = 2 * padded
        base = (call & 1) * half
        # rank 1's sums in rank 0's inbox, slot 1, as rank 1 would have stored them
        # (whole 16-byte pieces: the rows past M carry the tag too)
        inbox[0][base + slot: base + 2 * slot] = _tagged(torch.nn.functional.pad(peer, (0, padded - M)), call)
        result = torch.full((M,), float("nan"), device="cuda")
        st = lib.feather_gemv_fp8_allreduce(mw.data_ptr(), vw.data_ptr(), result.data_ptr(), M, n_local,
                                            fb._lib.mode_id(mode), inb, inbox_floats, flg, 0, world, None)
        assert st == 0 and lib.feather_device_status(None) == 0
        assert torch.equal(result, own + peer)
        # rank 0's sums went, tagged with the call number, to rank 1's inbox, slot 0
        assert torch.equal(inbox[1][base: base + 2 * M].view(torch.int32), _tagged(own, call).view(torch.int32))
        f0 = flags[0].cpu()
        assert int(f0[17]) == call and int(f0[16]) == 0
    # too small an inbox, bad shapes
    p = inbox[0].data_ptr()
    assert lib.feather_gemv_fp8_allreduce(p, p, p, 2048, 256, 0, inb, inbox_floats - 8, flg, 0, world, None) == -8
    assert lib.feather_gemv_fp8_allreduce(p, p, p, 2048, 250, 0, inb, inbox_floats, flg, 0, world, None) == -1
    assert lib.feather_gemv_fp8_allreduce(p, p, p, 2048, 256, 0, inb, inbox_floats, flg, 2, world, None) == -1
    big = 1 << 20   # far more CTAs than the GPU holds at once: refused, not deadlocked
    assert lib.feather_gemv_fp8_allreduce(p, p, p, big, 16, 0, inb, 8 * big * world, flg, 0, world, None) == -8


def test_gemv_chain_kernel_allreduce_ops_with_hand_fed_peer(fb):
    """feather_gemv_chain_fp8_tp as rank 0 of 2, the "peer" being a second inbox
    on the same GPU that the test fills by hand: a column-sharded op's output is
    own partial + peer partial (rank order), the own partials land tagged in
    the peer's inbox, local ops of the same launch are untouched, a dependent op
    waits for the all-reduced result, and the call counter advances so that the
    two inbox halves alternate over repeated launches."""
    from feather_b200._lib import ChainOp
    lib = fb._lib.load()
    world, M, n_local = 2, 2048, 704
    gen = torch.Generator(device="cuda").manual_seed(61)
    def packed(*shape):
        return fb.pack_fp8_tensor(torch.randn(*shape, device="cuda", generator=gen) * 0.05, "E4M3")
    w_ar = [packed(M, n_local), packed(300, 256)]          # two all-reduced ops
    v_ar = [packed(n_local), packed(256)]
    w_loc, v_loc = packed(512, 2048), packed(2048)         # a local op in between
    w_dep = packed(64, M)                                   # reads the first all-reduced result
    outs = [torch.zeros((M + 3) // 4, dtype=torch.int32, device="cuda"),
            torch.zeros(512, dtype=torch.float32, device="cuda"),
            torch.zeros(300, dtype=torch.float32, device="cuda"),
            torch.zeros(64, dtype=torch.float32, device="cuda")]
    table = (ChainOp * 4)()
    def fill(t, m, v, out, Mi, Ni, out_mode=-1, wait=-1, ar=0):
        t.m, t.v, t.out, t.M, t.N, t.mode, t.out_mode, t.wait_op, t.allreduce = (
            m.data_ptr(), v.data_ptr(), out.data_ptr(), Mi, Ni, 1, out_mode, wait, ar)
    fill(table[0], w_ar[0], v_ar[0], outs[0], M, n_local, out_mode=1, ar=1)   # packed E4M3 output
    fill(table[1], w_loc, v_loc, outs[1], 512, 2048)
    fill(table[2], w_ar[1], v_ar[1], outs[2], 300, 256, ar=1)
    fill(table[3], w_dep, outs[0], outs[3], 64, M, wait=0)
    nbytes = int(lib.feather_gemv_chain_plan_bytes(4))
    plan = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    assert lib.feather_gemv_chain_plan(ctypes.cast(table, ctypes.c_void_p), 4, plan.data_ptr(), nbytes, None) == 0
    n_ar, rows_cap = 2, 2048
    inbox_floats = int(lib.feather_gemv_chain_inbox_floats(n_ar, M, world))
    assert inbox_floats == 2 * n_ar * world * rows_cap * 2
    inbox = [torch.zeros(inbox_floats, dtype=torch.float32, device="cuda") for _ in range(world)]
    flags = [torch.zeros(32, dtype=torch.int32, device="cuda") for _ in range(world)]
    arr = ctypes.c_void_p * world
    inb, flg = arr(*[t.data_ptr() for t in inbox]), arr(*[t.data_ptr() for t in flags])
    own = [fb.gemv_fp8_acc_fp32_gpu(w_ar[0], v_ar[0], (M, n_local), "E4M3"),
           fb.gemv_fp8_acc_fp32_gpu(w_ar[1], v_ar[1], (300, 256), "E4M3")]
    local = fb.gemv_fp8_acc_fp32_gpu(w_loc, v_loc, (512, 2048), "E4M3")
    def region(call, ai, src, rows):   # floats of (parity, op, source rank), `rows` pairs
        base = 2 * ((((call & 1) * n_ar + ai) * world + src) * rows_cap)
        return slice(base, base + 2 * rows)
    for call in range(1, 5):
        peer = [torch.randn(M, device="cuda", generator=gen), torch.randn(300, device="cuda", generator=gen)]
        for ai, rows in ((0, M), (1, 300)):   # the peer's partial sums, as rank 1 would have stored them
            inbox[0][region(call, ai, 1, rows)] = _tagged(peer[ai], call)
        for o in outs:
            o.zero_()
        st = lib.feather_gemv_chain_fp8_tp(plan.data_ptr(), 4, 1 if call % 2 else 0, n_ar, M, inb, inbox_floats,
                                           flg, 0, world, None)
        assert st == 0 and lib.feather_device_status(None) == 0
        total0 = own[0] + peer[0]
        want0 = fb.pack_fp8_tensor(total0, "E4M3")
        assert torch.equal(outs[0], want0.view(torch.int32))
        assert torch.equal(outs[1], local)
        assert torch.equal(outs[2], own[1] + peer[1])
        assert torch.equal(outs[3], fb.gemv_fp8_acc_fp32_gpu(w_dep, want0, (64, M), "E4M3"))
        for ai, rows in ((0, M), (1, 300)):   # own partials, tagged, in the peer's inbox
            assert torch.equal(inbox[1][region(call, ai, 0, rows)].view(torch.int32),
                               _tagged(own[ai], call).view(torch.int32))
        assert int(flags[0][17]) == call
    # an inbox that is too small is refused before anything is launched
    assert lib.feather_gemv_chain_fp8_tp(plan.data_ptr(), 4, 0, n_ar, M, inb, inbox_floats - 1, flg, 0, world,
                                         None) == -8
    assert lib.feather_gemv_chain_fp8_tp(plan.data_ptr(), 4, 0, n_ar, M, inb, inbox_floats, flg, 2, world,
                                         None) == -1


def test_allreduce_gemv_world_1_and_missing_peer(fb):
    """World size 1 is a plain GEMV.  With a peer that never delivers the wait
    gives up after the limit, the status word reports it and the context stays
    usable (nothing faults, nothing hangs)."""
    lib = fb._lib.load()
    M, n_local = 2048, 512
    gen = torch.Generator(device="cuda").manual_seed(29)
    A = torch.randn(M, n_local, device="cuda", generator=gen, dtype=torch.float16)
    v = torch.randn(n_local, device="cuda", generator=gen, dtype=torch.float16)
    mw, vw = fb.pack_fp8_tensor(A, "E4M3"), fb.pack_fp8_tensor(v, "E4M3")
    own = fb.gemv_fp8_acc_fp32_gpu(mw, vw, (M, n_local), "E4M3")
    inbox = [torch.zeros(8 * M, dtype=torch.float32, device="cuda") for _ in range(2)]
    flags = [torch.zeros(32, dtype=torch.int32, device="cuda") for _ in range(2)]
    arr1, arr2 = ctypes.c_void_p * 1, ctypes.c_void_p * 2
    result = torch.zeros(M, dtype=torch.float32, device="cuda")
    for _ in range(3):
        result.zero_()
        st = lib.feather_gemv_fp8_allreduce(mw.data_ptr(), vw.data_ptr(), result.data_ptr(), M, n_local, 1,
                                            arr1(inbox[0].data_ptr()), 4 * M, arr1(flags[0].data_ptr()),
                                            0, 1, None)
        assert st == 0 and lib.feather_device_status(None) == 0
        assert torch.equal(result, own)
    flags[0].zero_()
    assert lib.feather_set_wait_limit_ms(100) == 0
    try:
        st = lib.feather_gemv_fp8_allreduce(mw.data_ptr(), vw.data_ptr(), result.data_ptr(), M, n_local, 1,
                                            arr2(*[t.data_ptr() for t in inbox]), 8 * M,
                                            arr2(*[t.data_ptr() for t in flags]), 0, 2, None)
        assert st == 0
        assert lib.feather_device_status(None) == -7
        assert lib.feather_device_status(None) == 0
        # call 1 uses the odd half; slot 0 = rank 0's tagged sums
        assert torch.equal(inbox[1][4 * M: 6 * M].view(torch.int32), _tagged(own, 1).view(torch.int32))
    finally:
        assert lib.feather_set_wait_limit_ms(2000) == 0


# ---------------------------------------------- GEMV with re-encoded output --
@pytest.mark.parametrize("mode,out_mode", [("E5M2", "E5M2"), ("E4M3", "E4M3"), ("E4M3", "E5M2")])
@pytest.mark.parametrize("shape", [(8, 16), (37, 2064), (2048, 2048), (2046, 2048), (5632, 2048),
                                   (2048, 5632), (32000, 2048), (19000, 1024), (33, 20), (7, 2052),
                                   (4736, 4096), (4801, 8192), (100, 40000)])
def test_gemv_packed_output_equals_gemv_then_pack(fb, c_oracle, mode, out_mode, shape):
    """The fused GEMV -> re-encode result is, bit for bit, the packer applied to
    the plain GEMV result (checked with the ORACLE packer on the GPU's FP32 sums,
    and against this package's own packer): every dispatch path -- one, two and
    four rows per warp, the word-load kernel, the large-matrix kernel -- ragged M
    (zero-padded last word), and a different output format."""
    M, N = shape
    gen = torch.Generator(device="cuda").manual_seed(M * 31 + N)
    # wide value range so that the sums hit subnormal, normal and overflowing codes
    A = (torch.randn(M, N, device="cuda", generator=gen) *
         torch.exp2(torch.randint(-9, 4, (M, 1), device="cuda", generator=gen).float())).to(torch.float16)
    v = torch.randn(N, device="cuda", generator=gen, dtype=torch.float16)
    mw, vw = fb.pack_fp8_tensor(A, mode), fb.pack_fp8_tensor(v, mode)
    y = fb.gemv_fp8_acc_fp32_gpu(mw, vw, (M, N), mode)
    got = fb.gemv_fp8_ret_packed_gpu(mw, vw, (M, N), mode, out_mode=out_mode)
    assert got.dtype == torch.uint32 and got.numel() == (M + 3) // 4 and got.feather_mode == out_mode
    want = c_oracle.pack(y.cpu().numpy(), out_mode)
    assert np.array_equal(got.view(torch.int32).cpu().numpy().view(np.uint32), want)
    assert torch.equal(got.view(torch.int32), fb.pack_fp8_tensor(y, out_mode).view(torch.int32))
    # static-matrix flag and a caller-supplied output buffer: same words
    out = torch.zeros((M + 3) // 4, dtype=torch.uint32, device="cuda")
    fb.gemv_fp8_ret_packed_gpu(mw, vw, (M, N), mode, out_mode=out_mode, out=out, static_matrix=True)
    assert torch.equal(out.view(torch.int32), got.view(torch.int32))


def test_gemv_packed_output_feeds_next_gemv_and_rejects(fb):
    lib = fb._lib.load()
    gen = torch.Generator(device="cuda").manual_seed(5)
    A = (0.05 * torch.randn(2048, 2048, device="cuda", generator=gen)).to(torch.float16)
    B = (0.05 * torch.randn(512, 2048, device="cuda", generator=gen)).to(torch.float16)
    x = torch.randn(2048, device="cuda", generator=gen, dtype=torch.float16)
    aw, bw, xw = (fb.pack_fp8_tensor(t, "E4M3") for t in (A, B, x))
    h = fb.gemv_fp8_ret_packed_gpu(aw, xw, A.shape, "E4M3")          # packed activation
    y = fb.gemv(bw, h, original_shape=B.shape)                        # mode read from the tag
    h_ref = fb.pack_fp8_tensor(fb.gemv(aw, xw, original_shape=A.shape), "E4M3")
    assert torch.equal(y, fb.gemv(bw, h_ref, original_shape=B.shape))
    # the large-matrix path needs a workspace; without one the C entry says so
    assert lib.feather_gemv_fp8_packed_workspace_bytes(2048, 2048) == 0
    assert lib.feather_gemv_fp8_packed_workspace_bytes(16384, 16384) == 4 * 16384
    assert lib.feather_gemv_fp8_packed_workspace_bytes(64, 20) == 4 * 64
    p = aw.data_ptr()
    assert lib.feather_gemv_fp8_packed(p, p, p, None, 64, 20, 0, 0, 0, None) == -6
    assert lib.feather_gemv_fp8_packed(p, p, p, None, 64, 16, 0, 5, 0, None) == -3
    assert lib.feather_gemv_fp8_packed(p, p, p, None, 64, 18, 0, 0, 0, None) == -1
    assert fb.gemv_fp8_ret_packed_gpu(aw, xw, (0, 2048), "E4M3").numel() == 0
    torch.cuda.synchronize()


# ------------------------------------------------------------ ReLU on unpack --
@pytest.mark.parametrize("mode", MODES)
def test_relu_all_codes_ragged_and_large_vs_oracle(fb, golden, mode):
    from feather_b200.routines.activations import relu1d_fp8_ret_fp32_feather_gpu as relu
    bits = lambda t: t.view(torch.int32).cpu().numpy()
    codes = torch.arange(256, dtype=torch.uint8).view(torch.int32).cuda()
    got = relu(codes, 256, mode=mode)
    assert np.array_equal(bits(got), O.relu(codes.cpu().numpy(), 256, mode).view(np.int32))  # sign of zero too
    if mode == "E5M2":  # the reference kernel's own output (NaN codes apart, see the oracle test)
        want = golden("relu")["all_codes_out"]
        keep = ~np.isnan(want)
        assert np.array_equal(got.cpu().numpy()[keep], want[keep])
        rng = np.random.default_rng(int(golden("relu")["n36004_seed"]))
        x = torch.from_numpy(rng.standard_normal(4 * 9000 + 4).astype(np.float16)).cuda()
        packed = fb.pack_fp8_tensor(x, "E5M2")
        assert np.array_equal(relu(packed, x.numel()).cpu().numpy(), golden("relu")["n36004_out"])
        assert torch.equal(relu(packed), relu(packed, x.numel()))    # n defaults to 4 per word, mode to the tag
    gen = torch.Generator(device="cuda").manual_seed(3)
    words = torch.randint(-2 ** 31, 2 ** 31 - 1, ((1 << 22) + 3,), device="cuda", generator=gen, dtype=torch.int32)
    for n in (4 * words.numel(), 4 * words.numel() - 3, 5, 1):
        out = relu(words, n, mode=mode)
        assert np.array_equal(bits(out), O.relu(words.cpu().numpy(), n, mode).view(np.int32))
    off = relu(words[1:], 4 * (words.numel() - 1) - 1, mode=mode,
               out=torch.empty(4 * words.numel() + 1, device="cuda")[1:4 * (words.numel() - 1)])  # unaligned dst
    assert np.array_equal(bits(off), O.relu(words[1:].cpu().numpy(), off.numel(), mode).view(np.int32))
    assert relu(words[:0], 0, mode=mode).numel() == 0
    with pytest.raises(ValueError):
        relu(words[:2], 9, mode=mode)
    with pytest.raises(NotImplementedError):
        relu(words[:2], 8, mode="E3M4")


# ------------------------------------------------------- multi-vector GEMV --
@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("shape,batch", [((2048, 2048), 4), ((2046, 2048), 3), ((5632, 2048), 2),
                                         ((37, 2064), 4), ((300, 40000), 4), ((4801, 8192), 4),
                                         ((32000, 2048), 9), ((64, 16), 1), ((33, 20), 3), ((2048, 5632), 5),
                                         ((9472, 4096), 8), ((9500, 8208), 5), ((9473, 2048), 2),
                                         ((12000, 16400), 3), ((9472, 528), 11), ((20000, 2048), 16),
                                         ((9999, 1536), 13), ((19000, 512), 33)])
def test_gemv_multi_vs_oracle_and_single_gemv(fb, c_oracle, mode, shape, batch):
    """B vectors in one pass: every out[b] against the f64 oracle, and against
    the single-vector GEMV -- bit for bit where both take FP32-FMA kernels with
    the same summation order, within rounding where the single call takes the
    large-matrix kernel or the batch takes the tensor-core kernel (M >= 64 rows
    per SM; its accumulation is the tensor core's)."""
    M, N = shape
    gen = torch.Generator(device="cuda").manual_seed(M + 7 * N + batch)
    A = torch.randn(M, N, device="cuda", generator=gen, dtype=torch.float16)
    V = torch.randn(batch, N, device="cuda", generator=gen, dtype=torch.float16)
    mw, vw = fb.pack_fp8_tensor(A, mode), fb.pack_fp8_tensor(V, mode)
    Y = fb.gemv_fp8_multi_acc_fp32_gpu(mw, vw, (M, N), mode)
    assert Y.shape == (batch, M) and Y.dtype == torch.float32
    host = lambda t: t.view(torch.int32).cpu().numpy().view(np.uint32)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    large = (M >= 32 * sms and N >= 4096) or (M >= 64 * sms and N % 16 == 0 and batch > 1)
    for b in range(batch):
        vb = vw[b * (N // 4):(b + 1) * (N // 4)]
        single = fb.gemv_fp8_acc_fp32_gpu(mw, vb, (M, N), mode)
        if large:
            assert O.normalised_error(Y[b].cpu().numpy(), single.cpu().numpy()) < 1e-5
        else:
            assert torch.equal(Y[b], single)
        ref = c_oracle.gemv(host(mw), host(vb), (M, N), mode, acc="f64")
        assert O.normalised_error(Y[b].cpu().numpy(), ref) < 1e-5
    out = torch.zeros(batch, M, device="cuda")
    fb.gemv_fp8_multi_acc_fp32_gpu(mw, vw, (M, N), mode, batch=batch, out=out, static_matrix=True)
    assert torch.equal(out, Y)


def test_gemv_multi_e5m2_kernels_agree(fb):
    """Large E5M2 matrices with rows of a multiple of 512 codes take the tcgen05 kernel (16
    vectors per pass); the mma.sync kernel beside it (8 per pass) gives the same sums to
    rounding, and both are within the bound of the float64 result."""
    M, N, B = 16384, 16384, 16
    gen = torch.Generator(device="cuda").manual_seed(77)
    mw = fb.pack_fp8_tensor(torch.randn(M, N, device="cuda", generator=gen, dtype=torch.float16), "E5M2")
    vw = fb.pack_fp8_tensor(torch.randn(B, N, device="cuda", generator=gen, dtype=torch.float16), "E5M2")
    lib = fb._lib.load()
    try:
        assert lib.feather_set_tuning(b"multi_tc=0") == 0
        a = fb.gemv_fp8_multi_acc_fp32_gpu(mw, vw, (M, N), "E5M2")
    finally:
        assert lib.feather_set_tuning(b"multi_tc=1") == 0
    b = fb.gemv_fp8_multi_acc_fp32_gpu(mw, vw, (M, N), "E5M2")
    fb.device_status()
    assert O.normalised_error(b.cpu().numpy(), a.cpu().numpy()) < 1e-5
    A = fb.unpack_fp8_tensor(mw, "E5M2").reshape(M, N).double()
    V = fb.unpack_fp8_tensor(vw, "E5M2").reshape(B, N).double()
    exact = (A @ V.T).T.cpu().numpy()
    assert O.normalised_error(b.cpu().numpy(), exact) < 5e-6
    assert O.normalised_error(a.cpu().numpy(), exact) < 5e-6


def test_gemv_multi_rejects(fb):
    w = torch.zeros(64, dtype=torch.int32, device="cuda")
    assert fb.gemv_fp8_multi_acc_fp32_gpu(w, w, (4, 16), "E5M2", batch=0).shape == (0, 4)
    with pytest.raises(ValueError):
        fb.gemv_fp8_multi_acc_fp32_gpu(w, w[:6], (4, 16), "E5M2")            # not whole vectors
    with pytest.raises(ValueError):
        fb.gemv_fp8_multi_acc_fp32_gpu(w, w, (4, 16), "E5M2", batch=65)
    with pytest.raises(ValueError):
        fb.gemv_fp8_multi_acc_fp32_gpu(w, w[:8], (4, 16), "E5M2", batch=3)   # too few words
    lib = fb._lib.load()
    p = w.data_ptr()
    assert lib.feather_gemv_fp8_multi(p, p, p, 4, 16, 2, 3, 0, None) == -3
    assert lib.feather_gemv_fp8_multi(p, p, p, 4, 16, -1, 0, 0, None) == -1
    assert lib.feather_gemv_fp8_multi(p, p, p, 4, 16, 2, 0, 2, None) == -1


# ------------------------------------------------------------------ attention --
@pytest.fixture
def attention_kernel(fb):
    """Select the attention kernel for one test; the library's default afterwards."""
    lib = fb._lib.load()
    knob = {"default": b"attn_tc=1", "tcgen05": b"attn_tc=2", "mma.sync": b"attn_tc=0"}

    def choose(name):
        assert lib.feather_set_tuning(knob[name]) == 0
    yield choose
    assert lib.feather_set_tuning(knob["default"]) == 0


def test_attention_kernels_agree_without_key_split(fb, attention_kernel):
    """One key tile per query block: the tcgen05 kernel and the register-fed kernel run the
    same arithmetic; they differ where the exponent's argument (one FMA in the scale of
    log2 against a division and a subtraction) rounds a probability to the other FP16
    neighbour, far below the fixture tolerance of 5e-4."""
    from feather_b200.routines.attention import flash_attention_fp8_e5m2_acc_fp32_gpu as attn
    for seq, d in ((64, 32), (50, 64), (64, 128)):
        rng = np.random.default_rng(seq * d)
        x = [torch.from_numpy(rng.standard_normal((seq, d)).astype(np.float16)).cuda() for _ in range(3)]
        q, k, v = (fb.pack_fp8_tensor(t, "E5M2") for t in x)
        attention_kernel("mma.sync")
        a = attn(q, k, v, seq, d // 4)
        attention_kernel("tcgen05")
        b = attn(q, k, v, seq, d // 4)
        fb.device_status()
        assert O.normalised_error(b.cpu().numpy(), a.cpu().numpy()) < 5e-5


@pytest.mark.parametrize("seq,d", [(128, 64), (100, 32), (200, 128), (64, 16), (1, 64), (1000, 128),
                                   (4096, 64), (2500, 32), (8192, 128), (130, 256), (64, 512),
                                   (1024, 256), (777, 512), (4096, 512)])
@pytest.mark.parametrize("kernel", ["default", "tcgen05", "mma.sync"])
def test_attention_vs_oracle_and_reference_outputs(fb, golden, seq, d, kernel, attention_kernel):
    """Packed-E5M2 attention against the oracle (same tiles, same FP16 rounding of the
    probabilities), the reference kernel's own outputs where the fixture has them, and
    torch's scaled_dot_product_attention when the key tiles are full.  Every shape runs
    through the library's own choice of kernel, through the tcgen05 kernel (rows of 32 to
    512 codes; rows of 16 have only the register-fed kernel) and through the
    register-fed kernel."""
    from feather_b200.routines.attention import flash_attention_fp8_e5m2_acc_fp32_gpu as attn
    if kernel != "default" and d not in (32, 64, 128, 256, 512):
        pytest.skip("one kernel only for this width")
    attention_kernel(kernel)
    g = golden("attention")
    key = f"s{seq}_d{d}"
    seed = int(g[key + "_seed"]) if key + "_seed" in g else seq + d
    rng = np.random.default_rng(seed)
    x = [torch.from_numpy(rng.standard_normal((seq, d)).astype(np.float16)).cuda() for _ in range(3)]
    q, k, v = (fb.pack_fp8_tensor(t, "E5M2") for t in x)
    out = attn(q, k, v, seq, d // 4)
    assert out.shape == (seq, d) and out.dtype == torch.float32
    got = out.cpu().numpy()
    if key + "_out" in g:
        assert O.normalised_error(got, g[key + "_out"]) < 5e-4
    if seq <= 1000:
        host = lambda t: t.view(torch.int32).cpu().numpy().view(np.uint32)
        assert O.normalised_error(got, O.flash_attention(host(q), host(k), host(v), seq, d // 4)) < 5e-4
    if seq % 64 == 0:
        dec = [fb.unpack_fp8_tensor(t, "E5M2").reshape(seq, d) for t in (q, k, v)]
        ref = torch.nn.functional.scaled_dot_product_attention(*(t[None] for t in dec))[0]
        assert O.normalised_error(got, ref.cpu().numpy()) < 2e-3
    assert torch.equal(attn(q, k, v, seq, d // 4), out)          # deterministic


def test_attention_operands_off_the_16_byte_grid(fb, attention_kernel):
    """The tcgen05 kernel fetches its operands by tensor-map copies, which want 16-byte
    aligned bases; operands that start 4 bytes off take the register-fed kernel instead and
    give its result."""
    from feather_b200.routines.attention import flash_attention_fp8_e5m2_acc_fp32_gpu as attn
    seq, d = 640, 128
    rng = np.random.default_rng(5)
    x = [torch.from_numpy(rng.standard_normal((seq, d)).astype(np.float16)).cuda() for _ in range(3)]
    q, k, v = (fb.pack_fp8_tensor(t, "E5M2").reshape(-1) for t in x)
    attention_kernel("mma.sync")
    want = attn(q, k, v, seq, d // 4)
    attention_kernel("tcgen05")
    shifted = []
    for t in (q, k, v):
        buf = torch.empty(t.numel() + 1, dtype=t.dtype, device=t.device)
        buf[1:].copy_(t)
        shifted.append(buf[1:])
    assert shifted[0].data_ptr() % 16 == 4
    assert torch.equal(attn(*shifted, seq, d // 4), want)
    fb.device_status()


def test_attention_back_to_back_launches_keep_stream_order(fb, attention_kernel):
    """The tcgen05 kernel is launched with programmatic stream serialization: a grid may
    start while the kernel before it still runs.  Operands produced by the kernel right
    before it, and a shared output buffer written by consecutive launches, must behave as
    if the launches ran one after the other."""
    from feather_b200.routines.attention import flash_attention_fp8_e5m2_acc_fp32_gpu as attn
    attention_kernel("tcgen05")
    seq, d = 2048, 128
    g = torch.Generator(device="cuda").manual_seed(11)
    xs = [[torch.randn(seq, d, device="cuda", generator=g, dtype=torch.float16) for _ in range(3)] for _ in range(2)]
    packed = [[fb.pack_fp8_tensor(t, "E5M2") for t in x] for x in xs]
    want = [attn(*p, seq, d // 4).clone() for p in packed]
    torch.cuda.synchronize()
    out = torch.empty(seq, d, dtype=torch.float32, device="cuda")
    for i in range(21):                       # alternating operands into ONE output: the last launch wins
        attn(*packed[i % 2], seq, d // 4, out=out)
    assert torch.equal(out, want[0])
    for i in range(6):                        # operands packed by the kernels right before the launch
        fresh = [fb.pack_fp8_tensor(t, "E5M2") for t in xs[i % 2]]
        assert torch.equal(attn(*fresh, seq, d // 4), want[i % 2])
    fb.device_status()


def test_attention_rejects(fb):
    from feather_b200.routines.attention import flash_attention_fp8_e5m2_acc_fp32_gpu as attn
    w = torch.zeros(64 * 16, dtype=torch.int32, device="cuda")
    assert attn(w, w, w, 0, 16).shape == (0, 64)
    with pytest.raises(ValueError):
        attn(w, w, w, 64, 12)
    with pytest.raises(ValueError):
        attn(w, w, w[:100], 64, 16)
    lib = fb._lib.load()
    p = w.data_ptr()
    assert lib.feather_attention_fp8_e5m2(p, p, p, p, 64, 256, None) == -8
    assert lib.feather_attention_fp8_e5m2(p, p, p, p, 64, 5, None) == -1
    assert lib.feather_attention_fp8_e5m2(p, p, p, p + 4, 64, 16, None) == -2
