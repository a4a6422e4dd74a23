"""Full-size parity against the REFERENCE ITSELF on the same GPU.

The reference package, installed unmodified under baseline/_ref by
baseline/install_reference.sh, runs in a process of its own
(baseline/reference_worker.py): its packer (feather/packers/fp8.py:260-281)
packs the seeded workload, its Triton kernels (feather/routines/gemv.py:136-235,
feather/routines/dot.py:220-260, feather/routines/attention.py:110-179) compute on
those words.  This process
generates the same workload from the same seed, packs it with the CUDA encoder
and runs the CUDA kernels through the C ABI:

* packed words must be bit-equal (SHA-256 of the whole buffer, plus a strided
  sample that localises a mismatch);
* GEMV results must agree within 1e-5 of the result's scale (FP32 accumulation,
  order-dependent -- the tolerance the path is specified with); dot likewise,
  the scale being sum |a_i * b_i| (the reference's own float atomics already
  make its last bits vary from run to run);
* attention results (both CUDA kernels) must agree with the reference kernel's within 5e-4
  of the result's scale, the tolerance of the fixtures (probabilities rounded to FP16).

Skipped when the reference install or Triton is not there.
"""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from baseline import workloads as W  # noqa: E402

pytestmark = pytest.mark.gpu
TOL = 1e-5
WORKER = os.path.join(ROOT, "baseline", "reference_worker.py")
GEMV_CASES = ["c1_e5m2_4096", "c1_e4m3_4096", "c2_e5m2_16384", "c3_e4m3_8192x8192",
              "c3_e4m3_16384x8192", "c3_e4m3_16384x16384"] + [n for n in W.CASES if n.startswith("int_")]
DOT_CASES = ["dot_e5m2_2pow26", "dot_e5m2_1500000", "dot_e5m2_10000"]
ATTENTION_CASES = [n for n in W.CASES if n.startswith("attn_")]


def run_worker(*argv, timeout=1500):
    res = subprocess.run([sys.executable, WORKER, *argv], capture_output=True, text=True, timeout=timeout,
                         cwd=os.path.join(ROOT, "baseline"))
    for line in res.stdout.splitlines():
        if line.startswith("REFERENCE_WORKER "):
            return json.loads(line[len("REFERENCE_WORKER "):])
    raise RuntimeError(f"reference worker gave no result (rc {res.returncode}): {res.stderr[-2000:]}")


@pytest.fixture(scope="module")
def reference_results(tmp_path_factory):
    if not os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "feather", "routines")):
        pytest.skip("baseline/_ref is not installed (baseline/install_reference.sh)")
    out = tmp_path_factory.mktemp("reference")
    res = run_worker("parity", "--cases", ",".join(GEMV_CASES + DOT_CASES + ATTENTION_CASES), "--outdir", str(out))
    if "unavailable" in res:
        pytest.skip("the reference cannot run here: " + res["unavailable"])
    return lambda name: np.load(os.path.join(str(out), name + ".npz"))


@pytest.fixture(scope="module")
def fb():
    import feather_b200
    feather_b200._lib.load()
    return feather_b200


def host_words(t: torch.Tensor) -> np.ndarray:
    return t.view(torch.int32).cpu().numpy().view(np.uint32)


def sha(words: np.ndarray) -> str:
    import hashlib
    return hashlib.sha256(np.ascontiguousarray(words).view(np.uint8).tobytes()).hexdigest()


def check_words(ours: torch.Tensor, ref, key: str):
    mine = host_words(ours)
    sample = ref[key + "_sample"]
    stride = 4099
    assert mine[::stride].shape == sample.shape
    bad = np.flatnonzero(mine[::stride] != sample)
    assert bad.size == 0, f"packed word {bad[0] * stride} differs from the reference packer's"
    assert sha(mine) == str(ref[key + "_sha"]), "packed buffer differs from the reference packer's"


@pytest.mark.parametrize("case", GEMV_CASES)
def test_gemv_full_size_against_the_reference_kernel(fb, reference_results, case):
    ref = reference_results(case)
    A, v, mode = W.make(case, "cuda")
    mw, vw = fb.pack_fp8_tensor(A, mode), fb.pack_fp8_tensor(v, mode)
    check_words(mw, ref, "a")
    check_words(vw, ref, "b")
    y = fb.gemv_fp8_acc_fp32_gpu(mw, vw, tuple(A.shape), mode).cpu().numpy()
    y_ref = ref["out"]
    assert np.isfinite(y_ref).all()
    err = np.abs(y.astype(np.float64) - y_ref).max() / max(np.abs(y_ref).max(), 1e-30)
    assert err < TOL, f"{case}: {err:.3e} of the result's scale away from the reference kernel"
    if case.startswith("int_"):
        # feather/benchmark/bench_gemv.py:75-93: integer inputs, exact in both formats
        assert np.array_equal(y, y_ref)
        assert torch.equal(torch.from_numpy(y).cuda(), torch.mv(A.float(), v.float()))
    fb.device_status()


@pytest.mark.parametrize("case", DOT_CASES)
def test_dot_against_the_reference_kernel(fb, reference_results, case):
    ref = reference_results(case)
    a, b, mode = W.make(case, "cuda")
    aw, bw = fb.pack_fp8_tensor(a, mode), fb.pack_fp8_tensor(b, mode)
    check_words(aw, ref, "a")
    check_words(bw, ref, "b")
    got = fb.dot_fp8_e5m2_acc_fp32_gpu(aw, bw).item()
    scale = float((fb.unpack_fp8_tensor(aw, mode).double().abs()
                   * fb.unpack_fp8_tensor(bw, mode).double().abs()).sum().item())
    for r in ref["out"]:   # two runs of the reference (atomics: not bit-stable)
        assert abs(got - float(r)) / scale < TOL
    assert fb.dot_fp8_e5m2_acc_fp32_gpu(aw, bw).item() == got
    fb.device_status()


@pytest.mark.parametrize("case", ATTENTION_CASES)
def test_attention_full_size_against_the_reference_kernel(fb, reference_results, case):
    from feather_b200.routines.attention import flash_attention_fp8_e5m2_acc_fp32_gpu as attn
    ref = reference_results(case)
    (q, k, v), _, mode = W.make(case, "cuda")
    seq, d = q.shape
    packed = [fb.pack_fp8_tensor(t, mode) for t in (q, k, v)]
    for words, key in zip(packed, "qkv"):
        assert sha(host_words(words)) == str(ref[key + "_sha"]), "packed buffer differs from the reference packer's"
    if "failed" in ref.files:
        pytest.skip("the reference kernel does not run this shape here: " + str(ref["failed"])[:120])
    y_ref = ref["out"]
    assert np.isfinite(y_ref).all()
    lib = fb._lib.load()
    for knob in (b"attn_tc=2", b"attn_tc=0"):        # the tcgen05 kernel, the mma.sync kernel
        assert lib.feather_set_tuning(knob) == 0
        try:
            y = attn(*packed, seq, d // 4).cpu().numpy()
        finally:
            assert lib.feather_set_tuning(b"attn_tc=1") == 0
        err = np.abs(y.astype(np.float64) - y_ref).max() / np.abs(y_ref).max()
        assert err < 5e-4, f"{case} ({knob.decode()}): {err:.3e} of the result's scale away from the reference kernel"
    fb.device_status()
