"""CPU-side checks of the boundary: the shared library loads, exports every
symbol include/feather_b200.h declares, and rejects bad arguments before it
touches a device.  No compute call is made here."""
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from feather_b200.csrc import build
    build.build()  # nvcc cross-compiles for sm_100a without a GPU
    from feather_b200 import _lib
    return _lib.load()


def test_every_declared_symbol_is_exported(lib):
    header = open(os.path.join(ROOT, "include", "feather_b200.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(feather_[a-z0-9_]+)\s*\(", header))
    from feather_b200 import _lib
    assert declared == set(_lib.SYMBOLS), declared ^ set(_lib.SYMBOLS)
    for name in declared:
        assert getattr(lib, name) is not None


def test_version_and_strerror(lib):
    assert lib.feather_version() >= 100
    assert lib.feather_strerror(0) == b"success"
    for code in range(-7, 0):
        assert lib.feather_strerror(code) not in (b"", b"unknown feather status")
    assert lib.feather_strerror(-99) == b"unknown feather status"
    assert lib.feather_dot_workspace_bytes(1 << 24) >= 16 + 4


def test_argument_rejection_needs_no_device(lib):
    # these return before any CUDA call
    assert lib.feather_gemv_fp8(None, None, None, 2, 6, 0, None) == -1   # N % 4
    assert lib.feather_gemv_fp8(None, None, None, -1, 8, 0, None) == -1
    assert lib.feather_gemv_fp8(None, None, None, 2, 8, 3, None) == -3   # mode
    assert lib.feather_gemv_fp8(None, None, None, 0, 8, 0, None) == 0    # empty
    assert lib.feather_encode_fp8(None, 0, None, -5, 0, None) == -1
    assert lib.feather_encode_fp8(None, 2, None, 4, 0, None) == -3       # dtype
    assert lib.feather_encode_fp8(None, 0, None, 0, 1, None) == 0
    assert lib.feather_decode_fp8(None, None, 4, 0, 2, None) == -3       # semantics
    assert lib.feather_dot_fp8(None, None, None, None, -1, 0, None) == -1
    assert lib.feather_dot_fp8(None, None, None, None, 4, 0, None) == -1  # out is null
    # the entry points added around the path
    assert lib.feather_relu_fp8(None, None, -1, 0, None) == -1
    assert lib.feather_relu_fp8(None, None, 4, 2, None) == -3
    assert lib.feather_relu_fp8(None, None, 0, 1, None) == 0
    assert lib.feather_gemv_fp8_multi(None, None, None, 4, 16, 65, 0, 0, None) == -1   # too many vectors
    assert lib.feather_gemv_fp8_multi(None, None, None, 4, 18, 2, 0, 0, None) == -1   # N % 4
    assert lib.feather_gemv_fp8_multi(None, None, None, 4, 16, 2, 5, 0, None) == -3
    assert lib.feather_gemv_fp8_multi(None, None, None, 4, 16, 0, 0, 0, None) == 0    # no vectors
    assert lib.feather_gemv_fp8_packed(None, None, None, None, 4, 16, 0, 7, 0, None) == -3  # output mode
    assert lib.feather_gemv_fp8_packed(None, None, None, None, 4, 16, 0, 0, 8, None) == -1  # flags
    assert lib.feather_gemv_fp8_packed(None, None, None, None, 0, 16, 0, 1, 0, None) == 0
    assert lib.feather_gemv_fp8_packed_workspace_bytes(0, 16) == 0
    assert lib.feather_attention_fp8_e5m2(None, None, None, None, -1, 16, None) == -1
    assert lib.feather_attention_fp8_e5m2(None, None, None, None, 64, 0, None) == -1
    assert lib.feather_attention_fp8_e5m2(None, None, None, None, 0, 16, None) == 0
    assert lib.feather_gemv_fp8_allreduce(None, None, None, 8, 16, 0, None, 0, None, 0, 1, None) == -1
    assert lib.feather_gemv_fp8_allreduce(None, None, None, 8, 20, 0, None, 0, None, 0, 1, None) == -1  # N % 16


def test_python_surface_without_gpu():
    import torch

    import feather
    import feather_b200
    assert feather.gemv is feather_b200.gemv and feather.dot is feather_b200.dot
    from feather.packers.fp8 import pack_fp8_tensor
    from feather.routines.dot import dot_fp8_e5m2_acc_fp32_gpu  # noqa: F401
    from feather.routines.gemv import gemv_fp8_e4m3_acc_fp32_gpu, gemv_fp8_e5m2_acc_fp32_gpu  # noqa: F401
    from feather.routines.activations import relu1d_fp8_ret_fp32_feather_gpu  # noqa: F401
    from feather.routines.attention import flash_attention_fp8_e5m2_acc_fp32_gpu  # noqa: F401
    with pytest.raises(NotImplementedError):
        pack_fp8_tensor(torch.zeros(4, dtype=torch.float16), mode="E3M4")
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError):  # no CPU fallback
            pack_fp8_tensor(torch.zeros(4, dtype=torch.float16))
        with pytest.raises(ValueError):
            feather.gemv(torch.zeros(4, dtype=torch.int32), torch.zeros(1, dtype=torch.int32),
                         original_shape=(4, 4))


def test_header_is_plain_c(tmp_path):
    """The boundary is a C ABI: the header must compile as C99 on its own (no C++, no
    CUDA or torch types), which is what a cgo / FFI binding would consume."""
    import subprocess
    src = tmp_path / "use_header.c"
    src.write_text('#include "feather_b200.h"\nint main(void) { return feather_version() == 0; }\n')
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Wextra", "-pedantic", "-Werror", "-fsyntax-only",
                    "-I", os.path.join(ROOT, "include"), str(src)], check=True)


def test_host_only_entry_points_of_the_newer_surface(lib):
    """Sizes, tuning specs and the debug query are pure host code."""
    # tuning: "key=value,..." ; unknown keys and bad values are rejected, good ones applied
    assert lib.feather_set_tuning(b"ring_pre_kb=64,dot_ring=2") == 0
    assert lib.feather_set_tuning(b"ring_pre_kb=128, ring_pre_kb_e4m3=-1") == 0
    assert lib.feather_set_tuning(b"no_such_knob=1") == -1
    assert lib.feather_set_tuning(b"dot_unroll=3") == -1
    assert lib.feather_set_tuning(b"attn_tc=0") == 0 and lib.feather_set_tuning(b"attn_tc=2") == 0
    assert lib.feather_set_tuning(b"attn_tc=3") == -1
    assert lib.feather_set_tuning(b"attn_tc=1") == 0
    assert lib.feather_set_tuning(b"ring_pre_kb") == -1
    assert lib.feather_set_tuning(None) == -1
    assert lib.feather_debug_bounds() in (0, 1)
    for code in (-8, -9):
        assert lib.feather_strerror(code) not in (b"", b"unknown feather status")
    # chain plan: counters (ticket + one per op, 16-byte granular) + 48 bytes per op
    assert lib.feather_gemv_chain_plan_bytes(0) == 0
    assert lib.feather_gemv_chain_plan_bytes(1) == 16 + 48
    assert lib.feather_gemv_chain_plan_bytes(155) == 624 + 155 * 48
    # tensor-parallel inbox: 2 call parities x ops x ranks x rows (rounded up to 16) x (sum, tag)
    assert lib.feather_gemv_chain_inbox_floats(44, 2048, 8) == 2 * 44 * 8 * 2048 * 2
    assert lib.feather_gemv_chain_inbox_floats(1, 100, 2) == 2 * 1 * 2 * 112 * 2
    assert lib.feather_gemv_chain_inbox_floats(0, 2048, 8) == 0
    # argument checks that come before any CUDA call
    assert lib.feather_gemv_chain_plan(None, 1, None, 0, None) == -1
    assert lib.feather_gemv_chain_fp8(None, 1, 0, None) == -1
    assert lib.feather_gemv_fp8_sharded_wait(None, 0, 1, 1, None, None) == -1
