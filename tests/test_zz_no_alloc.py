"""feather_dot_fp8_static: the dot product for callers that cannot allocate.

Some users of this library may not call cudaMalloc at all -- a host callback
running on a stream, a plug-in living inside another framework's pre-reserved
memory arena, a loop that cannot afford the allocator's device-wide
synchronisation -- so they cannot provide the workspace feather_dot_fp8 asks
for.  This entry point keeps its scratch in a fixed array inside the library.
The test drives it through the C ABI and holds it to the workspace-taking
entry point's answer bit for bit (both run the same kernel on the same grid)
and to the CPU oracle's float64 sum within the dot tests' tolerance: two calls
in a row on different data (the second call meets whatever the first left in
the shared array), both FP8 modes, plus the size limit.  The file name sorts
last so that a failure here cannot hide any other test from a run that stops
at the first failure.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
TOL = 1e-5  # same bar as the other dot tests: |difference| / sum of |products|


@pytest.fixture(scope="module")
def lib():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from feather_b200 import _lib
    return _lib.load()


def _operands(n_words: int, seed: int):
    rng = np.random.default_rng(seed)
    a = rng.integers(0, 2 ** 32, size=n_words, dtype=np.uint64).astype(np.uint32) & 0xBFBFBFBF
    b = rng.integers(0, 2 ** 32, size=n_words, dtype=np.uint64).astype(np.uint32) & 0xBFBFBFBF
    to_dev = lambda x: torch.from_numpy(x.view(np.int32)).cuda()  # finite codes only
    return a, b, to_dev(a), to_dev(b)


@pytest.mark.parametrize("mode", [0, 1])
def test_static_dot_matches_workspace_dot_twice_in_a_row(lib, mode, c_oracle):
    from oracle import feather_oracle as O
    ws = torch.zeros(int(lib.feather_dot_workspace_bytes(0)), dtype=torch.uint8, device="cuda")
    out_ref = torch.zeros((), dtype=torch.float32, device="cuda")
    out_new = torch.full((), float("nan"), dtype=torch.float32, device="cuda")
    # first a large call (long enough for the bulk-copy ring kernel: every CTA
    # fills its scratch slot), then a small one on other data that must not see
    # the leftovers, then an odd, unaligned length
    for n_words, seed, off in (((1 << 22) + 5, 1, 0), (4099, 2, 0), (70001, 3, 1)):
        a, b, ad, bd = _operands(n_words + off, seed)
        a, b, ad, bd = a[off:], b[off:], ad[off:], bd[off:]
        assert lib.feather_dot_fp8(ad.data_ptr(), bd.data_ptr(), out_ref.data_ptr(),
                                   ws.data_ptr(), n_words, mode, None) == 0
        assert lib.feather_dot_fp8_static(ad.data_ptr(), bd.data_ptr(), out_new.data_ptr(),
                                          n_words, mode, None) == 0
        torch.cuda.synchronize()
        name = "E5M2" if mode == 0 else "E4M3"
        scale = float(np.abs(O.unpack(a, name).astype(np.float64) * O.unpack(b, name)).sum())
        assert out_new.item() == out_ref.item()   # same kernel, same grid: same bits
        want = float(c_oracle.dot(a, b, name, acc="f64"))
        assert abs(out_new.item() - want) / scale < TOL
        # and once more on the same data: same bits as its own previous answer
        first = out_new.item()
        assert lib.feather_dot_fp8_static(ad.data_ptr(), bd.data_ptr(), out_new.data_ptr(),
                                          n_words, mode, None) == 0
        torch.cuda.synchronize()
        assert out_new.item() == first


def test_static_dot_limits_and_rejects(lib):
    z = torch.zeros(16, dtype=torch.int32, device="cuda")
    o = torch.full((), 7.0, dtype=torch.float32, device="cuda")
    limit = int(lib.feather_dot_fp8_static_max_words())
    assert limit == 1 << 28
    # beyond the limit: a clear error, nothing launched, output untouched
    assert lib.feather_dot_fp8_static(z.data_ptr(), z.data_ptr(), o.data_ptr(), limit + 1, 0, None) == -8
    assert b"scratch" in lib.feather_strerror(-8)
    assert lib.feather_dot_fp8_static(z.data_ptr(), z.data_ptr(), o.data_ptr(), 4, 5, None) == -3
    assert lib.feather_dot_fp8_static(z.data_ptr(), z.data_ptr(), None, 4, 0, None) == -1
    torch.cuda.synchronize()
    assert o.item() == 7.0
    # empty operands: the result is zero
    assert lib.feather_dot_fp8_static(z.data_ptr(), z.data_ptr(), o.data_ptr(), 0, 0, None) == 0
    torch.cuda.synchronize()
    assert o.item() == 0.0
