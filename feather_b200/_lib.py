"""ctypes binding of libfeather_b200.so (the C ABI in include/feather_b200.h).

There is no CPU or PyTorch fallback: if the shared library cannot be loaded
the import of any op fails loudly with the reason.
"""
from __future__ import annotations

import ctypes
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
# FEATHER_DEBUG_BOUNDS=1 selects the bounds-checking build (python -m feather_b200.csrc.build --debug-bounds)
LIB_PATH = os.path.join(_PKG, "libfeather_b200_debug.so" if os.environ.get("FEATHER_DEBUG_BOUNDS") == "1"
                        else "libfeather_b200.so")

MODE_IDS = {"E5M2": 0, "E4M3": 1}
SRC_F16, SRC_F32 = 0, 1
DECODE_KERNEL, DECODE_IEEE = 0, 1

# every symbol include/feather_b200.h declares: name -> (restype, argtypes)
_vp, _i32, _i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64
SYMBOLS = {
    "feather_version": (_i32, []),
    "feather_debug_bounds": (_i32, []),
    "feather_strerror": (ctypes.c_char_p, [_i32]),
    "feather_encode_fp8": (_i32, [_vp, _i32, _vp, _i64, _i32, _vp]),
    "feather_decode_fp8": (_i32, [_vp, _vp, _i64, _i32, _i32, _vp]),
    "feather_attention_fp8_e5m2": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _vp]),
    "feather_relu_fp8": (_i32, [_vp, _vp, _i64, _i32, _vp]),
    "feather_gemv_fp8": (_i32, [_vp, _vp, _vp, _i64, _i64, _i32, _vp]),
    "feather_gemv_fp8_multi": (_i32, [_vp, _vp, _vp, _i64, _i64, _i32, _i32, ctypes.c_uint32, _vp]),
    "feather_gemv_fp8_packed": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _i32, _i32, ctypes.c_uint32, _vp]),
    "feather_gemv_fp8_packed_workspace_bytes": (_i64, [_i64, _i64]),
    "feather_gemv_fp8_sharded": (_i32, [_vp, _vp, _i64, _i64, _i32, _vp, _vp, _i32, _i32,
                                        ctypes.c_uint32, _vp]),
    "feather_gemv_fp8_sharded_supported": (_i32, [_i64, _i64]),
    "feather_gemv_fp8_sharded_ex": (_i32, [_vp, _vp, _i64, _i64, _i32, _vp, _vp, _i32, _i32,
                                           ctypes.c_uint32, ctypes.c_uint32, _vp, _vp]),
    "feather_gemv_fp8_sharded_wait": (_i32, [_vp, _i32, _i32, ctypes.c_uint32, _vp, _vp]),
    "feather_gemv_fp8_allreduce": (_i32, [_vp, _vp, _vp, _i64, _i64, _i32, _vp, _i64, _vp, _i32, _i32,
                                          _vp]),
    "feather_enable_peer_access": (_i32, [_i32]),
    "feather_ipc_export": (_i32, [_vp, _vp, ctypes.POINTER(_i64)]),
    "feather_ipc_open": (_i32, [_vp, _i64, ctypes.POINTER(_vp)]),
    "feather_ipc_close": (_i32, [_vp, _i64]),
    "feather_device_status": (_i32, [_vp]),
    "feather_set_wait_limit_ms": (_i32, [_i32]),
    "feather_set_tuning": (_i32, [ctypes.c_char_p]),
    "feather_gemv_chain_plan_bytes": (_i64, [_i32]),
    "feather_gemv_chain_plan": (_i32, [_vp, _i32, _vp, _i64, _vp]),
    "feather_gemv_chain_fp8": (_i32, [_vp, _i32, ctypes.c_uint32, _vp]),
    "feather_gemv_chain_inbox_floats": (_i64, [_i32, _i32, _i32]),
    "feather_gemv_chain_fp8_tp": (_i32, [_vp, _i32, ctypes.c_uint32, _i32, _i32, _vp, _i64, _vp, _i32, _i32,
                                         _vp]),
    "feather_gemv_fp8_ex": (_i32, [_vp, _vp, _vp, _i64, _i64, _i32, ctypes.c_uint32, _vp]),
    "feather_dot_fp8": (_i32, [_vp, _vp, _vp, _vp, _i64, _i32, _vp]),
    "feather_dot_workspace_bytes": (_i64, [_i64]),
    "feather_dot_fp8_static": (_i32, [_vp, _vp, _vp, _i64, _i32, _vp]),
    "feather_dot_fp8_static_max_words": (_i64, []),
}



class ChainOp(ctypes.Structure):
    """feather_chain_op of include/feather_b200.h."""
    _fields_ = [("m", _vp), ("v", _vp), ("out", _vp), ("M", ctypes.c_int32), ("N", ctypes.c_int32),
                ("mode", ctypes.c_int32), ("out_mode", ctypes.c_int32), ("wait_op", ctypes.c_int32),
                ("allreduce", ctypes.c_int32)]


_lib = None


class FeatherError(RuntimeError):
    """A feather_status other than FEATHER_OK came back from the library."""

    def __init__(self, status: int, message: str):
        super().__init__(f"libfeather_b200: {message} (status {status})")
        self.status = status


def load() -> ctypes.CDLL:
    """Load the shared library once; raise if it is missing or incomplete."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m feather_b200.csrc.build` "
            "(needs nvcc); feather_b200 has no fallback path")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (restype, argtypes) in SYMBOLS.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def current_stream_ptr(device_index: int) -> int:
    """Raw cudaStream_t of torch's current stream on `device_index`."""
    import torch
    try:
        return torch._C._cuda_getCurrentRawStream(device_index)
    except AttributeError:  # older/newer torch without the private accessor
        return torch.cuda.current_stream(device_index).cuda_stream


def mode_id(mode: str) -> int:
    # the reference raises NotImplementedError for any other string
    # (feather/packers/fp8.py:113-114)
    if mode not in MODE_IDS:
        raise NotImplementedError(f"Mode {mode} not supported")
    return MODE_IDS[mode]


def check(status: int) -> None:
    if status == 0:
        return
    msg = load().feather_strerror(status).decode()
    if status in (-1, -2, -6, -8):
        raise ValueError(f"libfeather_b200: {msg} (status {status})")
    if status == -9:
        raise FeatherError(status, msg)
    if status == -7:
        raise FeatherError(status, msg + " (a device-side wait timed out; results are undefined)")
    if status == -3:
        raise NotImplementedError(f"libfeather_b200: {msg} (status {status})")
    raise FeatherError(status, msg)
