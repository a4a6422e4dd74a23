"""feather_b200: the packed-FP8 matrix-vector path of SuriyaaMM/feather, as
hand-written sm_100a CUDA behind a C ABI (include/feather_b200.h).

Two surfaces are exported:

* the reference's real module paths -- ``feather_b200.packers.fp8.pack_fp8_tensor``,
  ``feather_b200.routines.gemv.gemv_fp8_e5m2_acc_fp32_gpu`` /
  ``gemv_fp8_e4m3_acc_fp32_gpu``, ``feather_b200.routines.dot.dot_fp8_e5m2_acc_fp32_gpu``;
* the names the reference's README uses -- ``pack_fp8_tensor(t, mode=)``,
  ``gemv(m_packed, v_packed, original_shape=...)``, ``dot(a_packed, b_packed)``.

The top-level ``feather`` package of this repository re-exports both, so
``import feather`` code written against the reference runs unchanged.
There is no Triton, no backend dispatch and no CPU fallback.
"""
from __future__ import annotations

from . import _lib
from .packers.fp8 import PackedFP8, pack_fp8_tensor, unpack_fp8_tensor
from .routines.dot import (dot_fp8_acc_fp32_gpu, dot_fp8_e4m3_acc_fp32_gpu,
                           dot_fp8_e5m2_acc_fp32_gpu)
from .routines.gemv import (gemv_fp8_acc_fp32_gpu, gemv_fp8_e4m3_acc_fp32_gpu,
                            gemv_fp8_e5m2_acc_fp32_gpu, gemv_fp8_multi_acc_fp32_gpu,
                            gemv_fp8_ret_packed_gpu)

__version__ = "0.2.0"
__all__ = ["pack_fp8_tensor", "unpack_fp8_tensor", "gemv", "dot", "PackedFP8", "device_status",
           "gemv_fp8_acc_fp32_gpu", "gemv_fp8_e5m2_acc_fp32_gpu", "gemv_fp8_e4m3_acc_fp32_gpu",
           "gemv_fp8_ret_packed_gpu", "gemv_fp8_multi_acc_fp32_gpu", "dot_fp8_acc_fp32_gpu", "dot_fp8_e5m2_acc_fp32_gpu", "dot_fp8_e4m3_acc_fp32_gpu"]


def _mode_of(mode, *operands) -> str:
    """Mode resolution for the README-level calls, which have no mode
    argument in the reference: explicit ``mode=`` wins, else the mode the
    packer recorded on an operand, else the packer's default "E5M2"."""
    if mode is not None:
        return mode
    for t in operands:
        tagged = getattr(t, "feather_mode", None)
        if tagged is not None:
            return tagged
    return "E5M2"


def device_status() -> None:
    """Synchronise the current stream and raise if a device-side bounded wait
    timed out since the last check (``feather_device_status``)."""
    import torch
    _lib.check(_lib.load().feather_device_status(torch.cuda.current_stream().cuda_stream))


def gemv(m_packed, v_packed, original_shape=None, mode=None, out=None, static_matrix=False):
    """``feather.gemv(m_packed, v_packed, original_shape=matrix.shape)``."""
    if original_shape is None:
        raise TypeError("gemv() needs original_shape=(M, N), the matrix shape before packing")
    return gemv_fp8_acc_fp32_gpu(m_packed, v_packed, tuple(original_shape),
                                 _mode_of(mode, m_packed, v_packed), out=out,
                                 static_matrix=static_matrix)


def dot(a_packed, b_packed, mode=None):
    """``feather.dot(a_packed, b_packed)``: packed-FP8 dot product."""
    return dot_fp8_acc_fp32_gpu(a_packed, b_packed, _mode_of(mode, a_packed, b_packed))
