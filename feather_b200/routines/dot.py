"""Packed-FP8 dot product: the reference's ``feather.routines.dot`` FP8 surface.

``dot_fp8_e5m2_acc_fp32_gpu(x1, x2)`` keeps the reference signature and result
(feather/routines/dot.py:220-260: two packed vectors, a 0-dim FP32 CUDA
tensor).  The result is deterministic (fixed-order reduction), where the
reference's float atomics are not.  ``dot_fp8_e4m3_acc_fp32_gpu`` is an
extension: the reference has no E4M3 dot.
"""
from __future__ import annotations

import torch

from .. import _lib
from ..packers.fp8 import as_words

__all__ = ["dot_fp8_acc_fp32_gpu", "dot_fp8_e5m2_acc_fp32_gpu", "dot_fp8_e4m3_acc_fp32_gpu"]

# one zero-initialised workspace per (device, stream): the kernel hands its
# ticket counter back as zero, so the buffer is reused without clearing.
_workspaces: dict = {}


def _workspace(device: torch.device, stream: int, n_words: int) -> torch.Tensor:
    key = (device.index, stream)
    ws = _workspaces.get(key)
    need = int(_lib.load().feather_dot_workspace_bytes(n_words))
    if ws is None or ws.numel() < need:
        ws = torch.zeros(need, dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def dot_fp8_acc_fp32_gpu(x1: torch.Tensor, x2: torch.Tensor, mode: str = "E5M2") -> torch.Tensor:
    with torch._C.DisableTorchFunctionSubclass():  # operands may be PackedFP8 subclasses
        return _dot(x1, x2, mode)


def _dot(x1, x2, mode):
    mode_id = _lib.mode_id(mode)
    x1 = as_words(x1, "x1")
    x2 = as_words(x2, "x2")
    if x1.numel() != x2.numel():
        raise ValueError(f"operands differ in length: {x1.numel()} vs {x2.numel()} words")
    if x1.device != x2.device:
        raise ValueError("x1 and x2 must be on the same device")
    out = torch.empty((), dtype=torch.float32, device=x1.device)
    idx = x1.device.index
    with torch.cuda.device(idx):
        stream = _lib.current_stream_ptr(idx)
        ws = _workspace(x1.device, stream, x1.numel())
        _lib.check(_lib.load().feather_dot_fp8(x1.data_ptr(), x2.data_ptr(), out.data_ptr(),
                                               ws.data_ptr(), x1.numel(), mode_id, stream))
    return out


def dot_fp8_e5m2_acc_fp32_gpu(x1: torch.Tensor, x2: torch.Tensor) -> torch.Tensor:
    """Drop-in for feather/routines/dot.py:220-260."""
    return dot_fp8_acc_fp32_gpu(x1, x2, "E5M2")


def dot_fp8_e4m3_acc_fp32_gpu(x1: torch.Tensor, x2: torch.Tensor) -> torch.Tensor:
    """E4M3 dot with the kernel decode of feather/routines/gemv.py:83-88."""
    return dot_fp8_acc_fp32_gpu(x1, x2, "E4M3")
