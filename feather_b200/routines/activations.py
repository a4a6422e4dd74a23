"""ReLU on unpack: the reference's ``feather.routines.activations`` surface.

``relu1d_fp8_ret_fp32_feather_gpu(x, n)`` keeps the reference signature
(feather/routines/activations.py:32-41): ``x`` packed E5M2 words, ``n`` the
number of FP32 results; the result is ``max(0, decode(code))`` per code.  The
reference decodes E5M2 only (activations.py:19-22); ``mode="E4M3"`` is an
extension and uses the GEMV kernels' decode (feather/routines/gemv.py:83-88).
A NaN code gives 0 and -0 gives +0, as the compiled reference kernel's
``maximum`` does.
"""
from __future__ import annotations

import torch

from .. import _lib
from ..packers.fp8 import as_words

__all__ = ["relu1d_fp8_ret_fp32_feather_gpu"]


def relu1d_fp8_ret_fp32_feather_gpu(x: torch.Tensor, n: int | None = None, mode: str | None = None,
                                    out: torch.Tensor | None = None) -> torch.Tensor:
    """FP32 ``(n,)`` CUDA tensor of ``max(0, x_i)``; ``n`` defaults to four per
    packed word, ``mode`` to the mode the packer recorded on ``x`` (else E5M2)."""
    if mode is None:
        mode = getattr(x, "feather_mode", None) or "E5M2"
    mode_id = _lib.mode_id(mode)
    with torch._C.DisableTorchFunctionSubclass():
        w = as_words(x, "x")
        n = 4 * w.numel() if n is None else int(n)
        if n < 0 or n > 4 * w.numel():
            raise ValueError(f"n={n} exceeds the {4 * w.numel()} codes x holds")
        if out is None:
            out = torch.empty((n,), dtype=torch.float32, device=w.device)
        elif (out.dtype != torch.float32 or out.numel() != n or out.device != w.device
              or not out.is_contiguous()):
            raise ValueError("out must be a contiguous float32 tensor of n elements on x's device")
        if n:
            idx = w.device.index
            with torch.cuda.device(idx):
                _lib.check(_lib.load().feather_relu_fp8(w.data_ptr(), out.data_ptr(), n, mode_id,
                                                        _lib.current_stream_ptr(idx)))
    return out
