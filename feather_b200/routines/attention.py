"""Packed-E5M2 attention: the reference's ``feather.routines.attention`` surface.

``flash_attention_fp8_e5m2_acc_fp32_gpu(q, k, v, seq_len, h_dim)`` keeps the
reference signature (feather/routines/attention.py:110-179): packed E5M2 Q, K,
V of ``seq_len`` rows, ``h_dim`` = PACKED words per row (a quarter of the model
dimension, as the reference's docstring insists), result an FP32
``(seq_len, 4 * h_dim)`` CUDA tensor.  The arithmetic follows the reference
kernel tile by tile, including its unmasked zero keys when ``seq_len`` is not a
multiple of 64 (see ``feather_attention_fp8_e5m2`` in the C header).
"""
from __future__ import annotations

import torch

from .. import _lib
from ..packers.fp8 import as_words

__all__ = ["flash_attention_fp8_e5m2_acc_fp32_gpu"]


def flash_attention_fp8_e5m2_acc_fp32_gpu(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                                          seq_len: int, h_dim: int,
                                          out: torch.Tensor | None = None) -> torch.Tensor:
    seq_len, h_dim = int(seq_len), int(h_dim)
    if seq_len < 0 or h_dim not in (4, 8, 16, 32, 64, 128):
        raise ValueError("h_dim (packed words per row) must be a power of two from 4 to 128 and seq_len >= 0")
    with torch._C.DisableTorchFunctionSubclass():
        q, k, v = as_words(q, "q"), as_words(k, "k"), as_words(v, "v")
        need = seq_len * h_dim
        for name, t in (("q", q), ("k", k), ("v", v)):
            if t.numel() < need:
                raise ValueError(f"{name} holds {t.numel()} words, {seq_len} x {h_dim} needs {need}")
            if t.device != q.device:
                raise ValueError("q, k and v must be on the same device")
        if out is None:
            out = torch.empty((seq_len, 4 * h_dim), dtype=torch.float32, device=q.device)
        elif (out.dtype != torch.float32 or out.numel() != seq_len * 4 * h_dim or out.device != q.device
              or not out.is_contiguous()):
            raise ValueError("out must be a contiguous float32 (seq_len, 4 * h_dim) tensor on q's device")
        if seq_len:
            idx = q.device.index
            with torch.cuda.device(idx):
                _lib.check(_lib.load().feather_attention_fp8_e5m2(
                    q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), seq_len, h_dim,
                    _lib.current_stream_ptr(idx)))
    return out
