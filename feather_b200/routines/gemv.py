"""Packed-FP8 GEMV: the reference's ``feather.routines.gemv`` surface.

``gemv_fp8_e5m2_acc_fp32_gpu`` / ``gemv_fp8_e4m3_acc_fp32_gpu`` keep the
reference signatures (feather/routines/gemv.py:136, :187): packed matrix,
packed vector, the UNPACKED matrix shape; result an FP32 ``(M,)`` CUDA tensor,
enqueued on the current stream without synchronising.  Unlike the reference
wrappers, operands are validated (the reference computes garbage silently for
a short vector, a CPU tensor or N % 4 != 0) and the output is allocated on the
device directly.
"""
from __future__ import annotations

import torch

from .. import _lib
from ..packers.fp8 import as_words

__all__ = ["gemv_fp8_acc_fp32_gpu", "gemv_fp8_e5m2_acc_fp32_gpu", "gemv_fp8_e4m3_acc_fp32_gpu",
           "gemv_fp8_ret_packed_gpu", "gemv_fp8_multi_acc_fp32_gpu"]


def gemv_fp8_acc_fp32_gpu(m: torch.Tensor, v: torch.Tensor, m_shape, mode: str = "E5M2",
                          out: torch.Tensor | None = None,
                          static_matrix: bool = False) -> torch.Tensor:
    """out[r] = sum_j decode(m[r, j]) * decode(v[j]) with FP32 accumulation.

    ``static_matrix=True`` promises that no work still in flight on the stream
    writes ``m`` (weights packed earlier and synchronised): the kernel may then
    start streaming the matrix before it has waited for the previous kernel
    (``FEATHER_GEMV_STATIC_MATRIX``).  Leave it False when ``m`` was produced by
    the call right before."""
    # packed operands may be PackedFP8 (a Tensor subclass): skip the Python-level
    # __torch_function__ dispatch for the metadata reads below
    with torch._C.DisableTorchFunctionSubclass():
        return _gemv(m, v, m_shape, mode, out, 1 if static_matrix else 0)


def gemv_fp8_ret_packed_gpu(m: torch.Tensor, v: torch.Tensor, m_shape, mode: str = "E5M2",
                            out_mode: str | None = None, out: torch.Tensor | None = None,
                            static_matrix: bool = False, workspace: torch.Tensor | None = None):
    """The GEMV with its result re-encoded to packed FP8 in the same launch:
    ``pack_fp8_tensor(gemv(m, v, m_shape), out_mode)`` bit for bit -- the packed
    activation the next GEMV of a chain takes.  No reference counterpart (there
    the result goes through the CPU packer, feather/packers/fp8.py:260-281).

    Returns ``ceil(M / 4)`` packed words (a ``PackedFP8`` tagged ``out_mode``,
    default: ``mode``).  Small and mid-size matrices encode in the GEMV kernel's
    epilogue; large ones (and rows that are not whole 16-byte chunks) run the
    encoder behind the GEMV kernel on ``workspace`` (M floats, allocated here
    when not given)."""
    from ..packers.fp8 import _tag
    out_mode = mode if out_mode is None else out_mode
    with torch._C.DisableTorchFunctionSubclass():
        words = _gemv(m, v, m_shape, mode, out, 1 if static_matrix else 0,
                      out_mode_id=_lib.mode_id(out_mode), workspace=workspace)
        return words if out is not None else _tag(words, out_mode)


def gemv_fp8_multi_acc_fp32_gpu(m: torch.Tensor, v: torch.Tensor, m_shape, mode: str = "E5M2",
                                batch: int | None = None, out: torch.Tensor | None = None,
                                static_matrix: bool = False) -> torch.Tensor:
    """``out[b] = gemv(m, v[b])`` for ``batch`` packed vectors in ONE pass over
    the matrix (``feather_gemv_fp8_multi``).  No reference counterpart: there
    every vector is its own launch and re-reads the matrix.

    ``v`` holds the vectors one after the other, ``N / 4`` words each -- what
    ``pack_fp8_tensor`` returns for a ``(batch, N)`` tensor; ``batch`` defaults
    to ``v.numel() // (N / 4)``.  Returns a float32 ``(batch, M)`` tensor."""
    with torch._C.DisableTorchFunctionSubclass():
        mode_id = _lib.mode_id(mode)
        m = as_words(m, "m")
        v = as_words(v, "v")
        if len(m_shape) != 2:
            raise ValueError("m_shape must be the unpacked (M, N) of the matrix")
        M, N = int(m_shape[0]), int(m_shape[1])
        if M < 0 or N < 0 or N % 4:
            raise ValueError("N must be a non-negative multiple of 4: rows are whole packed words")
        n_words = N // 4
        if batch is None:
            if n_words == 0 or v.numel() % n_words:
                raise ValueError("v must hold a whole number of N/4-word vectors (or pass batch=)")
            batch = v.numel() // n_words
        batch = int(batch)
        if not 0 <= batch <= 64:
            raise ValueError("batch must be between 0 and 64")
        if m.numel() < M * n_words:
            raise ValueError(f"m holds {m.numel()} words, {M}x{N} needs {M * n_words}")
        if v.numel() < batch * n_words:
            raise ValueError(f"v holds {v.numel()} words, {batch} vectors of N={N} need {batch * n_words}")
        if v.device != m.device:
            raise ValueError("m and v must be on the same device")
        if out is None:
            out = torch.empty((batch, M), dtype=torch.float32, device=m.device)
        elif (out.dtype != torch.float32 or out.numel() != batch * M or out.device != m.device
              or not out.is_contiguous()):
            raise ValueError("out must be a contiguous float32 tensor of batch * M elements on m's device")
        if M and batch:
            idx = m.device.index
            with torch.cuda.device(idx):
                _lib.check(_lib.load().feather_gemv_fp8_multi(
                    m.data_ptr(), v.data_ptr(), out.data_ptr(), M, N, batch, mode_id,
                    1 if static_matrix else 0, _lib.current_stream_ptr(idx)))
        return out


def _gemv(m, v, m_shape, mode, out, flags, out_mode_id=None, workspace=None):
    mode_id = _lib.mode_id(mode)
    m = as_words(m, "m")
    v = as_words(v, "v")
    if len(m_shape) != 2:
        raise ValueError("m_shape must be the unpacked (M, N) of the matrix")
    M, N = int(m_shape[0]), int(m_shape[1])
    if M < 0 or N < 0 or N % 4:
        raise ValueError("N must be a non-negative multiple of 4: rows are whole packed words")
    if m.numel() < M * (N // 4):
        raise ValueError(f"m holds {m.numel()} words, {M}x{N} needs {M * (N // 4)}")
    if v.numel() < N // 4:
        raise ValueError(f"v holds {v.numel()} words, N={N} needs {N // 4}")
    if v.device != m.device:
        raise ValueError("m and v must be on the same device")
    if out_mode_id is not None:
        return _gemv_packed(m, v, M, N, mode_id, out_mode_id, out, flags, workspace)
    if out is None:
        out = torch.empty((M,), dtype=torch.float32, device=m.device)
    elif (out.dtype != torch.float32 or out.numel() != M or out.device != m.device
          or not out.is_contiguous()):
        raise ValueError("out must be a contiguous float32 tensor of M elements on m's device")
    if M:
        fn = _lib.load().feather_gemv_fp8_ex
        idx = m.device.index
        if torch.cuda.current_device() == idx:
            _lib.check(fn(m.data_ptr(), v.data_ptr(), out.data_ptr(), M, N, mode_id, flags,
                          _lib.current_stream_ptr(idx)))
        else:
            with torch.cuda.device(idx):
                _lib.check(fn(m.data_ptr(), v.data_ptr(), out.data_ptr(), M, N, mode_id, flags,
                              _lib.current_stream_ptr(idx)))
    return out


def _gemv_packed(m, v, M, N, mode_id, out_mode_id, out, flags, workspace):
    n_words = (M + 3) // 4
    if out is None:
        out = torch.empty((n_words,), dtype=torch.uint32, device=m.device)
    else:
        out = as_words(out, "out")
        if out.numel() != n_words or out.device != m.device:
            raise ValueError("out must hold ceil(M / 4) packed words on m's device")
    if M:
        lib = _lib.load()
        idx = m.device.index
        with torch.cuda.device(idx):
            ws_ptr = None
            need = int(lib.feather_gemv_fp8_packed_workspace_bytes(M, N))
            if m.data_ptr() % 16:
                need = 4 * M  # unaligned rows take the word-load kernel, which does not encode
            if need:
                if workspace is None:
                    workspace = torch.empty((M,), dtype=torch.float32, device=m.device)
                elif (workspace.dtype != torch.float32 or workspace.numel() < M
                      or workspace.device != m.device or not workspace.is_contiguous()):
                    raise ValueError("workspace must be a contiguous float32 tensor of >= M elements")
                ws_ptr = workspace.data_ptr()
            _lib.check(lib.feather_gemv_fp8_packed(m.data_ptr(), v.data_ptr(), out.data_ptr(), ws_ptr,
                                                   M, N, mode_id, out_mode_id, flags,
                                                   _lib.current_stream_ptr(idx)))
    return out


def gemv_fp8_e5m2_acc_fp32_gpu(m: torch.Tensor, v: torch.Tensor, m_shape) -> torch.Tensor:
    """Drop-in for feather/routines/gemv.py:136-184."""
    return gemv_fp8_acc_fp32_gpu(m, v, m_shape, "E5M2")


def gemv_fp8_e4m3_acc_fp32_gpu(m: torch.Tensor, v: torch.Tensor, m_shape) -> torch.Tensor:
    """Drop-in for feather/routines/gemv.py:187-235 (kernel decode of
    gemv.py:83-88: exponent-0 codes are +-m * 2^-17, 0x7F/0xFF are +-480)."""
    return gemv_fp8_acc_fp32_gpu(m, v, m_shape, "E4M3")
