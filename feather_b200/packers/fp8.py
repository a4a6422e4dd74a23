"""FP8 packers: the reference's ``feather.packers.fp8`` surface on the GPU.

``pack_fp8_tensor`` keeps the reference signature and result layout
(feather/packers/fp8.py:260-281: flatten, four codes per little-endian uint32,
zero-padded tail, 1-D ``torch.uint32``), but the encode runs as a CUDA kernel
(``feather_encode_fp8``) that is bit-exact with the reference's ml_dtypes
cast.  Differences allowed by the port:

* a CUDA input returns a CUDA tensor (the reference always returns a CPU
  tensor; the ``.cuda()`` the reference's users append is then a no-op);
* a CPU input is copied to the current CUDA device, encoded there, and the
  words are copied back, so the return device matches the reference's.  Without
  a CUDA device this raises: there is no CPU encoder in this package;
* dtypes other than float16/float32 raise ``TypeError`` (the reference logs a
  warning for non-fp16 and fails inside numpy for bfloat16).
"""
from __future__ import annotations

import torch

from .. import _lib

__all__ = ["PackedFP8", "pack_fp8_tensor", "unpack_fp8_tensor"]


class PackedFP8(torch.Tensor):
    """A packed-words tensor that remembers its FP8 mode.

    The README-level ``feather.gemv`` of the reference takes no mode argument,
    so the packer's result carries it (``.feather_mode``) through ``.cuda()``,
    ``.to()``, ``.view()`` and ``.contiguous()``.  It is an ordinary uint32
    tensor in every other respect.
    """

    feather_mode = None

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        out = super().__torch_function__(func, types, args, kwargs or {})
        if isinstance(out, PackedFP8) and out.feather_mode is None:
            for a in args:
                mode = getattr(a, "feather_mode", None)
                if mode is not None:
                    out.feather_mode = mode
                    break
        return out


def _tag(words: torch.Tensor, mode: str) -> torch.Tensor:
    t = words.as_subclass(PackedFP8)
    t.feather_mode = mode
    return t


def _require_cuda() -> None:
    if not torch.cuda.is_available():
        raise RuntimeError("feather_b200 needs a CUDA device (B200); there is no CPU path")


def pack_fp8_tensor(x: torch.Tensor, mode: str = "E5M2") -> torch.Tensor:
    """Pack a float16/float32 tensor of any shape into FP8 words.

    Mirrors feather/packers/fp8.py:260-281.  Returns a 1-D ``torch.uint32``
    tensor of ``ceil(x.numel() / 4)`` words on ``x``'s device.
    """
    mode_id = _lib.mode_id(mode)  # NotImplementedError for unknown modes
    if not isinstance(x, torch.Tensor):
        raise TypeError("pack_fp8_tensor expects a torch.Tensor")
    if x.dtype == torch.float16:
        src_dtype = _lib.SRC_F16
    elif x.dtype == torch.float32:
        src_dtype = _lib.SRC_F32
    else:
        raise TypeError(f"pack_fp8_tensor supports float16 and float32, got {x.dtype}")
    _require_cuda()
    lib = _lib.load()
    on_cpu = not x.is_cuda
    xd = x.cuda() if on_cpu else x
    xd = xd.reshape(-1).contiguous()
    n = xd.numel()
    words = torch.empty((n + 3) // 4, dtype=torch.int32, device=xd.device)
    if n:
        with torch.cuda.device(xd.device):
            stream = torch.cuda.current_stream().cuda_stream
            _lib.check(lib.feather_encode_fp8(xd.data_ptr(), src_dtype, words.data_ptr(), n,
                                              mode_id, stream))
    words = words.view(torch.uint32)
    if on_cpu:
        words = words.cpu()
    return _tag(words, mode)


def unpack_fp8_tensor(words: torch.Tensor, mode: str = "E5M2", semantics: str = "kernel",
                      n_elems: int | None = None) -> torch.Tensor:
    """Decode packed words to float32 on the GPU (``feather_decode_fp8``).

    ``semantics="kernel"`` gives the values the GEMV / dot kernels multiply
    with (feather/routines/gemv.py:31-34, 83-88); ``"ieee"`` gives what the
    reference CPU unpacker returns (feather/packers/fp8.py:336-432).
    """
    mode_id = _lib.mode_id(mode)
    sem = {"kernel": _lib.DECODE_KERNEL, "ieee": _lib.DECODE_IEEE}.get(semantics)
    if sem is None:
        raise ValueError(f"unknown semantics {semantics!r}")
    w = as_words(words, "words")
    n = w.numel() * 4 if n_elems is None else int(n_elems)
    if n < 0 or n > w.numel() * 4:
        raise ValueError("n_elems exceeds the packed length")
    out = torch.empty(n, dtype=torch.float32, device=w.device)
    if n:
        with torch.cuda.device(w.device):
            stream = torch.cuda.current_stream().cuda_stream
            _lib.check(_lib.load().feather_decode_fp8(w.data_ptr(), out.data_ptr(), n, mode_id,
                                                      sem, stream))
    return out


_WORD_DTYPES = (torch.uint32, torch.int32, torch.float32)


def as_words(t: torch.Tensor, name: str) -> torch.Tensor:
    """Validate a packed operand: CUDA, contiguous, 4-byte words.

    uint32 is what the packer returns; int32 and the float32 view
    (feather/packers/fp8.py:135) are what the reference's benchmarks pass.
    """
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor: feather_b200 has no CPU path")
    if t.dtype not in _WORD_DTYPES:
        raise ValueError(f"{name} must hold packed 32-bit words (uint32/int32/float32), got {t.dtype}")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    return t
