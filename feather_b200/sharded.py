"""Row-sharded multi-GPU GEMV.

The reference is single-GPU; this is the row split its GEMV admits: rows are
independent (feather/routines/gemv.py:17-18: one program per row, row stride
N/4 words), so rank r of W holds the contiguous packed rows
``[r*M/W, (r+1)*M/W)`` -- a contiguous slice of the flat packed tensor -- the
packed vector is replicated, every rank runs the single-GPU kernel on its
block, and the FP32 output slices are exchanged with one all-gather.

Two exchange paths:

* ``fused=False``: local GEMV into the rank's slice, then one in-place NCCL
  all-gather.
* ``fused=True`` (default on GPUs when the shape allows it): the GEMV kernel
  itself stores every finished row into all ranks' output buffers through
  peer-mapped memory (``feather_gemv_fp8_sharded``), so the exchange overlaps
  the streaming of the matrix and costs one NVLink round trip at the end
  instead of a collective launch.  The buffers are shared between the ranks'
  processes with CUDA IPC (torch's own tensor sharing).

One process per GPU over ``torch.distributed`` (NCCL on GPUs).  The local
compute is injectable so that the partition / gather plumbing can be tested
with the gloo backend on CPU ranks.
"""
from __future__ import annotations

import ctypes
from typing import Callable, List, Optional, Tuple

import torch
import torch.distributed as dist

__all__ = ["row_block", "local_words", "RowShardedGemv"]


def row_block(M: int, world_size: int, rank: int) -> Tuple[int, int]:
    """Rows [begin, end) owned by ``rank``.  M must divide evenly: the gather
    exchanges equal slices."""
    if world_size < 1 or not 0 <= rank < world_size:
        raise ValueError(f"bad rank {rank} for world size {world_size}")
    if M % world_size:
        raise ValueError(f"M={M} is not divisible by the number of ranks {world_size}")
    rows = M // world_size
    return rank * rows, (rank + 1) * rows


def local_words(m_packed: torch.Tensor, m_shape, world_size: int, rank: int) -> torch.Tensor:
    """This rank's slice of a FULL packed matrix (a view, no copy)."""
    M, N = int(m_shape[0]), int(m_shape[1])
    if N % 4:
        raise ValueError("N must be a multiple of 4")
    begin, end = row_block(M, world_size, rank)
    return m_packed.reshape(-1)[begin * (N // 4): end * (N // 4)]


class RowShardedGemv:
    """``y = A @ v`` with A's packed rows split over the ranks of a process group.

    Parameters
    ----------
    m_local : packed words of this rank's rows, ``(M/W) * N/4`` words.
    m_shape : the GLOBAL unpacked shape (M, N).
    mode    : "E5M2" or "E4M3".
    group   : process group (default: the world group).
    local_gemv : callable ``(m_local, v_packed, (rows, N), mode, out) -> out``;
        defaults to the CUDA kernel.  Tests on CPU ranks inject the oracle.
    fused   : True = exchange inside the kernel (raises if impossible), False =
        NCCL all-gather, None = fused when the operands are on GPUs, the world
        has more than one rank and the kernel supports the shape.

    The result of ``op(v)`` is the object's own buffer.  In fused mode two
    buffers alternate, so a result stays valid until the call after the next.
    """

    def __init__(self, m_local: torch.Tensor, m_shape, mode: str = "E5M2",
                 group: Optional[dist.ProcessGroup] = None,
                 local_gemv: Optional[Callable] = None, fused: Optional[bool] = None):
        if not dist.is_initialized():
            raise RuntimeError("torch.distributed is not initialised")
        self.group = group
        self.world_size = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.M, self.N = int(m_shape[0]), int(m_shape[1])
        if self.N % 4:
            raise ValueError("N must be a multiple of 4")
        self.row_begin, self.row_end = row_block(self.M, self.world_size, self.rank)
        self.rows = self.row_end - self.row_begin
        need = self.rows * (self.N // 4)
        if m_local.numel() != need:
            raise ValueError(f"rank {self.rank}: local block holds {m_local.numel()} words, "
                             f"{self.rows}x{self.N} needs {need}")
        self.m_local = m_local
        self.mode = mode
        custom_compute = local_gemv is not None
        if local_gemv is None:
            from .routines.gemv import gemv_fp8_acc_fp32_gpu
            local_gemv = gemv_fp8_acc_fp32_gpu
        self._local_gemv = local_gemv
        self._check_agreement()
        self.out = torch.empty(self.M, dtype=torch.float32, device=m_local.device)
        self.fused = False
        self._epoch = 0
        want = fused
        if want is None:
            want = (not custom_compute) and m_local.is_cuda and self.world_size > 1
        error = None
        if want:
            # Every rank runs the same sequence of collectives whatever fails locally.
            error = self._setup_fused()
        # all ranks must take the same path, or they would wait on each other
        agree = torch.tensor([int(want and error is None)], dtype=torch.int32, device=m_local.device)
        dist.all_reduce(agree, op=dist.ReduceOp.MIN, group=self.group)
        self.fused = bool(int(agree.item()))
        if fused and not self.fused:
            raise RuntimeError(f"fused exchange requested but not available: {error or 'a peer rank failed'}")

    # ------------------------------------------------------------ fused path --
    def _setup_fused(self):
        """Allocate the shared buffers and map every peer's.  Returns None on
        success or the exception that makes the fused path unusable here."""
        from . import _lib
        from .packers.fp8 import as_words
        dev = self.m_local.device
        error, payload = None, None
        try:
            lib = _lib.load()
            if self.world_size > 16:
                raise ValueError("fused exchange supports at most 16 ranks")
            as_words(self.m_local, "m_local")
            with torch.cuda.device(dev):
                if not lib.feather_gemv_fp8_sharded_supported(self.rows, self.N):
                    raise ValueError(f"{self.rows}x{self.N} per rank is outside the fused kernel's range")
                # [two output buffers | flag block]: one allocation per rank, exported by CUDA IPC
                self._shared = torch.zeros(2 * self.M + 32, dtype=torch.float32, device=dev)
                torch.cuda.synchronize(dev)
                handle = ctypes.create_string_buffer(64)
                offset = ctypes.c_int64(0)
                _lib.check(lib.feather_ipc_export(self._shared.data_ptr(), handle, ctypes.byref(offset)))
            payload = (handle.raw, int(offset.value), dev.index)
        except Exception as e:  # noqa: BLE001 - reported through the agreement step
            error = e
        gathered: List = [None] * self.world_size
        dist.all_gather_object(gathered, payload, group=self.group)
        if error is not None:
            return error
        try:
            if any(g is None for g in gathered):
                raise RuntimeError("a peer rank could not share its buffer")
            base, self._mapped = [], []
            with torch.cuda.device(dev):  # map with the device that runs the kernel current
                for r, (raw, off, peer_dev) in enumerate(gathered):
                    if r == self.rank:
                        base.append(self._shared.data_ptr())
                        continue
                    if not torch.cuda.can_device_access_peer(dev.index, peer_dev):
                        raise RuntimeError(f"GPU {dev.index} cannot access GPU {peer_dev} directly")
                    _lib.check(lib.feather_enable_peer_access(peer_dev))
                    mapped = ctypes.c_void_p(0)
                    _lib.check(lib.feather_ipc_open(raw, off, ctypes.byref(mapped)))
                    self._mapped.append((mapped.value, off))
                    base.append(mapped.value)
            arr = ctypes.c_void_p * self.world_size
            self._out_ptrs = [arr(*[b + 4 * self.M * k for b in base]) for k in (0, 1)]
            self._flag_ptrs = arr(*[b + 4 * 2 * self.M for b in base])
            self._views = [self._shared[: self.M], self._shared[self.M: 2 * self.M]]
            self._lib, self._check = lib, _lib.check
            self._fn = lib.feather_gemv_fp8_sharded
            self._m_ptr = self.m_local.data_ptr()
            self._n_words = self.N // 4
            self._dev, self._dev_index = dev, dev.index
            self._mode_id = _lib.mode_id(self.mode)
            self._stream_ptr = _lib.current_stream_ptr
            torch.cuda.synchronize(dev)
        except Exception as e:  # noqa: BLE001
            return e
        return None

    def close(self) -> None:
        """Unmap the peers' buffers (fused mode).  Call on every rank, after the
        last result has been consumed and before the process group goes away."""
        if getattr(self, "_mapped", None):
            torch.cuda.synchronize(self.m_local.device)
            dist.barrier(group=self.group)  # nobody is still writing into a buffer being unmapped
            with torch.cuda.device(self.m_local.device):
                for ptr, off in self._mapped:
                    self._lib.feather_ipc_close(ptr, off)
            self._mapped = []
            self.fused = False

    def _call_fused(self, v_packed: torch.Tensor) -> torch.Tensor:
        # hot path: everything that does not change between calls was prepared in
        # _setup_fused; operands may be PackedFP8 subclasses, so metadata reads
        # skip the Python-level __torch_function__ dispatch
        with torch._C.DisableTorchFunctionSubclass():
            if v_packed.numel() < self._n_words or v_packed.device != self._dev:
                raise ValueError("v must hold N/4 packed words on this rank's device")
            v_ptr = v_packed.data_ptr()
        self._epoch += 1
        k = self._epoch & 1
        idx = self._dev_index
        if torch.cuda.current_device() != idx:
            with torch.cuda.device(idx):
                return self._launch_fused(v_ptr, k, idx)
        return self._launch_fused(v_ptr, k, idx)

    def _launch_fused(self, v_ptr: int, k: int, idx: int) -> torch.Tensor:
        self._check(self._fn(self._m_ptr, v_ptr, self.rows, self.N, self._mode_id,
                             self._out_ptrs[k], self._flag_ptrs, self.rank, self.world_size,
                             (self._epoch & 0xFFFFFFFF) or 1, self._stream_ptr(idx)))
        return self._views[k]

    def _check_agreement(self) -> None:
        """Every rank must describe the same global problem."""
        mine = torch.tensor([self.M, self.N, {"E5M2": 0, "E4M3": 1}.get(self.mode, -1)],
                            dtype=torch.int64, device=self.m_local.device)
        lo, hi = mine.clone(), mine.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN, group=self.group)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX, group=self.group)
        if not (torch.equal(lo, mine) and torch.equal(hi, mine)):
            raise ValueError(f"rank {self.rank}: ranks disagree on (M, N, mode): "
                             f"min {lo.tolist()} max {hi.tolist()} mine {mine.tolist()}")

    def local(self, v_packed: torch.Tensor) -> torch.Tensor:
        """This rank's output rows, written into its slice of the full buffer."""
        mine = self.out[self.row_begin:self.row_end]
        self._local_gemv(self.m_local, v_packed, (self.rows, self.N), self.mode, out=mine)
        return mine

    def __call__(self, v_packed: torch.Tensor) -> torch.Tensor:
        """Full ``(M,)`` FP32 result on every rank.  The returned tensor is the
        object's own buffer and is overwritten by the next call."""
        if self.fused:
            return self._call_fused(v_packed)
        mine = self.local(v_packed)
        if self.world_size > 1:
            # in place: rank r's slice already sits at offset r * rows
            dist.all_gather_into_tensor(self.out, mine, group=self.group)
        return self.out
