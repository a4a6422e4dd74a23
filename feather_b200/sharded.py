"""Row-sharded multi-GPU GEMV.

The reference is single-GPU; this is the row split its GEMV admits: rows are
independent (feather/routines/gemv.py:17-18: one program per row, row stride
N/4 words), so rank r of W holds the contiguous packed rows
``[r*M/W, (r+1)*M/W)`` -- a contiguous slice of the flat packed tensor -- the
packed vector is replicated, every rank runs the single-GPU kernel on its
block, and the FP32 output slices are exchanged with one all-gather.

One process per GPU over ``torch.distributed`` (NCCL on GPUs).  The local
compute is injectable so that the partition / gather plumbing can be tested
with the gloo backend on CPU ranks.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

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
    """

    def __init__(self, m_local: torch.Tensor, m_shape, mode: str = "E5M2",
                 group: Optional[dist.ProcessGroup] = None,
                 local_gemv: Optional[Callable] = None):
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
        if local_gemv is None:
            from .routines.gemv import gemv_fp8_acc_fp32_gpu
            local_gemv = gemv_fp8_acc_fp32_gpu
        self._local_gemv = local_gemv
        self._check_agreement()
        self.out = torch.empty(self.M, dtype=torch.float32, device=m_local.device)

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
        mine = self.local(v_packed)
        if self.world_size > 1:
            # in place: rank r's slice already sits at offset r * rows
            dist.all_gather_into_tensor(self.out, mine, group=self.group)
        return self.out
