"""Multi-GPU GEMV: row-sharded (``RowShardedGemv``, below) and column-sharded
(``ColumnShardedGemv``: every rank holds a column block of all rows and the
matching slice of the vector, the partial row sums are all-reduced -- inside
the GEMV kernel through peer-mapped inboxes, or with the process group's
all-reduce).

Row-sharded GEMV
----------------

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
  peer-mapped memory (``feather_gemv_fp8_sharded_ex``), so the exchange
  overlaps the streaming of the matrix and there is no collective launch.
  ``op(v)`` returns when all slices have arrived; ``op(v, wait=False)`` ends
  the call as soon as this rank's rows are on their way and ``op.wait()``
  completes it later, so that the exchange latency and the skew between the
  ranks overlap whatever is enqueued in between (the next call, for one).  The
  buffers are shared between the ranks' processes with CUDA IPC.

One process per GPU over ``torch.distributed`` (NCCL on GPUs).  The local
compute is injectable so that the partition / gather plumbing can be tested
with the gloo backend on CPU ranks.
"""
from __future__ import annotations

import ctypes
from typing import Callable, List, Optional, Tuple

import torch
import torch.distributed as dist

__all__ = ["row_block", "local_words", "local_column_words", "local_vector_words", "RowShardedGemv",
           "PeerAllReduce", "ColumnShardedGemv"]


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


def _column_words(N: int, world_size: int, rank: int) -> Tuple[int, int]:
    """Words [begin, end) of a packed row (or of the packed vector) that hold
    rank's columns.  Column blocks are whole 16-byte chunks."""
    if world_size < 1 or not 0 <= rank < world_size:
        raise ValueError(f"bad rank {rank} for world size {world_size}")
    if N % (16 * world_size):
        raise ValueError(f"N={N} does not split into {world_size} blocks of whole 16-code chunks")
    words = N // world_size // 4
    return rank * words, (rank + 1) * words


def local_column_words(m_packed: torch.Tensor, m_shape, world_size: int, rank: int) -> torch.Tensor:
    """This rank's COLUMN block of a full packed matrix: columns
    ``[r*N/W, (r+1)*N/W)`` of every row, packed row-major (a copy: the block is
    strided in the full matrix)."""
    M, N = int(m_shape[0]), int(m_shape[1])
    begin, end = _column_words(N, world_size, rank)
    return m_packed.reshape(-1)[: M * (N // 4)].reshape(M, N // 4)[:, begin:end].contiguous().reshape(-1)


def local_vector_words(v_packed: torch.Tensor, N: int, world_size: int, rank: int) -> torch.Tensor:
    """The slice of the packed vector that goes with ``local_column_words`` (a view)."""
    begin, end = _column_words(int(N), world_size, rank)
    return v_packed.reshape(-1)[begin:end]


def _share_with_peers(shared: Optional[torch.Tensor], dev: torch.device, group, error=None):
    """Map every rank's ``shared`` buffer into this process (CUDA IPC).

    Collective over ``group``: every rank calls it, also a rank that already
    failed (``shared=None`` and its ``error``), so that nobody waits for a rank
    that gave up.  Returns ``(base, mapped, error)``: ``base[p]`` is the address
    of rank p's buffer here, ``mapped`` the (pointer, offset) pairs to hand to
    ``feather_ipc_close``; on failure ``error`` is the exception.
    """
    from . import _lib
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    payload = None
    if error is None:
        try:
            lib = _lib.load()
            with torch.cuda.device(dev):
                torch.cuda.synchronize(dev)
                handle = ctypes.create_string_buffer(64)
                offset = ctypes.c_int64(0)
                _lib.check(lib.feather_ipc_export(shared.data_ptr(), handle, ctypes.byref(offset)))
            payload = (handle.raw, int(offset.value), dev.index)
        except Exception as e:  # noqa: BLE001 - reported to the caller
            error = e
    gathered: List = [None] * world
    dist.all_gather_object(gathered, payload, group=group)
    if error is not None:
        return [], [], error
    base, mapped = [], []
    try:
        if any(g is None for g in gathered):
            raise RuntimeError("a peer rank could not share its buffer")
        with torch.cuda.device(dev):  # map with the device that runs the kernel current
            for r, (raw, off, peer_dev) in enumerate(gathered):
                if r == rank:
                    base.append(shared.data_ptr())
                    continue
                if not torch.cuda.can_device_access_peer(dev.index, peer_dev):
                    raise RuntimeError(f"GPU {dev.index} cannot access GPU {peer_dev} directly")
                _lib.check(lib.feather_enable_peer_access(peer_dev))
                ptr = ctypes.c_void_p(0)
                _lib.check(lib.feather_ipc_open(raw, off, ctypes.byref(ptr)))
                mapped.append((ptr.value, off))
                base.append(ptr.value)
    except Exception as e:  # noqa: BLE001
        return base, mapped, e
    return base, mapped, None


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

    static_matrix : promise that nothing in flight writes ``m_local`` (fused
        mode: the kernel starts streaming before its stream-order wait).

    The result of ``op(v)`` is the object's own buffer and stays valid until
    the next call on THIS rank is enqueued.  (In fused mode two buffers
    alternate, and a peer writes call k+2 into the buffer of call k only after
    every rank has delivered call k+1 -- which a rank does only once it has
    been launched for call k+1.)
    """

    def __init__(self, m_local: torch.Tensor, m_shape, mode: str = "E5M2",
                 group: Optional[dist.ProcessGroup] = None,
                 local_gemv: Optional[Callable] = None, fused: Optional[bool] = None,
                 static_matrix: bool = False):
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
        self.static_matrix = bool(static_matrix)
        self._pending = 0   # epoch of a fused call whose arrival wait has not been enqueued yet
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
        error = None
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
        except Exception as e:  # noqa: BLE001 - reported through the agreement step
            error = e
        base, self._mapped, error = _share_with_peers(
            None if error else self._shared, dev, self.group, error)
        if error is not None:
            return error
        try:
            lib = _lib.load()
            arr = ctypes.c_void_p * self.world_size
            self._out_ptrs = [arr(*[b + 4 * self.M * k for b in base]) for k in (0, 1)]
            self._flag_ptrs = arr(*[b + 4 * 2 * self.M for b in base])
            self._views = [self._shared[: self.M], self._shared[self.M: 2 * self.M]]
            self._lib, self._check = lib, _lib.check
            self._fn = lib.feather_gemv_fp8_sharded_ex
            self._wait_fn = lib.feather_gemv_fp8_sharded_wait
            self._stamps = None
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

    def _call_fused(self, v_packed: torch.Tensor, wait: bool) -> torch.Tensor:
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
                return self._launch_fused(v_ptr, k, idx, wait)
        return self._launch_fused(v_ptr, k, idx, wait)

    def _launch_fused(self, v_ptr: int, k: int, idx: int, wait: bool) -> torch.Tensor:
        flags = (1 if self.static_matrix else 0) | (0 if wait else 2)
        stamps = None if self._stamps is None else self._stamps.data_ptr()
        self._check(self._fn(self._m_ptr, v_ptr, self.rows, self.N, self._mode_id,
                             self._out_ptrs[k], self._flag_ptrs, self.rank, self.world_size,
                             (self._epoch & 0xFFFFFFFF) or 1, flags, stamps, self._stream_ptr(idx)))
        self._pending = 0 if wait else self._epoch
        return self._views[k]

    def wait(self) -> None:
        """Complete a call made with ``wait=False``: enqueue, on the current
        stream, the wait for all ranks' slices of the latest call.  Until then
        only this rank's own rows of the returned buffer are defined."""
        if not self.fused or not self._pending:
            return
        idx = self._dev_index
        with torch.cuda.device(idx):
            stamps = None if self._stamps is None else self._stamps.data_ptr()
            self._check(self._wait_fn(self._flag_ptrs, self.rank, self.world_size,
                                      (self._pending & 0xFFFFFFFF) or 1, stamps, self._stream_ptr(idx)))
        self._pending = 0

    def record_stamps(self, on: bool = True) -> None:
        """Have the kernels record the GPU timer of this rank's last CTA (rows
        pushed, epoch published, all epochs seen) into ``self.stamps()``."""
        self._stamps = (torch.zeros(3, dtype=torch.int64, device=self.m_local.device) if on else None)

    def stamps(self):
        torch.cuda.synchronize(self.m_local.device)
        return None if self._stamps is None else [int(x) for x in self._stamps.tolist()]

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

    def __call__(self, v_packed: torch.Tensor, wait: bool = True) -> torch.Tensor:
        """Full ``(M,)`` FP32 result on every rank.  The returned tensor is the
        object's own buffer and is valid until this rank's next call.
        ``wait=False`` (fused mode): see ``wait()``."""
        if self.fused:
            return self._call_fused(v_packed, wait)
        mine = self.local(v_packed)
        if self.world_size > 1:
            # in place: rank r's slice already sits at offset r * rows
            dist.all_gather_into_tensor(self.out, mine, group=self.group)
        return self.out


class PeerAllReduce:
    """Inbox and flag block for the all-reduce fused into column-sharded GEMVs.

    One object serves any number of ``ColumnShardedGemv`` operators, provided
    every rank calls them in the same order (the call counter lives in the flag
    block on the device, so a captured CUDA graph of calls can be replayed).
    ``max_rows`` is the largest M of those operators.  Collective: create it on
    every rank of ``group``; ``close()`` likewise.
    """

    def __init__(self, max_rows: int, device: Optional[torch.device] = None, group=None, n_ops: int = 1):
        """``n_ops`` > 1 sizes the inbox for a one-launch chain with that many
        all-reduced ops (``chain.PersistentGemvChain``); such a context serves
        that chain only."""
        from . import _lib
        if not dist.is_initialized():
            raise RuntimeError("torch.distributed is not initialised")
        self.group = group
        self.world_size, self.rank = dist.get_world_size(group), dist.get_rank(group)
        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.device, self.max_rows = dev, int(max_rows)
        error, self._mapped = None, []
        try:
            self._lib = _lib.load()
            if self.world_size > 16:
                raise ValueError("the fused all-reduce supports at most 16 ranks")
            # two halves x ops x world slots x (sum, tag) pairs for max_rows rounded up to 16
            self.n_ops = int(n_ops)
            self.inbox_floats = 2 * self.n_ops * self.world_size * 2 * ((self.max_rows + 15) // 16 * 16)
            # [inbox | flag block]
            self._shared = torch.zeros(self.inbox_floats + 32, dtype=torch.float32, device=dev)
        except Exception as e:  # noqa: BLE001 - every rank still takes part in the exchange below
            error = e
        base, self._mapped, error = _share_with_peers(None if error else self._shared, dev, group, error)
        ok = torch.tensor([int(error is None)], dtype=torch.int32, device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
        if not int(ok.item()):
            self.close(collective=False)
            raise RuntimeError(f"fused all-reduce not available: {error or 'a peer rank failed'}")
        arr = ctypes.c_void_p * self.world_size
        self.inbox_ptrs = arr(*base)
        self.flag_ptrs = arr(*[b + 4 * self.inbox_floats for b in base])

    def close(self, collective: bool = True) -> None:
        """Unmap the peers' buffers.  Call on every rank after the last result
        has been consumed and before the process group goes away."""
        if getattr(self, "_mapped", None):
            torch.cuda.synchronize(self.device)
            if collective:
                dist.barrier(group=self.group)  # nobody still writes into a buffer being unmapped
            with torch.cuda.device(self.device):
                for ptr, off in self._mapped:
                    self._lib.feather_ipc_close(ptr, off)
        self._mapped = []


class ColumnShardedGemv:
    """``y = A @ v`` with A's COLUMNS split over the ranks: rank r holds columns
    ``[r*N/W, (r+1)*N/W)`` of every row (packed row-major, row stride N/(4W)
    words; see ``local_column_words``) and is called with the matching slice of
    the packed vector.  Every rank's row sums are partial; the result is their
    sum, on every rank.

    * ``ctx`` given (a ``PeerAllReduce``): the partial sums are added inside the
      GEMV kernel through the ranks' peer-mapped inboxes
      (``feather_gemv_fp8_allreduce``): one launch per call, no collective, the
      same bits on every rank.
    * ``ctx=None``: local GEMV, then one all-reduce of the process group (NCCL
      on GPUs).  ``local_gemv`` -- ``(m_local, v_local, (M, N/W), mode, out) ->
      out`` -- replaces the CUDA kernel; tests on CPU ranks inject the oracle.

    ``m_shape`` is the LOCAL unpacked shape ``(M, N/W)``; N/W must be a
    multiple of 16.  The result is the object's own buffer.
    """

    def __init__(self, m_local: torch.Tensor, m_shape, mode: str, ctx: Optional[PeerAllReduce] = None,
                 out: Optional[torch.Tensor] = None, group: Optional[dist.ProcessGroup] = None,
                 local_gemv: Optional[Callable] = None):
        from . import _lib
        self.M, self.n_local = int(m_shape[0]), int(m_shape[1])
        if self.n_local % 16:
            raise ValueError("the local column count must be a multiple of 16")
        if m_local.numel() != self.M * (self.n_local // 4):
            raise ValueError(f"local block holds {m_local.numel()} words, {self.M}x{self.n_local} "
                             f"needs {self.M * (self.n_local // 4)}")
        self.m_local, self.ctx, self.mode = m_local, ctx, mode
        self._mode_id = _lib.mode_id(mode)
        self._n_words = self.n_local // 4
        if ctx is None and not dist.is_initialized():
            raise RuntimeError("torch.distributed is not initialised")
        self.group = ctx.group if ctx is not None else group
        self._check_agreement()
        if ctx is None:
            if local_gemv is None:
                from .routines.gemv import gemv_fp8_acc_fp32_gpu
                local_gemv = gemv_fp8_acc_fp32_gpu
            self._local_gemv = local_gemv
            self.out = (torch.empty(self.M, dtype=torch.float32, device=m_local.device)
                        if out is None else out)
            return
        if local_gemv is not None:
            raise ValueError("local_gemv cannot be combined with the fused all-reduce")
        from .packers.fp8 import as_words
        if self.M > ctx.max_rows:
            raise ValueError(f"M={self.M} exceeds the all-reduce inbox ({ctx.max_rows} rows)")
        words = as_words(m_local, "m_local")
        if words.device != ctx.device:
            raise ValueError("the matrix shard must live on the context's device")
        self.out = torch.empty(self.M, dtype=torch.float32, device=ctx.device) if out is None else out
        self._m_ptr, self._out_ptr = words.data_ptr(), self.out.data_ptr()
        self._fn, self._check = ctx._lib.feather_gemv_fp8_allreduce, _lib.check
        self._stream_ptr = _lib.current_stream_ptr

    def _check_agreement(self) -> None:
        """Every rank must hold a block of the same shape and format: the sums
        of blocks that differ would be added row by row all the same."""
        mine = torch.tensor([self.M, self.n_local, self._mode_id], dtype=torch.int64,
                            device=self.m_local.device)
        lo, hi = mine.clone(), mine.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN, group=self.group)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX, group=self.group)
        if not (torch.equal(lo, mine) and torch.equal(hi, mine)):
            raise ValueError(f"ranks disagree on the local block (M, N/W, mode): min {lo.tolist()} "
                             f"max {hi.tolist()} mine {mine.tolist()}")

    def __call__(self, v_local: torch.Tensor) -> torch.Tensor:
        ctx = self.ctx
        if ctx is None:
            self._local_gemv(self.m_local, v_local, (self.M, self.n_local), self.mode, out=self.out)
            if dist.get_world_size(self.group) > 1:
                dist.all_reduce(self.out, group=self.group)
            return self.out
        with torch._C.DisableTorchFunctionSubclass():
            if v_local.numel() < self._n_words or v_local.device != ctx.device:
                raise ValueError("v must hold the local N/4 packed words on this rank's device")
            v_ptr = v_local.data_ptr()
        idx = ctx.device.index
        if torch.cuda.current_device() != idx:
            with torch.cuda.device(idx):
                return self._launch(v_ptr, idx)
        return self._launch(v_ptr, idx)

    def _launch(self, v_ptr: int, idx: int) -> torch.Tensor:
        ctx = self.ctx
        self._check(self._fn(self._m_ptr, v_ptr, self._out_ptr, self.M, self.n_local, self._mode_id,
                             ctx.inbox_ptrs, ctx.inbox_floats, ctx.flag_ptrs, ctx.rank,
                             ctx.world_size, self._stream_ptr(idx)))
        return self.out
