"""Row-sharded GEMV plumbing on CPU ranks (gloo, world size 2).

The CUDA kernel cannot run here, so the oracle GEMV is injected as the local
compute; what is tested is the partition, the agreement check, the in-place
gather and the error paths.
"""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_local_gemv(m_local, v_packed, shape, mode, out):
    from oracle import feather_oracle as O
    y = O.gemv(m_local.numpy().view(np.uint32), v_packed.numpy().view(np.uint32), shape, mode)
    out.copy_(torch.from_numpy(y))
    return out


def _worker(rank: int, world: int, port: int, case: str, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from feather_b200.sharded import RowShardedGemv, local_words
        from oracle import feather_oracle as O
        rng = np.random.default_rng(42)  # same data on every rank
        M, N, mode = 24, 520, "E4M3"
        A = rng.standard_normal((M, N)).astype(np.float16)
        v = rng.standard_normal(N).astype(np.float16)
        mw = torch.from_numpy(O.pack_fp8_ndarray(A, mode).view(np.int32))
        vw = torch.from_numpy(O.pack_fp8_ndarray(v, mode).view(np.int32))
        if case == "ok":
            op = RowShardedGemv(local_words(mw, (M, N), world, rank), (M, N), mode,
                                local_gemv=_oracle_local_gemv)
            y = op(vw)
            ref = O.gemv(mw.numpy().view(np.uint32), vw.numpy().view(np.uint32), (M, N), mode)
            q.put((rank, bool(np.array_equal(y.numpy(), ref)), op.row_begin, op.row_end))
        elif case == "columns":
            # column-sharded GEMV, non-fused path: oracle partial sums + gloo all-reduce
            from feather_b200.sharded import ColumnShardedGemv, local_column_words, local_vector_words
            Mc, Nc = 24, 64 * world
            Ac = rng.standard_normal((Mc, Nc)).astype(np.float16)
            vc = rng.standard_normal(Nc).astype(np.float16)
            mwc = torch.from_numpy(O.pack_fp8_ndarray(Ac, mode).view(np.int32))
            vwc = torch.from_numpy(O.pack_fp8_ndarray(vc, mode).view(np.int32))
            cols = Nc // world
            op = ColumnShardedGemv(local_column_words(mwc, (Mc, Nc), world, rank), (Mc, cols), mode,
                                   local_gemv=_oracle_local_gemv)
            y = op(local_vector_words(vwc, Nc, world, rank)).numpy().copy()
            # the same block taken from the unpacked matrix, packed on its own
            blk = O.pack_fp8_ndarray(np.ascontiguousarray(Ac[:, rank * cols:(rank + 1) * cols]), mode)
            same_block = np.array_equal(blk.view(np.uint32), op.m_local.numpy().view(np.uint32))
            parts = [O.gemv(O.pack_fp8_ndarray(np.ascontiguousarray(Ac[:, r * cols:(r + 1) * cols]), mode).view(np.uint32),
                            O.pack_fp8_ndarray(vc[r * cols:(r + 1) * cols], mode).view(np.uint32),
                            (Mc, cols), mode) for r in range(world)]
            ref = O.gemv(mwc.numpy().view(np.uint32), vwc.numpy().view(np.uint32), (Mc, Nc), mode, acc="f64")
            q.put((rank, bool(np.array_equal(y, sum(parts[1:], parts[0]))) and same_block,
                   O.normalised_error(y, ref) < 1e-5))
        elif case == "columns_disagree":
            # the ranks pass different row counts for the column split
            from feather_b200.sharded import ColumnShardedGemv
            Mc = 24 if rank == 0 else 16
            try:
                ColumnShardedGemv(mw[: Mc * 16], (Mc, 64), mode, local_gemv=_oracle_local_gemv)
                q.put((rank, "no error"))
            except ValueError as e:
                q.put((rank, "ValueError" if "disagree" in str(e) else str(e)))
        elif case == "bad_columns":
            from feather_b200.sharded import local_column_words
            try:
                local_column_words(mw, (M, 520), world, rank)   # 520 / 2 is not whole 16-code chunks
                q.put((rank, "no error"))
            except ValueError:
                q.put((rank, "ValueError"))
        elif case == "disagree":
            shape = (M, N) if rank == 0 else (M, N)
            mode_r = mode if rank == 0 else "E5M2"
            try:
                RowShardedGemv(local_words(mw, shape, world, rank), shape, mode_r,
                               local_gemv=_oracle_local_gemv)
                q.put((rank, "no error"))
            except ValueError as e:
                q.put((rank, "ValueError" if "disagree" in str(e) else str(e)))
        elif case == "wrong_block":
            try:
                RowShardedGemv(mw[:17], (M, N), mode, local_gemv=_oracle_local_gemv)
                q.put((rank, "no error"))
            except ValueError:
                q.put((rank, "ValueError"))
    finally:
        dist.destroy_process_group()


def _run(case: str, world: int = 2):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, case, q)) for r in range(world)]
    for p in procs:
        p.start()
    out = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    return sorted(out)


def _lonely_worker(port: int, q):
    """Rank 0 of a world of 2 whose peer never starts."""
    import datetime
    import time
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    t0 = time.time()
    try:
        dist.init_process_group("gloo", rank=0, world_size=2, timeout=datetime.timedelta(seconds=5))
        q.put(("no error", time.time() - t0))
        dist.destroy_process_group()
    except Exception as e:  # noqa: BLE001 - the kind of exception is torch's business
        q.put((type(e).__name__, time.time() - t0))


def test_rank_missing_at_rendezvous_raises_within_the_timeout():
    """A rank that never joins: the others get an exception after the
    rendezvous timeout instead of waiting forever (host-side failure; nothing
    runs on a GPU)."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    p = ctx.Process(target=_lonely_worker, args=(_free_port(), q))
    p.start()
    kind, seconds = q.get(timeout=120)
    p.join(timeout=60)
    assert kind != "no error" and seconds < 60


def test_column_sharded_ranks_that_disagree_raise():
    assert _run("columns_disagree") == [(0, "ValueError"), (1, "ValueError")]


def test_row_sharded_gemv_matches_single_rank():
    res = _run("ok")
    assert res == [(0, True, 0, 12), (1, True, 12, 24)]


def test_ranks_that_disagree_raise():
    assert _run("disagree") == [(0, "ValueError"), (1, "ValueError")]


def test_wrong_local_block_raises():
    assert _run("wrong_block") == [(0, "ValueError"), (1, "ValueError")]


def test_row_block_partition():
    from feather_b200.sharded import row_block
    assert [row_block(65536, 8, r) for r in (0, 7)] == [(0, 8192), (57344, 65536)]
    with pytest.raises(ValueError):
        row_block(10, 4, 0)      # not divisible
    with pytest.raises(ValueError):
        row_block(8, 4, 4)       # rank out of range


def test_column_sharded_partition_and_all_reduce_world_2():
    assert _run("columns") == [(0, True, True), (1, True, True)]


def test_column_sharded_rejects_ragged_split():
    assert _run("bad_columns") == [(0, "ValueError"), (1, "ValueError")]
