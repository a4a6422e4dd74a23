"""Row-sharded GEMV on real GPUs (NCCL).  World size 1 always runs; world
sizes 2, 4 and 8 run when the box has that many GPUs."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    try:
        dist.init_process_group("nccl", rank=rank, world_size=world,
                                device_id=torch.device("cuda", rank))
    except Exception as e:  # e.g. the rendezvous port was taken: report, do not stall the parent
        q.put((rank, "init failed", repr(e)))
        return
    try:
        import feather_b200 as fb
        from feather_b200.sharded import RowShardedGemv, local_words
        from oracle import c_oracle as C
        from oracle import feather_oracle as O
        M, N, mode = 4736 * world, 8192, "E4M3"   # 4736 rows per rank: the ring kernel
        gen = torch.Generator(device="cuda").manual_seed(77)  # same data on every rank
        A = torch.randn(M, N, device="cuda", generator=gen, dtype=torch.float16)
        v = torch.randn(N, device="cuda", generator=gen, dtype=torch.float16)
        mw, vw = fb.pack_fp8_tensor(A, mode), fb.pack_fp8_tensor(v, mode)
        y_single = fb.gemv_fp8_acc_fp32_gpu(mw, vw, (M, N), mode)
        host = lambda t: t.view(torch.int32).cpu().numpy().view(np.uint32)
        ref = C.gemv(host(mw), host(vw), (M, N), mode, acc="f64")
        ok_bits, ok_err, modes = True, True, []
        for fused in ((False, True) if world > 1 else (False,)):
            op = RowShardedGemv(local_words(mw, (M, N), world, rank), (M, N), mode, fused=fused)
            modes.append(op.fused)
            for it in range(3):  # several calls: the fused path alternates buffers and counts epochs
                y = op(vw).clone()
                torch.cuda.synchronize()
                # rows never interact, so the sharded result has the single-GPU bits
                ok_bits &= bool(torch.equal(y, y_single))
                ok_err &= O.normalised_error(y.cpu().numpy(), ref) < 1e-5
            if op.fused:
                # split-phase: calls that do not wait for the peers' slices, back to back, then
                # one wait; each result is checked after the wait that completes it
                for it in range(5):
                    y = op(vw, wait=False)
                    if it % 2 == 0:
                        op.wait()
                        ok_bits &= bool(torch.equal(y, y_single))
                op.wait()
                ok_bits &= bool(torch.equal(y, y_single))
                # a different vector through the same buffers: no stale rows survive
                v2 = fb.pack_fp8_tensor(torch.randn(N, device="cuda", generator=gen, dtype=torch.float16), mode)
                y2 = op(v2, wait=False)
                op.wait()
                ok_bits &= bool(torch.equal(y2, fb.gemv_fp8_acc_fp32_gpu(mw, v2, (M, N), mode)))
                # the static-matrix variant
                op_s = RowShardedGemv(local_words(mw, (M, N), world, rank), (M, N), mode, fused=True,
                                      static_matrix=True)
                ok_bits &= bool(torch.equal(op_s(vw), y_single))
                op_s.close()
            fb.device_status()
        # tensor-parallel GEMV chain (one layer + lm_head) against the single-GPU chain
        from feather_b200 import chain
        tp = chain.TensorParallelChain(layers=1)
        single = chain.GemvChain(layers=1)
        tp.token(); single.token()
        torch.cuda.synchronize()
        ok_tp = len(tp.ops) == len(single.ops) == 8
        for (kind, _, _, shape, out_tp), (_, _, (m, n), out_1) in zip(tp.ops, single.ops):
            ref1 = out_1 if kind == "cols" else out_1[rank * shape[0]:(rank + 1) * shape[0]]
            ok_tp &= O.normalised_error(out_tp.cpu().numpy(), ref1.cpu().numpy()) < 1e-5
        ok_ar = True
        if world > 1:
            ok_ar = _check_fused_allreduce(rank, world, single)
            ok_ar &= _check_fused_allreduce(rank, world, single, persistent=True)
        q.put((rank, ok_bits and ok_tp and ok_ar and modes == ([False, True] if world > 1 else [False]),
               ok_err))
    except Exception as e:
        q.put((rank, "failed", repr(e)))
    finally:
        dist.destroy_process_group()


def _check_fused_allreduce(rank: int, world: int, single, persistent: bool = False) -> bool:
    """Column-sharded GEMVs with the all-reduce inside the kernel: equal to the
    partial sums added in rank order, the same bits on every rank, close to the
    single-GPU chain, over several calls (both inbox halves) and under CUDA
    graph replay (the call counter lives on the device).  ``persistent``: the
    rank's whole token as ONE launch, the all-reduces inside it."""
    import feather_b200 as fb
    from feather_b200 import chain
    from oracle import feather_oracle as O
    tp = chain.TensorParallelChain(layers=1, fused_allreduce=True, persistent=persistent)
    ok = tp.fused_allreduce
    fused = [(op, a, shape, out) for kind, op, a, shape, out in tp.ops if kind == "fused"]
    if persistent:   # the entries hold the packed shard itself, not an operator object
        class _Shard:
            def __init__(self, m):
                self.m_local = m
        fused = [(_Shard(op), a, shape, out) for op, a, shape, out in fused]
    refs = [single.ops[i][3] for i, (name, _, _) in enumerate(chain.LAYER_SHAPES) if name in ("o", "down")]
    ok &= len(fused) == len(refs) == 2
    expected = []
    for op, a, shape, out in fused:
        part = fb.gemv_fp8_acc_fp32_gpu(op.m_local, a, shape, tp.mode)
        parts = [torch.empty_like(part) for _ in range(world)]
        dist.all_gather(parts, part)
        total = parts[0].clone()
        for p in parts[1:]:
            total += p
        expected.append(total)

    def verify() -> bool:
        torch.cuda.synchronize()
        good = True
        for (op, a, shape, out), want, ref1 in zip(fused, expected, refs):
            good &= bool(torch.equal(out, want))
            good &= O.normalised_error(out.cpu().numpy(), ref1.cpu().numpy()) < 1e-5
            out.zero_()
        return good

    for _ in range(3):  # odd number of calls per op in total: both inbox halves, shifting parity
        tp.token()
        ok &= verify()
    stream, graph = torch.cuda.Stream(), torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        tp.token()
        torch.cuda.synchronize()
        with torch.cuda.graph(graph, stream=stream):
            tp.token()
    ok &= verify()  # capture does not run the kernels; the warm-up call above did
    for _ in range(3):
        graph.replay()
        ok &= verify()
    if persistent:   # the row-split ops of the same launch, against the single-GPU chain
        tp.token()
        torch.cuda.synchronize()
        for (kind, _, _, shape, out_tp), (_, _, _, out_1) in zip(tp.ops, single.ops):
            if kind == "rows":
                ok &= O.normalised_error(out_tp.cpu().numpy(),
                                         out_1[rank * shape[0]:(rank + 1) * shape[0]].cpu().numpy()) < 1e-5
    fb.device_status()
    tp.close()
    return bool(ok)


def _run(world: int):
    ctx = mp.get_context("spawn")
    for attempt in range(3):  # a rendezvous port can be taken between probing and binding
        q = ctx.Queue()
        port = _free_port()
        procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
        for p in procs:
            p.start()
        out = [q.get(timeout=420) for _ in range(world)]
        for p in procs:
            p.join(timeout=60)
        if any(o[1] == "init failed" for o in out) and attempt < 2:
            continue
        return sorted(out)


def test_row_sharded_world_1():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    assert _run(1) == [(0, True, True)]


@pytest.mark.parametrize("world", [2, 4, 8])
def test_row_sharded_world_n(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    assert _run(world) == [(r, True, True) for r in range(world)]
