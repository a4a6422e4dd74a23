"""TinyLlama-1.1B-shaped batch-1 decode GEMV chain on packed-FP8 weights.

The architecture's matrix shapes only (22 layers, hidden 2048, intermediate
5632 with SwiGLU, 32 query heads / 4 KV heads of dimension 64, vocabulary
32000); weights are random N(0, 0.02) packed E4M3, activations random N(0, 1)
packed E4M3.  One "token" runs, per layer, the q/k/v/o and gate/up/down GEMVs
and finally the lm_head GEMV through ``feather_b200.gemv`` -- 155 GEMVs that
read 1.03 GB of weights.  There is no attention, normalisation or sampling:
this measures the GEMV path only.  The reference has no such driver; it is the
batch-1 use its README motivates (feather README.md:5-21).

    python -m feather_b200.chain [--tokens 50] [--no-graph]
"""
from __future__ import annotations

import argparse

import torch

import feather_b200 as fb

HIDDEN, INTER, VOCAB, LAYERS = 2048, 5632, 32000, 22
KV_DIM = 4 * 64
#: (name, rows M, cols N) of the GEMVs of one layer
LAYER_SHAPES = (("q", HIDDEN, HIDDEN), ("k", KV_DIM, HIDDEN), ("v", KV_DIM, HIDDEN),
                ("o", HIDDEN, HIDDEN), ("gate", INTER, HIDDEN), ("up", INTER, HIDDEN),
                ("down", HIDDEN, INTER))


def weight_bytes() -> int:
    per_layer = sum(m * n for _, m, n in LAYER_SHAPES)
    return LAYERS * per_layer + VOCAB * HIDDEN


class GemvChain:
    """Weights, activations and output buffers of the chain; ``token()`` enqueues
    the 155 GEMVs of one token on the current stream."""

    def __init__(self, mode: str = "E4M3", seed: int = 6, device: str = "cuda",
                 layers: int = LAYERS, static_matrix: bool = True, merge_projections: bool = False,
                 reencode: str | None = None):
        """``reencode``: None = FP32 results only; "fused" = every GEMV writes its
        result as packed FP8 words from its own epilogue (``gemv_fp8_ret_packed_gpu``);
        "separate" = FP32 result, then the packer as a second launch."""
        if reencode not in (None, "fused", "separate"):
            raise ValueError("reencode must be None, 'fused' or 'separate'")
        gen = torch.Generator(device=device).manual_seed(seed)
        self.mode = mode
        self.static_matrix = static_matrix
        self.reencode = reencode
        self.packed = []  # per op: the packed-output buffer
        self.names = []   # per op: q, k, v, o, gate, up, down (or qkv, gate_up), lm_head
        self.ops = []  # (packed weights, packed activation, (M, N), out)
        acts = {}
        for n in (HIDDEN, INTER):
            a = torch.randn(n, device=device, generator=gen, dtype=torch.float16)
            acts[n] = fb.pack_fp8_tensor(a, mode)

        def add(m: int, n: int, name: str) -> None:
            w = (0.02 * torch.randn(m, n, device=device, generator=gen)).to(torch.float16)
            self.names.append(name)
            self.ops.append((fb.pack_fp8_tensor(w, mode), acts[n], (m, n),
                             torch.empty(m, dtype=torch.float32, device=device)))
            self.packed.append(torch.empty((m + 3) // 4, dtype=torch.uint32, device=device))
        # merge_projections: q/k/v share their input vector, and so do gate/up, so
        # each group is ONE GEMV over the row-concatenated weights (same results,
        # 89 instead of 155 launches per token)
        shapes = LAYER_SHAPES if not merge_projections else (
            ("qkv", HIDDEN + 2 * KV_DIM, HIDDEN), ("o", HIDDEN, HIDDEN),
            ("gate_up", 2 * INTER, HIDDEN), ("down", HIDDEN, INTER))
        for _ in range(layers):
            for name, m, n in shapes:
                add(m, n, name)
        add(VOCAB, HIDDEN, "lm_head")
        torch.cuda.synchronize()  # weights are final before any static_matrix GEMV runs

    def token(self) -> None:
        if self.reencode == "fused":
            for (w, a, shape, _), words in zip(self.ops, self.packed):
                fb.gemv_fp8_ret_packed_gpu(w, a, shape, self.mode, out=words,
                                           static_matrix=self.static_matrix)
            return
        for (w, a, shape, out), words in zip(self.ops, self.packed):
            fb.gemv_fp8_acc_fp32_gpu(w, a, shape, self.mode, out=out,
                                     static_matrix=self.static_matrix)
            if self.reencode == "separate":  # the packer's kernel on the FP32 result
                lib, idx = fb._lib.load(), out.device.index
                fb._lib.check(lib.feather_encode_fp8(out.data_ptr(), fb._lib.SRC_F32, words.data_ptr(),
                                                     out.numel(), fb._lib.mode_id(self.mode),
                                                     fb._lib.current_stream_ptr(idx)))

    def bytes_per_token(self) -> int:
        return sum(m * n + n + 4 * m for _, _, (m, n), _ in self.ops)


class PersistentGemvChain:
    """A table of GEMVs run by ONE persistent kernel launch
    (``feather_gemv_chain_fp8``): the matrix stream does not stop at the op
    boundaries, which is what the 155 separate launches of ``GemvChain`` pay for.

    ``ops`` is a list of dicts with keys ``m`` (packed matrix), ``v`` (packed
    vector), ``shape`` (unpacked (M, N)), optional ``mode`` (default the
    chain's), ``out`` (float32 (M,) tensor, or packed words with ``out_mode``),
    ``out_mode`` (None = FP32 sums, else "E5M2"/"E4M3": the sums re-encoded,
    bit for bit ``gemv_fp8_ret_packed_gpu``) and ``wait_op`` (index of the
    earlier op that writes ``v``).  Missing outputs are allocated.  Every op's
    result has the bits of the single-op call on the same operands.

    Tensor-parallel use (one process per GPU): ops with ``allreduce=True`` are
    column-sharded -- ``m`` is this rank's column block, ``shape`` its LOCAL
    (M, N/W), ``v`` the matching slice -- and their outputs are the sums over
    the ranks, exchanged inside the kernel through ``ctx``, a
    ``sharded.PeerAllReduce`` created with ``n_ops`` = the number of such ops.
    """

    def __init__(self, ops, mode: str = "E4M3", static_matrix: bool = True, ctx=None):
        import ctypes
        from ._lib import ChainOp
        from .packers.fp8 import as_words
        if not ops:
            raise ValueError("the chain needs at least one op")
        self.lib = fb._lib.load()
        self.static_matrix = static_matrix
        self.outs, self._keep = [], []
        self.specs = []   # per op: (matrix, vector, (M, N), mode, out_mode) as given
        table = (ChainOp * len(ops))()
        device = None
        for i, op in enumerate(ops):
            m, v = as_words(op["m"], "m"), as_words(op["v"], "v")
            M, N = int(op["shape"][0]), int(op["shape"][1])
            device = m.device if device is None else device
            if m.device != device or v.device != device:
                raise ValueError("all operands of a chain live on one device")
            if m.numel() < M * (N // 4) or v.numel() < N // 4:
                raise ValueError(f"op {i}: operands are shorter than {M}x{N} needs")
            out_mode = op.get("out_mode")
            out = op.get("out")
            if out is None:
                out = (torch.empty(M, dtype=torch.float32, device=device) if out_mode is None
                       else torch.empty((M + 3) // 4, dtype=torch.int32, device=device).view(torch.uint32))
            elif out_mode is None:
                if out.dtype != torch.float32 or out.numel() != M or out.device != device or not out.is_contiguous():
                    raise ValueError(f"op {i}: out must be a contiguous float32 tensor of M elements")
            else:
                out = as_words(out, "out")
                if out.numel() != (M + 3) // 4 or out.device != device:
                    raise ValueError(f"op {i}: out must hold ceil(M / 4) packed words")
            self.outs.append(out)
            self._keep.append((m, v))
            self.specs.append((m, v, (M, N), op.get("mode", mode), out_mode))
            t = table[i]
            t.m, t.v, t.out = m.data_ptr(), v.data_ptr(), out.data_ptr()
            t.M, t.N = M, N
            t.mode = fb._lib.mode_id(op.get("mode", mode))
            t.out_mode = -1 if out_mode is None else fb._lib.mode_id(out_mode)
            t.wait_op = int(op.get("wait_op", -1))
            t.allreduce = 1 if op.get("allreduce") else 0
        self.n_ops, self.device = len(ops), device
        self.ctx = ctx
        ar_rows = [int(op["shape"][0]) for op in ops if op.get("allreduce")]
        self.n_allreduce, self.max_allreduce_rows = len(ar_rows), max(ar_rows, default=0)
        if ar_rows:
            if ctx is None:
                raise ValueError("ops with allreduce=True need ctx=PeerAllReduce(max_rows, n_ops=...)")
            need = int(self.lib.feather_gemv_chain_inbox_floats(self.n_allreduce, self.max_allreduce_rows,
                                                                ctx.world_size))
            if ctx.inbox_floats < need or ctx.device != device:
                raise ValueError(f"the all-reduce context is too small ({ctx.inbox_floats} < {need} floats) "
                                 "or lives on another device")
        nbytes = int(self.lib.feather_gemv_chain_plan_bytes(self.n_ops))
        self.plan = torch.empty(nbytes, dtype=torch.uint8, device=device)
        with torch.cuda.device(device):
            fb._lib.check(self.lib.feather_gemv_chain_plan(
                ctypes.cast(table, ctypes.c_void_p), self.n_ops, self.plan.data_ptr(), nbytes,
                fb._lib.current_stream_ptr(device.index)))

    def token(self) -> None:
        idx = self.device.index
        with torch.cuda.device(idx):
            if self.ctx is None:
                fb._lib.check(self.lib.feather_gemv_chain_fp8(self.plan.data_ptr(), self.n_ops,
                                                              1 if self.static_matrix else 0,
                                                              fb._lib.current_stream_ptr(idx)))
            else:
                c = self.ctx
                fb._lib.check(self.lib.feather_gemv_chain_fp8_tp(
                    self.plan.data_ptr(), self.n_ops, 1 if self.static_matrix else 0, self.n_allreduce,
                    self.max_allreduce_rows, c.inbox_ptrs, c.inbox_floats, c.flag_ptrs, c.rank,
                    c.world_size, fb._lib.current_stream_ptr(idx)))

    __call__ = token

    @classmethod
    def from_chain(cls, chain: "GemvChain", dependent=False) -> "PersistentGemvChain":
        """The ops of a ``GemvChain`` as one launch.

        ``dependent=False``: the same independent GEMVs on the chain's fixed
        activations.  ``dependent="model"`` (or True): the data flow of the model
        whose shapes these are -- every op writes packed FP8; q, k and v read the
        layer's input (the previous layer's down output), o reads q's output
        (standing in for the attention output of the same length), gate and up
        read o's output, down reads gate's, lm_head the last down's; each reader
        waits for its writer: four dependent steps per layer.  ``dependent="serial"``:
        every op reads the latest output of matching length, k after q, v after k
        ...: 155 dependent steps, the worst case."""
        if dependent is True:
            dependent = "model"
        if dependent not in (False, "model", "serial"):
            raise ValueError("dependent must be False, 'model' or 'serial'")
        ops, last, src = [], {}, {}
        reads = {"q": "x", "k": "x", "v": "x", "qkv": "x", "o": "q", "gate": "o", "up": "o",
                 "gate_up": "o", "down": "gate", "lm_head": "x"}
        for i, ((w, a, (m, n), out), words, name) in enumerate(zip(chain.ops, chain.packed, chain.names)):
            op = {"m": w, "v": a, "shape": (m, n)}
            if dependent == "serial":
                op.update(out=words, out_mode=chain.mode)
                if n in last:
                    op.update(v=last[n][1], wait_op=last[n][0])
                last[m] = (i, words)
            elif dependent == "model":
                op.update(out=words, out_mode=chain.mode)
                want = reads[name]
                want = {"q": "qkv", "gate": "gate_up"}.get(want, want) if want not in src else want
                if want in src:   # the producer's first n codes (merged projections are longer)
                    op.update(v=src[want][1][: n // 4], wait_op=src[want][0])
                src[name] = (i, words)
                if name == "down":
                    src["x"] = (i, words)
            elif chain.reencode == "fused":
                op.update(out=words, out_mode=chain.mode)
            else:
                op.update(out=out)
            ops.append(op)
        return cls(ops, chain.mode, chain.static_matrix)


class TensorParallelChain:
    """The same chain split over the ranks of a process group (one process per GPU).

    * q/k/v/gate/up/lm_head are split by OUTPUT rows: rank r holds rows
      ``[r*M/W, (r+1)*M/W)`` of each and the whole activation; its outputs stay
      sharded (they feed the next, input-split, GEMV of a real model).
    * o and down are split by INPUT columns: rank r holds columns
      ``[r*N/W, (r+1)*N/W)`` of every row and the matching slice of the packed
      activation; each rank produces a full-length partial sum and the partials
      are added either inside the GEMV kernel through peer-mapped inboxes
      (``fused_allreduce=True``, sharded.ColumnShardedGemv) or with an NCCL
      all-reduce after it (2048 floats, 2 per layer).

    Weights are generated from the same seed, in the same order, as GemvChain's,
    so the two can be compared.
    """

    def __init__(self, mode: str = "E4M3", seed: int = 6, group=None, layers: int = LAYERS,
                 static_matrix: bool = True, fused_allreduce: bool = False,
                 merge_projections: bool = False, persistent: bool = False):
        """``persistent``: the rank's whole token is ONE launch
        (PersistentGemvChain) with the all-reduces of o and down inside it."""
        import torch.distributed as dist
        from .sharded import ColumnShardedGemv, PeerAllReduce
        self.dist, self.group = dist, group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        W, r = self.world, self.rank
        device = torch.device("cuda", torch.cuda.current_device())
        gen = torch.Generator(device=device).manual_seed(seed)
        self.mode, self.static_matrix = mode, static_matrix
        self.persistent = bool(persistent)
        self.fused_allreduce = (bool(fused_allreduce) or self.persistent) and self.world > 1
        self.ctx = None
        if self.fused_allreduce:
            self.ctx = PeerAllReduce(HIDDEN, device, group, n_ops=2 * layers if self.persistent else 1)
        self.ops = []  # (kind, packed weight shard, packed activation (slice), (rows, cols), out)
        acts = {}
        for n in (HIDDEN, INTER):
            a = torch.randn(n, device=device, generator=gen, dtype=torch.float16)
            acts[n] = fb.pack_fp8_tensor(a, mode)

        def add(name: str, m: int, n: int) -> None:
            w = (0.02 * torch.randn(m, n, device=device, generator=gen)).to(torch.float16)
            if name in ("o", "down"):  # input split
                if n % (4 * W):
                    raise ValueError(f"{name}: {n} columns do not split into {W} whole-word slices")
                cols = n // W
                shard = w[:, r * cols:(r + 1) * cols].contiguous()
                act = acts[n][r * cols // 4:(r + 1) * cols // 4]
                packed = fb.pack_fp8_tensor(shard, mode)
                out = torch.empty(m, dtype=torch.float32, device=device)
                if self.persistent:
                    self.ops.append(("fused" if self.world > 1 else "cols", packed, act, (m, cols), out))
                elif self.fused_allreduce:
                    self.ops.append(("fused", ColumnShardedGemv(packed, (m, cols), mode, self.ctx, out=out),
                                     act, (m, cols), out))
                else:
                    self.ops.append(("cols", packed, act, (m, cols), out))
            else:  # output split
                if m % W:
                    raise ValueError(f"{name}: {m} rows do not split over {W} ranks")
                rows = m // W
                shard = w[r * rows:(r + 1) * rows]
                self.ops.append(("rows", fb.pack_fp8_tensor(shard, mode), acts[n], (rows, n),
                                 torch.empty(rows, dtype=torch.float32, device=device)))
        # merge_projections: as in GemvChain, q/k/v and gate/up become one
        # row-split GEMV each (a rank's rows of the members, concatenated)
        shapes = LAYER_SHAPES if not merge_projections else (
            ("qkv", HIDDEN + 2 * KV_DIM, HIDDEN), ("o", HIDDEN, HIDDEN),
            ("gate_up", 2 * INTER, HIDDEN), ("down", HIDDEN, INTER))
        for _ in range(layers):
            for name, m, n in shapes:
                add(name, m, n)
        add("lm_head", VOCAB, HIDDEN)
        self.pchain = None
        if self.persistent:
            self.pchain = PersistentGemvChain(
                [{"m": w, "v": a, "shape": shape, "out": out, "allreduce": kind == "fused"}
                 for kind, w, a, shape, out in self.ops], mode, static_matrix, ctx=self.ctx)
        torch.cuda.synchronize()

    def token(self) -> None:
        if self.pchain is not None:
            return self.pchain.token()
        for kind, w, a, shape, out in self.ops:
            if kind == "fused":
                w(a)
                continue
            fb.gemv_fp8_acc_fp32_gpu(w, a, shape, self.mode, out=out, static_matrix=self.static_matrix)
            if kind == "cols" and self.world > 1:
                self.dist.all_reduce(out, group=self.group)

    def close(self) -> None:
        if self.ctx is not None:
            self.ctx.close()


def check_tp(tp: "TensorParallelChain", single: "GemvChain") -> float:
    """Largest error of a tensor-parallel token against the single-GPU chain
    built from the same seed, normalised per op by the largest reference value:
    row-split ops against their slice of the single-GPU result, column-split
    ops (after the all-reduce) against the whole of it.  Max over the ranks."""
    import torch.distributed as dist
    tp.token()
    single.token()
    torch.cuda.synchronize()
    worst = 0.0
    for (kind, _, _, shape, out_tp), (_, _, _, out_1) in zip(tp.ops, single.ops):
        ref = out_1 if kind in ("cols", "fused") else out_1[tp.rank * shape[0]:(tp.rank + 1) * shape[0]]
        scale = float(out_1.abs().max().item()) or 1.0
        worst = max(worst, float((out_tp.double() - ref.double()).abs().max().item()) / scale)
    t = torch.tensor([worst], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=tp.group)
    return float(t.item())


def measure_tp(tokens: int = 30, use_graph: bool = True, mode: str = "E4M3", group=None,
               fused_allreduce: bool = False, merge_projections: bool = False,
               check: bool = False, persistent: bool = False) -> dict:
    """Tokens per second of the tensor-parallel chain (call on every rank).
    ``check``: also compare one token with the single-GPU chain (check_tp)."""
    import torch.distributed as dist
    chain = TensorParallelChain(mode, group=group, fused_allreduce=fused_allreduce,
                                merge_projections=merge_projections, persistent=persistent)
    err = None
    if check:
        single = GemvChain(mode, merge_projections=merge_projections)
        err = check_tp(chain, single)
        del single
    # First token with a short wait limit: if the ranks cannot reach each other the
    # fused all-reduce gives up quickly and the status check raises here, instead of
    # every later call waiting out the default limit.
    lib = fb._lib.load()
    torch.cuda.synchronize()
    dist.barrier(group=group)  # all ranks have built their shards: they start the token together
    fb._lib.check(lib.feather_set_wait_limit_ms(200))
    try:
        chain.token()
        fb.device_status()
    finally:
        fb._lib.check(lib.feather_set_wait_limit_ms(2000))
    for _ in range(3):
        chain.token()
    torch.cuda.synchronize()
    run, graphed = chain.token, False
    if use_graph:
        try:
            stream = torch.cuda.Stream()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.stream(stream):
                chain.token()
                torch.cuda.synchronize()
                with torch.cuda.graph(graph, stream=stream):
                    chain.token()
            graph.replay()
            torch.cuda.synchronize()
            run, graphed = graph.replay, True
        except Exception:  # noqa: BLE001 - collectives that cannot be captured: time eagerly
            torch.cuda.synchronize()
    dist.barrier(group=group)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(tokens):
        run()
    end.record()
    torch.cuda.synchronize()
    t = torch.tensor([start.elapsed_time(end) / tokens], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    ms = float(t.item())
    chain.close()
    return {"tokens_per_s": round(1e3 / ms, 1), "us_per_token": round(ms * 1e3, 1),
            "gemvs_per_token_per_rank": len(chain.ops),
            "launches_per_token_per_rank": 1 if persistent else len(chain.ops),
            "all_reduces_per_token": sum(1 for o in chain.ops if o[0] in ("cols", "fused")),
            "fused_allreduce": chain.fused_allreduce, "merged_projections": merge_projections,
            "world": chain.world, "cuda_graph": graphed, "mode": mode,
            "max_norm_err_vs_single_gpu_chain": err}


def measure(tokens: int = 50, use_graph: bool = True, mode: str = "E4M3",
            merge_projections: bool = False, reencode: str | None = None,
            persistent: str | None = None) -> dict:
    """``persistent``: None = one launch per GEMV; "independent", "model" or
    "serial" = the whole token as one persistent launch with that data flow
    (PersistentGemvChain.from_chain)."""
    chain = GemvChain(mode, merge_projections=merge_projections, reencode=reencode)
    step = chain.token
    if persistent is not None:
        flow = {"independent": False, "dependent": "serial"}.get(persistent, persistent)
        step = PersistentGemvChain.from_chain(chain, dependent=flow).token
    for _ in range(3):
        step()
    torch.cuda.synchronize()
    if persistent is not None:
        fb.device_status()
    run = step
    if use_graph:
        stream = torch.cuda.Stream()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(stream):
            step()
            torch.cuda.synchronize()
            with torch.cuda.graph(graph, stream=stream):
                step()
        run = graph.replay
        run()
        torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(tokens):
        run()
    end.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(end) / tokens
    nbytes = chain.bytes_per_token()
    return {"tokens_per_s": round(1e3 / ms, 1), "us_per_token": round(ms * 1e3, 1),
            "gemvs_per_token": len(chain.ops), "launches_per_token": 1 if persistent else len(chain.ops),
            "GB/s": round(nbytes / ms / 1e6, 1),
            "bytes_per_token": nbytes, "cuda_graph": use_graph, "mode": mode,
            "merged_projections": merge_projections, "reencode": reencode, "persistent": persistent}


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=50)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--mode", default="E4M3")
    ap.add_argument("--merge-projections", action="store_true")
    a = ap.parse_args()
    print(measure(a.tokens, not a.no_graph, a.mode, a.merge_projections))
