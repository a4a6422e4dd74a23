#!/usr/bin/env python
"""Benchmark of the packed-FP8 GEMV path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Metric: achieved HBM GB/s of the packed-FP8 GEMV (algorithmic bytes = packed
matrix + packed vector + FP32 output, divided by time), whole job.

* N = 1: the single-GPU E5M2 GEMV, 16384 x 16384, seed 1 (256 MiB packed).  A
  step is one GEMV call; four distinct packed matrices are rotated so that no
  step finds its matrix in the 126 MB L2.
* N > 1 (launched by torch.distributed.run, one rank per GPU): the row-sharded
  E5M2 GEMV, 65536 x 65536 (4 GiB packed), rows split in contiguous blocks,
  vector replicated, output slices exchanged inside the GEMV kernel through
  peer-mapped buffers (the same step with an NCCL all-gather is reported in
  "extra").  A step is one call of the sharded operator; time is the max over
  ranks.  Total work is fixed ("strong" scaling).
* --impl reference: the reference's CPU path (decode with the kernel bit
  semantics + FP32 matvec, the C restatement in oracle/) on the host cores.

One JSON line is printed by rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "packed_fp8_gemv_hbm_gbps"
UNIT = "GB/s"
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0
# DRAM bytes of ONE launch of gemv_ring_kernel<E5M2> at 16384 x 16384 as ncu
# counted them (dram__bytes_read.sum + dram__bytes_write.sum of a single
# captured launch, clocks not locked): 268 522 240 read + 4 370 944 written.
NCU_TRAFFIC_BYTES_16384 = 272893184
REPEAT_BLOCKS = 8  # further blocks of K steps timed after the official one, for median / min


def gemv_bytes(M: int, N: int) -> int:
    """Algorithmic bytes of one GEMV: packed matrix + packed vector + output."""
    return M * N + 4 * ((N + 3) // 4) + 4 * M


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


def measured_tensor_peak():
    """Dense bf16 TFLOP/s of a cuBLAS GEMM timed alone (the burst figure), measured or fallback."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["bf16_tflops"]), "measured"
    except Exception:
        return 1590.0, "fallback"


_POLLER = r"""
import sys, time
import pynvml as nv
nv.nvmlInit()
h = nv.nvmlDeviceGetHandleByIndex(int(sys.argv[1]))
print("max", nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM), flush=True)
while True:
    t = time.time()
    print(t, nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM),
          nv.nvmlDeviceGetCurrentClocksEventReasons(h), flush=True)
    time.sleep(0.0005)
"""


class ClockSampler:
    """SM clock and throttle reasons while the timed region runs.

    NVML is polled (read-only queries, as fast as they return) by a CHILD
    process: polling from a thread of the benchmark process contends with its
    kernel launches for the driver's locks, which at 8 GPUs slowed the timed
    region by 25 %.  The child is started before the warm-up.  The official
    region of K steps can be shorter than one NVML query (20 x 40 us), so the
    sampler also knows an EXTENDED window: the official region plus the
    repeat blocks of the same step that follow it back to back.  The summary
    uses the samples inside the official region when there are at least three,
    else those of the extended window, and says which."""

    REASONS = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "hw_thermal_slowdown": 0x40,
               "sw_thermal_slowdown": 0x20, "hw_power_brake_slowdown": 0x80,
               "applications_clocks_setting": 0x2}

    def __init__(self, index: int):
        self.proc, self.t0, self.t1, self.t2 = None, None, None, None
        if index < 0:
            return
        try:
            import subprocess
            self.proc = subprocess.Popen([sys.executable, "-c", _POLLER, str(index)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.first = self.proc.stdout.readline()  # "max <MHz>": the poller is up and polling
        except Exception:
            self.proc = None

    def __enter__(self):
        self.t0 = time.time()
        return self

    def __exit__(self, *exc):
        self.t1 = time.time()

    def stop(self):
        """End of the extended window (call after the repeat blocks)."""
        self.t2 = time.time()
        if self.proc is not None:
            time.sleep(0.004)  # let the sample in flight be written
            self.proc.terminate()

    def summary(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        if self.t2 is None:
            self.stop()
        try:
            text, _ = self.proc.communicate(timeout=10)
        except Exception:
            self.proc.kill()
            return out
        official, extended = [], []
        for line in [self.first] + text.splitlines():
            f = line.split()
            if len(f) == 2 and f[0] == "max":
                out["sm_max_mhz"] = int(f[1])
            elif len(f) == 3:
                t, mhz, r = float(f[0]), int(f[1]), int(f[2])
                if self.t0 <= t <= self.t1:
                    official.append((mhz, r))
                if self.t0 <= t <= self.t2:
                    extended.append((mhz, r))
        use, out["window"] = (official, "official K steps") if len(official) >= 3 else (
            extended, "official K steps + the repeat blocks right behind them")
        if use:
            mhz = sorted(m for m, _ in use)
            reasons = 0
            for _, r in use:
                reasons |= r
            out["sm_mhz"] = mhz[len(mhz) // 2]
            out["sm_mhz_min"] = mhz[0]
            out["samples"] = len(use)
            out["samples_in_official_region"] = len(official)
            out["reasons"] = sorted(k for k, bit in self.REASONS.items() if reasons & bit)
        return out


def physical_gpu_index(local: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local])
        except Exception:
            return local
    return local


# ------------------------------------------------------------------ CPU arm --
def cpu_gemv_gbps(M: int, N: int, mode: str, budget_s: float, seed: int = 1):
    """Time the C oracle's GEMV (reference CPU path: kernel-semantics decode +
    FP32 matvec) on all host threads over a bounded row sample of the M x N
    workload.  Returns (GB/s, threads, description, seconds per pass)."""
    import numpy as np

    from oracle import c_oracle as C
    C.build()
    threads = C.use_all_cores()
    rng = np.random.default_rng(seed)
    rows = min(M, 2048)
    A = rng.standard_normal((rows, N)).astype(np.float16)
    v = rng.standard_normal(N).astype(np.float16)
    t0 = time.perf_counter()
    mw = C.pack(A, mode)
    pack_s = time.perf_counter() - t0
    vw = C.pack(v, mode)
    C.gemv(mw, vw, (rows, N), mode)  # warm
    t0 = time.perf_counter()
    C.gemv(mw, vw, (rows, N), mode)
    t_probe = time.perf_counter() - t0
    # a pass over `rows` rows costs t_probe; repeat passes to fill the budget
    reps = max(3, min(200, int(budget_s / max(t_probe, 1e-6))))
    t0 = time.perf_counter()
    for _ in range(reps):
        C.gemv(mw, vw, (rows, N), mode)
    dt = (time.perf_counter() - t0) / reps
    gbps = gemv_bytes(rows, N) / dt / 1e9
    sample = (f"{rows} of {M} rows x {N} cols {mode}, {reps} passes, C restatement of the "
              f"reference decode + FP32 matvec (OpenMP); packing those rows took {pack_s:.3f} s "
              f"({rows * N / pack_s / 1e9:.2f} Gelem/s)")
    return gbps, threads, sample, dt


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    M, N = (16384, 16384) if args.gpus == 1 else (65536, 65536)
    workload = ("gemv_e5m2_16384x16384" if args.gpus == 1 else "row_sharded_gemv_e5m2_65536x65536")
    import numpy as np

    from oracle import c_oracle as C
    C.build()
    threads = C.use_all_cores()
    rng = np.random.default_rng(1)
    # bounded sample: rows chosen so that warmup + steps end within ~2 minutes
    rows = min(M, 4096)
    A = rng.standard_normal((rows, N)).astype(np.float16)
    mw, vw = C.pack(A, "E5M2"), C.pack(rng.standard_normal(N).astype(np.float16), "E5M2")
    t0 = time.perf_counter()
    C.gemv(mw, vw, (rows, N), "E5M2")
    t1 = time.perf_counter() - t0
    total = (args.steps + args.warmup) * t1
    if total > 120.0:
        rows = max(64, int(rows * 120.0 / total))
        mw = mw[: rows * (N // 4)]
    for _ in range(args.warmup):
        C.gemv(mw, vw, (rows, N), "E5M2")
    t0 = time.perf_counter()
    for _ in range(args.steps):
        C.gemv(mw, vw, (rows, N), "E5M2")
    dt = (time.perf_counter() - t0) / max(args.steps, 1)
    gbps = gemv_bytes(rows, N) / dt / 1e9
    sample = f"{rows} of {M} rows x {N} cols per step, all host threads"
    line = {
        "impl": "reference", "metric": METRIC, "value": round(gbps, 3), "unit": UNIT,
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(dt * 1e3, 4), "higher_is_better": True,
        "scaling": "strong" if args.gpus > 1 else "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": {"workload": workload, "M": M, "N": N, "mode": "E5M2"},
        "cpu_baseline": {"value": round(gbps, 3), "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": sample},
        "e2e": {"value": round(gbps, 3), "unit": UNIT, "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def reference_worker(*argv, timeout: int = 900) -> dict:
    """Run baseline/reference_worker.py (the reference's own code, installed
    unmodified under baseline/_ref) in a process of its own; its JSON result, or
    {"unavailable": why}."""
    import subprocess
    worker = os.path.join(ROOT, "baseline", "reference_worker.py")
    try:
        res = subprocess.run([sys.executable, worker, *argv], capture_output=True, text=True,
                             timeout=timeout, cwd=os.path.join(ROOT, "baseline"))
        for ln in res.stdout.splitlines():
            if ln.startswith("REFERENCE_WORKER "):
                return json.loads(ln[len("REFERENCE_WORKER "):])
        return {"unavailable": f"worker exit code {res.returncode}: {res.stderr[-300:]}"}
    except Exception as e:  # noqa: BLE001
        return {"unavailable": repr(e)[:300]}


# ------------------------------------------------------------------ GPU arm --
def time_calls(torch, fn, n_iter: int, warmup: int) -> float:
    """Average milliseconds per call with CUDA events on the current stream."""
    for _ in range(warmup):
        fn()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for _ in range(n_iter):
        fn()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / n_iter


def check_sharded(torch, dist, fb, op, op_nccl, m_local, vw, M, N, mode, rank, world, dev) -> dict:
    """Correctness of the row-sharded operators on every rank: the fused
    exchange (waiting and split-phase) against the NCCL all-gather, bit for bit
    (rows never interact), and 1024 sampled rows PER RANK of the gathered
    result against the oracle's float64 GEMV of the same packed rows."""
    import numpy as np

    from oracle import c_oracle as C
    C.build()
    rows = M // world
    y_nccl = op_nccl(vw).clone()
    same_wait = same_split = True
    if op.fused:
        for _ in range(3):   # both buffers, several epochs
            same_wait &= bool(torch.equal(op(vw), y_nccl))
        for _ in range(3):
            y = op(vw, wait=False)
            op.wait()
            same_split &= bool(torch.equal(y, y_nccl))
        fb.device_status()
    n_sample = min(1024, rows)
    idx = np.sort(np.random.default_rng(100 + rank).choice(rows, n_sample, replace=False))
    idx_t = torch.from_numpy(idx).to(dev)
    sub = m_local.view(torch.int32).view(rows, N // 4)[idx_t].contiguous().cpu().numpy().view(np.uint32)
    v_host = vw.view(torch.int32).cpu().numpy().view(np.uint32)
    ref = C.gemv(sub.reshape(-1), v_host, (n_sample, N), mode, acc="f64")
    ref_t = torch.from_numpy(np.asarray(ref, dtype=np.float64)).to(dev)
    all_ref = [torch.empty_like(ref_t) for _ in range(world)]
    all_idx = [torch.empty_like(idx_t) for _ in range(world)]
    dist.all_gather(all_ref, ref_t)
    dist.all_gather(all_idx, idx_t)
    want = torch.cat(all_ref)
    where = torch.cat([all_idx[r] + r * rows for r in range(world)])
    got = (op(vw) if op.fused else y_nccl)[where].double()
    err = float(((got - want).abs().max() / want.abs().max()).item())
    t = torch.tensor([err, -float(same_wait), -float(same_split)], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return {"rows_checked_per_rank": world * n_sample, "max_norm_err_vs_oracle_f64": float(t[0].item()),
            "fused_equals_nccl": bool(t[1].item() == -1.0), "split_phase_equals_nccl": bool(t[2].item() == -1.0),
            "tolerance": 1e-5}


def run_ours(args) -> None:
    import torch
    import torch.distributed as dist

    import feather_b200 as fb
    from feather_b200.sharded import RowShardedGemv

    fb._lib.load()  # fail loudly if the CUDA library is missing
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus != world:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run (one rank per GPU)")
        raise SystemExit(f"--gpus {args.gpus} does not match WORLD_SIZE {world}")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    K, W = args.steps, args.warmup
    peak, peak_kind = measured_peak()
    mode = "E5M2"
    gen = torch.Generator(device=dev)

    def make_packed(rows: int, cols: int, seed: int, mode: str, dtype=torch.float16):
        gen.manual_seed(seed)
        out = torch.empty(rows * (cols // 4), dtype=torch.int32, device=dev).view(torch.uint32)
        blk = max(1, min(rows, (1 << 28) // cols))
        for r0 in range(0, rows, blk):
            r1 = min(rows, r0 + blk)
            a = torch.randn(r1 - r0, cols, device=dev, generator=gen, dtype=dtype)
            out[r0 * (cols // 4): r1 * (cols // 4)] = fb.pack_fp8_tensor(a, mode)
        return out

    extra = {}
    if world == 1:
        M = N = 16384
        workload = "gemv_e5m2_16384x16384"
        n_buf = 4
        mats = [make_packed(M, N, 1 + 100 * i, mode) for i in range(n_buf)]
        gen.manual_seed(1)
        v_f16 = torch.randn(N, device=dev, generator=gen, dtype=torch.float16)
        vw = fb.pack_fp8_tensor(v_f16, mode)
        out = torch.empty(M, dtype=torch.float32, device=dev)
        step_bytes = gemv_bytes(M, N)
        state = {"i": 0}

        def step():
            fb.gemv_fp8_acc_fp32_gpu(mats[state["i"] % n_buf], vw, (M, N), mode, out=out)
            state["i"] += 1

        def finish():
            pass
        l2_note = f"{n_buf} distinct 256 MiB packed matrices rotated (each larger than L2)"
    else:
        M = N = 65536
        workload = "row_sharded_gemv_e5m2_65536x65536"
        rows = M // world
        m_local = make_packed(rows, N, 5 + rank, mode)
        gen.manual_seed(5)
        vw = fb.pack_fp8_tensor(torch.randn(N, device=dev, generator=gen, dtype=torch.float16), mode)
        op = RowShardedGemv(m_local, (M, N), mode)  # fused peer-store exchange when available
        step_bytes = gemv_bytes(M, N)

        def step():
            # split-phase: the call ends when this rank's rows and epoch are on their way; the
            # arrival of the peers' slices is awaited once, after the last step (finish()),
            # still inside the timed region, and by every later call before it overwrites a buffer
            op(vw, wait=False)
        finish = op.wait
        l2_note = f"per-rank block {rows * N >> 20} MiB, larger than L2"
        extra["exchange"] = ("fused into the GEMV kernel (peer stores over NVLink), split-phase: the K "
                             "steps are enqueued back to back, the wait for the last step's slices is "
                             "inside the timed region" if op.fused
                             else "NCCL all-gather after the local GEMV")

    # ---- the timed region: W warm-up steps, then exactly K steps -----------
    # only rank 0 samples clocks; the poller process is up before the warm-up ends
    clocks = ClockSampler(physical_gpu_index(local_rank) if rank == 0 else -1)
    for _ in range(W):
        step()
    finish()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    if world > 1 and op.fused:
        # The host barrier leaves the ranks tens of microseconds apart, which K = 20 steps of
        # 90 us would carry as skew.  One more warm-up call that waits for every rank's slices
        # ends on all GPUs within a few microseconds; the start events are enqueued right
        # behind it, so the timed regions of the ranks begin together.
        op(vw)
    with clocks:
        start.record()
        for _ in range(K):
            step()
        finish()
        end.record()
        torch.cuda.synchronize()
    ms_total = start.elapsed_time(end)
    # the same K steps again, REPEAT_BLOCKS times, each block timed on its own: the spread
    # over blocks shows whether the official block (often under a millisecond) was typical
    block_us = [ms_total * 1e3 / K]
    for _ in range(REPEAT_BLOCKS):
        s_ev, e_ev = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s_ev.record()
        for _ in range(K):
            step()
        finish()
        e_ev.record()
        torch.cuda.synchronize()
        block_us.append(s_ev.elapsed_time(e_ev) * 1e3 / K)
    clocks.stop()
    if world > 1:
        dist.barrier()
        t = torch.tensor([ms_total] + block_us, device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total, block_us = float(t[0].item()), [float(x) for x in t[1:].tolist()]
    ms_per_step = ms_total / K
    value = step_bytes / (ms_per_step * 1e-3) / 1e9
    ordered = sorted(block_us)
    blocks = {"blocks": len(block_us), "steps_per_block": K, "official_us": round(block_us[0], 3),
              "median_us": round(ordered[len(ordered) // 2], 3), "min_us": round(ordered[0], 3),
              "max_us": round(ordered[-1], 3)}

    # ---- kernel-only duration for the roofline (local GEMV kernel) ---------
    if world == 1:
        kern_ms = ms_per_step
        kern_bytes = step_bytes
        kern_name = "gemv_ring_kernel<E5M2>"
    else:
        kern_ms = time_calls(torch, lambda: op.local(vw), max(20, K), 5)
        kern_bytes = gemv_bytes(M // world, N)
        parity = {}
        op_nccl = RowShardedGemv(m_local, (M, N), mode, fused=False)
        if op.fused:
            def rank_max(ms: float) -> float:
                t = torch.tensor([ms], device=dev, dtype=torch.float64)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                return round(float(t.item()) * 1e3, 3)
            # the same step (a) waiting for all slices at the end of every call, (b) with the
            # separate NCCL all-gather
            extra["fused_waiting_in_every_call_us"] = rank_max(time_calls(torch, lambda: op(vw), max(20, K), 5))
            extra["same_step_with_nccl_all_gather_us"] = rank_max(
                time_calls(torch, lambda: op_nccl(vw), max(20, K), 5))
            # where a waiting call's tail goes: GPU timer of the rank's last CTA
            op.record_stamps(True)
            lat, skew = [], []
            for _ in range(10):
                op(vw)
                st = op.stamps()
                lat.append((st[1] - st[0]) * 1e-3)
                skew.append((st[2] - st[1]) * 1e-3)
            op.record_stamps(False)
            t = torch.tensor([sorted(lat)[5], sorted(skew)[5]], device=dev, dtype=torch.float64)
            tmax, tmin = t.clone(), t.clone()
            dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
            dist.all_reduce(tmin, op=dist.ReduceOp.MIN)
            extra["exchange_tail_us"] = {
                "rows_pushed_to_epoch_published": {"max_over_ranks": round(float(tmax[0]), 2),
                                                   "min_over_ranks": round(float(tmin[0]), 2)},
                "epoch_published_to_all_epochs_seen": {"max_over_ranks": round(float(tmax[1]), 2),
                                                       "min_over_ranks": round(float(tmin[1]), 2)},
                "note": "median of 10 waiting calls per rank; the first is fence + flag stores, the "
                        "second the wait for the slowest rank"}
        extra["local_gemv_kernel_us"] = round(kern_ms * 1e3, 3)
        # ---- correctness of what was timed (outside the timed region) ------
        parity.update(check_sharded(torch, dist, fb, op, op_nccl, m_local, vw, M, N, mode, rank, world, dev))
        try:  # TinyLlama-shaped GEMV chain, tensor-parallel over the ranks (NCCL all-reduce)
            from feather_b200 import chain
            extra["tinyllama_gemv_chain_tensor_parallel"] = chain.measure_tp(tokens=20, check=True)
        except Exception as e:  # noqa: BLE001 - must not sink the headline
            extra["tinyllama_gemv_chain_tensor_parallel"] = {"error": repr(e)}
        try:  # the same with the all-reduce inside the column-sharded GEMV kernels
            extra["tinyllama_gemv_chain_tensor_parallel_fused_allreduce"] = chain.measure_tp(
                tokens=20, fused_allreduce=True, check=True)
            extra["tinyllama_gemv_chain_tensor_parallel_fused_allreduce_merged"] = chain.measure_tp(
                tokens=20, fused_allreduce=True, merge_projections=True, check=True)
        except Exception as e:  # noqa: BLE001
            extra["tinyllama_gemv_chain_tensor_parallel_fused_allreduce"] = {"error": repr(e)}
        try:  # each rank's whole token as ONE launch, the all-reduces inside it
            extra["tinyllama_gemv_chain_tensor_parallel_one_launch"] = chain.measure_tp(
                tokens=30, persistent=True, check=True)
            extra["tinyllama_gemv_chain_tensor_parallel_one_launch_merged"] = chain.measure_tp(
                tokens=30, persistent=True, merge_projections=True, check=True)
        except Exception as e:  # noqa: BLE001
            extra["tinyllama_gemv_chain_tensor_parallel_one_launch"] = {"error": repr(e)}
        parity["tp_chain_max_norm_err"] = {
            k.replace("tinyllama_gemv_chain_tensor_parallel", "tp"): v.get("max_norm_err_vs_single_gpu_chain")
            for k, v in extra.items() if k.startswith("tinyllama_gemv_chain_tensor_parallel")}
        extra["parity"] = parity
        kern_name = "gemv_ring_kernel<E5M2> (per-rank block)"
    achieved = kern_bytes / (kern_ms * 1e-3) / 1e9
    roofline = {"bound": "hbm", "kernel": kern_name, "achieved": round(achieved, 1),
                "peak": peak, "peak_kind": f"of {peak_kind}", "unit": "GB/s",
                "frac": round(achieved / peak, 4),
                "frac_of_nominal_8TBs": round(achieved / NOMINAL_HBM_GBS, 4),
                "algorithmic_bytes": kern_bytes, "us_per_launch": round(kern_ms * 1e3, 3),
                "traffic": NCU_TRAFFIC_BYTES_16384 if world == 1 else None}

    # ---- end to end: host buffers in, host result out, every step ----------
    if world == 1:
        m_host = mats[0].view(torch.int32).cpu().pin_memory()
        v_host = vw.view(torch.int32).cpu().pin_memory()
        out_host = torch.empty(M, dtype=torch.float32).pin_memory()
        m_dev = torch.empty_like(mats[0].view(torch.int32))
        v_dev = torch.empty_like(vw.view(torch.int32))

        def e2e_step():
            m_dev.copy_(m_host, non_blocking=True)
            v_dev.copy_(v_host, non_blocking=True)
            y = fb.gemv(m_dev, v_dev, original_shape=(M, N), mode=mode)
            out_host.copy_(y, non_blocking=True)
        h2d, d2h = m_host.numel() * 4 + v_host.numel() * 4, M * 4
        e2e_iters = max(3, min(K, 20))
    else:
        rows = M // world
        m_host = m_local.view(torch.int32).cpu().pin_memory()
        v_host = vw.view(torch.int32).cpu().pin_memory()
        out_host = torch.empty(M, dtype=torch.float32).pin_memory()
        v_dev = torch.empty_like(vw.view(torch.int32))

        def e2e_step():
            op.m_local.view(torch.int32).copy_(m_host, non_blocking=True)
            v_dev.copy_(v_host, non_blocking=True)
            out_host.copy_(op(v_dev), non_blocking=True)
        h2d, d2h = m_host.numel() * 4 + v_host.numel() * 4, M * 4
        e2e_iters = max(2, min(K, 5))
    e2e_ms = time_calls(torch, e2e_step, e2e_iters, 1)
    if world > 1:
        t = torch.tensor([e2e_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e = {"value": round(step_bytes / (e2e_ms * 1e-3) / 1e9, 3), "unit": UNIT,
           "ms_per_step": round(e2e_ms, 4), "h2d_bytes_per_step": h2d * world,
           "d2h_bytes_per_step": d2h * world,
           "path": "pinned host packed matrix+vector -> H2D -> feather.gemv -> D2H of the FP32 result"}

    # ---- other kernels of the path (single GPU only; outside the timed region)
    if world == 1:
        del m_host, m_dev
        n_it = max(20, min(K, 200))
        # E4M3 GEMV on the configuration-3 style data, same shape
        gen.manual_seed(4)
        m4 = []
        for i in range(n_buf):
            x = 4.0 * torch.randn(M, N, device=dev, generator=gen)
            u = torch.rand(M, N, device=dev, generator=gen)
            x = torch.where(u < 0.05, torch.copysign(2.0 ** -9 + u * 20 * (2.0 ** -6 - 2.0 ** -9), x),
                            torch.where(u < 0.10, torch.copysign(448.0 + (u - 0.05) * 20 * 552.0, x), x))
            m4.append(fb.pack_fp8_tensor(x, "E4M3"))
            del x, u
        v4 = fb.pack_fp8_tensor(v_f16, "E4M3")
        st = {"i": 0}

        def step4():
            fb.gemv_fp8_acc_fp32_gpu(m4[st["i"] % n_buf], v4, (M, N), "E4M3", out=out)
            st["i"] += 1
        ms4 = time_calls(torch, step4, n_it, 10)
        extra["gemv_e4m3_16384x16384"] = {
            "us_per_call": round(ms4 * 1e3, 3), "GB/s": round(step_bytes / ms4 / 1e6, 1),
            "frac_of_peak": round(step_bytes / ms4 / 1e6 / peak, 4)}
        for shape in ((8192, 8192), (16384, 8192)):
            mm, nn = shape
            views = [m4[i][: mm * nn // 4] for i in range(n_buf)]
            vv = v4[: nn // 4]
            o2 = out[:mm]
            st2 = {"i": 0}

            def step_s():
                fb.gemv_fp8_acc_fp32_gpu(views[st2["i"] % n_buf], vv, shape, "E4M3", out=o2)
                st2["i"] += 1
            ms_s = time_calls(torch, step_s, n_it, 10)
            b = gemv_bytes(mm, nn)
            extra[f"gemv_e4m3_{mm}x{nn}"] = {"us_per_call": round(ms_s * 1e3, 3),
                                             "GB/s": round(b / ms_s / 1e6, 1),
                                             "frac_of_peak": round(b / ms_s / 1e6 / peak, 4)}
        # several vectors in one pass over the matrix (feather_gemv_fp8_multi), both
        # formats; "matrix_GB/s" counts the matrix once, "vs_single_calls" is batch x
        # the single-vector time of this run divided by the multi-vector time
        # (E5M2 at this shape takes the tcgen05 kernel, 16 vectors per pass; E4M3 the mma.sync
        # kernel, 8 per pass)
        for name, mset, mmode, single_ms in (("e4m3", m4, "E4M3", ms4), ("e5m2", mats, mode, kern_ms)):
            for nb in (4, 8, 16):
                gen.manual_seed(21)
                Vn = fb.pack_fp8_tensor(torch.randn(nb, N, device=dev, generator=gen, dtype=torch.float16),
                                        mmode)
                outn = torch.empty(nb, M, dtype=torch.float32, device=dev)
                stm = {"i": 0}

                def step_m():
                    fb.gemv_fp8_multi_acc_fp32_gpu(mset[stm["i"] % n_buf], Vn, (M, N), mmode, batch=nb,
                                                   out=outn)
                    stm["i"] += 1
                ms_m = time_calls(torch, step_m, n_it, 10)
                extra[f"gemv_multi{nb}_{name}_16384x16384"] = {
                    "us_per_call": round(ms_m * 1e3, 3), "matrix_GB/s": round(M * N / ms_m / 1e6, 1),
                    "vs_single_calls": round(nb * single_ms / ms_m, 2)}
        del m4
        # the headline workload with FEATHER_GEMV_STATIC_MATRIX (weights promised static)
        st5 = {"i": 0}

        def step_static():
            fb.gemv_fp8_acc_fp32_gpu(mats[st5["i"] % n_buf], vw, (M, N), mode, out=out, static_matrix=True)
            st5["i"] += 1
        torch.cuda.synchronize()
        ms_st = time_calls(torch, step_static, max(n_it, 200), 10)
        extra["gemv_e5m2_16384x16384_static_matrix_flag"] = {
            "us_per_call": round(ms_st * 1e3, 3), "GB/s": round(step_bytes / ms_st / 1e6, 1),
            "frac_of_peak": round(step_bytes / ms_st / 1e6 / peak, 4)}
        # TinyLlama-shaped GEMV chain (155 GEMVs per token, E4M3 weights), CUDA graph replay
        try:
            from feather_b200 import chain
            extra["tinyllama_gemv_chain_1gpu"] = chain.measure(tokens=20, use_graph=True)
            extra["tinyllama_gemv_chain_1gpu_merged_qkv_gateup"] = chain.measure(
                tokens=20, use_graph=True, merge_projections=True)
            # every result re-encoded to packed FP8 (what a chained model needs):
            # in the GEMV epilogue, or as a second launch of the packer
            extra["tinyllama_gemv_chain_1gpu_reencode_fused"] = chain.measure(
                tokens=20, use_graph=True, reencode="fused")
            extra["tinyllama_gemv_chain_1gpu_reencode_separate_launch"] = chain.measure(
                tokens=20, use_graph=True, reencode="separate")
            # the whole token as ONE persistent launch (feather_gemv_chain_fp8): the same
            # independent GEMVs; with q/k/v and gate/up merged; with the model's data flow (every
            # op re-encodes its result, q/k/v read the previous layer's down output, o reads q's,
            # gate/up read o's, down reads gate's: four dependent steps per layer); and fully
            # serial (every op reads the latest output of matching length: 155 dependent steps)
            extra["tinyllama_gemv_chain_1gpu_one_launch"] = chain.measure(
                tokens=30, use_graph=True, persistent="independent")
            extra["tinyllama_gemv_chain_1gpu_one_launch_merged_qkv_gateup"] = chain.measure(
                tokens=30, use_graph=True, persistent="independent", merge_projections=True)
            extra["tinyllama_gemv_chain_1gpu_one_launch_model_dataflow"] = chain.measure(
                tokens=30, use_graph=True, persistent="model")
            extra["tinyllama_gemv_chain_1gpu_one_launch_model_dataflow_merged"] = chain.measure(
                tokens=30, use_graph=True, persistent="model", merge_projections=True)
            extra["tinyllama_gemv_chain_1gpu_one_launch_serial_dataflow"] = chain.measure(
                tokens=30, use_graph=True, persistent="serial")
        except Exception as e:  # noqa: BLE001 - the extra section must not sink the headline
            extra["tinyllama_gemv_chain_error"] = {"error": repr(e)}
        # dot on two 2^26-element E5M2 vectors: reuse the packed matrices as operands
        n_words = 1 << 24
        ops = [(mats[i][:n_words], mats[i][n_words:2 * n_words]) for i in range(n_buf)]
        st3 = {"i": 0}

        def step_d():
            a, b = ops[st3["i"] % n_buf]
            fb.dot_fp8_acc_fp32_gpu(a, b, "E5M2")
            st3["i"] += 1
        ms_d = time_calls(torch, step_d, n_it, 10)
        db = 2 * n_words * 4 + 4
        extra["dot_e5m2_2pow26"] = {"us_per_call": round(ms_d * 1e3, 3),
                                    "GB/s": round(db / ms_d / 1e6, 1),
                                    "frac_of_peak": round(db / ms_d / 1e6 / peak, 4)}
        # ReLU on unpack, 2^26 E5M2 codes -> FP32 (reads 1 B, writes 4 B per element);
        # inputs rotate, the 256 MiB output alone exceeds L2
        from feather_b200.routines.activations import relu1d_fp8_ret_fp32_feather_gpu as relu
        relu_out = torch.empty(4 * n_words, dtype=torch.float32, device=dev)
        st4 = {"i": 0}

        def step_r():
            relu(ops[st4["i"] % n_buf][0], 4 * n_words, mode="E5M2", out=relu_out)
            st4["i"] += 1
        ms_r = time_calls(torch, step_r, n_it, 10)
        rb = 5 * 4 * n_words
        extra["relu_unpack_e5m2_2pow26"] = {"us_per_call": round(ms_r * 1e3, 3),
                                            "GB/s": round(rb / ms_r / 1e6, 1),
                                            "frac_of_peak": round(rb / ms_r / 1e6 / peak, 4)}
        del relu_out
        # packed-E5M2 attention (single head, non-causal), tensor-core bound: 4 * seq^2 * d flops,
        # half of them (Q K^T) on E5M2 operands and half (P V) on FP16.  The library's choice
        # (the tcgen05 kernel at these lengths) with the register-fed mma.sync kernel beside it.
        from feather_b200.routines.attention import flash_attention_fp8_e5m2_acc_fp32_gpu as attn
        tpeak, tpeak_kind = measured_tensor_peak()
        lib = fb._lib.load()
        for seq, d in ((4096, 128), (8192, 64), (8192, 128), (4096, 256), (4096, 512)):
            gen.manual_seed(31)
            qkv = [fb.pack_fp8_tensor(torch.randn(seq, d, device=dev, generator=gen, dtype=torch.float16), "E5M2")
                   for _ in range(3)]
            o_attn = torch.empty(seq, d, dtype=torch.float32, device=dev)
            ms_a = time_calls(torch, lambda: attn(qkv[0], qkv[1], qkv[2], seq, d // 4, out=o_attn), 50, 5)
            lib.feather_set_tuning(b"attn_tc=0")
            try:
                ms_old = time_calls(torch, lambda: attn(qkv[0], qkv[1], qkv[2], seq, d // 4, out=o_attn), 20, 3)
            finally:
                lib.feather_set_tuning(b"attn_tc=1")
            tf = 4.0 * seq * seq * d / ms_a / 1e9
            extra[f"attention_e5m2_seq{seq}_d{d}"] = {
                "us_per_call": round(ms_a * 1e3, 2), "TFLOP/s": round(tf, 1),
                "frac_of_bf16_peak": round(tf / tpeak, 4), "peak_kind": tpeak_kind,
                "kernel": "tcgen05", "mma_sync_kernel_us": round(ms_old * 1e3, 2)}
        # encoder: fp16 16384^2 -> E5M2 (reads 2 B, writes 1 B per element)
        gen.manual_seed(9)
        src = torch.randn(M, N, device=dev, generator=gen, dtype=torch.float16)
        ms_e = time_calls(torch, lambda: fb.pack_fp8_tensor(src, "E5M2"), 20, 3)
        extra["encode_fp16_to_e5m2_16384x16384"] = {
            "us_per_call": round(ms_e * 1e3, 3), "GB/s": round(3 * M * N / ms_e / 1e6, 1),
            "frac_of_peak": round(3 * M * N / ms_e / 1e6 / peak, 4)}
        del src
        # the row-sharded workload (65536 x 65536, 4 GiB packed) on this ONE GPU: the
        # single-GPU point of the strong-scaling curve
        try:
            del mats, ops
            torch.cuda.empty_cache()
            Mb = Nb = 65536
            big = make_packed(Mb, Nb, 5, mode)
            gen.manual_seed(5)
            vb = fb.pack_fp8_tensor(torch.randn(Nb, device=dev, generator=gen, dtype=torch.float16), mode)
            ob = torch.empty(Mb, dtype=torch.float32, device=dev)
            ms_b = time_calls(torch, lambda: fb.gemv_fp8_acc_fp32_gpu(big, vb, (Mb, Nb), mode, out=ob), 20, 3)
            bb = gemv_bytes(Mb, Nb)
            extra["gemv_e5m2_65536x65536_1gpu"] = {
                "us_per_call": round(ms_b * 1e3, 2), "GB/s": round(bb / ms_b / 1e6, 1),
                "frac_of_peak": round(bb / ms_b / 1e6 / peak, 4),
                "note": "the N > 1 workload on one GPU: strong-scaling efficiency at N GPUs = this "
                        "time / (N x the N-GPU ms_per_step)"}
            del big, vb, ob
            torch.cuda.empty_cache()
        except Exception as e:  # noqa: BLE001
            extra["gemv_e5m2_65536x65536_1gpu"] = {"error": repr(e)}
        fb.device_status()

    if world > 1:
        op.close()  # unmap the peers' buffers (a collective: every rank calls it)
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    # ---- CPU baseline beside it (rank 0, bounded sample) --------------------
    cpu = None
    if world == 1:
        gbps, threads, sample, _ = cpu_gemv_gbps(M, N, mode, budget_s=12.0)
        cpu = {"value": round(gbps, 3), "unit": UNIT, "cores": threads, "kind": "port",
               "sample": sample}
        # the reference's OWN code beside it (a process of its own, baseline/reference_worker.py):
        # its Triton kernels on this GPU, and its packer + torch CPU decode + torch.mv on the host
        torch.cuda.empty_cache()
        extra["reference_triton_same_gpu"] = reference_worker("time", "--iters", "200")
        ref_cpu = reference_worker("cpu", "--M", "4096", "--N", "4096")
        if "unavailable" not in ref_cpu:
            e5 = ref_cpu["E5M2"]
            ref_cpu = {"value": e5["decode_mv_GB/s"], "unit": UNIT, "cores": ref_cpu["threads"],
                       "kind": "reference",
                       "sample": "4096 x 4096 (configuration 1): the reference packer "
                                 "(feather/packers/fp8.py:260-281), then a torch-CPU decode with the "
                                 "kernels' bit semantics + FP32 torch.mv; value = E5M2 decode+mv",
                       "detail": ref_cpu}
        extra["cpu_baseline_reference"] = ref_cpu
    line = {
        "metric": METRIC, "value": round(value, 1), "unit": UNIT, "n_gpus": world, "steps": K,
        "warmup": W, "ms_per_step": round(ms_per_step, 6), "higher_is_better": True,
        "scaling": "strong" if world > 1 else "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": workload, "M": M, "N": N, "mode": mode,
                   "bytes_per_step": step_bytes, "l2": l2_note,
                   "parallelism": f"rows/{world}" if world > 1 else "1 GPU"},
        "us_per_call": round(ms_per_step * 1e3, 3), "us_per_call_blocks": blocks,
        "frac_of_nominal_8TBs": round(value / world / NOMINAL_HBM_GBS, 4),
        "roofline": roofline, "e2e": e2e, "gpu_launches": K,
        "clocks": clocks.summary(), "extra": extra,
    }
    if cpu is not None:
        line["cpu_baseline"] = cpu
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
        par = extra.get("parity", {})
        errs = [par.get("max_norm_err_vs_oracle_f64", 0.0)] + [
            e for e in par.get("tp_chain_max_norm_err", {}).values() if e is not None]
        if not (par.get("fused_equals_nccl", True) and par.get("split_phase_equals_nccl", True)
                and all(e < 1e-5 for e in errs)):
            raise SystemExit("parity check of the multi-GPU run failed: " + json.dumps(par))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=400)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    args = ap.parse_args()
    if args.steps < 1 or args.warmup < 0:
        raise SystemExit("--steps must be >= 1 and --warmup >= 0")
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
