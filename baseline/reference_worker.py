#!/usr/bin/env python
"""Runs the reference's OWN code (installed unmodified under baseline/_ref by
install_reference.sh) in a process of its own and reports results as files /
one JSON line.  It is a checker and a baseline, never part of the product path:
only tests/ and bench.py's reference legs start it.

    python baseline/reference_worker.py parity --cases a,b,... --outdir DIR
    python baseline/reference_worker.py time   [--iters 200]
    python baseline/reference_worker.py cpu    [--M 4096 --N 4096]

A separate process because the reference's top-level package is called
``feather`` like this repository's drop-in alias, and because its kernels need
Triton, which the product never imports.  If the reference install or Triton is
missing, or the kernels cannot be compiled on this GPU, the JSON line is
``{"unavailable": "<why>"}`` and the exit code 0.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")


def _import_reference():
    if not os.path.isdir(os.path.join(REF, "feather", "routines")):
        raise RuntimeError("baseline/_ref is missing: run baseline/install_reference.sh")
    # the reference install first, this repository's root (and its `feather` alias) never
    sys.path[:] = [REF] + [p for p in sys.path if os.path.abspath(p or ".") != os.path.dirname(HERE)]
    import logging
    logging.disable(logging.WARNING)  # the packer logs whole arrays for non-fp16 input
    from feather.packers import fp8 as P
    from feather.routines import dot as D
    from feather.routines import gemv as G
    assert os.path.abspath(P.__file__).startswith(REF), P.__file__
    return P, G, D


def _workloads():
    import importlib.util
    spec = importlib.util.spec_from_file_location("ref_workloads", os.path.join(HERE, "workloads.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _sha(words) -> str:
    import numpy as np
    return hashlib.sha256(np.ascontiguousarray(words).view(np.uint8).tobytes()).hexdigest()


SAMPLE_STRIDE = 4099


def parity(args) -> dict:
    """For every case: the reference packer's words (hash + a strided sample)
    and the reference GPU kernel's result on them, saved to <outdir>/<case>.npz."""
    import numpy as np
    import torch
    P, G, D = _import_reference()
    W = _workloads()
    os.makedirs(args.outdir, exist_ok=True)
    done = {}
    for name in args.cases.split(","):
        t0 = time.time()
        a, b, mode = W.make(name, "cuda")
        if W.is_attention(name):
            # feather/routines/attention.py:110-179 on the reference packer's words of q, k, v
            from feather.routines import attention as A
            seq, d = a[0].shape
            words = [P.pack_fp8_tensor(t, mode=mode) for t in a]
            dev = [w.view(torch.uint32).to("cuda") for w in words]
            rec = {"q_sha": _sha(words[0].numpy().view(np.uint32)), "k_sha": _sha(words[1].numpy().view(np.uint32)),
                   "v_sha": _sha(words[2].numpy().view(np.uint32))}
            try:
                rec["out"] = A.flash_attention_fp8_e5m2_acc_fp32_gpu(dev[0], dev[1], dev[2], seq, d // 4).cpu().numpy()
                torch.cuda.synchronize()
            except Exception as e:      # e.g. the kernel's tiles do not fit this GPU
                rec["failed"] = type(e).__name__ + ": " + str(e)[:300]
            np.savez(os.path.join(args.outdir, name + ".npz"), **rec)
            done[name] = {"seconds": round(time.time() - t0, 2), "failed": "failed" in rec}
            continue
        aw = P.pack_fp8_tensor(a, mode=mode)          # CPU uint32, feather/packers/fp8.py:260
        bw = P.pack_fp8_tensor(b, mode=mode)
        t_pack = time.time() - t0
        ag, bg = aw.view(torch.uint32).to("cuda"), bw.view(torch.uint32).to("cuda")
        if W.is_dot(name):
            y = D.dot_fp8_e5m2_acc_fp32_gpu(ag, bg)    # feather/routines/dot.py:220
            y2 = D.dot_fp8_e5m2_acc_fp32_gpu(ag, bg)   # float atomics: a second run shows the spread
            out = np.array([y.item(), y2.item()], dtype=np.float32)
        else:
            fn = G.gemv_fp8_e5m2_acc_fp32_gpu if mode == "E5M2" else G.gemv_fp8_e4m3_acc_fp32_gpu
            out = fn(ag, bg, tuple(a.shape)).cpu().numpy()   # feather/routines/gemv.py:136, :187
        torch.cuda.synchronize()
        awn, bwn = aw.numpy().view(np.uint32), bw.numpy().view(np.uint32)
        np.savez(os.path.join(args.outdir, name + ".npz"), out=out,
                 a_sha=_sha(awn), b_sha=_sha(bwn), a_sample=awn[::SAMPLE_STRIDE].copy(),
                 b_sample=bwn[::SAMPLE_STRIDE].copy(), a_words=np.int64(awn.size))
        done[name] = {"seconds": round(time.time() - t0, 2), "pack_seconds": round(t_pack, 2)}
        del a, b, aw, bw, ag, bg
    return {"cases": done}


def _codes(torch, n_words: int, seed: int):
    g = torch.Generator(device="cuda").manual_seed(seed)
    w = torch.randint(-2 ** 31, 2 ** 31 - 1, (n_words,), device="cuda", dtype=torch.int64,
                      generator=g).to(torch.int32)
    # finite codes in both formats: clear the top exponent bit of every byte
    return (w & 0x3F3F3F3F | (w & (0x80808080 - 2 ** 32))).view(torch.uint32)


def _time(torch, fn, iters: int, warmup: int = 20) -> float:
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for i in range(iters):
        fn(i)
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) * 1e3 / iters   # microseconds


def timing(args) -> dict:
    """Microseconds per call of the reference's Triton kernels on this GPU:
    kernel only (the jitted kernel launched as its wrapper launches it, output
    pre-allocated) and through the public wrapper (which allocates the output on
    the CPU and copies it to the device on every call).  Four operand sets are
    rotated so that no call finds its matrix in L2."""
    import torch
    P, G, D = _import_reference()
    res = {"gpu": torch.cuda.get_device_name(0)}
    import triton
    res["triton"] = triton.__version__
    n_buf = 4
    for mode, kern, wrap, shapes in (
            ("E5M2", G._gemv_fp8_e5m2_acc_fp32_kernel, G.gemv_fp8_e5m2_acc_fp32_gpu,
             ((16384, 16384), (8192, 8192), (16384, 8192))),
            ("E4M3", G._gemv_fp8_e4m3_acc_fp32_kernel, G.gemv_fp8_e4m3_acc_fp32_gpu,
             ((16384, 16384), (8192, 8192), (16384, 8192)))):
        mats = [_codes(torch, 16384 * 16384 // 4, 1 + s) for s in range(n_buf)]
        v_all = _codes(torch, 16384 // 4, 9)
        for M, N in shapes:
            ms = [m[: M * N // 4] for m in mats]
            v = v_all[: N // 4]
            out = torch.empty(M, dtype=torch.float32, device="cuda")
            k_us = _time(torch, lambda i: kern[(M,)](ms[i % n_buf], v, out, N // 4, BLOCK_SIZE=1024),
                         args.iters)
            w_us = _time(torch, lambda i: wrap(ms[i % n_buf], v, (M, N)), args.iters)
            nbytes = M * N + N + 4 * M
            res[f"gemv_{mode.lower()}_{M}x{N}"] = {
                "kernel_us": round(k_us, 2), "kernel_GB/s": round(nbytes / k_us / 1e3, 1),
                "wrapper_us": round(w_us, 2), "wrapper_GB/s": round(nbytes / w_us / 1e3, 1)}
        del mats
    n_words = 1 << 24
    xs = [(_codes(torch, n_words, 20 + s), _codes(torch, n_words, 30 + s)) for s in range(n_buf)]
    out0 = torch.zeros((), dtype=torch.float32, device="cuda")
    grid = ((n_words + 1023) // 1024,)
    k_us = _time(torch, lambda i: D._dot_fp8_e5m2_acc_fp32_kernel[grid](*xs[i % n_buf], out0, n_words,
                                                                      BLOCK_SIZE=1024), args.iters)
    w_us = _time(torch, lambda i: D.dot_fp8_e5m2_acc_fp32_gpu(*xs[i % n_buf]), args.iters)
    res["dot_e5m2_2pow26"] = {"kernel_us": round(k_us, 2), "kernel_GB/s": round((8 * n_words + 4) / k_us / 1e3, 1),
                              "wrapper_us": round(w_us, 2)}
    del xs
    # attention through the public wrapper (its kernel is autotuned with a single
    # configuration; the wrapper allocates the output on the device)
    from feather.routines import attention as A
    for seq, d in ((4096, 128), (8192, 64), (8192, 128), (4096, 256), (4096, 512)):
        qkv = [_codes(torch, seq * d // 4, 50 + s) for s in range(3)]
        try:
            us = _time(torch, lambda i: A.flash_attention_fp8_e5m2_acc_fp32_gpu(qkv[0], qkv[1], qkv[2], seq, d // 4),
                       max(10, args.iters // 4), 3)
            res[f"attention_e5m2_seq{seq}_d{d}"] = {"wrapper_us": round(us, 2),
                                                      "TFLOP/s": round(4.0 * seq * seq * d / us / 1e6, 1)}
        except Exception as e:      # e.g. the kernel's tiles do not fit this GPU's shared memory
            res[f"attention_e5m2_seq{seq}_d{d}"] = {"failed": type(e).__name__ + ": " + str(e)[:200]}
    # torch.mv on the unpacked operands, for context
    for dt, name in ((torch.float16, "fp16"), (torch.float32, "fp32")):
        As = [torch.randn(16384, 16384, device="cuda", dtype=dt) for _ in range(2)]
        x = torch.randn(16384, device="cuda", dtype=dt)
        us = _time(torch, lambda i: torch.mv(As[i % 2], x), max(20, args.iters // 4), 5)
        res[f"torch_mv_{name}_16384x16384_us"] = round(us, 2)
        del As
    return res


def cpu_path(args) -> dict:
    """The reference's CPU path on the host cores: its packer
    (feather/packers/fp8.py:260-281), then a torch-CPU decode with the GPU
    kernels' bit semantics (feather/routines/gemv.py:31-34 and :83-88) and an
    FP32 torch.mv."""
    import numpy as np
    import torch
    P, _, _ = _import_reference()
    M, N = args.M, args.N
    torch.manual_seed(0)
    A = torch.randn(M, N).half()
    v = torch.randn(N).half()
    res = {"threads": torch.get_num_threads(), "cpu_count": os.cpu_count(), "M": M, "N": N}

    def decode(words: torch.Tensor, mode: str) -> torch.Tensor:
        c = words.view(torch.uint8).to(torch.int32)
        if mode == "E5M2":
            bits = c << 8
        else:
            e = (c >> 3) & 0xF
            bits = ((c & 0x80) << 8) | (torch.where(e > 0, e + 8, 0) << 10) | ((c & 7) << 7)
        return bits.to(torch.int16).view(torch.float16).float()

    for mode in ("E5M2", "E4M3"):
        t0 = time.perf_counter()
        mw = P.pack_fp8_tensor(A, mode=mode)
        t_pack = time.perf_counter() - t0
        vw = P.pack_fp8_tensor(v, mode=mode)
        reps, best = 3, 1e9
        for _ in range(reps):
            t0 = time.perf_counter()
            y = torch.mv(decode(mw, mode).view(M, N), decode(vw, mode))
            best = min(best, time.perf_counter() - t0)
        nbytes = M * N + N + 4 * M
        res[mode] = {"pack_s": round(t_pack, 4), "pack_Melem_per_s": round(M * N / t_pack / 1e6, 1),
                     "decode_mv_s": round(best, 4), "decode_mv_GB/s": round(nbytes / best / 1e9, 3),
                     "checksum": float(y.double().abs().sum())}
    return res


def main() -> None:
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="op", required=True)
    p = sub.add_parser("parity")
    p.add_argument("--cases", required=True)
    p.add_argument("--outdir", required=True)
    t = sub.add_parser("time")
    t.add_argument("--iters", type=int, default=200)
    c = sub.add_parser("cpu")
    c.add_argument("--M", type=int, default=4096)
    c.add_argument("--N", type=int, default=4096)
    args = ap.parse_args()
    try:
        res = {"parity": parity, "time": timing, "cpu": cpu_path}[args.op](args)
    except Exception as e:  # noqa: BLE001 - reported, not raised: the caller skips
        res = {"unavailable": f"{type(e).__name__}: {e}"[:400]}
    print("REFERENCE_WORKER " + json.dumps(res), flush=True)


if __name__ == "__main__":
    main()
