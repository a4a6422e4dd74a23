"""Small launch driver for profiling one kernel of the path under ncu.

    python benchmark/ncu/profile_kernels.py --op gemv --mode E5M2 --M 16384 --N 16384

Modelled on the reference's feather/benchmark/ncu/profile_gemv.py (a warm-up
call, the measured calls, a synchronize).  Operands are random finite FP8 codes
generated on the device; two operand sets alternate so that a call never finds
its data in L2.  Prints one line per op with the CUDA-event time.
"""
from __future__ import annotations

import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import feather_b200 as fb  # noqa: E402


def _codes(n_words: int, seed: int) -> torch.Tensor:
    g = torch.Generator(device="cuda").manual_seed(seed)
    w = torch.randint(-2 ** 31, 2 ** 31 - 1, (n_words,), device="cuda", dtype=torch.int64,
                      generator=g).to(torch.int32)
    return w & 0x3F3F3F3F | (w & (0x80808080 - 2 ** 32))  # keep sign, clear the top exponent bit


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", choices=("gemv", "dot", "encode", "decode", "relu", "multi", "packed", "attention",
                                     "chain"), default="gemv")
    ap.add_argument("--layers", type=int, default=1, help="layers of the TinyLlama-shaped chain for --op chain")
    ap.add_argument("--batch", type=int, default=8, help="vectors per call for --op multi")
    ap.add_argument("--mode", choices=("E5M2", "E4M3"), default="E5M2")
    ap.add_argument("--M", type=int, default=16384)
    ap.add_argument("--N", type=int, default=16384)
    ap.add_argument("--launches", type=int, default=3)
    a = ap.parse_args()
    M, N = a.M, a.N
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if a.op == "chain":
        # the TinyLlama-shaped GEMV chain (a.layers layers + lm_head) as ONE launch; two weight
        # sets alternate so that a launch never finds its weights in L2
        from feather_b200 import chain
        chains = [chain.PersistentGemvChain.from_chain(chain.GemvChain(a.mode, seed=6 + i, layers=a.layers))
                  for i in range(2)]
        call = lambda i: chains[i % 2].token()
        nbytes = a.layers * sum(m * n for _, m, n in chain.LAYER_SHAPES) + chain.VOCAB * chain.HIDDEN
        M, N = a.layers, 0
    elif a.op == "gemv":
        mats = [_codes(M * N // 4, s) for s in (1, 2)]
        v = _codes(N // 4, 3)
        out = torch.empty(M, dtype=torch.float32, device="cuda")
        call = lambda i: fb.gemv_fp8_acc_fp32_gpu(mats[i % 2], v, (M, N), a.mode, out=out)
        nbytes = M * N + N + 4 * M
    elif a.op == "dot":
        xs = [(_codes(M * N // 4, s), _codes(M * N // 4, s + 10)) for s in (1, 2)]
        call = lambda i: fb.dot_fp8_acc_fp32_gpu(*xs[i % 2], a.mode)
        nbytes = 2 * M * N + 4
    elif a.op == "encode":
        g = torch.Generator(device="cuda").manual_seed(1)
        xs = [torch.randn(M, N, device="cuda", generator=g, dtype=torch.float16) for _ in range(2)]
        call = lambda i: fb.pack_fp8_tensor(xs[i % 2], a.mode)
        nbytes = 3 * M * N
    elif a.op == "multi":
        mats = [_codes(M * N // 4, s) for s in (1, 2)]
        v = _codes(a.batch * N // 4, 3)
        out = torch.empty(a.batch, M, dtype=torch.float32, device="cuda")
        call = lambda i: fb.gemv_fp8_multi_acc_fp32_gpu(mats[i % 2], v, (M, N), a.mode, batch=a.batch, out=out)
        nbytes = M * N + a.batch * (N + 4 * M)
    elif a.op == "packed":
        mats = [_codes(M * N // 4, s) for s in (1, 2)]
        v = _codes(N // 4, 3)
        out = torch.empty((M + 3) // 4, dtype=torch.uint32, device="cuda")
        call = lambda i: fb.gemv_fp8_ret_packed_gpu(mats[i % 2], v, (M, N), a.mode, out=out)
        nbytes = M * N + N + M
    elif a.op == "attention":   # --M = sequence length, --N = model dimension (16 .. 128)
        from feather_b200.routines.attention import flash_attention_fp8_e5m2_acc_fp32_gpu as attn
        qkv = [[_codes(M * N // 4, s + 3 * i) for s in (1, 2, 3)] for i in range(2)]
        out = torch.empty(M, N, dtype=torch.float32, device="cuda")
        call = lambda i: attn(*qkv[i % 2], M, N // 4, out=out)
        nbytes = 3 * M * N + 4 * M * N
    elif a.op == "relu":
        from feather_b200.routines.activations import relu1d_fp8_ret_fp32_feather_gpu as relu
        ws = [_codes(M * N // 4, s) for s in (1, 2)]
        out = torch.empty(M * N, dtype=torch.float32, device="cuda")
        call = lambda i: relu(ws[i % 2], M * N, mode=a.mode, out=out)
        nbytes = 5 * M * N
    else:
        ws = [_codes(M * N // 4, s) for s in (1, 2)]
        call = lambda i: fb.unpack_fp8_tensor(ws[i % 2], a.mode)
        nbytes = 5 * M * N
    call(0)  # warm-up
    torch.cuda.synchronize()
    start.record()
    for i in range(a.launches):
        call(i + 1)
    end.record()
    torch.cuda.synchronize()
    us = start.elapsed_time(end) * 1e3 / a.launches
    print(f"{a.op} {a.mode} {M}x{N}: {us:.2f} us/launch, {nbytes / us / 1e3:.1f} GB/s algorithmic")


if __name__ == "__main__":
    main()
