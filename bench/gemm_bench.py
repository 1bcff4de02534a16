#!/usr/bin/env python
"""Times the tcgen05 GEMM on the shapes of the decoder configurations against
torch.matmul (cuBLAS), one shape per line.

Each measurement: 5 warm-up launches, then `--iters` launches between CUDA
events with a 256 MB buffer rewritten before every launch so that operands
are not served from L2.  Prints TFLOP/s for both and the fraction of the
measured cuBLAS bf16 peak read from MEASURED_PEAKS.json when present.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import mccl_b200  # noqa: E402

C = mccl_b200._C


def shapes(model: str):
    d, ff, v, t = {"70m": (512, 2048, 32000, 4096), "110m": (768, 3072, 32000, 4096), "1.3b": (2048, 8192, 32000, 16384)}[model]
    fwd = [(t, 3 * d, d), (t, d, d), (t, ff, d), (t, d, ff), (t, v, d)]
    out = []
    for (m, n, k) in fwd:
        out.append(("fwd", m, n, k, False, False))
        out.append(("dgrad", m, k, n, False, True))     # dx[M,K] = dy[M,N] W[N,K]
        out.append(("wgrad", n, k, m, True, True))      # dW[N,K] = dy^T x
    return out


def time_fn(fn, iters, flush):
    for _ in range(5):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        flush.add_(1.0)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    return total / iters * 1e3  # us


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="70m")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--shape", type=int, nargs=3, metavar=("M", "N", "K"), help="time one forward GEMM of this shape only")
    ap.add_argument("--kernel", default="", choices=["", "pair", "persistent", "tile"],
                    help="which of this package's GEMM kernels to time (default: the package's default, CTA pairs)")
    args = ap.parse_args()
    if args.kernel:
        C.set_gemm_kernel(args.kernel)
    peak = None
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        peak = json.load(open(p)).get("bf16_tflops")
    flush = torch.zeros(64 << 20, device="cuda")
    print(f"{'kind':6} {'M':>6} {'N':>6} {'K':>6} {'ours us':>9} {'TF/s':>7} {'cublas us':>10} {'TF/s':>7} {'ours/cublas':>11} {'of peak':>8}")
    todo = [("fwd", *args.shape, False, False)] if args.shape else shapes(args.model)
    for kind, m, n, k, a_t, b_t in todo:
        a = torch.randn(m, k, device="cuda").bfloat16()
        b = torch.randn(n, k, device="cuda").bfloat16()
        aa = a.t().contiguous() if a_t else a
        bb = b.t().contiguous() if b_t else b
        fp32 = kind == "wgrad"
        ours = time_fn(lambda: C.gemm_bf16(aa, bb, None, "none", fp32, None, False, a_t, b_t), args.iters, flush)
        if kind == "fwd":
            ref = time_fn(lambda: torch.matmul(a, b.t()), args.iters, flush)
        elif kind == "dgrad":
            ref = time_fn(lambda: torch.matmul(a, bb), args.iters, flush)
        else:
            ref = time_fn(lambda: torch.matmul(aa.t(), bb).float(), args.iters, flush)
        fl = 2.0 * m * n * k
        frac = f"{fl / ours / 1e6 / peak:8.2f}" if peak else "     n/a"
        print(f"{kind:6} {m:6d} {n:6d} {k:6d} {ours:9.1f} {fl / ours / 1e6:7.1f} {ref:10.1f} {fl / ref / 1e6:7.1f} {ref / ours:11.2f} {frac}")
    assert C.gemm_error_flag() == 0


if __name__ == "__main__":
    main()
