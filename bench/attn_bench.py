#!/usr/bin/env python
"""Causal attention on the fused QKV projection's output: this package's tcgen05 kernels against PyTorch's
scaled_dot_product_attention reached through views of the same tensor (what the model did before).

    python bench/attn_bench.py [--batch 16] [--seq 256] [--heads 8,12] [--iters 50]

Device time with CUDA events, a buffer larger than the L2 written between iterations, 5 warm-up iterations.
Both arms start from qkv [B, S, 3*H*64] and end with the [B, S, H*64] output (forward) or the gradient of qkv
(forward + backward), so the slices, transposes and concatenations the library path needs are part of its time.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import mccl_b200  # noqa: E402,F401
from mccl_b200 import ops  # noqa: E402


def sdpa_path(qkv: torch.Tensor, heads: int) -> torch.Tensor:
    B, S = qkv.shape[:2]
    q, k, v = (t.transpose(1, 2) for t in qkv.view(B, S, 3, heads, 64).unbind(2))
    return F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(B, S, heads * 64)


def timed(fn, iters: int, flush: torch.Tensor) -> float:
    for _ in range(5):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    return total / iters * 1e3


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--seq", type=int, default=256)
    ap.add_argument("--heads", default="8,12")
    ap.add_argument("--iters", type=int, default=50)
    args = ap.parse_args()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for heads in [int(h) for h in args.heads.split(",")]:
        B, S = args.batch, args.seq
        qkv = (torch.randn(B, S, 3 * heads * 64, device="cuda") * 0.5).bfloat16().requires_grad_(True)
        d_out = (torch.randn(B, S, heads * 64, device="cuda") * 0.5).bfloat16()
        flops_fwd = 2 * 2 * B * heads * S * S * 64 / 2     # two products, causal half
        row = {"batch": B, "seq": S, "heads": heads}
        for name, fn in (("mccl", lambda: ops.causal_attention(qkv, heads)), ("sdpa", lambda: sdpa_path(qkv, heads))):
            with torch.no_grad():
                row[f"{name}_fwd_us"] = round(timed(fn, args.iters, flush), 2)

            def both(f=fn):
                qkv.grad = None
                f().backward(d_out)
            row[f"{name}_fwd_bwd_us"] = round(timed(both, args.iters, flush), 2)
        row["fwd_speedup"] = round(row["sdpa_fwd_us"] / row["mccl_fwd_us"], 2)
        row["fwd_bwd_speedup"] = round(row["sdpa_fwd_bwd_us"] / row["mccl_fwd_bwd_us"], 2)
        row["mccl_fwd_tflops"] = round(flops_fwd / (row["mccl_fwd_us"] * 1e-6) / 1e12, 1)
        print(json.dumps(row), flush=True)


if __name__ == "__main__":
    main()
