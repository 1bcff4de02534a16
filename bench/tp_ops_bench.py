"""Fused tensor-parallel GEMMs against the unfused baseline, shape by shape.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29521 \
        bench/tp_ops_bench.py --iters 20

For every GEMM of one 1.3B decoder layer under N-way tensor parallelism (tokens 16384, d_model
2048, FFN 8192) it times

* ``ag_gemm``   (one kernel: all-gather of the activation shard overlapped with the tcgen05 tiles)
  against ``all_gather_into_tensor`` + ``torch.matmul`` on the same `mccl` group's NCCL twin, and
* ``gemm_rs``   (one kernel: tiles stored into the owner's staging slot, in-kernel reduction)
  against ``torch.matmul`` + ``reduce_scatter_tensor``.

Device time from CUDA events around `iters` back-to-back calls, max over ranks.  The roofline
column is max(FLOPs / measured GEMM peak, NVLink bytes per GPU / 770 GB/s) / achieved time.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def timed(fn, iters, dev, group=None):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier(group=group)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters * 1e3], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return t.item()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--d-model", type=int, default=2048)
    ap.add_argument("--d-ff", type=int, default=8192)
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    import mccl_b200
    from mccl_b200 import _C
    dist.init_process_group(backend="mccl")
    nccl = dist.new_group(backend="nccl", device_id=dev)
    comm = mccl_b200.get_backend().device_comm(local)
    T, D, FF = args.tokens, args.d_model, args.d_ff
    rows = T // world
    tp = _C.TpGemm(comm, rows * D)
    sym = comm.symm_alloc(rows * D * 2)
    peak = 1.38e15
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        peak = json.load(open(p)).get("bf16_tflops_sustained", 1381.0) * 1e12
    link = 770e9
    results = []
    torch.manual_seed(rank)
    # all-gather -> GEMM: (name, N_out, weight stored [K, N]?)
    for name, n_out, w_kn in [("qkv fwd", 3 * D // world, False), ("gate_up fwd", 2 * FF // world, False),
                              ("proj dgrad", D // world, True), ("down dgrad", FF // world, True)]:
        x = torch.randn(rows, D, device=dev).bfloat16()
        sym.tensor(rank, 0, [rows, D], torch.bfloat16, local).copy_(x)
        w = (torch.randn(D, n_out, device=dev) if w_kn else torch.randn(n_out, D, device=dev)).bfloat16()
        full = torch.empty(T, D, dtype=torch.bfloat16, device=dev)

        def base():
            dist.all_gather_into_tensor(full, x, group=nccl)
            return torch.matmul(full, w if w_kn else w.t())

        t_f = timed(lambda: tp.ag_gemm(sym, 0, rows, w, w_kn), args.iters, dev)
        t_b = timed(base, args.iters, dev)
        flops = 2.0 * T * n_out * D
        nv = (world - 1) * rows * D * 2
        ideal = max(flops / peak, nv / link) * 1e6
        results.append(("ag_gemm " + name, T, n_out, D, t_f, t_b, ideal))
    # GEMM -> reduce-scatter: (name, K_local)
    for name, k_loc, w_kn in [("proj fwd", D // world, False), ("down fwd", FF // world, False),
                              ("qkv dgrad", 3 * D // world, True), ("gate_up dgrad", 2 * FF // world, True)]:
        x = torch.randn(T, k_loc, device=dev).bfloat16()
        w = (torch.randn(k_loc, D, device=dev) if w_kn else torch.randn(D, k_loc, device=dev)).bfloat16()
        out = torch.empty(rows, D, dtype=torch.bfloat16, device=dev)

        def base():
            y = torch.matmul(x, w if w_kn else w.t())
            dist.reduce_scatter_tensor(out, y, group=nccl)
            return out

        t_f = timed(lambda: tp.gemm_rs(x, w, w_kn), args.iters, dev)
        t_b = timed(base, args.iters, dev)
        flops = 2.0 * T * D * k_loc
        nv = (world - 1) * rows * D * 2
        ideal = max(flops / peak, nv / link) * 1e6
        results.append(("gemm_rs " + name, T, D, k_loc, t_f, t_b, ideal))
    torch.cuda.synchronize()
    tp.check_status()
    if rank == 0:
        print(f"world {world}; times in us (max over ranks); roofline = max(FLOPs / {peak / 1e12:.0f} TFLOP/s, NVLink bytes / 770 GB/s)")
        print(f"{'op':24} {'M':>6} {'N':>6} {'K':>6} {'fused':>8} {'nccl+cublas':>12} {'speedup':>8} {'roofline':>9} {'fused/roof':>10}")
        for name, m, n, k, tf, tb, ideal in results:
            print(f"{name:24} {m:6d} {n:6d} {k:6d} {tf:8.1f} {tb:12.1f} {tb / tf:8.2f} {ideal:9.1f} {ideal / tf:10.2f}")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
