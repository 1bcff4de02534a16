#!/usr/bin/env python
"""Collective sweep: bus bandwidth of every schedule against NCCL, 1 KB - 1 GB.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port 29533 bench/collective_sweep.py [--max-mb 1024] [--ops allreduce,allgather,...]

One process per GPU.  The default group uses backend "mccl"; a second group on
backend "nccl" runs the same operations on the same buffers for comparison.
Values are N(0,1) per rank from seed=rank.  Every number is device-timed (CUDA
events around `iters` back-to-back calls after warm-up), reduced with MAX over
ranks, and reported as bus bandwidth with the usual factors (allreduce
2(N-1)/N, allgather / reduce_scatter / alltoall (N-1)/N) next to the 900 GB/s
per-direction NVLink 5 figure.  Buffers rotate through a pool larger than the
L2 for small messages so that repeated calls do not just hit in cache.

Follows the reference's own sweep (tests/multinode/bench.py:66-111: allreduce
timing at 1 KB ... 4 MB), extended to every collective, schedule and wire type.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import mccl_b200  # noqa: E402

NVLINK_GBS = 900.0


def bus_factor(op: str, n: int) -> float:
    return 2.0 * (n - 1) / n if op == "allreduce" else (n - 1) / n


def timed(fn, iters: int, device) -> float:
    for _ in range(max(3, iters // 10)):
        fn()
    torch.cuda.synchronize(device)
    dist.barrier()
    torch.cuda.synchronize(device)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize(device)
    t = torch.tensor([e0.elapsed_time(e1) / iters * 1e3], device=device)  # us
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--max-mb", type=float, default=1024.0)
    ap.add_argument("--min-kb", type=float, default=1.0)
    ap.add_argument("--ops", default="allreduce,allgather,reduce_scatter,alltoall")
    ap.add_argument("--algos", default="oneshot,twoshot,twoshot_push,ring,tree,nvls,symm,auto")
    ap.add_argument("--size-step", type=int, default=2, help="ratio between consecutive message sizes")
    ap.add_argument("--ctas", type=int, default=0, help="cap on CTAs per collective kernel (0 = default)")
    ap.add_argument("--threads", type=int, default=0, help="threads per collective CTA (0 = default)")
    ap.add_argument("--dtypes", default="fp32,fp32+bf16wire,bf16")
    ap.add_argument("--out", default="")
    args = ap.parse_args()

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    os.environ.setdefault("MCCL_ARENA_MB", "1024")
    dist.init_process_group("mccl", rank=rank, world_size=world)
    nccl = dist.new_group(backend="nccl")
    comm = mccl_b200.get_backend().device_comm(local)
    if args.ctas or args.threads:
        comm.set_launch_shape(args.ctas, args.threads)
    warm = torch.ones(1024, device=device)
    dist.all_reduce(warm, group=nccl)

    sizes = []
    s = int(args.min_kb * 1024)
    while s <= int(args.max_mb * (1 << 20)):
        sizes.append(s)
        s *= max(args.size_step, 2)
    rows = []
    symm_cache = {}
    ops = args.ops.split(",")
    for op in ops:
        for dt_name in args.dtypes.split(","):
            dtype = torch.bfloat16 if dt_name == "bf16" else torch.float32
            wire = "bf16" if dt_name.endswith("bf16wire") else "native"
            if op != "allreduce" and dt_name != "fp32":
                continue
            es = 2 if dtype == torch.bfloat16 else 4
            for nbytes in sizes:
                numel = max(world, nbytes // es // world * world)
                if op == "allgather":
                    numel = max(1, numel // world)   # per-rank input; the gathered buffer has `nbytes`
                pool = max(1, min(16, (256 << 20) // max(nbytes, 1)))
                g = torch.Generator(device="cpu").manual_seed(rank)
                base = torch.randn(min(numel, 1 << 20), generator=g).to(dtype)
                bufs = [base.repeat((numel + base.numel() - 1) // base.numel())[:numel].to(device).contiguous() for _ in range(pool)]
                iters = 200 if nbytes <= (1 << 20) else (50 if nbytes <= (64 << 20) else 10)
                state = {"i": 0}

                def nxt():
                    state["i"] = (state["i"] + 1) % pool
                    return bufs[state["i"]]

                variants = []
                if op == "allreduce":
                    for algo in args.algos.split(","):
                        if algo == "symm":
                            continue
                        if algo == "nvls" and not comm.nvls_available:
                            continue
                        if algo in ("oneshot", "tree") and nbytes > (64 << 20):
                            continue  # latency schedules: not meaningful (and arena-bound) for huge messages
                        variants.append((f"mccl:{algo}", lambda a=algo: (lambda t: comm.allreduce([t], [t], op="sum", algo=a, wire=wire))(nxt())))
                    if wire == "native" and nbytes >= (64 << 10) and "symm" in args.algos.split(","):
                        # buffer registered in the symmetric heap: reduced in place, no staging copies
                        padded = ((numel + world - 1) // world + 15) // 16 * 16 * world
                        if nbytes not in symm_cache:
                            symm_cache.clear()
                            symm_cache[nbytes] = comm.symm_alloc(padded * es)
                        sb = symm_cache[nbytes]
                        variants.append(("mccl:symm", lambda: comm.allreduce_symm(sb, 0, numel, dtype, "sum")))
                    if wire == "native":
                        variants.append(("nccl", lambda: dist.all_reduce(nxt(), group=nccl)))
                elif op == "allgather":
                    outs = [torch.empty(numel * world, dtype=dtype, device=device) for _ in range(min(pool, 2))]
                    variants.append(("mccl", lambda: comm.allgather([nxt()], [outs[state["i"] % len(outs)]])))
                    variants.append(("nccl", lambda: dist.all_gather_into_tensor(outs[state["i"] % len(outs)], nxt(), group=nccl)))
                elif op == "reduce_scatter":
                    outs = [torch.empty(numel // world, dtype=dtype, device=device)]
                    variants.append(("mccl", lambda: comm.reduce_scatter([nxt()], [outs[0]], op="sum", wire=wire)))
                    variants.append(("nccl", lambda: dist.reduce_scatter_tensor(outs[0], nxt(), group=nccl)))
                elif op == "alltoall":
                    outs = [torch.empty(numel, dtype=dtype, device=device)]
                    sp = [[numel // world] * world]
                    variants.append(("mccl", lambda: comm.alltoallv([nxt()], [outs[0]], sp, sp)))
                    variants.append(("nccl", lambda: dist.all_to_all_single(outs[0], nxt(), group=nccl)))
                for name, fn in variants:
                    us = timed(fn, iters, device)
                    comm.check_status()
                    # message size in the nccl-tests sense: the full gathered buffer for allgather
                    msg = numel * es * (world if op == "allgather" else 1)
                    busbw = msg / (us * 1e-6) / 1e9 * bus_factor(op, world)
                    row = {"op": op, "dtype": dt_name, "bytes": msg, "impl": name, "us": round(us, 2),
                           "busbw_gbs": round(busbw, 2), "frac_of_900": round(busbw / NVLINK_GBS, 3), "world": world,
                           "ctas": comm.max_ctas, "threads": comm.launch_threads}
                    rows.append(row)
                    if rank == 0:
                        print(json.dumps(row), flush=True)
                del bufs
    if rank == 0 and args.out:
        with open(args.out, "w") as f:
            json.dump(rows, f, indent=1)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
