"""Times the host (TCP) path: allreduce of 1 048 576 fp32 elements with every algorithm and wire type, then
allgather / reduce_scatter / alltoall, between CPU ranks on loopback.  No GPU needed.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 bench/cpu_plumbing.py
"""
from __future__ import annotations

import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import mccl_b200  # noqa: E402,F401


def timed(fn, iters=10):
    fn()
    dist.barrier()
    t0 = time.perf_counter()
    for _ in range(iters):
        fn()
    dist.barrier()
    return (time.perf_counter() - t0) / iters * 1e3


def main() -> None:
    dist.init_process_group("mccl")
    rank, world = dist.get_rank(), dist.get_world_size()
    n = 1 << 20
    g = torch.Generator().manual_seed(rank)
    x = torch.randn(n, generator=g)
    rows = []
    for algo in ("ring", "tree", "butterfly"):
        for wire in ("", "bf16"):
            os.environ["MCCL_ALLREDUCE_ALGO"] = algo
            if wire:
                os.environ["MCCL_WIRE_DTYPE"] = wire
            else:
                os.environ.pop("MCCL_WIRE_DTYPE", None)
            t = x.clone()
            ms = timed(lambda: dist.all_reduce(t))
            rows.append((f"allreduce {algo}{' + bf16 wire' if wire else ''}", ms))
    os.environ.pop("MCCL_ALLREDUCE_ALGO", None)
    os.environ.pop("MCCL_WIRE_DTYPE", None)
    out = torch.empty(world * n)
    rows.append(("allgather", timed(lambda: dist.all_gather_into_tensor(out, x))))
    rs = torch.empty(n // world)
    rows.append(("reduce_scatter", timed(lambda: dist.reduce_scatter_tensor(rs, x[: n // world * world]))))
    a2a = torch.empty(n // world * world)
    rows.append(("alltoall", timed(lambda: dist.all_to_all_single(a2a, x[: n // world * world]))))
    if rank == 0:
        print(f"world {world}, 1 048 576 fp32 elements (4 MiB) per rank, loopback TCP, wall time per call")
        for name, ms in rows:
            print(f"  {name:32s} {ms:8.2f} ms   {4.194304 / ms:6.2f} GB/s of payload")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
