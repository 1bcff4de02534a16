"""Tensor-parallel decoder step with the fused all-gather→GEMM and GEMM→reduce-scatter kernels.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 examples/tensor_parallel.py

The reference ships ``tensor_parallel_split`` only and points to hand-wired column / row
parallel layers (mccl/distributed/sharding.py:54-69, README.md:76); these are the layers.
"""
from __future__ import annotations

import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import mccl_b200  # noqa: E402,F401
from mccl_b200.parallel import TensorParallelContext, TPDecoder  # noqa: E402


def main() -> None:
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("mccl")
    world = dist.get_world_size()
    cfg = dict(vocab=8192, d_model=1024, n_layers=4, n_heads=16, d_ff=4096, batch=4, seq=1024)
    ctx = TensorParallelContext(device=dev, max_rows_local=cfg["batch"] * cfg["seq"] // world, max_features=cfg["d_model"])
    torch.manual_seed(1 + dist.get_rank())
    model = TPDecoder(ctx, **cfg).to(dev)
    for p in model.replicated_parameters():
        dist.broadcast(p.data, 0)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-4, fused=True)
    g = torch.Generator().manual_seed(0)
    tokens = torch.randint(0, cfg["vocab"], (cfg["batch"], cfg["seq"] + 1), generator=g).to(dev)
    for step in range(10):
        opt.zero_grad(set_to_none=True)
        loss = model(tokens[:, :-1].contiguous(), tokens[:, 1:].contiguous())
        loss.backward()
        model.sync_replicated_grads()
        opt.step()
        total = loss.detach().clone()
        dist.all_reduce(total)
        if dist.get_rank() == 0:
            print(f"step {step}: loss {total.item():.4f}")
    ctx.check()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
