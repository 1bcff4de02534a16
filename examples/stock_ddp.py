"""Stock torch DistributedDataParallel over backend "mccl", with the bf16-wire hook.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 examples/stock_ddp.py

This is how the reference is used (README.md:20-40): nothing but the backend name changes.
"""
from __future__ import annotations

import os
import sys

import torch
import torch.distributed as dist
import torch.nn as nn
from torch.nn.parallel import DistributedDataParallel as DDP

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import mccl_b200  # noqa: E402,F401
from mccl_b200.parallel import bf16_wire_hook  # noqa: E402


def main() -> None:
    local = int(os.environ.get("LOCAL_RANK", "0"))
    use_cuda = torch.cuda.is_available()
    dev = torch.device("cuda", local) if use_cuda else torch.device("cpu")
    if use_cuda:
        torch.cuda.set_device(local)
    dist.init_process_group("mccl")
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(256, 1024), nn.GELU(), nn.Linear(1024, 256)).to(dev)
    ddp = DDP(model, device_ids=[local] if use_cuda else None)
    ddp.register_comm_hook(None, bf16_wire_hook)
    opt = torch.optim.AdamW(ddp.parameters(), lr=1e-3)
    x = torch.randn(64, 256, device=dev)
    for step in range(20):
        opt.zero_grad()
        loss = (ddp(x) - x).pow(2).mean()
        loss.backward()
        opt.step()
    if dist.get_rank() == 0:
        print(f"final loss {loss.item():.5f}")
        mccl_b200.metrics.log_metrics()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
