"""Data-parallel training of a decoder with the graph-captured engine.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 examples/ddp_train.py --model 70m

Mirrors the reference's example trainer (examples/ddp_dummy_train.py): synthetic
token batches, a fixed number of steps, throughput and the backend's metrics at
the end.  Runs on one GPU without a process group as well.
"""
from __future__ import annotations

import argparse
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import mccl_b200  # noqa: E402
from mccl_b200.models import build_decoder  # noqa: E402
from mccl_b200.parallel import DDPTrainer  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="70m", choices=["tiny", "70m", "110m"])
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--batch", type=int, default=16, help="per GPU")
    ap.add_argument("--seq", type=int, default=256)
    ap.add_argument("--wire", default="bf16", choices=["bf16", "native"])
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("mccl")
    torch.manual_seed(0)
    model = build_decoder(args.model, native=True).to(dev)
    seq = min(args.seq, model.cfg.max_seq)
    trainer = DDPTrainer(model, dev, lr=3e-4, wire=args.wire)
    g = torch.Generator().manual_seed(1 + (dist.get_rank() if world > 1 else 0))
    tokens = torch.randint(0, model.cfg.vocab, (args.batch, seq + 1), generator=g).pin_memory()
    inp, tgt = tokens[:, :-1].contiguous().pin_memory(), tokens[:, 1:].contiguous().pin_memory()
    for _ in range(5):
        trainer.step_from_host(inp, tgt)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for step in range(args.steps):
        loss = trainer.step_from_host(inp, tgt)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    trainer.check()
    if world == 1 or dist.get_rank() == 0:
        print(f"{args.model}: {args.steps} steps, loss {loss:.4f}, {args.steps * args.batch * world / dt:.1f} samples/s "
              f"({dt / args.steps * 1e3:.2f} ms/step, {trainer.launches_per_step} kernel launches per step)")
        mccl_b200.metrics.log_metrics()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
