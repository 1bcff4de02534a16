#!/usr/bin/env python
"""A/B runs of the data-parallel step: how the bucket collectives share the GPU with backward.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench/ddp_overlap_sweep.py [--model 70m] [--steps 20] [--configs a,b,...] [--out FILE]

One process per GPU runs every configuration in turn (same model, same data), times K steps with CUDA
events (max over ranks) and then records one step with the device timeline (stamps written by the GEMM
and collective kernels themselves), whose summary says for every bucket collective when it started, how
long it ran, on how many SMs, and which share of its lifetime a GEMM was running beside it.
"""
from __future__ import annotations

import argparse
import gc
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# name: (overlap, comm_sms, comm_threads, wire, bucket_mb, overlap_optimizer)
CONFIGS = {
    "inline": (False, 0, 0, "bf16", 25.0, False),
    "shared256": (True, 0, 0, "bf16", 25.0, True),
    "shared256_noopt": (True, 0, 0, "bf16", 25.0, False),
    "sm12": (True, 12, 512, "bf16", 25.0, True),
    "sm20": (True, 20, 512, "bf16", 25.0, True),
    "sm12nvls": (True, 12, 512, "native", 25.0, True),
    "sm8": (True, 8, 512, "bf16", 25.0, True),
    "sm16": (True, 16, 512, "bf16", 25.0, True),
    "sm16_noopt": (True, 16, 512, "bf16", 25.0, False),
    "sm24": (True, 24, 512, "bf16", 25.0, True),
    "sm16x256": (True, 16, 256, "bf16", 25.0, True),
    "nvls": (True, 0, 0, "native", 25.0, True),
    "sm16nvls": (True, 16, 512, "native", 25.0, True),
    "sm8nvls": (True, 8, 512, "native", 25.0, True),
    "shared256b10": (True, 0, 0, "bf16", 10.0, True),
    "shared256b50": (True, 0, 0, "bf16", 50.0, True),
}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="70m")
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--seq", type=int, default=256)
    ap.add_argument("--configs", default="inline,shared256,sm8,sm16,sm24,sm16nvls")
    ap.add_argument("--out", default="")
    ap.add_argument("--no-timeline", action="store_true")
    ap.add_argument("--gemm-shapes", action="store_true", help="also list the in-step time of every GEMM shape")
    args = ap.parse_args()

    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    os.environ.setdefault("MCCL_DEVICE_TIMEOUT_MS", "20000")

    import mccl_b200  # noqa: F401
    from mccl_b200.models import build_decoder
    from mccl_b200.parallel import DDPTrainer
    from mccl_b200.utils import timeline

    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group(backend="mccl", rank=rank, world_size=world)
    if not args.no_timeline:
        timeline.enable(local_rank, capacity=1 << 17, every=1)

    g = torch.Generator().manual_seed(0)
    tokens = torch.randint(0, 32000, (4, world, args.batch, args.seq + 1), generator=g)
    toks = [tokens[i, rank, :, :-1].contiguous().to(device) for i in range(4)]
    tgts = [tokens[i, rank, :, 1:].contiguous().to(device) for i in range(4)]

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    lines = []
    for name in args.configs.split(","):
        overlap, comm_sms, comm_threads, wire, bucket_mb, overlap_opt = CONFIGS[name]
        torch.manual_seed(0)
        model = build_decoder(args.model, native=True, max_seq=args.seq).to(device)
        trainer = DDPTrainer(model, device, lr=3e-4, wire=wire, bucket_mb=bucket_mb, overlap=overlap,
                             comm_sms=comm_sms, comm_threads=comm_threads, overlap_optimizer=overlap_opt)
        for i in range(4):
            trainer.step(toks[i % 4], tgts[i % 4])
        best = None
        for rep in range(3):
            sync()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(args.steps):
                trainer.step(toks[i % 4], tgts[i % 4])
            e1.record()
            sync()
            ms = e0.elapsed_time(e1) / args.steps
            if world > 1:
                t = torch.tensor([ms], device=device)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = float(t.item())
            best = ms if best is None else min(best, ms)
        trainer.check()
        summary = ""
        if not args.no_timeline:
            sync()
            timeline.drain(local_rank)
            trainer.step(toks[0], tgts[0])
            torch.cuda.synchronize(device)
            recs = timeline.drain(local_rank)
            summary = timeline.summarize(recs, shapes=args.gemm_shapes)
        if rank == 0:
            head = {"config": name, "n_gpus": world, "model": args.model, "ms_per_step": round(best, 4),
                    "overlap": overlap, "comm_sms": comm_sms, "comm_threads": comm_threads, "wire": wire,
                    "bucket_mb": bucket_mb, "overlap_optimizer": trainer.overlap_optimizer, "buckets": len(trainer.buckets)}
            lines.append(json.dumps(head))
            if summary:
                lines.append(summary)
            print(lines[-2] if summary else lines[-1], flush=True)
            if summary:
                print(summary, flush=True)
        del trainer, model
        gc.collect()
        torch.cuda.empty_cache()
        sync()
    if rank == 0 and args.out:
        with open(args.out, "w") as f:
            f.write("\n".join(lines) + "\n")
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
