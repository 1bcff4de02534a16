#!/usr/bin/env python
"""Flagship benchmark: DDP training throughput (samples/s) of the 70M decoder.

    python bench.py --gpus N --steps K --warmup W [--impl mccl|nccl|reference] [--model 70m|110m]

The metric and configuration are the reference's headline benchmark
(README.md:44-54): 70M decoder-only transformer (d_model 512, 16 layers,
8 heads, FFN 2048 GELU, pre-LayerNorm, learned positions, vocab 32000, tied
embeddings), batch 16 per GPU, sequence 256, AdamW lr 3e-4, bf16 compute with
fp32 master weights, synthetic token ids uniform in [0, 32000) from seed 0,
random-init weights.  Weak scaling: per-GPU batch fixed.

Arms:
  mccl       this repository: DDPTrainer over backend "mccl" (own kernels)
  nccl       stock PyTorch: DistributedDataParallel over backend "nccl", autocast bf16,
             fused AdamW (the measured baseline this repository has to beat)
  reference  the unmodified reference package from baseline/_ref; it only builds on
             macOS/arm64 (Metal), so this arm reports itself unavailable

Timing: W warm-up steps, then exactly K steps between CUDA events, bracketed by
barrier + synchronize on both sides, max over ranks.  The working set of one
step (fp32 parameters, gradients and both Adam moments, >1 GB) is far larger
than the 126 MB L2, so no explicit flush is needed between steps.  The
end-to-end figure repeats the K steps through DDPTrainer.step_from_host:
pinned-host tokens copied to the device and the loss read back every step.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

PUBLISHED_SAMPLES_PER_S = {"70m": 56.9, "110m": 35.9}  # reference, 3x Mac mini M4 (README.md:50,54)


def parse() -> argparse.Namespace:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="mccl", choices=["mccl", "nccl", "reference"])
    ap.add_argument("--model", default="70m", choices=["70m", "110m", "tiny"])
    ap.add_argument("--batch", type=int, default=16, help="per-GPU batch")
    ap.add_argument("--seq", type=int, default=256)
    ap.add_argument("--wire", default="bf16", choices=["bf16", "native"])
    ap.add_argument("--algo", default="auto")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-overlap", action="store_true")
    ap.add_argument("--bucket-mb", type=float, default=25.0)
    return ap.parse_args()


def reference_unavailable() -> None:
    print(json.dumps({
        "impl": "reference",
        "unavailable": "reference builds only on macOS/arm64 (Metal/MPS): its setup.py raises 'MCCL can only be built "
                       "on macOS' during the offline pip install into baseline/_ref",
    }))


def main() -> None:
    args = parse()
    if args.impl == "reference":
        reference_unavailable()
        return

    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)

    import mccl_b200
    from mccl_b200.models import build_decoder
    from mccl_b200.utils import ClockSampler

    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group(backend=("mccl" if args.impl == "mccl" else "nccl"), rank=rank, world_size=world,
                                device_id=device if args.impl == "nccl" else None)

    torch.manual_seed(0)
    model = build_decoder(args.model, native=(args.impl == "mccl"), max_seq=args.seq).to(device)
    cfg = model.cfg
    B, S = args.batch, args.seq

    # synthetic data: uniform token ids from seed 0 (each rank draws its own slice of the stream)
    g = torch.Generator().manual_seed(0)
    n_batches = 8
    stream = torch.randint(0, cfg.vocab, (n_batches, world, B, S + 1), generator=g)
    host_tokens = [stream[i, rank, :, :-1].contiguous().pin_memory() for i in range(n_batches)]
    host_targets = [stream[i, rank, :, 1:].contiguous().pin_memory() for i in range(n_batches)]
    dev_tokens = [t.to(device) for t in host_tokens]
    dev_targets = [t.to(device) for t in host_targets]

    launches = 0
    if args.impl == "mccl":
        from mccl_b200.parallel import DDPTrainer
        trainer = DDPTrainer(model, device, lr=3e-4, wire=args.wire, bucket_mb=args.bucket_mb,
                             overlap=not args.no_overlap, use_graph=not args.no_graph, algo=args.algo)

        def run_step(i):
            return trainer.step(dev_tokens[i % n_batches], dev_targets[i % n_batches])

        def run_step_e2e(i):
            return trainer.step_from_host(host_tokens[i % n_batches], host_targets[i % n_batches])
    else:
        from torch.nn.parallel import DistributedDataParallel as DDP
        net = DDP(model, device_ids=[local_rank], bucket_cap_mb=args.bucket_mb, gradient_as_bucket_view=True) if world > 1 else model
        opt = torch.optim.AdamW(model.parameters(), lr=3e-4, fused=True)

        def run_step(i):
            opt.zero_grad(set_to_none=True)
            with torch.autocast("cuda", dtype=torch.bfloat16):
                loss = net(dev_tokens[i % n_batches], dev_targets[i % n_batches])
            loss.backward()
            opt.step()
            return loss.detach()

        def run_step_e2e(i):
            tok = host_tokens[i % n_batches].to(device, non_blocking=True)
            tgt = host_targets[i % n_batches].to(device, non_blocking=True)
            opt.zero_grad(set_to_none=True)
            with torch.autocast("cuda", dtype=torch.bfloat16):
                loss = net(tok, tgt)
            loss.backward()
            opt.step()
            return float(loss.item())

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    def timed(fn, steps):
        sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        last = None
        for i in range(steps):
            last = fn(i)
        e1.record()
        sync()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, last

    for i in range(max(args.warmup, 3)):
        run_step(i)
    sampler = ClockSampler(local_rank).start() if rank == 0 else None
    ms, last_loss = timed(run_step, args.steps)
    clocks = sampler.stop() if sampler is not None else None
    if args.impl == "mccl":
        launches = trainer.launches_per_step * args.steps
        trainer.check()

    for i in range(3):
        run_step_e2e(i)
    ms_e2e, last_e2e = timed(run_step_e2e, args.steps)

    if rank == 0:
        global_batch = B * world
        value = global_batch * args.steps / (ms / 1e3)
        e2e_value = global_batch * args.steps / (ms_e2e / 1e3)
        pub = PUBLISHED_SAMPLES_PER_S.get(args.model)
        line = {
            "metric": "ddp_train_samples_per_sec",
            "value": round(value, 2),
            "unit": "samples/s",
            "impl": args.impl,
            "n_gpus": world,
            "steps": args.steps,
            "warmup": max(args.warmup, 3),
            "ms_per_step": round(ms / args.steps, 4),
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": round(value / pub, 2) if pub else None,
            "dtype": "bf16",
            "data": "synthetic: token ids uniform in [0, vocab) from seed 0; random-init weights",
            "config": {
                "model": f"decoder-{args.model} (d_model {cfg.d_model}, {cfg.n_layers} layers, {cfg.n_heads} heads, "
                         f"ffn {cfg.d_ff} {cfg.act}, {cfg.norm}, {cfg.pos} positions, vocab {cfg.vocab}, tied={cfg.tied})",
                "global_batch": global_batch,
                "per_gpu_batch": B,
                "seq_len": S,
                "optimizer": "AdamW lr 3e-4, fp32 master weights",
                "parallelism": f"dp{world}",
                "wire": args.wire if args.impl == "mccl" else "fp32 (NCCL)",
                "l2": "per-step working set (params, grads, Adam moments > 1 GB) exceeds the 126 MB L2; no flush needed",
                "cuda_graph": (args.impl == "mccl" and not args.no_graph),
            },
            "clocks": clocks,
            "e2e": {
                "value": round(e2e_value, 2),
                "unit": "samples/s",
                "ms_per_step": round(ms_e2e / args.steps, 4),
                "h2d_bytes_per_step": int(host_tokens[0].numel() * 8 * 2),
                "d2h_bytes_per_step": 4,
            },
            "gpu_launches": int(launches),
            "final_loss": float(last_loss.item()) if hasattr(last_loss, "item") else float(last_loss),
        }
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
