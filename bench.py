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

Timing: W warm-up steps, then a region of exactly K steps between CUDA events,
bracketed by barrier + synchronize on both sides, max over ranks.  The region
is repeated R times (--repeats, 5 by default); `value` is the median region and
`repeats` carries every region's time.  The working set of one step (fp32
parameters, gradients and both Adam moments, >1 GB) is far larger than the
126 MB L2, so no explicit flush is needed between steps.  The end-to-end figure
repeats the K steps through DDPTrainer.step_from_host: pinned-host tokens copied
to the device and the loss read back every step.  SM clocks and throttle reasons
are sampled with nvidia-smi over the whole measured span.  Unless --no-nccl-arm
is given, the same invocation then times the `nccl` arm (same model, data, K and
W) and reports it under `nccl_arm`, so one record carries both.
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

# The reference's published numbers are for other hardware (3x Mac mini M4 over Thunderbolt, README.md:50,54); they
# are carried as context, not as a denominator: nothing was published for this hardware, so vs_baseline is null.
PUBLISHED_OTHER_HARDWARE = {"70m": 56.9, "110m": 35.9}


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
    ap.add_argument("--repeats", type=int, default=5, help="timed regions of --steps steps each; the median is reported")
    ap.add_argument("--no-nccl-arm", action="store_true", help="do not also time the nccl arm in this invocation")
    ap.add_argument("--comm-sms", type=int, default=None)
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

    import statistics

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

    def make_mccl_arm():
        from mccl_b200.parallel import DDPTrainer
        trainer = DDPTrainer(model, device, lr=3e-4, wire=args.wire, bucket_mb=args.bucket_mb,
                             overlap=not args.no_overlap, use_graph=not args.no_graph, algo=args.algo, comm_sms=args.comm_sms)

        def run_step(i):
            return trainer.step(dev_tokens[i % n_batches], dev_targets[i % n_batches])

        def run_step_e2e(i):
            return trainer.step_from_host(host_tokens[i % n_batches], host_targets[i % n_batches])
        return trainer, run_step, run_step_e2e

    def make_nccl_arm(net_model, group):
        from torch.nn.parallel import DistributedDataParallel as DDP
        net = (DDP(net_model, device_ids=[local_rank], bucket_cap_mb=args.bucket_mb, gradient_as_bucket_view=True,
                   process_group=group) if world > 1 else net_model)
        opt = torch.optim.AdamW(net_model.parameters(), lr=3e-4, fused=True)

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
        return run_step, run_step_e2e

    def measure(run_step, run_step_e2e, repeats):
        """W warm-up steps, `repeats` regions of K steps each, then the same through the end-to-end call."""
        for i in range(max(args.warmup, 3)):
            run_step(i)
        regions, last = [], None
        for _ in range(max(repeats, 1)):
            ms, last = timed(run_step, args.steps)
            regions.append(ms)
        for i in range(3):
            run_step_e2e(i)
        e2e_regions, last_e2e = [], None
        for _ in range(max(min(repeats, 3), 1)):
            ms, last_e2e = timed(run_step_e2e, args.steps)
            e2e_regions.append(ms)
        return regions, e2e_regions, last

    launches = 0
    trainer = None
    sampler = ClockSampler(local_rank, period_ms=100).start() if rank == 0 else None
    if args.impl == "mccl":
        trainer, run_step, run_step_e2e = make_mccl_arm()
    else:
        run_step, run_step_e2e = make_nccl_arm(model, None)
    regions, e2e_regions, last_loss = measure(run_step, run_step_e2e, args.repeats)
    clocks = sampler.stop() if sampler is not None else None
    ms = statistics.median(regions)
    ms_e2e = statistics.median(e2e_regions)
    if trainer is not None:
        launches = trainer.launches_per_step * args.steps
        trainer.check()

    # The comparison arm in the same invocation: stock eager model, DistributedDataParallel over NCCL, fused AdamW.
    nccl_arm = None
    if args.impl == "mccl" and not args.no_nccl_arm:
        try:
            torch.manual_seed(0)
            ref_model = build_decoder(args.model, native=False, max_seq=args.seq).to(device)
            group = dist.new_group(backend="nccl") if world > 1 else None
            r_step, r_e2e = make_nccl_arm(ref_model, group)
            r_regions, r_e2e_regions, _ = measure(r_step, r_e2e, min(args.repeats, 3))
            r_ms, r_ms_e2e = statistics.median(r_regions), statistics.median(r_e2e_regions)
            nccl_arm = {
                "value": round(B * world * args.steps / (r_ms / 1e3), 2),
                "ms_per_step": round(r_ms / args.steps, 4),
                "e2e": round(B * world * args.steps / (r_ms_e2e / 1e3), 2),
                "what": "stock eager PyTorch model, DistributedDataParallel over backend nccl, autocast bf16, fused AdamW; "
                        "same data, steps and warm-up",
            }
        except Exception as e:  # noqa: BLE001  (the comparison arm must not take the headline number with it)
            nccl_arm = {"unavailable": f"{type(e).__name__}: {e}"[:200]}

    if rank == 0:
        global_batch = B * world
        value = global_batch * args.steps / (ms / 1e3)
        e2e_value = global_batch * args.steps / (ms_e2e / 1e3)
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
            "vs_baseline": None,
            "published_other_hardware": {"samples_per_s": PUBLISHED_OTHER_HARDWARE.get(args.model),
                                         "hardware": "3x Mac mini M4 over Thunderbolt (reference README.md:50,54)"},
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
            "repeats": {"n": len(regions), "ms_per_step_min": round(min(regions) / args.steps, 4),
                        "ms_per_step_max": round(max(regions) / args.steps, 4),
                        "ms_per_step_all": [round(r / args.steps, 4) for r in regions], "value_is": "median region"},
            "nccl_arm": nccl_arm,
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
