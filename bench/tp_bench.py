"""Tensor-parallel training step of the 1.3B decoder on one NVSwitch box.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29511 \
        bench/tp_bench.py --impl mccl --steps 10 --warmup 3

``--impl mccl`` runs the layers on this package's fused all-gather→GEMM and
GEMM→reduce-scatter kernels over the `mccl` process group; ``--impl nccl`` runs the
same modules on stock ``torch.distributed`` (NCCL) collectives and library
matmuls, which is the comparison the reference's tensor-parallel note implies
(README.md:76: hand-wired column / row parallelism over the backend's
collectives).  Prints one JSON line (tokens/s over the whole job; device time,
max over ranks).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

MODELS = {
    "1.3b": dict(vocab=32000, d_model=2048, n_layers=24, n_heads=16, d_ff=8192, batch=8, seq=2048),
    "small": dict(vocab=4096, d_model=1024, n_layers=4, n_heads=16, d_ff=4096, batch=4, seq=1024),
}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", default="mccl", choices=["mccl", "nccl"])
    ap.add_argument("--model", default="1.3b", choices=sorted(MODELS))
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    import mccl_b200  # noqa: F401  (registers backend "mccl")
    from mccl_b200.parallel.tp import TensorParallelContext, TPDecoder
    from mccl_b200.utils.clocks import ClockSampler
    dist.init_process_group(backend=args.impl, device_id=dev if args.impl == "nccl" else None)
    cfg = MODELS[args.model]
    rows_local = cfg["batch"] * cfg["seq"] // world
    ctx = TensorParallelContext(device=dev, max_rows_local=rows_local, max_features=cfg["d_model"],
                                fused=args.impl == "mccl", ag_slots=4 * cfg["n_layers"] + 8)
    torch.manual_seed(1234 + rank)
    model = TPDecoder(ctx, **cfg).to(dev)
    for p in model.replicated_parameters():
        dist.broadcast(p.data, 0)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-4, fused=True)
    g = torch.Generator().manual_seed(99)
    tokens = torch.randint(0, cfg["vocab"], (cfg["batch"], cfg["seq"] + 1), generator=g).to(dev)
    inp, tgt = tokens[:, :-1].contiguous(), tokens[:, 1:].contiguous()

    def step():
        opt.zero_grad(set_to_none=True)
        loss = model(inp, tgt)
        loss.backward()
        model.sync_replicated_grads()
        opt.step()
        return loss

    for _ in range(max(args.warmup, 3)):
        loss = step()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        loss = step()
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop() if sampler else None
    ms = torch.tensor([e0.elapsed_time(e1) / args.steps], device=dev)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    total = loss.detach().clone()
    dist.all_reduce(total)
    ctx.check()
    if rank == 0:
        tokens_per_step = cfg["batch"] * cfg["seq"]
        print(json.dumps({
            "metric": "tp_decoder_train_tokens_per_sec", "impl": args.impl, "value": tokens_per_step / (ms.item() / 1e3),
            "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms.item(),
            "loss": total.item(), "dtype": "bf16", "data": "synthetic",
            "config": {"model": args.model, **cfg, "parallelism": f"tp{world}", "inputs": "activations larger than L2"},
            "clocks": clocks,
        }), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
