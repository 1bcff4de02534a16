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
    ap.add_argument("--pp", type=int, default=1, help="pipeline stages; tensor parallelism runs over world / pp ranks per stage")
    ap.add_argument("--microbatches", type=int, default=4, help="micro-batches per step when --pp > 1")
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    import mccl_b200  # noqa: F401  (registers backend "mccl")
    from mccl_b200.parallel.tp import TensorParallelContext, TPDecoder
    from mccl_b200.utils.clocks import ClockSampler
    dist.init_process_group(backend=args.impl, device_id=dev if args.impl == "nccl" else None)
    cfg = dict(MODELS[args.model])
    pp = args.pp
    tp_size = world // pp
    stage, tp_rank = rank // tp_size, rank % tp_size
    tp_group = None
    if pp > 1:
        for s in range(pp):   # every rank creates every group
            g_ = dist.new_group(list(range(s * tp_size, (s + 1) * tp_size)), backend=args.impl)
            if s == stage:
                tp_group = g_
    n_mb = args.microbatches if pp > 1 else 1
    mb_batch = cfg["batch"] // n_mb
    rows_local = mb_batch * cfg["seq"] // tp_size
    from mccl_b200.parallel.pp import PipelineStage, split_layers
    layers = split_layers(cfg["n_layers"], pp)[stage]
    ctx = TensorParallelContext(group=tp_group, device=dev, max_rows_local=rows_local, max_features=cfg["d_model"],
                                fused=args.impl == "mccl")
    torch.manual_seed(1234 + rank)
    mcfg = dict(cfg, batch=mb_batch)
    model = TPDecoder(ctx, layers_range=(layers.start, layers.stop), **mcfg).to(dev)
    for p in model.replicated_parameters():
        dist.broadcast(p.data, stage * tp_size, group=tp_group)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-4, fused=True)
    g = torch.Generator().manual_seed(99)
    tokens = torch.randint(0, cfg["vocab"], (cfg["batch"], cfg["seq"] + 1), generator=g).to(dev)
    inp, tgt = tokens[:, :-1].contiguous(), tokens[:, 1:].contiguous()

    if pp == 1:
        def step():
            opt.zero_grad(set_to_none=True)
            loss = model(inp, tgt)
            loss.backward()
            model.sync_replicated_grads()
            opt.step()
            return loss
    else:
        def fn(x, mb):
            sl = slice(mb * mb_batch, (mb + 1) * mb_batch)
            if stage == 0:
                return model(inp[sl], None)
            out = model(inp[sl] if stage == 0 else None, tgt[sl] if stage == pp - 1 else None, hidden=x)
            return out / n_mb if stage == pp - 1 else out

        pipe = PipelineStage(fn, stage, pp, rank - tp_size if stage > 0 else None, rank + tp_size if stage < pp - 1 else None,
                             (rows_local, cfg["d_model"]), torch.bfloat16, dev)

        def step():
            opt.zero_grad(set_to_none=True)
            loss = pipe.run(n_mb)
            model.sync_replicated_grads()
            opt.step()
            return loss if loss is not None else torch.zeros((), device=dev)

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
    total = loss.detach().clone().float()
    dist.all_reduce(total)
    ctx.check()
    if rank == 0:
        tokens_per_step = cfg["batch"] * cfg["seq"]
        print(json.dumps({
            "metric": "tp_decoder_train_tokens_per_sec", "impl": args.impl, "value": tokens_per_step / (ms.item() / 1e3),
            "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms.item(),
            "loss": total.item(), "dtype": "bf16", "data": "synthetic",
            "config": {"model": args.model, **cfg, "parallelism": f"tp{tp_size}" + (f" x pp{pp} ({n_mb} micro-batches, 1F1B)" if pp > 1 else ""),
                       "inputs": "activations larger than L2"},
            "clocks": clocks,
        }), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
