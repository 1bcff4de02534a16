#!/usr/bin/env python
"""Kernel-time shares of one replayed training step of the 70M decoder on one GPU.

    python bench/step_profile.py

Runs the trainer's CUDA graph three times under torch.profiler (CUPTI kernel records) and prints, per kernel name,
launches per step, mean duration and share of the summed kernel time.  Kernels of the weight-gradient stream overlap
the main chain, so the sum exceeds the step time; durations are taken with the profiler attached and serve to compare
shares, not as benchmark numbers (those come from bench.py).
"""
import os, sys, collections
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch
from torch.profiler import profile, ProfilerActivity
import mccl_b200
from mccl_b200.models import build_decoder
from mccl_b200.parallel import DDPTrainer

dev = torch.device("cuda", 0)
torch.manual_seed(0)
model = build_decoder("70m", native=True, max_seq=256).to(dev)
tr = DDPTrainer(model, dev, lr=3e-4)
tok = torch.randint(0, 32000, (16, 257), device=dev)
x, y = tok[:, :-1].contiguous(), tok[:, 1:].contiguous()
for _ in range(6): tr.step(x, y)
torch.cuda.synchronize()
with profile(activities=[ProfilerActivity.CUDA]) as prof:
    for _ in range(3): tr.step(x, y)
    torch.cuda.synchronize()
agg = collections.defaultdict(lambda: [0, 0.0])
for e in prof.events():
    if e.device_type == torch.autograd.DeviceType.CUDA:
        n = e.name
        for a, b in (("mccl::ops::(anonymous namespace)::", ""), ("mccl::(anonymous namespace)::", ""), ("void ", "")):
            n = n.replace(a, b)
        n = n[:80]
        agg[n][0] += 1; agg[n][1] += e.device_time_total if hasattr(e, "device_time_total") else e.cuda_time_total
tot = sum(v[1] for v in agg.values())
print(f"total kernel time per step {tot/3:.1f} us")
for n, (c, t) in sorted(agg.items(), key=lambda kv: -kv[1][1])[:40]:
    print(f"{t/3:9.1f} us {c//3:5d}x {t/c:8.1f} us  {100*t/tot:5.1f}%  {n}")
