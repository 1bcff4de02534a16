"""Soak loops and stock DistributedDataParallel on CPU ranks over the TCP mesh.

Scaled-down forms of the reference's soak suite (tests/test_soak.py: 10 000 small allreduces, mixed sizes,
interleaved allreduce / broadcast / barrier, three ranks, odd sizes) and of its DDP integration test
(tests/test_ddp.py: gradients equal on every rank, a few optimizer steps of a small MLP).
"""
import pytest
import torch
import torch.distributed as dist
import torch.nn as nn
from torch.nn.parallel import DistributedDataParallel as DDP

from tests.common import spawn


def _soak(rank, world):
    # many small allreduces: results stay exact, no work object leaks an error
    t = torch.ones(1024)
    for i in range(1500):
        t.fill_(float(rank + 1 + (i % 3)))
        dist.all_reduce(t)
        if i % 250 == 0:
            assert t[0].item() == sum(r + 1 + (i % 3) for r in range(world))
    # mixed sizes, odd ones included
    for n in (1, 3, 64, 1023, 4097, 65536, 1 << 20, 77777):
        x = torch.full((n,), float(rank + 1))
        dist.all_reduce(x)
        assert x[0].item() == x[-1].item() == world * (world + 1) / 2
    # interleaved collectives keep their order
    acc = torch.zeros(8)
    for i in range(200):
        a = torch.full((8,), float(i + rank))
        dist.all_reduce(a)
        b = torch.full((8,), float(i)) if rank == i % world else torch.zeros(8)
        dist.broadcast(b, i % world)
        assert b[0].item() == i
        if i % 20 == 0:
            dist.barrier()
        acc += a
    expect = sum(world * i + world * (world - 1) / 2 for i in range(200))
    assert acc[0].item() == expect
    # a few large ones
    big = torch.full((8 << 20,), 1.0)
    for _ in range(3):
        dist.all_reduce(big)
        big.div_(world)
    assert big[12345].item() == 1.0
    from mccl_b200 import metrics
    m = metrics.get_metrics()
    assert m.total_errors == 0 and m.total_ops >= 1500
    return True


@pytest.mark.parametrize("world", [2, 3])
def test_soak(world):
    assert all(spawn(_soak, world, timeout=300))


def _ddp(rank, world):
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(32, 64), nn.ReLU(), nn.Linear(64, 64), nn.ReLU(), nn.Linear(64, 8))
    ddp = DDP(model)
    opt = torch.optim.SGD(ddp.parameters(), lr=0.05)
    g = torch.Generator().manual_seed(100 + rank)
    x, y = torch.randn(16, 32, generator=g), torch.randn(16, 8, generator=g)
    losses = []
    for step in range(5):
        opt.zero_grad()
        loss = (ddp(x) - y).pow(2).mean()
        loss.backward()
        # every rank holds the same (averaged) gradients
        flat = torch.cat([p.grad.reshape(-1) for p in model.parameters()])
        ref = flat.clone()
        dist.broadcast(ref, 0)
        assert torch.equal(flat, ref)
        opt.step()
        losses.append(loss.item())
    w = torch.cat([p.detach().reshape(-1) for p in model.parameters()])
    ref = w.clone()
    dist.broadcast(ref, 0)
    assert torch.equal(w, ref)
    return losses


@pytest.mark.parametrize("world", [2, 3])
def test_stock_ddp_on_cpu_ranks(world):
    losses = spawn(_ddp, world, timeout=300)
    assert all(l[-1] < l[0] for l in losses)
