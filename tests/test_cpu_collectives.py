"""Collectives on CPU tensors over the TCP mesh (world_size > 1, no GPU).

Covers the CPU plumbing run of the baseline spec (world 2 over loopback,
1 048 576 fp32 elements drawn N(0,1) with seed=rank, ring / tree / butterfly
with and without the bf16 wire, then allgather / reduce_scatter / alltoall) and
the per-op suites of the reference (tests/collectives/test_allreduce.py,
test_broadcast.py, allgather.py, test_reduce_scatter.py, test_alltoall.py,
test_p2p.py, test_barrier.py), each checked against fp64 goldens on every rank.
"""
import os

import pytest
import torch
import torch.distributed as dist

from tests.common import (DTYPES, FLOAT_DTYPES, REDUCE_OPS, WORLD, assert_close, golden_allreduce, randn_tensor,
                          rank_tensor, reduce_op, spawn)


# ---------------------------------------------------------------- config 0 --
def _plumbing(rank, world, numel):
    import mccl_b200
    be = mccl_b200.get_backend()
    inputs = [randn_tensor(r, numel) for r in range(world)]
    gold = torch.stack([t.double() for t in inputs]).sum(0)
    report = {}
    for algo in ("ring", "tree", "butterfly"):
        for wire in ("", "bf16"):
            os.environ["MCCL_ALLREDUCE_ALGO"] = algo
            if wire:
                os.environ["MCCL_WIRE_DTYPE"] = wire
            else:
                os.environ.pop("MCCL_WIRE_DTYPE", None)
            t = inputs[rank].clone()
            dist.all_reduce(t)
            assert be.last_algo() == algo, (be.last_algo(), algo)
            if wire:  # bf16 rounding of each input: error relative to the magnitude of the result
                err = ((t.double() - gold).abs().max() / gold.abs().max()).item()
            else:
                err = ((t.double() - gold).abs() / gold.abs().clamp_min(1.0)).max().item()
            assert err <= (1e-2 if wire else 1e-6), (algo, wire, err)
            report[(algo, wire)] = err
    os.environ.pop("MCCL_ALLREDUCE_ALGO", None)
    os.environ.pop("MCCL_WIRE_DTYPE", None)
    # allgather
    mine = inputs[rank]
    out = torch.empty(world * numel)
    dist.all_gather_into_tensor(out, mine)
    assert torch.equal(out, torch.cat(inputs))
    # reduce_scatter
    per = numel // world
    rs = torch.empty(per)
    dist.reduce_scatter_tensor(rs, mine)
    assert_close(rs, gold[rank * per:(rank + 1) * per], torch.float32, "reduce_scatter")
    # alltoall
    a2a = torch.empty(numel)
    dist.all_to_all_single(a2a, mine)
    want = torch.cat([inputs[p][rank * per:(rank + 1) * per] for p in range(world)])
    assert torch.equal(a2a, want)
    return report


def test_cpu_plumbing_run():
    reports = spawn(_plumbing, 2, numel=1 << 20, timeout=180)
    assert all(len(r) == 6 for r in reports)


# ------------------------------------------------------ algorithm selection --
def _selection(rank, world):
    import mccl_b200
    be = mccl_b200.get_backend()
    seen = {}
    small = torch.ones(1024)          # 4 KB  <= 256 KB  -> tree under auto
    big = torch.ones(128 * 1024)      # 512 KB > 256 KB  -> ring under auto
    os.environ.pop("MCCL_ALLREDUCE_ALGO", None)
    dist.all_reduce(small); seen["auto_small"] = be.last_algo()
    dist.all_reduce(big); seen["auto_big"] = be.last_algo()
    os.environ["MCCL_TREE_BELOW"] = "1024"
    dist.all_reduce(small); seen["auto_small_low_cut"] = be.last_algo()
    os.environ["MCCL_TREE_BELOW"] = str(4096)   # inclusive bound
    dist.all_reduce(small); seen["auto_inclusive"] = be.last_algo()
    os.environ.pop("MCCL_TREE_BELOW")
    os.environ["MCCL_ALLREDUCE_ALGO"] = "ring"
    tiny = torch.ones(1)
    dist.all_reduce(tiny); seen["ring_tiny"] = be.last_algo()      # numel < world -> tree
    os.environ["MCCL_ALLREDUCE_ALGO"] = "butterfly"
    dist.all_reduce(tiny); seen["butterfly_tiny"] = be.last_algo()
    os.environ["MCCL_ALLREDUCE_ALGO"] = "no-such-algo"
    dist.all_reduce(big); seen["unknown"] = be.last_algo()          # anything else -> tree
    os.environ.pop("MCCL_ALLREDUCE_ALGO")
    assert tiny.item() == world ** 2
    return seen


def test_allreduce_algorithm_selection_semantics():
    seen = spawn(_selection, 2)[0]
    assert seen == {"auto_small": "tree", "auto_big": "ring", "auto_small_low_cut": "ring", "auto_inclusive": "tree",
                    "ring_tiny": "tree", "butterfly_tiny": "tree", "unknown": "tree"}


# ------------------------------------------------------- dtype x op matrix --
def _allreduce_matrix(rank, world, numel):
    for algo in ("ring", "tree", "butterfly"):
        os.environ["MCCL_ALLREDUCE_ALGO"] = algo
        for dt in DTYPES:
            for op in REDUCE_OPS:
                if op == "avg" and not dt.is_floating_point:
                    continue
                if op == "product" and dt == torch.float16:
                    continue
                inputs = [rank_tensor(r, numel, dt) for r in range(world)]
                t = inputs[rank].clone()
                dist.all_reduce(t, op=reduce_op(op))
                assert_close(t, golden_allreduce(inputs, op), dt, f"{algo}/{dt}/{op}")
    os.environ.pop("MCCL_ALLREDUCE_ALGO")
    return True


@pytest.mark.parametrize("world", sorted({2, 3, WORLD}))
def test_allreduce_dtype_op_matrix(world):
    assert all(spawn(_allreduce_matrix, world, numel=128))


def _allreduce_sizes(rank, world):
    """Odd sizes exercise the short / empty tail chunks of ring and butterfly."""
    for algo in ("ring", "butterfly", "tree"):
        os.environ["MCCL_ALLREDUCE_ALGO"] = algo
        for wire in ("", "bf16"):
            if wire:
                os.environ["MCCL_WIRE_DTYPE"] = wire
            for n in (1, 2, 3, 7, 33, 997, 4097):
                inputs = [randn_tensor(r, n) for r in range(world)]
                t = inputs[rank].clone()
                dist.all_reduce(t)
                gold = torch.stack([x.double() for x in inputs]).sum(0)
                err = ((t.double() - gold).abs().max() / gold.abs().max().clamp_min(1.0)).item()
                assert err <= (1e-2 if wire else 1e-5), (algo, wire, n, err)
                # every rank must hold the same bits
                gathered = [torch.empty_like(t) for _ in range(world)]
                dist.all_gather(gathered, t)
                assert all(torch.equal(g, gathered[0]) for g in gathered), (algo, wire, n)
            os.environ.pop("MCCL_WIRE_DTYPE", None)
    os.environ.pop("MCCL_ALLREDUCE_ALGO")
    return True


@pytest.mark.parametrize("world", [2, 3, 4])
def test_allreduce_odd_sizes_and_bitwise_agreement(world):
    assert all(spawn(_allreduce_sizes, world))


# ---------------------------------------------------------------- broadcast --
def _broadcast(rank, world):
    for dt in DTYPES:
        for root in (0, world - 1):
            t = rank_tensor(rank, 64, dt)
            dist.broadcast(t, root)
            assert torch.equal(t, rank_tensor(root, 64, dt)), (dt, root)
    return True


def test_broadcast():
    assert all(spawn(_broadcast, 3))


# ---------------------------------------------------------------- allgather --
def _allgather(rank, world):
    for dt in DTYPES:
        mine = rank_tensor(rank, 48, dt)
        want = [rank_tensor(r, 48, dt) for r in range(world)]
        out = torch.empty(world * 48, dtype=dt)
        dist.all_gather_into_tensor(out, mine)
        assert torch.equal(out, torch.cat(want)), dt
        # in place: input is the rank's slice of the output
        buf = torch.zeros(world * 48, dtype=dt)
        buf[rank * 48:(rank + 1) * 48] = mine
        dist.all_gather_into_tensor(buf, buf[rank * 48:(rank + 1) * 48])
        assert torch.equal(buf, torch.cat(want)), dt
        outs = [torch.empty(48, dtype=dt) for _ in range(world)]
        dist.all_gather(outs, mine)
        assert all(torch.equal(o, w) for o, w in zip(outs, want)), dt
    return True


def test_allgather():
    assert all(spawn(_allgather, 3))


# ----------------------------------------------------------- reduce_scatter --
def _reduce_scatter(rank, world):
    for dt in FLOAT_DTYPES + [torch.int32, torch.int64]:
        for op in REDUCE_OPS:
            if op == "avg" and not dt.is_floating_point:
                continue
            if op == "product" and dt == torch.float16:
                continue
            per = 40
            inputs = [rank_tensor(r, world * per, dt) for r in range(world)]
            gold = golden_allreduce(inputs, op)[rank * per:(rank + 1) * per]
            out = torch.empty(per, dtype=dt)
            dist.reduce_scatter_tensor(out, inputs[rank].clone(), op=reduce_op(op))
            assert_close(out, gold, dt, f"rs/{dt}/{op}")
            # in place: output aliases the rank's slice of the input
            buf = inputs[rank].clone()
            dist.reduce_scatter_tensor(buf[rank * per:(rank + 1) * per], buf, op=reduce_op(op))
            assert_close(buf[rank * per:(rank + 1) * per], gold, dt, f"rs-inplace/{dt}/{op}")
            # list form
            out2 = torch.empty(per, dtype=dt)
            dist.reduce_scatter(out2, list(inputs[rank].clone().chunk(world)), op=reduce_op(op))
            assert_close(out2, gold, dt, f"rs-list/{dt}/{op}")
    return True


def test_reduce_scatter():
    assert all(spawn(_reduce_scatter, 3))


# ----------------------------------------------------------------- alltoall --
def _alltoall(rank, world):
    # even split, 2-D rows
    rows = 2
    x = (torch.arange(world * rows * 3, dtype=torch.float32) + 1000 * rank).reshape(world * rows, 3)
    out = torch.empty_like(x)
    dist.all_to_all_single(out, x)
    want = torch.cat([(torch.arange(world * rows * 3, dtype=torch.float32) + 1000 * p).reshape(world * rows, 3)
                      [rank * rows:(rank + 1) * rows] for p in range(world)])
    assert torch.equal(out, want)
    # uneven splits: rank r sends 4*(r+1) elements to every peer
    send = 4 * (rank + 1)
    inp = torch.full((send * world,), float(rank))
    in_splits = [send] * world
    out_splits = [4 * (p + 1) for p in range(world)]
    o = torch.empty(sum(out_splits))
    dist.all_to_all_single(o, inp, out_splits, in_splits)
    assert torch.equal(o, torch.cat([torch.full((4 * (p + 1),), float(p)) for p in range(world)]))
    # list form with per-peer sizes
    ins = [torch.full((rank + p + 1,), float(rank * 10 + p)) for p in range(world)]
    outs = [torch.empty(p + rank + 1) for p in range(world)]
    dist.all_to_all(outs, ins)
    for p in range(world):
        assert torch.equal(outs[p], torch.full((p + rank + 1,), float(p * 10 + rank)))
    return True


def test_alltoall():
    assert all(spawn(_alltoall, 3))


# --------------------------------------------------- reduce / gather / scatter --
def _rooted(rank, world):
    for root in (0, world - 1):
        t = rank_tensor(rank, 32, torch.float32)
        keep = t.clone()
        dist.reduce(t, root, op=dist.ReduceOp.SUM)
        if rank == root:
            assert_close(t, golden_allreduce([rank_tensor(r, 32, torch.float32) for r in range(world)], "sum"), torch.float32)
        else:
            assert torch.equal(t, keep)
        outs = [torch.empty(32) for _ in range(world)] if rank == root else None
        dist.gather(keep, outs, dst=root)
        if rank == root:
            assert all(torch.equal(outs[r], rank_tensor(r, 32, torch.float32)) for r in range(world))
        got = torch.empty(32)
        ins = [rank_tensor(r + 5, 32, torch.float32) for r in range(world)] if rank == root else None
        dist.scatter(got, ins, src=root)
        assert torch.equal(got, rank_tensor(rank + 5, 32, torch.float32))
    return True


def test_reduce_gather_scatter():
    assert all(spawn(_rooted, 3))


# ---------------------------------------------------------------- send/recv --
def _p2p(rank, world):
    nxt, prv = (rank + 1) % world, (rank - 1) % world
    for tag in (0, 7, 12345):
        msg = torch.full((257,), float(rank * 100 + (tag % 97)))
        got = torch.empty(257)
        # order by parity so that a posted recv never blocks the send it waits for
        if rank % 2 == 0:
            dist.send(msg, nxt, tag=tag)
            dist.recv(got, prv, tag=tag)
        else:
            dist.recv(got, prv, tag=tag)
            dist.send(msg, nxt, tag=tag)
        assert torch.equal(got, torch.full((257,), float(prv * 100 + (tag % 97))))
    return True


def test_send_recv_ring():
    assert all(spawn(_p2p, 2))
    assert all(spawn(_p2p, 4))


# ------------------------------------------------------------------ barrier --
def _barrier(rank, world):
    import time
    t0 = time.time()
    time.sleep(0.2 * rank)
    dist.barrier()
    waited = time.time() - t0
    assert waited >= 0.2 * (world - 1) - 0.05, waited   # nobody leaves before the slowest arrives
    for _ in range(20):
        dist.barrier()
    return waited


def test_barrier_staggered():
    waits = spawn(_barrier, 3)
    assert max(waits) < 10


# ---------------------------------------------------- ordering and sub-groups --
def _ordering_and_groups(rank, world):
    works = []
    tensors = [torch.full((100 + i,), float(rank + i)) for i in range(10)]
    for t in tensors:
        works.append(dist.all_reduce(t, async_op=True))
    for w in works:
        w.wait()
    for i, t in enumerate(tensors):
        assert torch.equal(t, torch.full((100 + i,), float(sum(r + i for r in range(world)))))
    # sub-group of the even ranks
    evens = list(range(0, world, 2))
    g = dist.new_group(evens, backend="mccl")
    if rank in evens:
        t = torch.ones(16) * (rank + 1)
        dist.all_reduce(t, group=g)
        assert torch.equal(t, torch.ones(16) * sum(r + 1 for r in evens))
    dist.barrier()
    return True


def test_async_ordering_and_subgroups():
    assert all(spawn(_ordering_and_groups, 4))
