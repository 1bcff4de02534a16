"""Kernel dispatch over a group: data-parallel split of one logical grid, tensor transfer, forward pipeline
(CPU ranks).  The reference designs these (csrc/runtime/ShaderDispatch.hpp:88-122,
csrc/runtime/DistributedMetalRuntime.cpp dispatch_data_parallel / dispatch_pipeline / transfer_tensor) without tests."""
import pytest
import torch
import torch.distributed as dist

from tests.common import spawn


def _runtime(rank, world):
    from mccl_b200.distributed.runtime import DistributedRuntime
    rt = DistributedRuntime()
    total = 1003                      # not divisible: the remainder goes to the last node
    a = torch.arange(total, dtype=torch.float32)
    out = torch.zeros(total)

    def saxpy(offset, count, x, y):
        y[offset:offset + count] = 2.0 * x[offset:offset + count] + 1.0

    assert rt.load_library({"saxpy": saxpy}) == ["saxpy"]
    with pytest.raises(KeyError):
        rt.dispatch_data_parallel("missing", total)
    offset, count = rt.dispatch_data_parallel("saxpy", total, a, out)
    rt.sync_all()
    # every rank did exactly its slice; together they cover the grid once
    mine = torch.zeros(total)
    mine[offset:offset + count] = 1.0
    dist.all_reduce(mine)
    assert torch.equal(mine, torch.ones(total))
    dist.all_reduce(out)              # slices are disjoint, so the sum is the whole result
    assert torch.equal(out, 2.0 * a + 1.0)
    # tensor transfer between two ranks
    t = torch.full((5,), float(rank))
    got = rt.transfer_tensor(t, src=0, dst=world - 1)
    if rank == world - 1:
        assert got is not None and torch.equal(got, torch.zeros(5))
    else:
        assert got is None
    # forward pipeline: stage r adds r + 1; the last stage sees the sum of all stages
    mbs = [torch.full((4,), float(i)) for i in range(5)]
    outs = rt.dispatch_pipeline(lambda x: x + (rank + 1), mbs, (4,), torch.float32, torch.device("cpu"))
    if rank == world - 1:
        assert len(outs) == 5
        for i, o in enumerate(outs):
            assert torch.equal(o, torch.full((4,), float(i + world * (world + 1) // 2)))
    else:
        assert outs == []
    rt.sync_all()
    return offset, count


@pytest.mark.parametrize("world", [2, 3])
def test_dispatch_transfer_and_pipeline(world):
    slices = spawn(_runtime, world, timeout=120)
    assert sum(c for _, c in slices) == 1003
    assert [o for o, _ in slices] == sorted(o for o, _ in slices)
