"""Distributed memory, coherence and the tensor layer between real GPUs (one process per GPU).

What the reference sketches for RDMA (DistributedMemoryManager put / get / put_with_imm / fence:
csrc/dmem/DistributedMemoryManager.cpp:215-300; gpu_acquire / gpu_release left as stubs:
csrc/coherence/CoherenceProtocol.cpp:163-174; DistributedTensor: mccl/distributed/tensor.py:123-327)
runs here over NVLink: regions live in symmetric heaps every rank maps, device-side atomics hit a
peer's words, and acquire / release are stream-ordered kernels with bounded waits.  NVLS is off in
these tests and every wait has a short limit, so a failing rank cannot take its peers' GPUs with it.
"""
import os

import pytest
import torch
import torch.distributed as dist

from tests.common import spawn

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]

_ENV = {"MCCL_NVLS": "0", "NCCL_NVLS_ENABLE": "0", "MCCL_DEVICE_TIMEOUT_MS": "20000", "MCCL_ARENA_MB": "64"}


def _world():
    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    return min(n, int(os.environ.get("MCCL_TEST_GPUS", "8")))


def _dmem_put_get(rank, world):
    import mccl_b200
    from mccl_b200 import _C
    dev = torch.device("cuda", torch.cuda.current_device())
    be = mccl_b200.get_backend()
    _C.init_dmem_symm(be, dev.index)
    n = 1 << 16
    heap_id, heap = _C.alloc_symm_heap(n * 4 * 2)
    mine = heap.tensor(rank, 0, [2, n], torch.float32, dev.index)
    mine.zero_()
    region = _C.register_region(heap.ptr(rank), n * 4 * 2, _C.REGION_READABLE | _C.REGION_WRITABLE | _C.REGION_SHARED | _C.REGION_DEVICE,
                                heap_id, 0)
    torch.cuda.synchronize()
    dist.barrier()
    nxt, prv = (rank + 1) % world, (rank - 1) % world
    # put: row 0 of the next rank's region receives my pattern, followed by an immediate
    g = torch.Generator().manual_seed(rank)
    src = torch.randn(n, generator=g).to(dev)
    wr = _C.put_with_imm(nxt, region, 0, src.data_ptr(), n * 4, 1000 + rank)
    assert wr > 0
    assert _C.poll_completion(wr)
    torch.cuda.synchronize()
    dist.barrier()
    want = torch.randn(n, generator=torch.Generator().manual_seed(prv))
    assert torch.equal(mine[0].cpu(), want), "put landed wrong"
    imms = _C.take_immediates()
    assert imms == [(prv, region, 0, n * 4, 1000 + prv)], imms
    # get: read row 0 of the previous rank's region (which holds prv-1's pattern)
    out = torch.empty(n, device=dev)
    wr = _C.get(prv, region, 0, out.data_ptr(), n * 4)
    assert wr > 0 and _C.poll_completion(wr)
    torch.cuda.synchronize()
    want2 = torch.randn(n, generator=torch.Generator().manual_seed((prv - 1) % world))
    assert torch.equal(out.cpu(), want2), "get read wrong"
    # out-of-range access is refused and counted
    assert _C.put(nxt, region, n * 4 * 2 - 8, src.data_ptr(), 64) == 0
    # many immediates in a row arrive in order (ring of 256 per pair; stay below it between drains)
    dist.barrier()
    for i in range(100):
        _C.put_with_imm(nxt, region, n * 4, src.data_ptr(), 16, i)
    torch.cuda.synchronize()
    dist.barrier()
    got = [t[4] for t in _C.take_immediates()]
    assert got == list(range(100)), got[:10]
    stats = _C.get_stats()
    assert stats["total_put_ops"] >= 101 and stats["total_get_ops"] == 1 and stats["total_errors"] >= 1
    # SM-driven copy and device-side atomics on a peer's words
    peer_row = heap.ptr(nxt) + n * 4          # row 1 of the next rank
    _C.dmem_copy(peer_row, src.data_ptr(), n * 4, dev.index)
    torch.cuda.synchronize()
    dist.barrier()
    assert torch.equal(mine[1].cpu(), want), "dmem_copy landed wrong"
    dist.barrier()
    # all ranks hammer three words of rank 0: a counter, a CAS slot and a float sum
    cheap_id, cheap = _C.alloc_symm_heap(4096)
    cnt = cheap.tensor(0, 0, [1], torch.int32, dev.index)
    slot = cheap.tensor(0, 8, [1], torch.int64, dev.index)
    fsum = cheap.tensor(0, 16, [1], torch.float32, dev.index)
    dist.barrier()
    _C.dmem_atomic_selftest(cnt, slot, fsum, 1000)
    torch.cuda.synchronize()
    dist.barrier()
    if rank == 0:
        assert cnt.item() == 1000 * world, cnt.item()
        assert slot.item() == 42
        assert abs(fsum.item() - 500.0 * world) < 1e-3
    dist.barrier()
    _C.shutdown_dmem()
    return True


def test_dmem_put_get_imm_atomics_between_gpus():
    assert all(spawn(_dmem_put_get, _world(), timeout=90, _cuda=True, env=_ENV))


def _coherence_pingpong(rank, world):
    import mccl_b200
    from mccl_b200 import _C
    dev = torch.device("cuda", torch.cuda.current_device())
    comm = mccl_b200.get_backend().device_comm(dev.index)
    coh = _C.GpuCoherence(comm)
    buf = comm.symm_alloc(4096)
    mine = buf.tensor(rank, 0, [256], torch.float32, dev.index)
    nxt = (rank + 1) % world
    peer = buf.tensor(nxt, 0, [256], torch.float32, dev.index)
    prv = (rank - 1) % world
    dist.barrier()
    # 100 epochs: write into the next rank's buffer, release, acquire, read what the previous rank wrote
    for epoch in range(1, 101):
        peer.fill_(float(epoch * 10 + rank))     # plain elementwise store over NVLink
        e = coh.gpu_release(dev.index)
        assert e == 2 * epoch - 1   # two releases per round: data, then "done reading"
        coh.gpu_acquire(e, 5000, dev.index)
        got = mine.clone()
        torch.cuda.synchronize()
        assert coh.status() == 0
        assert got[0].item() == epoch * 10 + prv and got[-1].item() == epoch * 10 + prv, (epoch, got[0].item())
        # nobody overwrites a buffer that is still being read: meet before the next epoch's writes
        coh.gpu_release(dev.index)
        coh.gpu_acquire(coh.epoch, 5000, dev.index)
        torch.cuda.synchronize()
    assert coh.epoch == 200
    dist.barrier()
    # a release that never comes: the acquire gives up after its limit and says whom it waited for
    if rank == 0:
        coh.gpu_acquire(coh.epoch + 1, 300, dev.index)
        torch.cuda.synchronize()
        assert coh.status() == 2, coh.status()   # 1 + the first peer that did not release: rank 1
        coh.clear_status()
        assert (torch.ones(4, device=dev) * 2).sum().item() == 8   # the context is fine
    dist.barrier()
    return True


def test_gpu_acquire_release_pingpong_and_timeout():
    assert all(spawn(_coherence_pingpong, min(_world(), 4), timeout=180, _cuda=True, env=_ENV))


def _dist_tensor(rank, world):
    from mccl_b200.distributed import DistributedModel, DistributedTensor, ShardingSpec
    dev = torch.device("cuda", torch.cuda.current_device())
    n = 4096 * world + 0
    for dt, tol in ((torch.float32, 1e-5), (torch.bfloat16, 2e-2)):
        inputs = [torch.randn(n, generator=torch.Generator().manual_seed(10 + r)).to(dt) for r in range(world)]
        gold = torch.stack([x.double() for x in inputs]).sum(0)
        t = DistributedTensor(inputs[rank].to(dev), ShardingSpec.DATA_PARALLEL)
        assert t.in_symmetric_heap
        out = t.all_reduce("sum")
        torch.cuda.synchronize()
        err = ((out.double().cpu() - gold).abs().max() / gold.abs().max()).item()
        assert err < tol, (dt, err)
        # mean of a gradient
        t2 = DistributedTensor(torch.zeros(n, dtype=dt, device=dev), ShardingSpec.DATA_PARALLEL)
        m = t2.sync_gradient(inputs[rank].to(dev))
        torch.cuda.synchronize()
        err = ((m.double().cpu() - gold / world).abs().max() / (gold / world).abs().max()).item()
        assert err < tol, (dt, "avg", err)
        # gather / scatter forms
        t3 = DistributedTensor(inputs[rank].to(dev).view(world, -1), ShardingSpec.TENSOR_PARALLEL, shard_dim=1)
        full = t3.all_gather()
        want = torch.cat([x.view(world, -1) for x in inputs], dim=1)
        assert torch.equal(full.cpu(), want)
        rs = DistributedTensor(inputs[rank].to(dev)).reduce_scatter("sum")
        per = n // world
        err = ((rs.double().cpu() - gold[rank * per:(rank + 1) * per]).abs().max() / gold.abs().max()).item()
        assert err < tol, (dt, "rs", err)
        # a peer's shard can be copied out (plain elementwise copy over NVLink)
        pv = t.peer_view((rank + 1) % world).clone()
        torch.cuda.synchronize()
        assert torch.equal(pv, out)   # after the allreduce every shard holds the same values
    # PGAS gradient sync of a model
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(32, 64), torch.nn.Tanh(), torch.nn.Linear(64, 4)).to(dev)
    dm = DistributedModel(model)
    dm.register_parameters()
    x = torch.randn(8, 32, generator=torch.Generator().manual_seed(50 + rank)).to(dev)
    dm(x).square().mean().backward()
    local = [p.grad.clone() for p in model.parameters()]
    dm.sync_gradients()
    for p, lg in zip(model.parameters(), local):
        gathered = [torch.empty_like(lg) for _ in range(world)]
        dist.all_gather(gathered, lg)
        mean = torch.stack(gathered).double().mean(0)
        assert ((p.grad.double() - mean).abs().max() / mean.abs().max().clamp_min(1e-6)).item() < 1e-5
    return True


def test_distributed_tensor_and_model_on_gpus():
    env = dict(_ENV)
    env.pop("MCCL_NVLS")   # the symmetric in-place path may use in-switch reduction here: no rank fails in this test
    assert all(spawn(_dist_tensor, _world(), timeout=180, _cuda=True, env=env))


def _kernel_dispatch(rank, world):
    from mccl_b200.distributed import DistributedRuntime
    dev = torch.device("cuda", torch.cuda.current_device())
    rt = DistributedRuntime()
    total = 1000 * world + 3
    data = torch.zeros(total, device=dev)

    def saxpy(offset, count, buf, a):
        buf[offset:offset + count] += a * torch.arange(offset, offset + count, device=buf.device, dtype=buf.dtype)
    rt.load_library({"saxpy": saxpy})
    off, cnt = rt.dispatch_data_parallel("saxpy", total, data, 2.0, device=dev)
    rt.sync_all(dev)
    # every rank computed only its slice; together the slices cover the grid once
    dist.all_reduce(data)
    assert torch.equal(data.cpu(), 2.0 * torch.arange(total, dtype=torch.float32))
    counts = [torch.zeros(1, device=dev) for _ in range(world)]
    dist.all_gather(counts, torch.tensor([float(cnt)], device=dev))
    assert sum(int(c.item()) for c in counts) == total
    # forward pipeline over send / recv: stage r adds r + 1
    mbs = [torch.full((4, 8), float(i), device=dev) for i in range(6)]
    outs = rt.dispatch_pipeline(lambda x: x + (rank + 1), mbs, (4, 8), torch.float32, dev)
    torch.cuda.synchronize()
    if rank == world - 1:
        extra = sum(range(1, world + 1))
        assert [o[0, 0].item() for o in outs] == [i + extra for i in range(6)]
    return True


def test_kernel_dispatch_and_pipeline_on_gpus():
    assert all(spawn(_kernel_dispatch, _world(), timeout=180, _cuda=True, env=_ENV))
