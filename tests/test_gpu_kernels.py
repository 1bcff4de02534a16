"""Device kernels against plain PyTorch references (single GPU).

* The stand-alone element-wise kernels, on the size list the reference uses to
  hit the vector body and the scalar tail (tests/test_local_kernels.py:
  sizes {1,3,7,13,97,997,1M}, scale 1/N for N in {2,3,4,8}).
* Every collective kernel, run as `world` virtual ranks on one GPU in one
  cooperative launch, so that the index arithmetic, the wire cast and the
  flag protocol are checked without a second device.  Goldens are fp64 sums
  of the inputs computed by PyTorch.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

import os

os.environ.setdefault("MCCL_ARENA_MB", "64")  # small arenas: eight virtual ranks share one GPU

SIZES = [1, 3, 7, 13, 97, 997, 4097, 1 << 20]


def _C():
    import mccl_b200
    return mccl_b200._C


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16, torch.float64, torch.int32, torch.int64])
def test_elementwise_kernels(dtype):
    C = _C()
    dev = torch.device("cuda", 0)
    for n in SIZES:
        a = (torch.arange(n, device=dev) % 7 + 1).to(dtype)
        b = (torch.arange(n, device=dev) % 3 + 1).to(dtype)
        for off in (0, 1):  # offset 1 element: unaligned pointers take the scalar path
            if n <= off:
                continue
            aa, bb = a[off:], b[off:]
            assert torch.equal(C._mccl_accumulate_chunk(aa.clone(), bb), aa + bb), (n, off)
            assert torch.equal(C._mccl_elementwise_min(aa.clone(), bb), torch.minimum(aa, bb))
            assert torch.equal(C._mccl_elementwise_max(aa.clone(), bb), torch.maximum(aa, bb))
            assert torch.equal(C._mccl_elementwise_product(aa.clone(), bb), aa * bb)
    if dtype.is_floating_point:
        for world in (2, 3, 4, 8):
            x = torch.randn(997, device=dev).to(dtype)
            y = torch.randn(997, device=dev).to(dtype)
            ref = (x.float() * (1.0 / world)).to(dtype)
            got = C._mccl_scale_inplace(x.clone(), 1.0 / world)
            assert torch.allclose(got.float(), ref.float(), rtol=1e-2 if dtype != torch.float32 else 1e-6, atol=1e-6)
            ref2 = ((x.float() + y.float()) * (1.0 / world)).to(dtype)
            got2 = C._mccl_accumulate_and_scale(x.clone(), y, 1.0 / world)
            assert torch.allclose(got2.float(), ref2.float(), rtol=1e-2 if dtype != torch.float32 else 1e-6, atol=1e-5)


@pytest.fixture(scope="module", params=[2, 4, 8])
def comm(request):
    c = _C().DeviceComm(request.param, 0)
    yield c
    torch.cuda.synchronize()
    assert c.status() == 0


def _inputs(world, n, dtype, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    if dtype.is_floating_point:
        return [torch.randn(n, generator=g).to(dtype).cuda() for _ in range(world)]
    return [torch.randint(-50, 50, (n,), generator=g).to(dtype).cuda() for _ in range(world)]


def _gold(inputs, op):
    st = torch.stack([t.double().cpu() for t in inputs])
    return {"sum": st.sum(0), "avg": st.mean(0), "min": st.min(0).values, "max": st.max(0).values,
            "product": st.prod(0)}[op]


@pytest.mark.parametrize("algo", ["oneshot", "twoshot", "twoshot_push", "ring", "tree"])
@pytest.mark.parametrize("dtype,wire", [(torch.float32, "native"), (torch.float32, "bf16"), (torch.bfloat16, "native"),
                                        (torch.float16, "native"), (torch.float64, "native"), (torch.int32, "native"),
                                        (torch.int64, "native")])
def test_allreduce_emulated(comm, algo, dtype, wire):
    world = comm.world
    for n in (1, 5, 16, 997, 4097, 300_001):
        for op in (["sum", "avg", "max"] if dtype.is_floating_point else ["sum", "min"]):
            ins = _inputs(world, n, dtype, seed=n)
            outs = [torch.full_like(t, 7) for t in ins]
            ran = comm.allreduce(ins, outs, op=op, algo=algo, wire=wire)
            torch.cuda.synchronize()
            assert comm.status() == 0
            if not (algo == "ring" and n < world):
                assert ran == ("butterfly" if algo == "twoshot" else algo), ran
            gold = _gold(ins, op)
            tol = 2e-2 if (wire == "bf16" or dtype in (torch.bfloat16, torch.float16)) else (1e-5 if dtype == torch.float32 else 1e-12)
            for r in range(world):
                got = outs[r].double().cpu()
                if dtype.is_floating_point:
                    err = ((got - gold).abs().max() / gold.abs().max().clamp_min(1.0)).item()
                    assert err <= tol, (algo, dtype, wire, n, op, r, err)
                else:
                    assert torch.equal(got, gold), (algo, dtype, n, op, r)
                assert torch.equal(outs[r], outs[0]), "ranks must agree bit for bit"
            # in place
            bufs = [t.clone() for t in ins]
            comm.allreduce(bufs, bufs, op=op, algo=algo, wire=wire)
            torch.cuda.synchronize()
            for r in range(world):
                assert torch.equal(bufs[r], outs[r]), (algo, dtype, wire, n, op, "in-place differs")


def test_allreduce_unaligned_pointers(comm):
    world = comm.world
    ins = [t[1:] for t in _inputs(world, 1001, torch.float32)]
    outs = [torch.zeros(1003, device="cuda")[3:] for _ in range(world)]
    for algo in ("oneshot", "twoshot", "ring", "tree"):
        comm.allreduce(ins, outs, op="sum", algo=algo)
        torch.cuda.synchronize()
        gold = _gold(ins, "sum")
        for r in range(world):
            assert ((outs[r].double().cpu() - gold).abs().max() / gold.abs().max()).item() < 1e-5, algo


def test_allreduce_larger_than_arena_piece(comm):
    """Forces the piecewise path with a message bigger than one arena half can stage."""
    world = comm.world
    n = comm.arena_bytes // 4  # fp32 elements == whole arena; one-shot needs world x that
    n = min(n, 48 << 20)
    ins = _inputs(world, n, torch.float32, seed=3)
    outs = [torch.empty_like(t) for t in ins]
    for algo in ("twoshot", "twoshot_push", "oneshot"):
        comm.allreduce(ins, outs, op="sum", algo=algo)
        torch.cuda.synchronize()
        assert comm.status() == 0
        gold = torch.stack(ins).double().sum(0)
        assert ((outs[0].double() - gold).abs().max() / gold.abs().max()).item() < 1e-5, algo


@pytest.mark.parametrize("dtype,wire", [(torch.float32, "native"), (torch.float32, "bf16"), (torch.bfloat16, "native"), (torch.int32, "native")])
def test_reduce_scatter_emulated(comm, dtype, wire):
    world = comm.world
    for per in (1, 13, 1000, 65_537):
        ins = _inputs(world, per * world, dtype, seed=per)
        outs = [torch.empty(per, dtype=dtype, device="cuda") for _ in range(world)]
        comm.reduce_scatter(ins, outs, op="sum", wire=wire)
        torch.cuda.synchronize()
        gold = _gold(ins, "sum")
        for r in range(world):
            g = gold[r * per:(r + 1) * per]
            got = outs[r].double().cpu()
            if dtype.is_floating_point:
                assert ((got - g).abs().max() / gold.abs().max().clamp_min(1.0)).item() <= (2e-2 if (wire == "bf16" or dtype != torch.float32) else 1e-5)
            else:
                assert torch.equal(got, g)


def test_allgather_broadcast_alltoall_emulated(comm):
    world = comm.world
    for n in (1, 3, 17, 4099, 250_001):
        for dtype in (torch.uint8, torch.float32, torch.bfloat16):
            ins = [(torch.arange(n) % 251 + r).to(dtype).cuda() for r in range(world)]
            outs = [torch.zeros(n * world, dtype=dtype, device="cuda") for _ in range(world)]
            comm.allgather(ins, outs)
            torch.cuda.synchronize()
            want = torch.cat(ins)
            for r in range(world):
                assert torch.equal(outs[r], want), ("allgather", n, dtype, r)
            for root in (0, world - 1):
                bufs = [t.clone() for t in ins]
                comm.broadcast(bufs, root)
                torch.cuda.synchronize()
                for r in range(world):
                    assert torch.equal(bufs[r], ins[root]), ("broadcast", n, dtype, root, r)
    # all-to-all with uneven splits: rank r sends (r + p + 1) elements to peer p
    ins, outs, isp, osp = [], [], [], []
    for r in range(world):
        isp.append([r + p + 1 for p in range(world)])
        osp.append([p + r + 1 for p in range(world)])
        ins.append(torch.cat([torch.full((r + p + 1,), float(r * 10 + p)) for p in range(world)]).cuda())
        outs.append(torch.zeros(sum(osp[-1]), device="cuda"))
    comm.alltoallv(ins, outs, isp, osp)
    torch.cuda.synchronize()
    for r in range(world):
        want = torch.cat([torch.full((p + r + 1,), float(p * 10 + r)) for p in range(world)]).cuda()
        assert torch.equal(outs[r], want), ("alltoall", r)
    # segments longer than an arena slot: the kernel agrees on the number of rounds on the device.  Only rank 0
    # sends long segments (so the other ranks learn the round count from it), of different lengths per peer.
    slot = comm.arena_bytes // 2 // world
    long_elems = (slot // 4) * 2 + 1001          # fp32: a little over two slots
    ins, outs, isp, osp = [], [], [], []
    for r in range(world):
        isp.append([(long_elems + 7 * p) if r == 0 else 5 for p in range(world)])
        osp.append([(long_elems + 7 * r) if p == 0 else 5 for p in range(world)])
        ins.append(torch.cat([torch.arange(isp[-1][p], dtype=torch.float32) + 1000.0 * (r * world + p) for p in range(world)]).cuda())
        outs.append(torch.zeros(sum(osp[-1]), device="cuda"))
    comm.alltoallv(ins, outs, isp, osp)
    torch.cuda.synchronize()
    assert comm.status() == 0
    for r in range(world):
        want = torch.cat([torch.arange(osp[r][p], dtype=torch.float32) + 1000.0 * (p * world + r) for p in range(world)]).cuda()
        if not torch.equal(outs[r], want):
            bad = (outs[r] != want).nonzero().flatten()
            raise AssertionError(("alltoall rounds", r, "mismatches", bad.numel(), "first", int(bad[0]), "last", int(bad[-1]),
                                  "slot elements", slot // 4, "got", outs[r][bad[0]].item(), "want", want[bad[0]].item()))
    comm.barrier()
    torch.cuda.synchronize()
    assert comm.status() == 0


def test_allgather_larger_than_a_slot(comm):
    """A block longer than its slot (arena half / world) goes in pieces."""
    world = comm.world
    n = (comm.arena_bytes // 2 // world) // 4 * 2 + 333    # fp32 elements: a little over two slots per rank
    ins = [(torch.arange(n, dtype=torch.float32) * 0.5 + r).cuda() for r in range(world)]
    outs = [torch.zeros(n * world, device="cuda") for _ in range(world)]
    comm.allgather(ins, outs)
    torch.cuda.synchronize()
    want = torch.cat(ins)
    for r in range(world):
        assert torch.equal(outs[r], want), r
    assert comm.status() == 0


def test_symmetric_heap_allreduce_emulated(comm):
    world = comm.world
    n = 100_003
    per = ((n + world - 1) // world + 15) // 16 * 16
    buf = comm.symm_alloc(per * world * 4)
    views = [buf.tensor(r, 0, [per * world], torch.float32, 0) for r in range(world)]
    ins = _inputs(world, n, torch.float32, seed=11)
    for r in range(world):
        views[r].zero_()
        views[r][:n] = ins[r]
    ran = comm.allreduce_symm(buf, 0, n, torch.float32, "avg")
    torch.cuda.synchronize()
    assert comm.status() == 0 and ran == "butterfly"
    gold = _gold(ins, "avg")
    for r in range(world):
        assert ((views[r][:n].double().cpu() - gold).abs().max()).item() < 1e-5
        assert torch.equal(views[r][:n], views[0][:n])


def test_replay_in_cuda_graph(comm):
    """Epochs and the arena half live on the device, so a captured collective can be replayed."""
    world = comm.world
    ins = _inputs(world, 5000, torch.float32, seed=5)
    outs = [torch.empty_like(t) for t in ins]
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        comm.allreduce(ins, outs, op="sum", algo="twoshot")
        comm.allreduce(ins, outs, op="sum", algo="oneshot")
        comm.allreduce(ins, outs, op="sum", algo="twoshot")  # odd count: replays alternate the arena half
    torch.cuda.current_stream().wait_stream(s)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        comm.allreduce(ins, outs, op="sum", algo="twoshot")
        comm.allreduce(outs, outs, op="max", algo="oneshot")
        comm.allreduce(ins, outs, op="sum", algo="twoshot")
    gold = _gold(ins, "sum")
    for it in range(5):
        for t in outs:
            t.zero_()
        g.replay()
        torch.cuda.synchronize()
        assert comm.status() == 0
        assert ((outs[0].double().cpu() - gold).abs().max() / gold.abs().max()).item() < 1e-5, it


@pytest.mark.parametrize("world", [2, 4])
def test_send_recv_emulated(world):
    """send / recv through the per-pair slots: a sender and a receiver run as two virtual ranks of one
    cooperative launch.  Sizes cover one partial chunk, an unaligned tail and a message longer than the
    two slot buffers (streamed: the sender waits for the receiver to drain)."""
    C = _C()
    c = C.DeviceComm(world, 0)
    slot = c.p2p_slot_bytes
    dev = torch.device("cuda", 0)
    for it, nbytes in enumerate([100, 4096, (1 << 20) + 3, 2 * slot, 5 * slot + 17]):
        src_rank, dst_rank = it % world, (it + 1) % world
        g = torch.Generator().manual_seed(it)
        payload = torch.randint(0, 256, (nbytes,), generator=g, dtype=torch.uint8).to(dev)
        bufs, peers, sends = [], [], []
        for v in range(world):
            if v == src_rank:
                bufs.append(payload); peers.append(dst_rank); sends.append(True)
            elif v == dst_rank:
                bufs.append(torch.zeros(nbytes, dtype=torch.uint8, device=dev)); peers.append(src_rank); sends.append(False)
            else:
                bufs.append(torch.zeros(1, dtype=torch.uint8, device=dev)); peers.append(-1); sends.append(False)
        c.p2p_emulated(bufs, peers, sends)
        torch.cuda.synchronize()
        assert c.status() == 0, nbytes
        assert torch.equal(bufs[dst_rank], payload), nbytes
    # the same pair again, many small messages: sequence numbers and buffer parity keep alternating
    for i in range(20):
        payload = torch.full((1000,), float(i), device=dev)
        out = torch.zeros(1000, device=dev)
        bufs = [payload, out] + [torch.zeros(1, device=dev)] * (world - 2)
        c.p2p_emulated(bufs, [1, 0] + [-1] * (world - 2), [True, False] + [False] * (world - 2))
    torch.cuda.synchronize()
    assert c.status() == 0 and out[0].item() == 19.0


def test_bounded_wait_reports_timeout_and_context_survives():
    """A rank that withholds its signal makes the peers' waits run out: the kernels
    return, the status word names the silent peer, and the GPU stays usable."""
    C = _C()
    c = C.DeviceComm(2, 0)
    c.set_device_timeout_ms(200)
    ins = _inputs(2, 1024, torch.float32)
    outs = [torch.empty_like(t) for t in ins]
    c.allreduce(ins, outs, algo="twoshot")
    torch.cuda.synchronize()
    assert c.status() == 0
    c.inject_skip_signals(1)   # virtual rank 0 stays silent in the next collective
    c.allreduce(ins, outs, algo="twoshot")
    torch.cuda.synchronize()    # returns after ~200 ms, no hang
    assert c.status() != 0
    with pytest.raises(Exception, match="timed out"):
        c.check_status()
    # the context still works
    x = torch.ones(10, device="cuda")
    assert (x + x).sum().item() == 20


def test_debug_bounds_poison_canaries_and_refusal(monkeypatch):
    """MCCL_DEBUG_BOUNDS=1: the staging arena starts out poisoned and ends in a canary, results are unchanged,
    and a kernel whose staging extent would leave its arena half records a violation and touches nothing."""
    monkeypatch.setenv("MCCL_DEBUG_BOUNDS", "1")
    C = _C()
    c = C.DeviceComm(4, 0)
    assert c.debug_bounds
    for algo in ("oneshot", "twoshot", "ring", "tree"):
        for n in (5, 4097, 1 << 18):
            ins = _inputs(4, n, torch.float32, seed=n)
            outs = [torch.empty_like(t) for t in ins]
            c.allreduce(ins, outs, algo=algo)
            torch.cuda.synchronize()
            gold = _gold(ins, "sum")
            assert not torch.isnan(outs[0]).any(), (algo, n)      # no poisoned staging was consumed
            assert ((outs[0].double().cpu() - gold).abs().max() / gold.abs().max()).item() < 1e-5, (algo, n)
    outs2 = [torch.empty(4 * 1000, device="cuda") for _ in range(4)]
    c.allgather([torch.full((1000,), float(v), device="cuda") for v in range(4)], outs2)
    torch.cuda.synchronize()
    c.check_status()          # also verifies the canary behind the arena
    c.check_canaries()
    # pretend the arena is 64 KiB long: a 1 MiB two-shot needs more, so the kernel must refuse
    c.set_debug_arena_limit(64 << 10)
    ins = _inputs(4, 1 << 18, torch.float32, seed=3)
    outs = [torch.full_like(t, -7.0) for t in ins]
    c.allreduce(ins, outs, algo="twoshot")
    torch.cuda.synchronize()
    assert c.status() != 0
    assert all((o == -7.0).all() for o in outs), "a refused kernel must not write its outputs"
    with pytest.raises(Exception, match="MCCL_DEBUG_BOUNDS"):
        c.check_status()
    c.clear_status()
    c.set_debug_arena_limit(0)
    c.allreduce(ins, outs, algo="twoshot")
    torch.cuda.synchronize()
    c.check_status()
