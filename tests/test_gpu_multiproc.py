"""Collectives between real GPUs: one process per GPU over backend "mccl".

World size = min(visible GPUs, MCCL_TEST_GPUS or 8).  Every result is checked
against fp64 goldens on every rank, following the reference's per-op suites
(tests/collectives/*.py) and its DDP integration tests (tests/test_ddp.py,
tests/test_ddp_e2e.py: loss decreases, parameters stay identical across ranks).
"""
import os

import pytest
import torch
import torch.distributed as dist

from tests.common import assert_close, golden_allreduce, randn_tensor, rank_tensor, reduce_op, spawn

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _world():
    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    return min(n, int(os.environ.get("MCCL_TEST_GPUS", "8")))


def _allreduce_all(rank, world):
    import mccl_b200
    be = mccl_b200.get_backend()
    dev = torch.device("cuda", torch.cuda.current_device())
    info = {}
    for algo in ("oneshot", "twoshot", "ring", "tree", "nvls", "auto"):
        os.environ["MCCL_ALLREDUCE_ALGO"] = algo
        for wire in ("", "bf16"):
            if wire:
                os.environ["MCCL_WIRE_DTYPE"] = wire
            else:
                os.environ.pop("MCCL_WIRE_DTYPE", None)
            for n in (1, 7, 1000, 4097, 1 << 20, (1 << 22) + 5):
                inputs = [randn_tensor(r, n) for r in range(world)]
                gold = torch.stack([x.double() for x in inputs]).sum(0)
                t = inputs[rank].to(dev)
                dist.all_reduce(t)
                torch.cuda.synchronize()
                be.check_device_status()
                err = ((t.double().cpu() - gold).abs().max() / gold.abs().max().clamp_min(1.0)).item()
                # With bf16 on the wire every hop rounds to 8 mantissa bits (2^-8 = 3.9e-3 relative).  One-shot and
                # two-shot round each addend once; ring rounds the running partial sum at each of its N - 1 steps
                # and tree at each of its log2(N) levels, so the error grows with the hop count: N - 1 = 7
                # roundings of up to 3.9e-3 each, on sums whose partials can exceed the final value, is what
                # 2.5e-2 allows for.  Without the wire cast the result must match fp64 to fp32 accuracy.
                assert err <= (2.5e-2 if wire else 1e-5), (algo, wire, n, err)
                gathered = [torch.empty_like(t) for _ in range(world)]
                dist.all_gather(gathered, t)
                assert all(torch.equal(g, gathered[0]) for g in gathered), (algo, wire, n, "ranks differ")
            info[(algo, wire)] = be.last_algo()
    os.environ.pop("MCCL_ALLREDUCE_ALGO", None)
    os.environ.pop("MCCL_WIRE_DTYPE", None)
    for dt in (torch.float32, torch.float16, torch.bfloat16, torch.float64, torch.int32, torch.int64, torch.uint8, torch.bool):
        for op in ("sum", "min", "max", "product", "avg"):
            if (op == "avg" and not dt.is_floating_point) or (op == "product" and dt == torch.float16):
                continue
            inputs = [rank_tensor(r, 300, dt) for r in range(world)]
            t = inputs[rank].to(dev)
            dist.all_reduce(t, op=reduce_op(op))
            assert_close(t, golden_allreduce(inputs, op), dt, f"{dt}/{op}")
    info["mode"] = be.device_comm(dev.index).symm_mode
    info["nvls"] = be.device_comm(dev.index).nvls_available
    return info


def test_allreduce_every_algorithm():
    w = _world()
    infos = spawn(_allreduce_all, w, timeout=300, _cuda=True)
    print(infos[0])
    assert infos[0][("twoshot", "")] == "butterfly"
    assert infos[0][("ring", "")] == "ring" and infos[0][("tree", "")] == "tree"


def _other_collectives(rank, world):
    dev = torch.device("cuda", torch.cuda.current_device())
    for dt in (torch.float32, torch.bfloat16, torch.int64, torch.uint8):
        for n in (1, 48, 100_003):
            mine = rank_tensor(rank, n, dt).to(dev)
            want = torch.cat([rank_tensor(r, n, dt) for r in range(world)]).to(dev)
            out = torch.empty(world * n, dtype=dt, device=dev)
            dist.all_gather_into_tensor(out, mine)
            assert torch.equal(out, want), ("allgather", dt, n)
            outs = [torch.empty(n, dtype=dt, device=dev) for _ in range(world)]
            dist.all_gather(outs, mine)
            assert torch.equal(torch.cat(outs), want)
            for root in (0, world - 1):
                t = rank_tensor(rank, n, dt).to(dev)
                dist.broadcast(t, root)
                assert torch.equal(t, rank_tensor(root, n, dt).to(dev)), ("broadcast", dt, n, root)
    for dt in (torch.float32, torch.bfloat16, torch.int32):
        for op in ("sum", "max", "avg"):
            if op == "avg" and not dt.is_floating_point:
                continue
            per = 1001
            inputs = [rank_tensor(r, world * per, dt) for r in range(world)]
            gold = golden_allreduce(inputs, op)[rank * per:(rank + 1) * per]
            out = torch.empty(per, dtype=dt, device=dev)
            dist.reduce_scatter_tensor(out, inputs[rank].to(dev), op=reduce_op(op))
            assert_close(out, gold, dt, f"rs/{dt}/{op}")
    # all-to-all: even 2-D and uneven
    rows = 3
    x = (torch.arange(world * rows * 5, dtype=torch.float32) + 1000 * rank).reshape(world * rows, 5).to(dev)
    out = torch.empty_like(x)
    dist.all_to_all_single(out, x)
    want = torch.cat([(torch.arange(world * rows * 5, dtype=torch.float32) + 1000 * p).reshape(world * rows, 5)
                      [rank * rows:(rank + 1) * rows] for p in range(world)]).to(dev)
    assert torch.equal(out, want)
    send = 4 * (rank + 1)
    inp = torch.full((send * world,), float(rank), device=dev)
    o = torch.empty(sum(4 * (p + 1) for p in range(world)), device=dev)
    dist.all_to_all_single(o, inp, [4 * (p + 1) for p in range(world)], [send] * world)
    assert torch.equal(o, torch.cat([torch.full((4 * (p + 1),), float(p)) for p in range(world)]).to(dev))
    ins = [torch.full((rank + p + 1,), float(rank * 10 + p), device=dev) for p in range(world)]
    outs = [torch.empty(p + rank + 1, device=dev) for p in range(world)]
    dist.all_to_all(outs, ins)
    for p in range(world):
        assert torch.equal(outs[p], torch.full((p + rank + 1,), float(p * 10 + rank), device=dev))
    # rooted
    t = rank_tensor(rank, 64, torch.float32).to(dev)
    keep = t.clone()
    dist.reduce(t, 0)
    if rank == 0:
        assert_close(t, golden_allreduce([rank_tensor(r, 64, torch.float32) for r in range(world)], "sum"), torch.float32)
    else:
        assert torch.equal(t, keep)
    outs = [torch.empty(64, device=dev) for _ in range(world)] if rank == 0 else None
    dist.gather(keep, outs, dst=0)
    if rank == 0:
        assert all(torch.equal(outs[r].cpu(), rank_tensor(r, 64, torch.float32)) for r in range(world))
    got = torch.empty(64, device=dev)
    dist.scatter(got, [rank_tensor(r + 5, 64, torch.float32).to(dev) for r in range(world)] if rank == 0 else None, src=0)
    assert torch.equal(got.cpu(), rank_tensor(rank + 5, 64, torch.float32))
    # send / recv: this backend's own kernels over per-pair slots in peer-mapped memory
    nxt, prv = (rank + 1) % world, (rank - 1) % world
    msg = torch.full((1000,), float(rank), device=dev)
    buf = torch.empty(1000, device=dev)
    if rank % 2 == 0:
        dist.send(msg, nxt); dist.recv(buf, prv)
    else:
        dist.recv(buf, prv); dist.send(msg, nxt)
    assert torch.equal(buf, torch.full((1000,), float(prv), device=dev))
    # both directions at once (isend + irecv), a message longer than the two slot buffers of a pair
    import mccl_b200
    slot = mccl_b200.get_backend().device_comm(dev.index).p2p_slot_bytes
    n = (5 * slot) // 4 + 3
    big = torch.arange(n, dtype=torch.float32, device=dev) + rank
    got = torch.empty(n, dtype=torch.float32, device=dev)
    reqs = [dist.isend(big, nxt), dist.irecv(got, prv)]
    for r in reqs:
        r.wait()
    torch.cuda.synchronize()
    assert torch.equal(got, torch.arange(n, dtype=torch.float32, device=dev) + prv)
    for i in range(50):   # many small messages in a row keep their order
        m = torch.full((17,), float(i * world + rank), device=dev)
        o = torch.empty(17, device=dev)
        reqs = [dist.isend(m, nxt), dist.irecv(o, prv)]
        for r in reqs:
            r.wait()
        assert o[0].item() == i * world + prv
    mccl_b200.get_backend().check_device_status()
    for _ in range(10):
        dist.barrier()
    return True


def test_other_collectives():
    assert all(spawn(_other_collectives, _world(), timeout=300, _cuda=True))


def _stock_ddp(rank, world):
    import torch.nn as nn
    from torch.nn.parallel import DistributedDataParallel as DDP
    from mccl_b200.parallel import bf16_wire_hook
    dev = torch.device("cuda", torch.cuda.current_device())
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(64, 256), nn.GELU(), nn.Linear(256, 256), nn.GELU(), nn.Linear(256, 64), nn.GELU(),
                          nn.Linear(64, 8)).to(dev)
    ddp = DDP(model, device_ids=[dev.index], bucket_cap_mb=1)
    if os.environ.get("MCCL_TEST_HOOK") == "1":
        ddp.register_comm_hook(None, bf16_wire_hook)
    opt = torch.optim.Adam(ddp.parameters(), lr=1e-2)
    g = torch.Generator().manual_seed(100 + rank)
    x = torch.randn(32, 64, generator=g).to(dev)   # one fixed batch per rank
    y = x[:, :8] * 2.0
    losses = []
    for step in range(12):
        loss = ((ddp(x) - y) ** 2).mean()
        opt.zero_grad()
        loss.backward()
        opt.step()
        losses.append(loss.item())
    sig = torch.stack([p.detach().double().sum() for p in model.parameters()])
    sigs = [torch.empty_like(sig) for _ in range(world)]
    dist.all_gather(sigs, sig)
    for s in sigs:
        assert torch.allclose(s, sigs[0], rtol=0, atol=1e-6), "parameters diverged across ranks"
    assert losses[-1] < losses[0]
    return losses


@pytest.mark.parametrize("hook", ["0", "1"])
def test_stock_ddp_trains_and_stays_in_sync(hook):
    spawn(_stock_ddp, _world(), timeout=300, _cuda=True, env={"MCCL_TEST_HOOK": hook})


def _engine(rank, world, wire):
    from mccl_b200.models import build_decoder
    from mccl_b200.parallel import DDPTrainer
    dev = torch.device("cuda", torch.cuda.current_device())
    torch.manual_seed(0)
    model = build_decoder("tiny", native=True).to(dev)
    trainer = DDPTrainer(model, dev, lr=1e-3, wire=wire, bucket_mb=0.25, use_graph=True)
    g = torch.Generator().manual_seed(7 + rank)
    tokens = torch.randint(0, model.cfg.vocab, (4, 65), generator=g).to(dev)
    losses = []
    for _ in range(6):
        losses.append(float(trainer.step(tokens[:, :-1].contiguous(), tokens[:, 1:].contiguous()).item()))
    trainer.check()
    # every rank must hold bit-identical parameters: compare against rank 0's copy
    ref = trainer.flat_p.clone()
    dist.broadcast(ref, 0)
    bad = (ref != trainer.flat_p).nonzero().flatten()
    if bad.numel():
        where = [(b.start, b.numel, int(((bad >= b.start) & (bad < b.start + b.numel)).sum())) for b in trainer.buckets]
        raise AssertionError(f"flat parameters diverged in {bad.numel()} of {ref.numel()} elements; (bucket start, size, bad): {where}; "
                             f"max diff {(ref - trainer.flat_p).abs().max().item():.3e}")
    assert losses[-1] < losses[0], losses
    return losses


@pytest.mark.parametrize("wire", ["bf16", "native"])
def test_engine_trains_and_stays_in_sync(wire):
    spawn(_engine, _world(), timeout=300, _cuda=True, wire=wire)


def _fault(rank, world):
    """Rank 1 withholds one round of signals: rank 0's bounded wait runs out and reports it."""
    import mccl_b200
    be = mccl_b200.get_backend()
    dev = torch.device("cuda", torch.cuda.current_device())
    t = torch.ones(1000, device=dev)
    dist.all_reduce(t)
    torch.cuda.synchronize()
    comm = be.device_comm(dev.index)
    comm.set_device_timeout_ms(300)
    if rank == 1:
        comm.inject_skip_signals(1)
    work = dist.all_reduce(t, async_op=True)
    work.wait()                  # stream-ordered: returns at once
    torch.cuda.synchronize()     # the kernel gives up after ~300 ms
    status = comm.status()
    raised = ""
    if rank == 0:
        # the Work of the failing collective reports it, with no explicit status check by the caller
        import time
        deadline = time.time() + 5
        while work.is_success() and time.time() < deadline:   # the completion thread marks it within microseconds
            time.sleep(0.01)
        try:
            work.wait()
        except Exception as e:   # noqa: BLE001
            raised = f"{type(e).__name__}: {e}"
        assert not work.is_success()
    # the context survives on every rank
    assert (torch.ones(4, device=dev) * 2).sum().item() == 8
    return status, raised


def test_skipped_signal_times_out_without_hanging():
    # NVLS off: a rank must never die or stall while bound to a multicast object in a fault test
    out = spawn(_fault, 2, timeout=120, _cuda=True, env={"MCCL_NVLS": "0", "NCCL_NVLS_ENABLE": "0"}, _skip_final_barrier=True)
    assert out[0][0] != 0
    assert "timed out" in out[0][1], out


def _fault_env(rank, world):
    """The same fault, configured from the environment: MCCL_FAULT_INJECT makes rank 1 withhold the signals
    of its second collective; rank 0's wait runs out and the Work of that collective reports it."""
    import mccl_b200
    dev = torch.device("cuda", torch.cuda.current_device())
    t = torch.ones(1000, device=dev)
    dist.all_reduce(t)            # collective 0: healthy
    torch.cuda.synchronize()
    assert t[0].item() == world
    work = dist.all_reduce(t, async_op=True)   # collective 1: rank 1 stays silent
    torch.cuda.synchronize()
    raised = ""
    if rank == 0:
        try:
            work.wait()
        except Exception as e:   # noqa: BLE001
            raised = f"{type(e).__name__}: {e}"
    assert (torch.ones(4, device=dev) * 2).sum().item() == 8
    return raised


def test_fault_injection_from_environment():
    out = spawn(_fault_env, 2, timeout=120, _cuda=True, _skip_final_barrier=True,
                env={"MCCL_NVLS": "0", "NCCL_NVLS_ENABLE": "0", "MCCL_DEVICE_TIMEOUT_MS": "300",
                     "MCCL_FAULT_INJECT": "rank=1,skip_signals=1,after=1"})
    assert "timed out" in out[0], out


def _tp_gemms(rank, world):
    import mccl_b200
    from mccl_b200 import _C
    dev = torch.device("cuda", torch.cuda.current_device())
    comm = mccl_b200.get_backend().device_comm(dev.index)
    rows, K, N = 256, 512, 384
    tp = _C.TpGemm(comm, rows * max(N, K))
    sym = comm.symm_alloc(rows * K * 2)
    mine = sym.tensor(rank, 0, [rows, K], torch.bfloat16, dev.index)
    worst = 0.0
    for it in range(3):   # several epochs: both staging parities and flag reuse
        g = torch.Generator(device="cpu").manual_seed(100 * it + rank)
        x = torch.randn(rows, K, generator=g).to(dev).bfloat16()
        gw = torch.Generator(device="cpu").manual_seed(1000 + it)
        w = (torch.randn(N, K, generator=gw) * 0.05).to(dev).bfloat16()
        # all-gather -> GEMM, both weight layouts
        mine.copy_(x)
        full = torch.empty(world * rows, K, dtype=torch.bfloat16, device=dev)
        dist.all_gather_into_tensor(full, x)
        gold = full.float() @ w.float().t()
        y, gathered, _ = tp.ag_gemm(sym, 0, rows, w, False)
        assert torch.equal(gathered, full)
        worst = max(worst, ((y.float() - gold).abs().max() / gold.abs().max()).item())
        y2, _, _ = tp.ag_gemm(sym, 0, rows, w.t().contiguous(), True)
        worst = max(worst, ((y2.float() - gold).abs().max() / gold.abs().max()).item())
        # GEMM -> reduce-scatter
        xr = torch.randn(world * rows, K, generator=g).to(dev).bfloat16()
        part = xr.float() @ w.float().t()
        dist.all_reduce(part)
        gold_rs = part[rank * rows:(rank + 1) * rows]
        out = tp.gemm_rs(xr, w, False)
        worst = max(worst, ((out.float() - gold_rs).abs().max() / gold_rs.abs().max()).item())
        out2 = tp.gemm_rs(xr, w.t().contiguous(), True)
        worst = max(worst, ((out2.float() - gold_rs).abs().max() / gold_rs.abs().max()).item())
        torch.cuda.synchronize()
        tp.check_status()
    assert _C.gemm_error_flag() == 0
    return worst


def test_fused_tensor_parallel_gemms():
    """All-gather -> GEMM and GEMM -> reduce-scatter against fp32 matmuls of the gathered / summed operands.

    Tolerance: the reduce-scatter fusion rounds every rank's partial product to bf16 before the owner adds the
    `world` partials in fp32 and rounds the sum once more, so the result carries up to world + 1 bf16 roundings
    (relative 2^-8 each) of values of magnitude sqrt(K) ~ 23 where an unfused fp32 reduction would carry one;
    2e-2 relative to the largest output covers 8 ranks with margin."""
    worst = spawn(_tp_gemms, _world(), timeout=300, _cuda=True)
    assert max(worst) < 2e-2, worst


def _tp_model(rank, world):
    from mccl_b200.parallel.tp import TensorParallelContext, TPDecoder
    dev = torch.device("cuda", torch.cuda.current_device())
    B, S, V, D, H, FF, L = 2, 128 * world // 2, 512, 256, 8, 512, 2
    losses = {}
    grads = {}
    for fused in (True, False):
        torch.manual_seed(7)   # same replicated weights; shards differ by rank below
        ctx = TensorParallelContext(device=dev, max_rows_local=B * S // world, max_features=max(3 * D, FF), fused=fused)
        torch.manual_seed(7 + rank)
        model = TPDecoder(ctx, vocab=V, d_model=D, n_layers=L, n_heads=H, d_ff=FF, batch=B, seq=S).to(dev)
        for p in model.replicated_parameters():   # replicated parameters must agree
            dist.broadcast(p.data, 0)
        g = torch.Generator().manual_seed(3)
        tokens = torch.randint(0, V, (B, S), generator=g).to(dev)
        targets = torch.randint(0, V, (B, S), generator=g).to(dev)
        loss = model(tokens, targets)
        loss.backward()
        model.sync_replicated_grads()
        total = loss.detach().clone()
        dist.all_reduce(total)
        losses[fused] = total.item()
        grads[fused] = torch.cat([p.grad.reshape(-1).float() for p in model.parameters()])
        ctx.check()
    assert abs(losses[True] - losses[False]) < 2e-2 * abs(losses[False]), losses
    rel = ((grads[True] - grads[False]).norm() / grads[False].norm()).item()
    assert rel < 3e-2, rel
    return losses[True], rel


def test_tensor_parallel_decoder_fused_matches_collectives():
    spawn(_tp_model, _world(), timeout=300, _cuda=True)


def _gpu_soak(rank, world):
    dev = torch.device("cuda", torch.cuda.current_device())
    expect_sum = world * (world + 1) / 2
    t = torch.empty(1024, device=dev)
    # The reference soaks 10 000 iterations over TCP (tests/test_soak.py:66-76); here 2 000 back-to-back small
    # allreduces, 9 odd sizes, 200 interleaved allreduce / broadcast / barrier rounds and 5 x 128 MiB keep the
    # test inside a minute of GPU time while still wrapping every epoch counter's parity many times.
    for i in range(2000):           # small messages back to back: epochs and arena halves keep alternating
        t.fill_(float(rank + 1))
        dist.all_reduce(t)
    assert t[0].item() == expect_sum and t[-1].item() == expect_sum
    for n in (1, 3, 1023, 4097, 65536, 262145, 1 << 20, 3 << 20, (16 << 20) + 5):    # odd sizes, every schedule of `auto`
        x = torch.full((n,), float(rank + 1), device=dev)
        dist.all_reduce(x)
        assert x[0].item() == expect_sum and x[-1].item() == expect_sum, n
    for i in range(200):            # interleaved collectives keep their order
        a = torch.full((4096,), float(i + rank), device=dev)
        dist.all_reduce(a)
        b = torch.full((4096,), float(i), device=dev) if rank == i % world else torch.zeros(4096, device=dev)
        dist.broadcast(b, i % world)
        if i % 25 == 0:
            dist.barrier()
        assert b[0].item() == i and a[0].item() == world * i + world * (world - 1) / 2
    big = torch.ones(32 << 20, device=dev)
    for _ in range(5):
        dist.all_reduce(big, op=dist.ReduceOp.AVG)
    assert big[12345].item() == 1.0
    torch.cuda.synchronize()
    import mccl_b200
    mccl_b200.get_backend().device_comm(dev.index).check_status()
    return True


def test_soak_on_gpus():
    assert all(spawn(_gpu_soak, _world(), timeout=300, _cuda=True))


def _subgroups(rank, world):
    """Collectives on a sub-group of the GPUs leave the non-members' tensors untouched
    (the reference's multi-node check: tests/multinode/bench.py:53-64)."""
    dev = torch.device("cuda", torch.cuda.current_device())
    members = list(range(max(2, world // 2))) if world > 2 else [0, 1]
    sub = dist.new_group(members, backend="mccl")
    solo = dist.new_group([world - 1], backend="mccl")
    t = torch.full((5000,), float(rank + 1), device=dev)
    if rank in members:
        dist.all_reduce(t, group=sub)
        torch.cuda.synchronize()
        want = float(sum(m + 1 for m in members))
        assert t[0].item() == want and t[-1].item() == want
        big = torch.full((3 << 20,), float(rank + 1), device=dev)
        dist.all_reduce(big, op=dist.ReduceOp.AVG, group=sub)
        assert abs(big[7].item() - want / len(members)) < 1e-5
        out = torch.empty(len(members) * 10, device=dev)
        dist.all_gather_into_tensor(out, torch.full((10,), float(rank), device=dev), group=sub)
        assert out[::10].tolist() == [float(m) for m in members]
    else:
        torch.cuda.synchronize()
        assert t[0].item() == rank + 1      # untouched
    if rank == world - 1:
        s = torch.full((16,), 3.0, device=dev)
        dist.all_reduce(s, group=solo)       # a group of one is a no-op
        assert s[0].item() == 3.0
    # the world group still works afterwards, interleaved with the sub-group
    w = torch.ones(100, device=dev)
    dist.all_reduce(w)
    assert w[0].item() == world
    if rank in members:
        dist.barrier(group=sub)
    return True


def test_subgroup_collectives_on_gpus():
    assert all(spawn(_subgroups, _world(), timeout=300, _cuda=True, env={"MCCL_SUBGROUP_ARENA_MB": "32"}))


def _ddp_tiny_buckets(rank, world):
    """Stock DDP over 15 small layers with a bucket cap that gives one bucket per layer: many tiny
    allreduces back to back, on the comm stream, while backward runs (tests/test_ddp_e2e.py:102-129)."""
    import torch.nn as nn
    from torch.nn.parallel import DistributedDataParallel as DDP
    dev = torch.device("cuda", torch.cuda.current_device())
    torch.manual_seed(0)
    layers = []
    for _ in range(15):
        layers += [nn.Linear(64, 64), nn.Tanh()]
    model = nn.Sequential(*layers, nn.Linear(64, 1)).to(dev)
    import copy
    plain = copy.deepcopy(model)
    ddp = DDP(model, device_ids=[dev.index], bucket_cap_mb=0.01)
    opt = torch.optim.SGD(ddp.parameters(), lr=0.01)
    g = torch.Generator().manual_seed(200 + rank)
    x = torch.randn(64, 64, generator=g).to(dev)
    y = x.sum(1, keepdim=True) * 0.1
    # one step against the definition: DDP's gradients are the mean over ranks of the local gradients
    ((plain(x) - y) ** 2).mean().backward()
    ((ddp(x) - y) ** 2).mean().backward()
    for p_ddp, p_plain in zip(model.parameters(), plain.parameters()):
        want = p_plain.grad.clone()
        dist.all_reduce(want, op=dist.ReduceOp.AVG)
        assert torch.allclose(p_ddp.grad, want, rtol=1e-5, atol=1e-7), (p_ddp.grad - want).abs().max().item()
    for _ in range(30):
        loss = ((ddp(x) - y) ** 2).mean()
        opt.zero_grad()
        loss.backward()
        opt.step()
    flat = torch.cat([p.detach().reshape(-1) for p in model.parameters()])
    ref = flat.clone()
    dist.broadcast(ref, 0)
    assert torch.equal(ref, flat), "parameters diverged across ranks"
    assert torch.isfinite(flat).all()
    import mccl_b200
    mccl_b200.get_backend().check_device_status()
    return len(list(ddp.parameters()))


def test_ddp_many_tiny_buckets():
    spawn(_ddp_tiny_buckets, _world(), timeout=300, _cuda=True)


def _fsdp2(rank, world):
    """FSDP2 (fully_shard) over this backend: all-gather of parameter shards before use,
    reduce-scatter of gradients after backward, both as coalesced tensor forms."""
    import torch.nn as nn
    from torch.distributed.fsdp import fully_shard
    dev = torch.device("cuda", torch.cuda.current_device())
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(64, 128), nn.GELU(), nn.Linear(128, 128), nn.GELU(), nn.Linear(128, 8)).to(dev)
    ref = nn.Sequential(nn.Linear(64, 128), nn.GELU(), nn.Linear(128, 128), nn.GELU(), nn.Linear(128, 8)).to(dev)
    ref.load_state_dict(model.state_dict())
    for layer in model:
        if isinstance(layer, nn.Linear):
            fully_shard(layer)
    fully_shard(model)
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    ropt = torch.optim.SGD(ref.parameters(), lr=0.1)
    for step in range(4):
        xs = [torch.randn(16, 64, generator=torch.Generator().manual_seed(1000 * step + r)).to(dev) for r in range(world)]
        loss = model(xs[rank]).square().mean()
        opt.zero_grad()
        loss.backward()
        opt.step()
        # the unsharded reference sees the mean gradient over all ranks' batches
        ropt.zero_grad()
        (sum(ref(x).square().mean() for x in xs) / world).backward()
        ropt.step()
    full = [p.full_tensor() if hasattr(p, "full_tensor") else p for p in model.parameters()]
    for a, b in zip(full, ref.parameters()):
        assert torch.allclose(a, b, rtol=1e-4, atol=1e-5), (a - b).abs().max().item()
    return True


def test_fsdp2_fully_shard_smoke():
    spawn(_fsdp2, min(_world(), 2) if _world() >= 2 else _world(), timeout=300, _cuda=True)
