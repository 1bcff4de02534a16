"""Distributed memory and coherence between PROCESSES of one box: shared-memory fabric and mailboxes."""
import ctypes
import multiprocessing as mp
import os
import time
import traceback

import numpy as np

PAGE = 64 * 1024


def _view(addr, n):
    return np.ctypeslib.as_array((ctypes.c_uint8 * n).from_address(addr))


def _node(rank, world, name, barrier, queue):
    try:
        import mccl_b200
        C = mccl_b200._C
        fab = C.ShmFabric(name, rank, world)
        dm = C.DmemManager(rank, fab)
        heap_id, ptr = fab.alloc_heap(2 * PAGE)
        mine = _view(ptr, 2 * PAGE)
        mine[:] = rank + 1
        rid = dm.register_region(ptr, 2 * PAGE, heap_id=heap_id, heap_offset=0)
        barrier.wait()
        # ---- dmem: put into the right-hand neighbour, get from the left-hand one ----
        right, left = (rank + 1) % world, (rank - 1) % world
        src = np.full(128, 100 + rank, dtype=np.uint8)
        assert dm.put(right, rid, 1000, src.ctypes.data, 128) != 0
        dm.fence()
        barrier.wait()
        assert (mine[1000:1128] == 100 + left).all() and mine[999] == rank + 1
        dst = np.zeros(64, dtype=np.uint8)
        assert dm.get(left, rid, 0, dst.ctypes.data, 64) != 0
        assert (dst == left + 1).all()
        barrier.wait()
        assert dm.put_with_imm(right, rid, 0, src.ctypes.data, 8, 7000 + rank) != 0
        barrier.wait()
        imms = fab.collect_imm()
        assert [(i[0], i[4]) for i in imms] == [(left, 7000 + left)], imms
        barrier.wait()
        # ---- coherence over the shared mailboxes: node 0 is the home of page 0 of its region ----
        mine[:PAGE] = 9 if rank == 0 else mine[:PAGE]
        bus = C.ShmBus(fab)
        co = C.CoherenceProtocol(rank, bus, dm, 3000)
        co.start()
        barrier.wait()
        try:
            if rank != 0:
                a = co.read_page(0, rid, 5)
                assert _view(a, PAGE)[5] == 9 and co.local_state(0, rid, 0) == 1      # SHARED copy
            barrier.wait()
            if rank == 1:
                w = co.read_page(0, rid, 5, write=True)                                 # invalidates the other readers
                _view(w, PAGE)[:16] = 55
                co.write_page_done(0, rid, 5)
                co.release()                                                            # writes the page home
            barrier.wait()
            if rank == 0:
                time.sleep(0.05)
                assert mine[0] == 55 and mine[16] == 9
                assert co.directory_lookup(rid, 0)[0] == 0                              # UNCACHED again
            if rank >= 2:
                assert co.local_state(0, rid, 0) == 0                                   # invalidated by the writer
            co.barrier_all()
            co.fence()
            stats = co.stats()
            barrier.wait()      # nobody stops serving while a peer still waits for fence acknowledgements
        finally:
            co.shutdown()
        barrier.wait()
        queue.put((rank, "ok", stats["messages_handled"]))
    except BaseException as e:  # noqa: BLE001
        queue.put((rank, "error", f"{type(e).__name__}: {e}\n{traceback.format_exc()}"))
        try:
            barrier.abort()
        except Exception:
            pass


def test_dmem_and_coherence_between_processes():
    world = 3
    ctx = mp.get_context("spawn")
    barrier, queue = ctx.Barrier(world), ctx.Queue()
    name = f"t{os.getpid()}"
    procs = [ctx.Process(target=_node, args=(r, world, name, barrier, queue), daemon=True) for r in range(world)]
    for p in procs:
        p.start()
    results = [queue.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=10)
    bad = [r for r in results if r[1] != "ok"]
    assert not bad, "\n".join(str(b[2]) for b in bad)
    assert all(r[2] > 0 for r in results)
    assert not [f for f in os.listdir("/dev/shm") if f.startswith(f"mccl-{name}")]   # segments are unlinked


def _module_api(rank, world, name, barrier, queue):
    try:
        import mccl_b200
        C = mccl_b200._C
        C.init_dmem(node_id=rank, num_peers=world - 1, shm_name=name)
        heap_id, ptr = C.alloc_dmem_heap(4096)
        rid = C.register_region(ptr, 4096, heap_id=heap_id, heap_offset=0)
        mine = _view(ptr, 4096)
        barrier.wait()
        peer = (rank + 1) % world
        src = np.arange(256, dtype=np.uint8) ^ rank
        assert C.put(peer, rid, 512, src.ctypes.data, 256) != 0
        assert C.drain_pending() >= 0
        barrier.wait()
        left = (rank - 1) % world
        assert (mine[512:768] == (np.arange(256, dtype=np.uint8) ^ left)).all()
        back = np.zeros(256, dtype=np.uint8)
        assert C.get(peer, rid, 512, back.ctypes.data, 256) != 0
        assert (back == src).all()
        st = C.get_stats()
        assert st["total_put_ops"] == 1 and st["total_get_ops"] == 1 and st["total_errors"] == 0
        # memory that is not in a shared heap cannot be reached from another process: the call fails cleanly
        private = np.zeros(64, dtype=np.uint8)
        prid = C.register_region(private.ctypes.data, 64)
        barrier.wait()
        assert C.put(peer, prid, 0, src.ctypes.data, 8) == 0
        assert C.get_stats()["total_errors"] == 1
        barrier.wait()
        C.shutdown_dmem()
        queue.put((rank, "ok", 1))
    except BaseException as e:  # noqa: BLE001
        queue.put((rank, "error", f"{type(e).__name__}: {e}\n{traceback.format_exc()}"))
        try:
            barrier.abort()
        except Exception:
            pass


def test_module_level_dmem_between_processes():
    world = 2
    ctx = mp.get_context("spawn")
    barrier, queue = ctx.Barrier(world), ctx.Queue()
    name = f"m{os.getpid()}"
    procs = [ctx.Process(target=_module_api, args=(r, world, name, barrier, queue), daemon=True) for r in range(world)]
    for p in procs:
        p.start()
    results = [queue.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=10)
    bad = [r for r in results if r[1] != "ok"]
    assert not bad, "\n".join(str(b[2]) for b in bad)
