"""Distributed runtime on the host: scheduler, node agent, cluster manager with
heartbeat failure detection, distributed memory, coherence protocol, kernel
dispatch.  The reference has no tests for dmem, coherence, scheduler, cluster
manager or agent (its tests/ directory covers the process group only); the cases
follow the behaviour its sources describe.  Failures are made on the host: an
agent that stops answering, a dropped protocol message.
"""
import ctypes
import time

import numpy as np
import pytest

import mccl_b200

C = mccl_b200._C
GB = 1 << 30


# ------------------------------------------------------------------ scheduler --
def _loads(n, total=80 * GB, used=0):
    return [(i, True, total, used) for i in range(n)]


def test_scheduler_priority_then_fcfs():
    s = C.Scheduler()
    a = s.submit("a", priority="LOW", memory_per_node=60 * GB)
    b = s.submit("b", priority="HIGH", memory_per_node=60 * GB)
    c = s.submit("c", priority="NORMAL", memory_per_node=60 * GB)
    d = s.submit("d", priority="NORMAL", memory_per_node=60 * GB)
    r = s.schedule_tick(_loads(2))
    assert [j for j, _ in r["started"]] == [b, c]          # high first, then the older NORMAL
    assert s.get(a)["state"] == "PENDING" and s.get(d)["state"] == "PENDING"
    s.complete(b)
    r = s.schedule_tick(_loads(2))
    assert [j for j, _ in r["started"]] == [d]              # NORMAL before LOW
    assert s.get(b)["state"] == "COMPLETED"


def test_scheduler_first_fit_memory_and_multinode():
    s = C.Scheduler()
    big = s.submit("big", nodes=2, memory_per_node=50 * GB)
    small = s.submit("small", nodes=1, memory_per_node=40 * GB)
    r = s.schedule_tick([(0, True, 80 * GB, 40 * GB), (1, True, 80 * GB, 0), (2, True, 80 * GB, 0), (3, False, 80 * GB, 0)])
    placed = dict(r["started"])
    assert placed[big] == [1, 2]         # node 0 lacks memory, node 3 is offline
    assert placed[small] == [0]
    too_big = s.submit("huge", memory_per_node=100 * GB)
    assert s.schedule_tick(_loads(4))["started"] == []
    assert s.cancel(too_big) and s.get(too_big)["state"] == "CANCELLED"


def test_scheduler_preemption_and_requeue():
    s = C.Scheduler()
    low = s.submit("low", priority="LOW", memory_per_node=70 * GB)
    s.schedule_tick(_loads(1))
    crit = s.submit("crit", priority="CRITICAL", memory_per_node=70 * GB)
    r = s.schedule_tick(_loads(1))
    assert r["preempted"] == [low] and [j for j, _ in r["started"]] == [crit]
    assert s.get(low)["state"] == "PENDING" and s.get(low)["preemptions"] == 1
    normal = s.submit("normal", priority="NORMAL", memory_per_node=70 * GB)
    assert s.schedule_tick(_loads(1))["started"] == []     # NORMAL does not preempt


def test_scheduler_evict_node_fails_single_and_requeues_multi():
    s = C.Scheduler()
    single = s.submit("single", nodes=1, memory_per_node=30 * GB)
    multi = s.submit("multi", nodes=2, memory_per_node=30 * GB)
    later = s.submit("later", nodes=3, memory_per_node=30 * GB)     # node 0 is full after the first two
    placed = dict(s.schedule_tick(_loads(3))["started"])
    assert placed[single] == [0] and placed[multi] == [0, 1]
    touched = s.evict_node(0)
    assert set(touched) == {single, multi}
    assert s.get(single)["state"] == "FAILED" and "offline" in s.get(single)["reason"]
    assert s.get(multi)["state"] == "RESCHEDULING"
    assert [j["id"] for j in s.queue()][0] == multi         # requeued at the front
    placed = dict(s.schedule_tick([(1, True, 80 * GB, 0), (2, True, 80 * GB, 0)])["started"])
    assert placed[multi] == [1, 2] and later not in placed


def test_scheduler_fair_share_bump_and_accounting():
    s = C.Scheduler()
    hog = s.submit("hog", tenant="hog", priority="NORMAL", memory_per_node=GB)
    s.schedule_tick(_loads(1, total=GB))
    time.sleep(0.05)
    s.complete(hog)
    assert s.tenant_node_seconds("hog") > 0.04
    # hog has used the machine, newcomer has not: newcomer's LOW job counts as NORMAL and, being
    # older than hog's next NORMAL job, goes first
    newcomer = s.submit("n1", tenant="newcomer", priority="LOW", memory_per_node=GB)
    hog2 = s.submit("hog2", tenant="hog", priority="NORMAL", memory_per_node=GB)
    r = s.schedule_tick(_loads(1, total=GB))
    assert [j for j, _ in r["started"]] == [newcomer]
    assert s.get(hog2)["state"] == "PENDING"


# ---------------------------------------------------------------------- agent --
def test_agent_protocol_roundtrip():
    a = C.AgentServer()
    port = a.start()
    try:
        ok, status, payload, err = C.agent_request("127.0.0.1", port, C.AGENT_PING)
        assert ok and status == 0 and a.pings == 1
        reg = (7).to_bytes(4, "little") + (4096).to_bytes(8, "little")
        assert C.agent_request("127.0.0.1", port, C.AGENT_REGISTER, reg)[1] == 0
        assert a.regions() == {7: 4096}
        calls = []
        a.set_run_handler(lambda k, off, cnt: calls.append((k, off, cnt)) or 0)
        run = (5).to_bytes(2, "little") + b"scale" + (128).to_bytes(8, "little") + (64).to_bytes(8, "little")
        assert C.agent_request("127.0.0.1", port, C.AGENT_KERNEL_RUN, run)[1] == 3      # NOT_FOUND: not loaded yet
        assert C.agent_request("127.0.0.1", port, C.AGENT_KERNEL_LOAD, b"scale")[1] == 0
        assert C.agent_request("127.0.0.1", port, C.AGENT_KERNEL_RUN, run)[1] == 0
        assert calls == [("scale", 128, 64)]
        ok, status, payload, _ = C.agent_request("127.0.0.1", port, C.AGENT_STATS)
        stats = dict(line.split("=") for line in payload.decode().split())
        assert stats["pings"] == "1" and stats["runs"] == "1" and stats["regions"] == "1"
        assert C.agent_request("127.0.0.1", port, 99)[1] == 2                           # UNKNOWN_COMMAND
        assert C.agent_request("127.0.0.1", port, C.AGENT_DEREGISTER, (7).to_bytes(4, "little"))[1] == 0
    finally:
        a.stop()
    ok, _, _, err = C.agent_request("127.0.0.1", port, C.AGENT_PING, b"", 200)
    assert not ok and err


# ------------------------------------------------------------ cluster manager --
def test_cluster_membership_and_leader():
    cm = C.ClusterManager(0)
    assert cm.leader() == -1
    assert cm.join(2) and cm.join(1) and cm.join(5)
    assert cm.leader() == 1 and cm.online_count() == 3
    cm.node_failure(1)
    assert cm.leader() == 2 and cm.online_count() == 2
    assert cm.heartbeat(1) and cm.leader() == 1            # a node that answers again is back
    assert cm.leave(1) and cm.leader() == 2
    assert not cm.join(8)                                   # ids 0..7 only


def test_heartbeat_failure_detection_evicts_jobs_and_reelects():
    agents = [C.AgentServer() for _ in range(3)]
    ports = [a.start() for a in agents]
    cm = C.ClusterManager(0, heartbeat_interval_ms=40, heartbeat_timeout_ms=250, ping_socket_timeout_ms=100, scheduler_tick_ms=40)
    for i, p in enumerate(ports):
        cm.join(i, "127.0.0.1", p, 80 * GB)
    cm.publish_region(0, 1, 0x1000, 4096)
    cm.publish_region(1, 1, 0x2000, 4096)
    sched = cm.scheduler()
    single = sched.submit("on-node-0", nodes=1, memory_per_node=GB)
    multi = sched.submit("spans", nodes=3, memory_per_node=GB)
    cm.start()
    try:
        deadline = time.time() + 3
        while time.time() < deadline and sched.running_count() < 2:
            time.sleep(0.02)
        assert sched.get(single)["nodes"] == [0] and sched.get(multi)["nodes"] == [0, 1, 2]
        assert all(a.pings > 0 for a in agents) or time.sleep(0.2) is None
        agents[0].set_unresponsive(True)                    # the node hangs: connections open, no answers
        deadline = time.time() + 3
        while time.time() < deadline and cm.online_count() == 3:
            time.sleep(0.02)
        assert cm.online_count() == 2 and cm.leader() == 1
        assert sched.get(single)["state"] == "FAILED"
        assert sched.get(multi)["state"] in ("RESCHEDULING", "PENDING")   # requeued, cannot run on 2 nodes
        assert cm.lookup_region(0, 1) is None and cm.lookup_region(1, 1) == (0x2000, 4096)
        states = {n["node_id"]: n["status"] for n in cm.nodes()}
        assert states == {0: "OFFLINE", 1: "ONLINE", 2: "ONLINE"}
    finally:
        cm.stop()
        for a in agents:
            a.set_unresponsive(False)
            a.stop()


# ----------------------------------------------------------------------- dmem --
def _buf(n, fill=0):
    a = np.full(n, fill, dtype=np.uint8)
    return a, a.ctypes.data


def test_dmem_put_get_imm_and_stats():
    fab = C.LocalFabric(3)
    nodes = [C.DmemManager(i, fab) for i in range(3)]
    mem1, p1 = _buf(1 << 16)
    r1 = nodes[1].register_region(p1, mem1.nbytes)
    assert nodes[0].catalog_size() == 1 and nodes[2].catalog_size() == 1     # replicated directory
    src, ps = _buf(1000, 7)
    wr = nodes[0].put(1, r1, 128, ps, 1000)
    assert wr > 0 and nodes[0].poll_completion(wr)
    assert (mem1[128:1128] == 7).all() and mem1[127] == 0 and mem1[1128] == 0
    dst, pd = _buf(1000)
    assert nodes[2].get(1, r1, 128, pd, 1000) > 0
    assert (dst == 7).all()
    assert nodes[0].put_with_imm(1, r1, 0, ps, 16, 0xBEEF) > 0
    assert nodes[1].take_immediates() == [(0, r1, 0, 16, 0xBEEF)] and nodes[1].take_immediates() == []
    # bounds: past the end of the region, unknown region, unknown node's region
    assert nodes[0].put(1, r1, (1 << 16) - 10, ps, 100) == 0
    assert nodes[0].get(1, 99, 0, pd, 10) == 0
    st = nodes[0].stats()
    assert st["total_put_ops"] == 2 and st["total_put_bytes"] == 1016 and st["total_errors"] == 2
    assert nodes[2].stats()["total_get_bytes"] == 1000
    # read-only region refuses remote writes
    ro, pro = _buf(256, 3)
    rr = nodes[2].register_region(pro, 256, C.REGION_READABLE | C.REGION_SHARED)
    assert nodes[0].put(2, rr, 0, ps, 16) == 0 and nodes[0].get(2, rr, 0, pd, 16) > 0
    assert nodes[1].unregister_region(r1) and nodes[0].put(1, r1, 0, ps, 16) == 0
    assert nodes[0].drain_pending() == 0
    assert nodes[2].catalog_roundtrip()[0] == nodes[2].catalog_roundtrip()[1]


def test_global_address_wire_format():
    raw, node, region, off, packed = C.global_address_wire(3, 0x01020304, 0x1122334455667788)
    assert len(raw) == 14 and (node, region, off) == (3, 0x01020304, 0x1122334455667788)
    assert raw == (3).to_bytes(2, "little") + (0x01020304).to_bytes(4, "little") + (0x1122334455667788).to_bytes(8, "little")
    assert packed == (3 << 48) | (0x01020304 << 16)


def test_module_level_dmem_api():
    C.init_dmem(node_id=0, num_peers=1)
    try:
        peer_mem, pp = _buf(4096)
        rid = C.register_region_on(1, pp, 4096)
        src, ps = _buf(64, 9)
        wr = C.put(1, rid, 100, ps, 64)
        assert wr > 0 and C.poll_completion(wr) and (peer_mem[100:164] == 9).all()
        assert C.get_stats()["total_put_bytes"] == 64 and C.drain_pending() == 0
        mine, pm = _buf(128)
        my_id = C.register_region(pm, 128)
        assert my_id > 0 and C.unregister_region(my_id)
        C.metal_sync()
    finally:
        C.shutdown_dmem()
    assert C.get_stats()["total_put_bytes"] == 0


# ------------------------------------------------------------------ coherence --
PAGE = C.COHERENCE_PAGE_SIZE


def _cluster(n, timeout_ms=2000):
    fab, bus = C.LocalFabric(n), C.LocalBus(n)
    dm = [C.DmemManager(i, fab) for i in range(n)]
    co = [C.CoherenceProtocol(i, bus, dm[i], timeout_ms) for i in range(n)]
    for c in co:
        c.start()
    return fab, bus, dm, co


def _view(addr, n):
    return np.ctypeslib.as_array((ctypes.c_uint8 * n).from_address(addr))


def test_coherence_read_share_write_invalidate_writeback():
    fab, bus, dm, co = _cluster(3)
    try:
        home, ph = _buf(2 * PAGE, 1)
        rid = dm[0].register_region(ph, home.nbytes)
        # two readers share page 0
        a1 = co[1].read_page(0, rid, 10)
        a2 = co[2].read_page(0, rid, 20)
        assert _view(a1, PAGE)[10] == 1 and _view(a2, PAGE)[20] == 1
        assert co[0].directory_lookup(rid, 0) == (1, 0b110, 0xff, 2)            # SHARED by nodes 1 and 2
        assert co[1].local_state(0, rid, 0) == 1
        # node 1 wants to write: node 2's copy is invalidated first
        w = co[1].read_page(0, rid, 10, write=True)
        _view(w, PAGE)[:100] = 42
        co[1].write_page_done(0, rid, 10)
        assert co[2].local_state(0, rid, 0) == 0 and co[1].local_state(0, rid, 0) == 2
        state, sharers, owner, _ = co[0].directory_lookup(rid, 0)
        assert (state, sharers, owner) == (2, 0b010, 1)                          # EXCLUSIVE, owner 1
        assert home[0] == 1                                                      # not written back yet
        # node 2 reads again: the home makes node 1 write its dirty copy back first
        a2 = co[2].read_page(0, rid, 0)
        assert home[0] == 42 and _view(a2, PAGE)[99] == 42 and _view(a2, PAGE)[100] == 1
        assert co[1].local_state(0, rid, 0) == 0 and co[1].stats()["writebacks"] == 1
        # release writes a dirty exclusive page home and forgets every cached page
        w = co[2].read_page(0, rid, PAGE + 5, write=True)                        # page 1
        _view(w, PAGE)[5] = 77
        co[2].write_page_done(0, rid, PAGE + 5)
        co[2].release()
        assert home[PAGE + 5] == 77 and co[2].local_state(0, rid, PAGE) == 0
        time.sleep(0.05)
        assert co[0].directory_lookup(rid, 1)[0] == 0                            # UNCACHED again
        # the home itself goes through the directory too
        h = co[0].read_page(0, rid, 0)
        assert h == ph
        for c in co:
            c.acquire()
        assert co[0].global_epoch() >= 1
    finally:
        for c in co:
            c.shutdown()


def test_coherence_barrier_fence_and_lost_message_times_out():
    import threading
    fab, bus, dm, co = _cluster(3, timeout_ms=400)
    try:
        done = []
        ts = [threading.Thread(target=lambda c=c: (c.barrier_all(), done.append(1))) for c in co]
        for t in ts[:2]:
            t.start()
        time.sleep(0.1)
        assert done == []                 # nobody leaves before the last node arrives
        ts[2].start()
        for t in ts:
            t.join()
        assert len(done) == 3
        co[0].fence()
        # a lost reply makes the requester give up with an error instead of waiting for ever
        home, ph = _buf(PAGE, 5)
        rid = dm[0].register_region(ph, home.nbytes)
        bus.drop_op(2, 1)                 # READ_REPLY messages to node 1 vanish
        with pytest.raises(C.TimeoutError):
            co[1].read_page(0, rid, 0)
        assert co[1].stats()["timeouts"] == 1
        bus.drop_nothing()
        assert _view(co[1].read_page(0, rid, 0), PAGE)[0] == 5     # the protocol still works afterwards
    finally:
        for c in co:
            c.shutdown()


# ------------------------------------------------------------ kernel dispatch --
def test_data_parallel_split_and_pipeline_schedule():
    assert C.data_parallel_split(10, 3) == [(0, 0, 3), (1, 3, 3), (2, 6, 4)]   # remainder to the last node
    assert C.data_parallel_split(2, 4) == [(0, 0, 0), (1, 0, 0), (2, 0, 0), (3, 0, 2)]
    assert C.data_parallel_split(0, 2) == [(0, 0, 0), (1, 0, 0)]
    sched = C.pipeline_schedule(2, 3)   # fill, steady, drain
    assert sched == [(0, 0, 0), (1, 0, 1), (1, 1, 0), (2, 0, 2), (2, 1, 1), (3, 1, 2)]
