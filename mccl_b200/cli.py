"""``mccl`` command line.

Parity: ``mccl check | test | status | submit | jobs | cancel | watch`` plus
the flag forms ``--check``, ``--test`` and ``--worlds``, ``parse_memory("16GB")``
and a ``test`` command that shells out to pytest with ``MCCL_TEST_WORLDS``
(mccl/cli.py:111-218).  ``bench`` (collective sweep) and ``tune`` (write the
algorithm-selection table) are additions.  Job commands talk to a cluster
manager living in this process, with agents reachable over TCP.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time
from typing import List, Optional

_UNITS = {"B": 1, "KB": 1 << 10, "MB": 1 << 20, "GB": 1 << 30, "TB": 1 << 40}


def parse_memory(text: str) -> int:
    """"16GB" → bytes.  Accepts B / KB / MB / GB / TB (binary multiples), case-insensitive."""
    t = text.strip().upper()
    for unit in ("TB", "GB", "MB", "KB", "B"):
        if t.endswith(unit):
            return int(float(t[: -len(unit)]) * _UNITS[unit])
    return int(t)


def _state_path() -> str:
    return os.environ.get("MCCL_STATE_FILE", os.path.join(os.path.expanduser("~"), ".mccl_jobs.json"))


def _manager():
    """A cluster manager restored from the state file: nodes from MCCL_AGENTS ("host:port,..."), jobs from disk."""
    from . import _C
    cm = _C.ClusterManager(0, 200, 1000, 300, 200)
    for i, ep in enumerate(p for p in os.environ.get("MCCL_AGENTS", "").split(",") if p):
        host, _, port = ep.partition(":")
        cm.join(i, host, int(port), parse_memory(os.environ.get("MCCL_NODE_MEMORY", "180GB")))
    if os.path.exists(_state_path()):
        with open(_state_path()) as f:
            for j in json.load(f):
                if j["state"] in ("PENDING", "RUNNING", "RESCHEDULING"):
                    cm.scheduler().submit(j["name"], j["tenant"], j["priority"], j["nodes_required"], j["memory_per_node"],
                                          j["command"])
    return cm


def _save(cm) -> None:
    with open(_state_path(), "w") as f:
        json.dump(cm.scheduler().jobs(), f, indent=1)


def cmd_check(_args) -> int:
    from .check import run_all
    return run_all()


def cmd_test(args) -> int:
    env = dict(os.environ)
    if args.worlds:
        env["MCCL_TEST_WORLDS"] = args.worlds
        env["MCCL_TEST_WORLD"] = args.worlds.split(",")[0]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    marker = "gpu" if args.gpu else "not gpu"
    return subprocess.call([sys.executable, "-m", "pytest", os.path.join(root, "tests"), "-q", "-m", marker], env=env)


def cmd_status(_args) -> int:
    from . import _C, get_metrics
    m = get_metrics()
    print(f"collectives: ops={m.total_ops} bytes={m.total_bytes} errors={m.total_errors} avg={m.avg_latency_ms:.3f} ms")
    s = _C.get_stats()
    print(f"dmem: put {s['total_put_ops']} ops / {s['total_put_bytes']} B, get {s['total_get_ops']} ops / "
          f"{s['total_get_bytes']} B, errors {s['total_errors']}")
    cm = _manager()
    for n in cm.nodes():
        ok, status, payload, err = _C.agent_request(n["host"], n["agent_port"], _C.AGENT_STATS, b"", 500)
        print(f"node {n['node_id']} {n['host']}:{n['agent_port']} " + (payload.decode().replace("\n", " ") if ok else f"unreachable ({err})"))
    return 0


def cmd_submit(args) -> int:
    cm = _manager()
    jid = cm.scheduler().submit(args.name, args.tenant, args.priority.upper(), args.nodes, parse_memory(args.memory),
                                " ".join(args.command))
    _save(cm)
    print(jid)
    return 0


def cmd_jobs(_args) -> int:
    cm = _manager()
    for j in cm.scheduler().jobs():
        print(f"{j['id']:4d} {j['state']:12s} {j['priority']:8s} {j['tenant']:10s} nodes={j['nodes_required']} {j['name']}")
    return 0


def cmd_cancel(args) -> int:
    cm = _manager()
    ok = cm.scheduler().cancel(args.job_id)
    _save(cm)
    print("cancelled" if ok else "no such active job")
    return 0 if ok else 1


def cmd_watch(args) -> int:
    for _ in range(args.count):
        cmd_status(args)
        time.sleep(args.interval)
    return 0


def cmd_bench(args) -> int:
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    return subprocess.call([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
                            "--master-addr", "127.0.0.1", "--master-port", str(args.port),
                            os.path.join(root, "bench", "collective_sweep.py"), "--max-mb", str(args.max_mb)] + (["--out", args.out] if args.out else []))


def cmd_tune(args) -> int:
    """Turns a sweep result (JSON written by ``mccl bench --out``) into the algorithm-selection table."""
    from .tuning import save_tuning_table
    with open(args.sweep) as f:
        rows = [r for r in json.load(f) if r["op"] == "allreduce" and r["dtype"] == "fp32" and r["impl"].startswith("mccl:")]
    table_rows = [{"bytes": r["bytes"], "algo": r["impl"].split(":", 1)[1], "us": r["us"]} for r in rows
                  if r["impl"].split(":", 1)[1] in ("oneshot", "twoshot", "twoshot_push", "nvls")]
    world = rows[0]["world"] if rows else 0
    path = save_tuning_table(table_rows, world, args.out or None)
    print(path)
    return 0


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="mccl", description="mccl_b200 command line")
    ap.add_argument("--check", action="store_true", help="same as `mccl check`")
    ap.add_argument("--test", action="store_true", help="same as `mccl test`")
    ap.add_argument("--worlds", default="", help="world sizes for the tests, e.g. 2,3")
    sub = ap.add_subparsers(dest="cmd")
    sub.add_parser("check")
    t = sub.add_parser("test")
    t.add_argument("--worlds", default="")
    t.add_argument("--gpu", action="store_true")
    sub.add_parser("status")
    s = sub.add_parser("submit")
    s.add_argument("--name", default="job")
    s.add_argument("--tenant", default="default")
    s.add_argument("--priority", default="normal")
    s.add_argument("--nodes", type=int, default=1)
    s.add_argument("--memory", default="16GB")
    s.add_argument("command", nargs=argparse.REMAINDER)
    sub.add_parser("jobs")
    c = sub.add_parser("cancel")
    c.add_argument("job_id", type=int)
    w = sub.add_parser("watch")
    w.add_argument("--interval", type=float, default=1.0)
    w.add_argument("--count", type=int, default=10)
    b = sub.add_parser("bench")
    b.add_argument("--gpus", type=int, default=2)
    b.add_argument("--max-mb", type=float, default=256)
    b.add_argument("--port", type=int, default=29533)
    b.add_argument("--out", default="")
    tu = sub.add_parser("tune")
    tu.add_argument("sweep")
    tu.add_argument("--out", default="")
    args = ap.parse_args(argv)
    if args.check and not args.cmd:
        return cmd_check(args)
    if args.test and not args.cmd:
        args.gpu = False
        return cmd_test(args)
    handlers = {"check": cmd_check, "test": cmd_test, "status": cmd_status, "submit": cmd_submit, "jobs": cmd_jobs,
                "cancel": cmd_cancel, "watch": cmd_watch, "bench": cmd_bench, "tune": cmd_tune}
    if not args.cmd:
        ap.print_help()
        return 0
    return handlers[args.cmd](args)


if __name__ == "__main__":
    sys.exit(main())
