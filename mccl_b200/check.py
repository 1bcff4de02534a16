"""Read-only environment checks (``mccl check``).

Parity: the reference runs seven checks (platform, python version, toolchain,
backend registered, interconnect interface, VPN, peers reachable), prints a
table and exits 1 when a required check fails (mccl/check.py:1-167).  The
checks here are the ones that matter on an NVSwitch box; none changes a setting.
"""
from __future__ import annotations

import os
import socket
import subprocess
import sys
from typing import Callable, List, NamedTuple


class CheckResult(NamedTuple):
    name: str
    ok: bool
    required: bool
    detail: str


def _check_python() -> CheckResult:
    ok = sys.version_info >= (3, 10)
    return CheckResult("python >= 3.10", ok, True, sys.version.split()[0])


def _check_torch() -> CheckResult:
    try:
        import torch
        return CheckResult("torch importable", True, True, f"torch {torch.__version__}, CUDA build {torch.version.cuda}")
    except Exception as e:  # noqa: BLE001
        return CheckResult("torch importable", False, True, str(e))


def _check_extension() -> CheckResult:
    try:
        import mccl_b200
        return CheckResult("native extension loads", True, True, f"mccl_b200._C {mccl_b200._C.__version__}")
    except Exception as e:  # noqa: BLE001
        return CheckResult("native extension loads", False, True, str(e))


def _check_backend() -> CheckResult:
    try:
        import torch.distributed as dist
        import mccl_b200  # noqa: F401
        ok = "mccl" in dist.Backend.backend_list
        return CheckResult("backend 'mccl' registered", ok, True, "dist.Backend.backend_list")
    except Exception as e:  # noqa: BLE001
        return CheckResult("backend 'mccl' registered", False, True, str(e))


def _check_gpus() -> CheckResult:
    try:
        import torch
        if not torch.cuda.is_available():
            return CheckResult("CUDA devices", False, False, "no GPU visible: only CPU tensors (TCP) will work")
        n = torch.cuda.device_count()
        caps = {torch.cuda.get_device_capability(i) for i in range(n)}
        ok = caps == {(10, 0)}
        return CheckResult("CUDA devices are sm_100", ok, False, f"{n} device(s), capability {sorted(caps)}")
    except Exception as e:  # noqa: BLE001
        return CheckResult("CUDA devices", False, False, str(e))


def _check_p2p() -> CheckResult:
    try:
        import torch
        n = torch.cuda.device_count() if torch.cuda.is_available() else 0
        if n < 2:
            return CheckResult("peer access matrix", True, False, "fewer than two GPUs: nothing to check")
        bad = [(i, j) for i in range(n) for j in range(n) if i != j and not torch.cuda.can_device_access_peer(i, j)]
        return CheckResult("peer access matrix", not bad, False, "all pairs" if not bad else f"no P2P between {bad[:4]}")
    except Exception as e:  # noqa: BLE001
        return CheckResult("peer access matrix", False, False, str(e))


def _check_nvlink() -> CheckResult:
    try:
        out = subprocess.run(["nvidia-smi", "nvlink", "--status", "-i", "0"], capture_output=True, text=True, timeout=10).stdout
        links = [l for l in out.splitlines() if "GB/s" in l]
        return CheckResult("NVLink links up (GPU 0)", bool(links), False, f"{len(links)} link(s)")
    except Exception as e:  # noqa: BLE001
        return CheckResult("NVLink links up (GPU 0)", False, False, f"nvidia-smi unavailable: {e}")


def _check_nccl() -> CheckResult:
    try:
        import torch.distributed as dist
        ok = dist.is_nccl_available()
        return CheckResult("NCCL available (CUDA send/recv)", ok, False, "torch.distributed.is_nccl_available()")
    except Exception as e:  # noqa: BLE001
        return CheckResult("NCCL available (CUDA send/recv)", False, False, str(e))


def _check_peers() -> CheckResult:
    peers = [p for p in os.environ.get("MCCL_PEERS", "").split(",") if p]
    if not peers:
        return CheckResult("MCCL_PEERS reachable", True, False, "MCCL_PEERS not set")
    bad = []
    for p in peers:
        host, _, port = p.partition(":")
        try:
            with socket.create_connection((host, int(port or 29500)), timeout=1.0):
                pass
        except OSError:
            bad.append(p)
    return CheckResult("MCCL_PEERS reachable", not bad, False, "all reachable" if not bad else f"unreachable: {bad}")


CHECKS: List[Callable[[], CheckResult]] = [_check_python, _check_torch, _check_extension, _check_backend, _check_gpus,
                                           _check_p2p, _check_nvlink, _check_nccl, _check_peers]


def run_all(file=None) -> int:
    """Prints a table; returns 1 when a required check failed, else 0."""
    out = file or sys.stdout
    results = [c() for c in CHECKS]
    width = max(len(r.name) for r in results)
    failed = False
    for r in results:
        mark = "ok  " if r.ok else ("FAIL" if r.required else "warn")
        print(f"[{mark}] {r.name.ljust(width)}  {r.detail}", file=out)
        failed = failed or (r.required and not r.ok)
    return 1 if failed else 0


if __name__ == "__main__":
    sys.exit(run_all())
