"""Python face of the native per-operation metrics.

Parity: the reference's example trainer calls ``mccl.get_metrics()`` and reads
``total_ops, avg_latency_ms, avg_sync_ms, avg_network_ms, avg_reduce_ms`` from
the result (examples/ddp_dummy_train.py:211-224); the summary fields follow
its C++ ``Metrics::summarize`` (csrc/runtime/Metrics.cpp:69-116).
"""
from __future__ import annotations

import sys


def get_metrics():
    from . import _C
    return _C.get_metrics()


def reset_metrics() -> None:
    from . import _C
    _C.reset_metrics()


def metrics_history():
    from . import _C
    return _C.metrics_history()


def set_trace(path: str) -> None:
    """Appends every finished collective to ``<path>.<pid>`` as a Chrome-trace event (one JSON object per
    line); ``""`` stops.  ``MCCL_TRACE=<path>`` in the environment does the same from the first op on."""
    from . import _C
    _C.set_trace(path)


def enable_nvtx(on: bool = True) -> None:
    """Brackets every collective with an NVTX range (``MCCL_NVTX=1`` switches it on at import)."""
    from . import _C
    _C.enable_nvtx(on)


def log_metrics(file=None) -> None:
    m = get_metrics()
    out = file or sys.stderr
    print(
        f"[mccl metrics] ops={m.total_ops} bytes={m.total_bytes} errors={m.total_errors} "
        f"lat avg/p50/p99={m.avg_latency_ms:.3f}/{m.p50_latency_ms:.3f}/{m.p99_latency_ms:.3f} ms "
        f"peak={m.peak_gbps:.2f} Gbps queue={m.avg_queue_wait_ms:.3f} ms exec={m.avg_execution_ms:.3f} ms",
        file=out,
    )
