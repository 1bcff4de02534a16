"""MCCL_TRACE-style op tracing and the NVTX switch (CPU ranks over the TCP mesh)."""
import glob
import json
import os
import tempfile

import torch
import torch.distributed as dist

from tests.common import spawn


def _traced(rank, world, path):
    from mccl_b200 import metrics
    metrics.enable_nvtx(True)      # ranges are no-ops without a profiler attached; must not disturb the ops
    metrics.set_trace(path)
    t = torch.full((1024,), float(rank + 1))
    dist.all_reduce(t)
    dist.barrier()
    metrics.set_trace("")
    metrics.enable_nvtx(False)
    assert t[0].item() == sum(range(1, world + 1))
    return os.getpid()


def test_trace_file_has_one_event_per_op():
    d = tempfile.mkdtemp()
    path = os.path.join(d, "trace")
    pids = spawn(_traced, 2, path=path)
    files = sorted(glob.glob(path + ".*"))
    assert len(files) == 2 and {int(f.rsplit(".", 1)[1]) for f in files} == set(pids)
    for f in files:
        events = [json.loads(line.rstrip().rstrip(",")) for line in open(f) if line.strip()]
        names = [e["name"] for e in events]
        assert any("allreduce" in n for n in names) and any("barrier" in n for n in names), names
        for e in events:
            assert e["ph"] == "X" and e["dur"] >= 0 and e["args"]["failed"] is False
        ar = next(e for e in events if "allreduce" in e["name"])
        assert ar["args"]["bytes"] == 4096
