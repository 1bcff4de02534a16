"""Helpers for stock ``DistributedDataParallel`` on backend "mccl".

DDP needs nothing special: ``DDP(model)`` over a group created with
``backend="mccl"`` all-reduces its gradient buckets through the backend, as
with the reference (README.md:27-35).  ``bf16_wire_hook`` is a DDP
communication hook that sends fp32 gradient buckets as bf16 on the wire with
fp32 accumulation and the 1/world scale fused into the same kernel, which is
what ``MCCL_WIRE_DTYPE=bf16`` selects globally.
"""
import contextlib
import os

import torch
import torch.distributed as dist


@contextlib.contextmanager
def wire_dtype(name: str):
    """Temporarily sets ``MCCL_WIRE_DTYPE`` (the backend re-reads it on every allreduce)."""
    old = os.environ.get("MCCL_WIRE_DTYPE")
    if name:
        os.environ["MCCL_WIRE_DTYPE"] = name
    else:
        os.environ.pop("MCCL_WIRE_DTYPE", None)
    try:
        yield
    finally:
        if old is None:
            os.environ.pop("MCCL_WIRE_DTYPE", None)
        else:
            os.environ["MCCL_WIRE_DTYPE"] = old


def bf16_wire_hook(group, bucket: dist.GradBucket) -> torch.futures.Future[torch.Tensor]:
    """``model.register_comm_hook(group, bf16_wire_hook)``: averaged gradients, bf16 on the wire.

    The wire dtype is an argument of the backend call, so nothing here touches ``os.environ`` (the hook
    runs on autograd's thread while other threads may be issuing collectives of their own)."""
    from .._backend import get_backend
    buf = bucket.buffer()
    be = get_backend(group)
    if be is None:   # not an mccl group: plain averaged allreduce
        work = dist.all_reduce(buf, op=dist.ReduceOp.AVG, group=group, async_op=True)
    else:
        work = be.allreduce_with(buf, op="avg", wire="bf16" if buf.dtype == torch.float32 else "native")
    return work.get_future().then(lambda fut: fut.value()[0])
