"""Registration of the ``mccl`` backend with ``torch.distributed``.

Parity: the reference registers a creator ``(prefix_store, rank, world_size,
timeout)`` under the name "mccl" for ``["cpu", "mps"]``, idempotently, and
offers ``set_iface_priority`` to steer interface selection
(mccl/_backend.py:21-75).  Here the devices are ``["cpu", "cuda"]`` and no
interface filter is installed by default (single-box runs use loopback).
"""
from __future__ import annotations

import os
from datetime import timedelta
from typing import Iterable

import torch
import torch.distributed as dist

_REGISTERED = False


def set_iface_priority(prefixes: Iterable[str]) -> None:
    """IPv4 prefixes (e.g. ``["10.0.1.", "192.168.5."]``) the TCP mesh may use.

    Must be called before ``init_process_group``; an empty list removes the filter.
    """
    prefixes = list(prefixes)
    if prefixes:
        os.environ["MCCL_IFACE_PRIORITY"] = ",".join(prefixes)
    else:
        os.environ.pop("MCCL_IFACE_PRIORITY", None)


def _nccl_p2p_factory(store, rank: int, world_size: int, timeout: timedelta):
    """Builds the NCCL group that carries CUDA send/recv (pipeline stages)."""
    def make():
        if not hasattr(dist, "ProcessGroupNCCL"):
            raise RuntimeError("mccl: CUDA send/recv needs torch built with NCCL")
        pstore = dist.PrefixStore("mccl_p2p", store)
        opts = dist.ProcessGroupNCCL.Options()
        try:
            opts._timeout = timeout
        except Exception:  # attribute name differs across torch versions
            pass
        return dist.ProcessGroupNCCL(pstore, rank, world_size, opts)
    return make


def _create(store, rank: int, world_size: int, timeout: timedelta):
    from . import _C
    # The first group of a process is the world group and gets the full staging arena (MCCL_ARENA_MB,
    # 512 MB).  Groups made later with new_group() are sub-groups (tensor / pipeline / data-parallel
    # dimensions): several of them coexist on a GPU, so each gets MCCL_SUBGROUP_ARENA_MB (128 MB) and
    # larger messages are staged in pieces.
    arena_mb = 0
    try:
        is_sub = dist.distributed_c10d._world.default_pg is not None
    except Exception:  # private attribute moved: treat every group as a world group
        is_sub = False
    if is_sub:
        arena_mb = int(os.environ.get("MCCL_SUBGROUP_ARENA_MB", "128"))
    pg = _C._create_process_group_mccl(store, rank, world_size, timeout, arena_mb)
    pg.set_p2p_factory(_nccl_p2p_factory(store, rank, world_size, timeout))
    return pg


def register() -> None:
    """Idempotent; called by ``import mccl_b200`` (and ``import mccl``)."""
    global _REGISTERED
    if _REGISTERED:
        return
    try:
        dist.Backend.register_backend("mccl", _create, extended_api=False, devices=["cpu", "cuda"])
    except TypeError:  # older signature without extended_api / devices
        dist.Backend.register_backend("mccl", _create)
    _REGISTERED = True


def get_backend(group=None):
    """The native ProcessGroupMCCL object behind a torch process group (or None)."""
    group = group or dist.group.WORLD
    for dev in ("cuda", "cpu"):
        try:
            be = group._get_backend(torch.device(dev))
        except Exception:
            continue
        if be is not None and be.__class__.__name__ == "ProcessGroupMCCL":
            return be
    return None
