"""Data-parallel and pipeline dispatch of registered kernels over the ranks of a group.

Parity: the reference's DistributedMetalRuntime loads a shader library on every
agent, splits a 1-D grid over the nodes (remainder to the last), surrounds the
launch with coherence barriers, and runs pipelines with warm-up / steady /
cool-down phases and double buffering (csrc/runtime/DistributedMetalRuntime.cpp:120-372,
csrc/runtime/ShaderDispatch.hpp:88-122).  Here every rank is its own "agent"
(one process per GPU, SPMD): ``dispatch_data_parallel`` runs the rank's slice of
a registered kernel between a stream-ordered acquire / release pair, and
``dispatch_pipeline`` moves activations between stages with send / recv.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Sequence

import torch
import torch.distributed as dist

from .. import _C


class DistributedRuntime:
    def __init__(self, group=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self._kernels: Dict[str, Callable] = {}
        self._coh = None

    # ------------------------------------------------------------- registry --
    def load_library(self, kernels: Dict[str, Callable]) -> List[str]:
        """Registers kernels by name.  A kernel is ``fn(offset, count, *bindings)`` operating on
        elements [offset, offset + count) of its bindings."""
        self._kernels.update(kernels)
        return sorted(self._kernels)

    def _coherence(self, device: torch.device):
        if self._coh is None and self.world > 1 and device.type == "cuda":
            import mccl_b200
            be = mccl_b200.get_backend(self.group)
            if be is not None:
                self._coh = _C.GpuCoherence(be.device_comm(device.index))
        return self._coh

    # ----------------------------------------------------------- dispatchers --
    def dispatch_data_parallel(self, kernel: str, total: int, *bindings, device: Optional[torch.device] = None):
        """Runs this rank's slice of `kernel` over a grid of `total` elements; returns (offset, count)."""
        if kernel not in self._kernels:
            raise KeyError(f"kernel '{kernel}' is not loaded")
        _, offset, count = _C.data_parallel_split(total, self.world)[self.rank]
        coh = self._coherence(device) if device is not None else None
        if coh is not None:
            coh.gpu_acquire(coh.epoch, 10000, device.index)   # peers' earlier writes are visible
        if count:
            self._kernels[kernel](offset, count, *bindings)
        if coh is not None:
            coh.gpu_release(device.index)                     # publish this slice's writes
        return offset, count

    def sync_all(self, device: Optional[torch.device] = None) -> None:
        if device is not None and device.type == "cuda":
            torch.cuda.synchronize(device)
        if self.world > 1:
            dist.barrier(group=self.group)

    def transfer_tensor(self, t: torch.Tensor, src: int, dst: int) -> Optional[torch.Tensor]:
        """Point-to-point move of a tensor between two ranks (the backend's send / recv kernels for CUDA tensors)."""
        if self.rank == src:
            dist.send(t, dst, group=self.group)
            return None
        if self.rank == dst:
            dist.recv(t, src, group=self.group)
            return t
        return None

    def dispatch_pipeline(self, stage_fn: Callable[[torch.Tensor], torch.Tensor], micro_batches: Sequence[torch.Tensor],
                          act_shape, dtype, device) -> List[torch.Tensor]:
        """Runs `stage_fn` as stage `rank` of a `world`-stage pipeline (fill, steady, drain).  Stage 0
        consumes `micro_batches`; the last stage returns its outputs.  Activations arrive in two
        alternating buffers: the receive of micro-batch i + 1 is posted before micro-batch i is
        computed, and sends are asynchronous, so transfers overlap the neighbouring compute."""
        n = len(micro_batches)
        outs: List[torch.Tensor] = []
        if n == 0:
            return outs
        bufs = [torch.empty(act_shape, dtype=dtype, device=device) for _ in range(2)]
        pending_recv = None
        if self.rank > 0:
            pending_recv = dist.irecv(bufs[0], self.rank - 1, group=self.group)
        sends = []
        for mb in range(n):
            if self.rank == 0:
                x = micro_batches[mb]
            else:
                pending_recv.wait()
                x = bufs[mb & 1]
                if mb + 1 < n:   # the other buffer was consumed by micro-batch mb - 1, whose compute was enqueued before
                    pending_recv = dist.irecv(bufs[(mb + 1) & 1], self.rank - 1, group=self.group)
            y = stage_fn(x)
            if self.rank < self.world - 1:
                y = y.contiguous()
                sends.append((dist.isend(y, self.rank + 1, group=self.group), y))
            else:
                outs.append(y)
        for work, _ in sends:
            work.wait()
        return outs
