"""A tensor shard that knows how it relates to its peers' shards.

Parity: the reference's ``DistributedTensor`` registers its shard with the
distributed-memory layer and offers ``sync_gradient``, ``all_reduce(op)``,
``all_gather`` and ``reduce_scatter`` built from one-sided put / get
(mccl/distributed/tensor.py:30-345).  Its ``sync_gradient`` writes every
peer's scaled gradient to the same offset, so the last writer wins; here it
produces the true mean.  On a CUDA group created with backend "mccl" the shard
lives in the group's symmetric heap, so reductions run in place over NVLink
(in-switch where available) without staging copies; on any other group the
same methods fall back to ``torch.distributed`` collectives.
"""
from __future__ import annotations

import enum
from typing import Optional

import torch
import torch.distributed as dist


class ShardingSpec(enum.Enum):
    REPLICATED = "replicated"
    DATA_PARALLEL = "data_parallel"
    TENSOR_PARALLEL = "tensor_parallel"
    PIPELINE_PARALLEL = "pipeline_parallel"


_OPS = {"sum": dist.ReduceOp.SUM, "avg": dist.ReduceOp.AVG, "min": dist.ReduceOp.MIN, "max": dist.ReduceOp.MAX}


class DistributedTensor:
    def __init__(self, tensor: torch.Tensor, spec: ShardingSpec = ShardingSpec.REPLICATED, group=None, shard_dim: int = 0):
        self.spec, self.group, self.shard_dim = spec, group, shard_dim
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self._symm = None
        self._comm = None
        self.local = tensor
        if tensor.is_cuda and self.world > 1:
            import mccl_b200
            be = mccl_b200.get_backend(group)
            if be is not None and tensor.dtype in (torch.float32, torch.float16, torch.bfloat16):
                comm = be.device_comm(tensor.device.index)
                n = tensor.numel()
                per = ((n + self.world - 1) // self.world + 15) // 16 * 16
                self._symm = comm.symm_alloc(per * self.world * tensor.element_size())
                self._comm = comm
                view = self._symm.tensor(self.rank, 0, [per * self.world], tensor.dtype, tensor.device.index)
                view.zero_()
                view[:n].copy_(tensor.reshape(-1))
                self.local = view[:n].view(tensor.shape)

    # ------------------------------------------------------------------ info --
    @property
    def in_symmetric_heap(self) -> bool:
        return self._symm is not None

    def peer_view(self, rank: int) -> torch.Tensor:
        """This process's mapping of a peer's shard (symmetric heap only): every access is a load / store over NVLink.

        The returned tensor aliases ANOTHER GPU's memory.  Copy it with a plain elementwise copy
        (``.clone()``, ``dst.copy_(view)``, ``view.copy_(src)``) or hand it to this package's own kernels;
        never pass it to a library kernel (``matmul``, attention, convolutions, ...): such kernels may read
        their operands with cluster-multicast bulk loads, which must not touch a peer's memory."""
        if self._symm is None:
            raise RuntimeError("peer views need a CUDA shard on a backend='mccl' group")
        n = self.local.numel()
        return self._symm.tensor(rank, 0, [n], self.local.dtype, self.local.device.index).view(self.local.shape)

    # ------------------------------------------------------------- reductions --
    def all_reduce(self, op: str = "sum") -> torch.Tensor:
        if self.world == 1:
            return self.local
        if self._symm is not None and op in ("sum", "avg"):
            self._comm.allreduce_symm(self._symm, 0, self.local.numel(), self.local.dtype, op)
        else:
            dist.all_reduce(self.local, op=_OPS[op], group=self.group)
        return self.local

    def sync_gradient(self, grad: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Mean of the gradient over the group (in place)."""
        if grad is not None:
            self.local.copy_(grad)
        return self.all_reduce("avg")

    def all_gather(self) -> torch.Tensor:
        """Concatenation of every rank's shard along ``shard_dim``."""
        if self.world == 1:
            return self.local
        flat = torch.empty(self.world * self.local.numel(), dtype=self.local.dtype, device=self.local.device)
        dist.all_gather_into_tensor(flat, self.local.contiguous().reshape(-1), group=self.group)
        parts = [p.view(self.local.shape) for p in flat.chunk(self.world)]
        return torch.cat(parts, dim=self.shard_dim)

    def reduce_scatter(self, op: str = "sum") -> torch.Tensor:
        """Reduces the full tensor over the group and returns this rank's 1/world slice (flattened)."""
        if self.world == 1:
            return self.local.reshape(-1)
        n = self.local.numel()
        if n % self.world != 0:
            raise ValueError(f"reduce_scatter needs numel ({n}) divisible by the world size ({self.world})")
        out = torch.empty(n // self.world, dtype=self.local.dtype, device=self.local.device)
        dist.reduce_scatter_tensor(out, self.local.contiguous().reshape(-1), op=_OPS[op], group=self.group)
        return out
