"""Split helpers and a model wrapper that keeps replicas in sync.

Parity: ``ModelParallelPlan.{data_parallel_split, tensor_parallel_split,
pipeline_parallel_split}`` and ``DistributedModel.{register_parameters,
deregister_parameters, sync_gradients, parameters, train, eval, __call__}``
(mccl/distributed/sharding.py:24-228).  ``sync_gradients`` averages all
gradients with one fused collective over a flat buffer.
"""
from __future__ import annotations

from typing import List, Sequence

import torch
import torch.distributed as dist

from .tensor import DistributedTensor, ShardingSpec


class ModelParallelPlan:
    @staticmethod
    def data_parallel_split(batch: torch.Tensor, world: int, rank: int) -> torch.Tensor:
        """This rank's slice of a batch along dim 0 (the last rank also takes the remainder)."""
        per = batch.shape[0] // world
        start = rank * per
        end = batch.shape[0] if rank == world - 1 else start + per
        return batch[start:end]

    @staticmethod
    def tensor_parallel_split(weight: torch.Tensor, dim: int, world: int) -> List[torch.Tensor]:
        return list(torch.chunk(weight, world, dim=dim))

    @staticmethod
    def pipeline_parallel_split(layers: Sequence, stages: int) -> List[list]:
        """Contiguous blocks of layers; the last stage also takes the remainder."""
        per = len(layers) // stages
        out = []
        for s in range(stages):
            start = s * per
            end = len(layers) if s == stages - 1 else start + per
            out.append(list(layers[start:end]))
        return out


class DistributedModel:
    def __init__(self, model: torch.nn.Module, group=None):
        self.model, self.group = model, group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self._flat: DistributedTensor | None = None
        self._params: List[torch.nn.Parameter] = []

    def register_parameters(self) -> int:
        """Allocates the flat gradient buffer (symmetric heap on CUDA / backend "mccl") and
        broadcasts rank 0's parameters.  Returns the number of gradient elements."""
        self._params = [p for p in self.model.parameters() if p.requires_grad]
        total = sum(p.numel() for p in self._params)
        if not self._params:
            return 0
        ref = self._params[0]
        self._flat = DistributedTensor(torch.zeros(total, dtype=torch.float32, device=ref.device), ShardingSpec.DATA_PARALLEL,
                                       self.group)
        if self.world > 1:
            for p in self._params:
                dist.broadcast(p.data, src=0, group=self.group)
        return total

    def deregister_parameters(self) -> None:
        self._flat = None
        self._params = []

    def sync_gradients(self) -> None:
        """Averages every parameter's gradient over the group."""
        if self.world == 1 or not self._params:
            return
        if self._flat is None:
            self.register_parameters()
        flat = self._flat.local
        off = 0
        for p in self._params:
            n = p.numel()
            if p.grad is None:
                flat[off:off + n].zero_()
            else:
                flat[off:off + n].copy_(p.grad.reshape(-1))
            off += n
        self._flat.all_reduce("avg")
        off = 0
        for p in self._params:
            n = p.numel()
            if p.grad is not None:
                p.grad.copy_(flat[off:off + n].view_as(p.grad))
            off += n

    def parameters(self):
        return self.model.parameters()

    def train(self, mode: bool = True):
        self.model.train(mode)
        return self

    def eval(self):
        return self.train(False)

    def __call__(self, *args, **kwargs):
        return self.model(*args, **kwargs)
