"""Tensor-level distributed runtime: sharded tensors, model wrappers, split helpers.

Same public names as the reference's ``mccl.distributed`` (mccl/distributed/__init__.py:5-13).
"""
from .sharding import DistributedModel, ModelParallelPlan  # noqa: F401
from .tensor import DistributedTensor, ShardingSpec  # noqa: F401
from .runtime import DistributedRuntime  # noqa: F401
