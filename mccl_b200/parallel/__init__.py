"""Parallelism strategies: data parallel (engine + stock-DDP hook), tensor
parallel, pipeline parallel and sequence-parallel helpers."""
from .ddp import bf16_wire_hook, wire_dtype  # noqa: F401
from .trainer import DDPTrainer  # noqa: F401
