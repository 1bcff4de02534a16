"""Parallelism strategies: data parallel (engine + stock-DDP hook), tensor
parallel with sequence-parallel activations (fused all-gather→GEMM and
GEMM→reduce-scatter kernels) and pipeline parallel (1F1B over send / recv)."""
from .ddp import bf16_wire_hook, wire_dtype  # noqa: F401
from .pp import PipelineStage, split_layers  # noqa: F401
from .tp import (ColumnParallelLinear, ParallelAttention, ParallelMLP, RowParallelLinear, TensorParallelContext,  # noqa: F401
                 TPDecoder)
from .trainer import DDPTrainer  # noqa: F401
