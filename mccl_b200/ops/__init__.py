"""Model operators backed by this package's sm_100a kernels.

Each function is differentiable (a ``torch.autograd.Function`` around the
native forward and backward kernels) and has a plain-PyTorch twin in
``mccl_b200.ops.reference`` that the numerics tests compare against.
"""
from .functional import (adamw_step, causal_attention, embedding, launch_count, linear, linear_cross_entropy, mlp_gelu, native_ops_available, norm,
                         norm_residual)  # noqa: F401
