"""Differentiable operators.  CUDA tensors run the native kernels; the
fallbacks below only serve CPU tensors (tests without a GPU)."""
from __future__ import annotations

import os

import torch
import torch.nn.functional as F

from .. import _C

_HAS = {name: hasattr(_C, name) for name in ("gemm_bf16", "norm_fwd", "norm_bwd", "adamw_flat", "ce_fwd_bwd", "embed_fwd",
                                             "attn_fwd")}
_launches = 0


def native_ops_available() -> dict:
    return dict(_HAS)


def launch_count() -> int:
    """Number of this package's model-operator kernels launched so far in this process."""
    native = _C.op_launch_count() if hasattr(_C, "op_launch_count") else 0
    return native + _launches


def norm(x: torch.Tensor, weight: torch.Tensor, bias, eps: float) -> torch.Tensor:
    if x.is_cuda and _HAS["norm_fwd"]:
        from .native import NormFn
        return NormFn.apply(x, weight, bias, eps)
    v = x.float()
    if bias is not None:
        return F.layer_norm(v, v.shape[-1:], weight, bias, eps).to(x.dtype)
    return (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps) * weight).to(x.dtype)


def norm_residual(x: torch.Tensor, weight: torch.Tensor, bias, eps: float):
    """``(norm(x), x)``: use the second value as the residual input of the branch so that the two gradients
    of x are added inside the norm-backward kernel."""
    if x.is_cuda and _HAS["norm_fwd"]:
        from .native import NormResidualFn
        return NormResidualFn.apply(x, weight, bias, eps)
    return norm(x, weight, bias, eps), x


def linear(x: torch.Tensor, weight: torch.Tensor, bias=None, act: str = "none", residual=None) -> torch.Tensor:
    """act(x @ W^T + b) + residual, in one kernel on CUDA."""
    if x.is_cuda and _HAS["gemm_bf16"]:
        from .native import LinearFn
        return LinearFn.apply(x, weight, bias, act, residual)
    y = F.linear(x, weight.to(x.dtype), None if bias is None else bias.to(x.dtype))
    y = F.gelu(y) if act == "gelu" else y
    return y if residual is None else y + residual


def native_attention_supported(seq: int, head_dim: int) -> bool:
    """Shapes the attention kernels cover: head dimension 64, sequences of 128 or 256 (training needs backward)."""
    return bool(_HAS.get("attn_fwd")) and head_dim == 64 and seq in (128, 256) and os.environ.get("MCCL_NATIVE_ATTN", "1") != "0"


def causal_attention(qkv: torch.Tensor, n_heads: int) -> torch.Tensor:
    """Causal self-attention.  qkv: [B, S, 3 * n_heads * head_dim] (or already [B, S, 3, H, Dh]), the output of a
    fused QKV projection; returns [B, S, n_heads * head_dim].  On CUDA with head dimension 64 and S in {128, 256}
    this is one kernel each way; otherwise PyTorch's scaled_dot_product_attention on views of the same tensor."""
    B, S = qkv.shape[0], qkv.shape[1]
    hd = qkv.numel() // (B * S * 3 * n_heads)
    q5 = qkv.view(B, S, 3, n_heads, hd)
    if qkv.is_cuda and qkv.dtype == torch.bfloat16 and native_attention_supported(S, hd):
        from .native import CausalAttentionFn
        return CausalAttentionFn.apply(q5, 1.0 / (hd ** 0.5))
    q, k, v = (t.transpose(1, 2) for t in q5.unbind(2))
    a = F.scaled_dot_product_attention(q, k, v, is_causal=True)
    return a.transpose(1, 2).reshape(B, S, n_heads * hd)


def mlp_gelu(x: torch.Tensor, w1: torch.Tensor, b1, w2: torch.Tensor, b2, residual=None) -> torch.Tensor:
    """gelu(x @ w1^T + b1) @ w2^T + b2 (+ residual).  On CUDA the whole block is one autograd node whose backward
    fuses the GELU derivative into the input-gradient GEMM of the second layer."""
    d_in, d_ff, d_out = w1.shape[1], w1.shape[0], w2.shape[0]
    if (x.is_cuda and _HAS["gemm_bf16"] and d_in % 64 == 0 and d_ff % 64 == 0 and d_out % 8 == 0
            and os.environ.get("MCCL_FUSE_MLP", "1") != "0"):
        from .native import MlpGeluFn
        return MlpGeluFn.apply(x, w1, b1, w2, b2, residual)
    h = linear(x, w1, b1, "gelu")
    return linear(h, w2, b2, "none", residual)


def embedding(ids: torch.Tensor, tok: torch.Tensor, pos=None) -> torch.Tensor:
    """bf16(tok[ids] + pos[:seq]) for ids [..., seq]; tok / pos are fp32 tables."""
    seq = ids.shape[-1]
    if (ids.is_cuda and _HAS.get("embed_fwd") and tok.dtype == torch.float32 and tok.shape[1] % 8 == 0
            and os.environ.get("MCCL_NATIVE_EMBED", "1") != "0"):
        from .native import EmbeddingFn
        return EmbeddingFn.apply(ids, tok, pos, seq)
    x = F.embedding(ids, tok)
    if pos is not None:
        x = x + pos[:seq]
    return x.to(torch.bfloat16)


def linear_cross_entropy(h: torch.Tensor, weight: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    """Mean cross entropy of (h @ weight.T) against targets; h [T, D] bf16, weight [V, D]."""
    if h.is_cuda and _HAS["ce_fwd_bwd"] and _HAS["gemm_bf16"]:
        from .native import LinearCrossEntropyFn
        return LinearCrossEntropyFn.apply(h, weight, targets)
    logits = F.linear(h, weight.to(h.dtype))
    return F.cross_entropy(logits.float(), targets)


def adamw_step(p, g, m, v, lr, beta1, beta2, eps, wd, step, p_bf16=None, grad_scale=1.0, zero_grad=False, ctas_per_sm=8):
    """In-place fused AdamW over flat fp32 tensors (optionally refreshing a bf16 copy of p and clearing g)."""
    if p.is_cuda and _HAS["adamw_flat"]:
        _C.adamw_flat(p, g, m, v, p_bf16, lr, beta1, beta2, eps, wd, step, grad_scale, zero_grad, ctas_per_sm)
        return
    g_buf = g
    g = g * grad_scale if grad_scale != 1.0 else g
    m.mul_(beta1).add_(g, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    bc1, bc2 = 1 - beta1 ** step, 1 - beta2 ** step
    p.mul_(1 - lr * wd).addcdiv_(m / bc1, (v / bc2).sqrt_().add_(eps), value=-lr)
    if p_bf16 is not None:
        p_bf16.copy_(p)
    if zero_grad:
        g_buf.zero_()
