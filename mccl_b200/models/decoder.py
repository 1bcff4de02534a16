"""Decoder-only transformer family.

The reference's headline numbers are DDP samples/s on a 70M and a 110M decoder
(README.md:44-54; the training script itself is not in its tree, only a toy
model: examples/ddp_utils.py:41-147).  The architectures here are the ones the
baseline configurations spell out:

  70m   d_model 512,  16 layers,  8 heads, FFN 2048 GELU,   pre-LayerNorm, learned positions, vocab 32000, tied
  110m  d_model 768,  12 layers, 12 heads, FFN 3072 GELU,   pre-LayerNorm, learned positions, vocab 32000, tied
  1.3b  d_model 2048, 24 layers, 16 heads, FFN 8192 SwiGLU, RMSNorm, RoPE, vocab 32000

`Decoder` is a plain ``nn.Module`` (fp32 master parameters) whose forward runs
in bf16.  On a CUDA device its matmuls, normalisations, activation and loss go
through this package's sm_100a operators (``mccl_b200.ops``); with
``native=False`` or on CPU the same math runs on stock PyTorch operators, which
is also the numerics reference in the tests.
"""
from __future__ import annotations

import dataclasses
import os
import math
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclasses.dataclass
class DecoderConfig:
    vocab: int = 32000
    d_model: int = 512
    n_layers: int = 16
    n_heads: int = 8
    d_ff: int = 2048
    max_seq: int = 256
    act: str = "gelu"          # "gelu" | "swiglu"
    norm: str = "layernorm"    # "layernorm" | "rmsnorm"
    pos: str = "learned"       # "learned" | "rope"
    tied: bool = True
    eps: float = 1e-5

    @property
    def head_dim(self) -> int:
        return self.d_model // self.n_heads

    def param_count(self) -> int:
        ff = (3 if self.act == "swiglu" else 2) * self.d_model * self.d_ff
        attn = 4 * self.d_model * self.d_model
        per_layer = ff + attn
        emb = self.vocab * self.d_model * (1 if self.tied else 2)
        pos = self.max_seq * self.d_model if self.pos == "learned" else 0
        return self.n_layers * per_layer + emb + pos


PRESETS = {
    "70m": DecoderConfig(d_model=512, n_layers=16, n_heads=8, d_ff=2048, max_seq=256),
    "110m": DecoderConfig(d_model=768, n_layers=12, n_heads=12, d_ff=3072, max_seq=256),
    "1.3b": DecoderConfig(d_model=2048, n_layers=24, n_heads=16, d_ff=8192, max_seq=2048, act="swiglu",
                          norm="rmsnorm", pos="rope", tied=False),
    "tiny": DecoderConfig(vocab=512, d_model=128, n_layers=2, n_heads=4, d_ff=512, max_seq=64),
}


# Residual gradients are added inside the norm-backward kernel (one launch less per norm in backward:
# 6.63 -> 6.38 ms per step of the 70M decoder on one GPU); MCCL_FUSE_RESIDUAL_GRAD=0 switches it off.
_FUSE_RESIDUAL_GRAD = os.environ.get("MCCL_FUSE_RESIDUAL_GRAD", "1") != "0"


def _rope_tables(seq: int, dim: int, device, base: float = 10000.0):
    inv = 1.0 / (base ** (torch.arange(0, dim, 2, device=device, dtype=torch.float32) / dim))
    t = torch.arange(seq, device=device, dtype=torch.float32)
    f = torch.outer(t, inv)
    return f.cos(), f.sin()


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x: [B, H, S, D]; rotates pairs (even, odd)."""
    x1, x2 = x[..., 0::2], x[..., 1::2]
    c, s = cos[None, None, : x.shape[2]], sin[None, None, : x.shape[2]]
    out = torch.stack((x1 * c - x2 * s, x1 * s + x2 * c), dim=-1)
    return out.flatten(-2).to(x.dtype)


class Norm(nn.Module):
    def __init__(self, cfg: DecoderConfig):
        super().__init__()
        self.kind, self.eps = cfg.norm, cfg.eps
        self.weight = nn.Parameter(torch.ones(cfg.d_model))
        self.bias = nn.Parameter(torch.zeros(cfg.d_model)) if cfg.norm == "layernorm" else None

    def forward(self, x: torch.Tensor, native: bool) -> torch.Tensor:
        if native:
            from .. import ops
            return ops.norm(x, self.weight, self.bias, self.eps)
        if self.kind == "layernorm":
            return F.layer_norm(x.float(), x.shape[-1:], self.weight, self.bias, self.eps).to(x.dtype)
        v = x.float()
        return (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + self.eps) * self.weight).to(x.dtype)

    def with_residual(self, x: torch.Tensor, native: bool):
        """(norm(x), x as it should be fed to the residual connection).  The native path hands x through the
        norm operator so that backward adds the residual gradient in the norm-backward kernel
        (MCCL_FUSE_RESIDUAL_GRAD=0: x is returned untouched)."""
        if native and _FUSE_RESIDUAL_GRAD:
            from .. import ops
            return ops.norm_residual(x, self.weight, self.bias, self.eps)
        return self.forward(x, native), x


class Linear(nn.Module):
    """Weight [out, in] (fp32 master); computes in bf16."""

    def __init__(self, d_in: int, d_out: int, bias: bool, std: float):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(d_out, d_in).normal_(0.0, std))
        self.bias = nn.Parameter(torch.zeros(d_out)) if bias else None

    def forward(self, x: torch.Tensor, native: bool, act: str = "none", residual=None) -> torch.Tensor:
        if native:
            from .. import ops
            return ops.linear(x, self.weight, self.bias, act, residual)
        y = F.linear(x, self.weight.to(x.dtype), None if self.bias is None else self.bias.to(x.dtype))
        y = F.gelu(y) if act == "gelu" else y
        return y if residual is None else y + residual


class Block(nn.Module):
    def __init__(self, cfg: DecoderConfig):
        super().__init__()
        self.cfg = cfg
        d, std = cfg.d_model, 0.02
        out_std = 0.02 / math.sqrt(2 * cfg.n_layers)
        bias = cfg.norm == "layernorm"
        self.ln1 = Norm(cfg)
        self.qkv = Linear(d, 3 * d, bias, std)
        self.proj = Linear(d, d, bias, out_std)
        self.ln2 = Norm(cfg)
        if cfg.act == "swiglu":
            self.gate_up = Linear(d, 2 * cfg.d_ff, False, std)
        else:
            self.up = Linear(d, cfg.d_ff, bias, std)
        self.down = Linear(cfg.d_ff, d, bias, out_std)

    def forward(self, x: torch.Tensor, rope, native: bool) -> torch.Tensor:
        cfg = self.cfg
        B, S, D = x.shape
        h, x = self.ln1.with_residual(x, native)
        qkv = self.qkv(h, native)
        if native and rope is None:
            from .. import ops
            a = ops.causal_attention(qkv, cfg.n_heads)   # own kernels for head dimension 64, S in {128, 256}
        else:
            qkv = qkv.view(B, S, 3, cfg.n_heads, cfg.head_dim)
            # unbind, not three selects: its backward is one stack instead of three zero-filled tensors and two adds
            q, k, v = (t.transpose(1, 2) for t in qkv.unbind(2))
            if rope is not None:
                q, k = apply_rope(q, *rope), apply_rope(k, *rope)
            a = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(B, S, D)
        x = self.proj(a, native, residual=x)
        h, x = self.ln2.with_residual(x, native)
        if cfg.act == "swiglu":
            g, u = self.gate_up(h, native).chunk(2, dim=-1)
            h = F.silu(g) * u
        elif native:
            from .. import ops
            return ops.mlp_gelu(h, self.up.weight, self.up.bias, self.down.weight, self.down.bias, residual=x)
        else:
            h = self.up(h, native, act="gelu")
        return self.down(h, native, residual=x)


class Decoder(nn.Module):
    def __init__(self, cfg: DecoderConfig, native: Optional[bool] = None):
        super().__init__()
        self.cfg = cfg
        self.native = native
        self.tok = nn.Embedding(cfg.vocab, cfg.d_model)
        nn.init.normal_(self.tok.weight, 0.0, 0.02)
        self.pos = nn.Embedding(cfg.max_seq, cfg.d_model) if cfg.pos == "learned" else None
        if self.pos is not None:
            nn.init.normal_(self.pos.weight, 0.0, 0.02)
        self.blocks = nn.ModuleList(Block(cfg) for _ in range(cfg.n_layers))
        self.ln_f = Norm(cfg)
        self.head = None if cfg.tied else Linear(cfg.d_model, cfg.vocab, False, 0.02)
        if cfg.tied:
            # the embedding lookup contributes to this gradient through autograd as well
            self.tok.weight._shared_grad = True

    def _native(self, x: torch.Tensor) -> bool:
        if self.native is not None:
            return self.native and x.is_cuda
        return x.is_cuda

    def hidden(self, tokens: torch.Tensor) -> torch.Tensor:
        B, S = tokens.shape
        native = self._native(tokens)
        if native:
            from .. import ops
            x = ops.embedding(tokens, self.tok.weight, None if self.pos is None else self.pos.weight)
        else:
            x = self.tok(tokens)
            if self.pos is not None:
                x = x + self.pos.weight[:S]
            x = x.to(torch.bfloat16)
        rope = _rope_tables(S, self.cfg.head_dim, tokens.device) if self.cfg.pos == "rope" else None
        for blk in self.blocks:
            x = blk(x, rope, native)
        return self.ln_f(x, native)

    def head_weight(self) -> torch.Tensor:
        return self.tok.weight if self.head is None else self.head.weight

    def forward(self, tokens: torch.Tensor, targets: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Returns logits [B, S, V] (bf16), or the mean next-token loss when targets are given."""
        h = self.hidden(tokens)
        native = self._native(tokens)
        w = self.head_weight()
        if targets is None:
            return F.linear(h, w.to(h.dtype))
        if native:
            from .. import ops
            return ops.linear_cross_entropy(h.reshape(-1, h.shape[-1]), w, targets.reshape(-1))
        logits = F.linear(h, w.to(h.dtype))
        return F.cross_entropy(logits.float().view(-1, logits.shape[-1]), targets.reshape(-1))


def build_decoder(name: str, native: Optional[bool] = None, **overrides) -> Decoder:
    cfg = dataclasses.replace(PRESETS[name], **overrides)
    return Decoder(cfg, native=native)
