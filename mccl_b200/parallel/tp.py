"""Hand-wired tensor parallelism with sequence-parallel activations.

The reference offers ``tensor_parallel_split`` and notes that hand-wired
column / row parallel layers work over its collectives while the DeviceMesh API
does not (mccl/distributed/sharding.py:54-69, README.md:76).  These modules are
that hand wiring for one NVSwitch box:

* activations between layers are sharded by token rows (sequence parallel);
* ``ColumnParallelLinear`` computes ``all_gather(x) @ W_shard^T`` and
  ``RowParallelLinear`` computes ``reduce_scatter(x @ W_shard^T)``, each as ONE
  kernel that overlaps the NVLink transfer with the tcgen05 tiles
  (``_C.TpGemm``); the backward passes reuse the same two kernels (the input
  gradient of a column-parallel layer is a GEMM→reduce-scatter, that of a
  row-parallel layer an all-gather→GEMM);
* with ``fused=False`` the same modules run on ``torch.distributed`` collectives
  plus library matmuls, which is the comparison baseline and the CPU path.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from .. import _C


class TensorParallelContext:
    """Per-group state of the fused tensor-parallel kernels."""

    def __init__(self, group=None, device: Optional[torch.device] = None, max_rows_local: int = 2048, max_features: int = 8192,
                 fused: bool = True):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.device = device
        self.fused = bool(fused and self.world > 1 and device is not None and device.type == "cuda")
        self.native = self.fused   # fused arm: this package's kernels everywhere; otherwise stock PyTorch operators
        self.tp = None
        self.comm = None
        self._act = None
        if self.fused:
            import mccl_b200
            be = mccl_b200.get_backend(group)
            if be is None:
                raise RuntimeError("fused tensor parallelism needs a process group created with backend='mccl'")
            self.comm = be.device_comm(device.index)
            self.tp = _C.TpGemm(self.comm, max_rows_local * max_features)
            # symmetric staging for the shard a fused all-gather reads from the peers
            self._act_bytes = max_rows_local * max_features * 2
            self._act = self.comm.symm_alloc(self._act_bytes)

    def stage(self, x: torch.Tensor):
        """Copies a [rows, features] bf16 shard into the symmetric staging buffer (peers read it from there)."""
        n = x.numel() * 2
        if n > self._act_bytes:
            raise ValueError(f"shard of {n} bytes exceeds the symmetric staging buffer ({self._act_bytes})")
        view = self._act.tensor(self.rank, 0, list(x.shape), torch.bfloat16, self.device.index)
        view.copy_(x)
        return self._act

    def check(self) -> None:
        if self.tp is not None:
            self.tp.check_status()


def _w16(weight: torch.Tensor) -> torch.Tensor:
    w = getattr(weight, "_bf16", None)
    if w is not None:
        return w
    return weight if weight.dtype == torch.bfloat16 else weight.detach().to(torch.bfloat16)


def _all_gather_rows(x: torch.Tensor, ctx: TensorParallelContext) -> torch.Tensor:
    out = torch.empty(ctx.world * x.shape[0], x.shape[1], dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(out, x.contiguous(), group=ctx.group)
    return out


def _reduce_scatter_rows(y: torch.Tensor, ctx: TensorParallelContext) -> torch.Tensor:
    out = torch.empty(y.shape[0] // ctx.world, y.shape[1], dtype=y.dtype, device=y.device)
    dist.reduce_scatter_tensor(out, y.contiguous(), group=ctx.group)
    return out


def _wgrad(dy: torch.Tensor, x: torch.Tensor, native: bool) -> torch.Tensor:
    """dW[N, K] = dy[M, N]^T @ x[M, K]; fp32 from this package's GEMM, else a library matmul in the input dtype."""
    M, N, K = dy.shape[0], dy.shape[1], x.shape[1]
    if native and dy.is_cuda and M % 64 == 0 and N % 8 == 0 and K % 8 == 0:
        return _C.gemm_bf16(dy.contiguous(), x.contiguous(), None, "none", True, None, False, True, True)[0]
    return dy.t() @ x


class _ColumnParallelFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, ctxp: TensorParallelContext):
        w16 = _w16(weight)
        rows_local = x.shape[0]
        if ctxp.fused and rows_local % 128 == 0 and x.shape[1] % 64 == 0 and w16.shape[0] % 8 == 0:
            sym = ctxp.stage(x)
            y, gathered, _ = ctxp.tp.ag_gemm(sym, 0, rows_local, w16, False)
            ctx.fused_path = True
        else:
            gathered = _all_gather_rows(x, ctxp) if ctxp.world > 1 else x
            y = F.linear(gathered, w16)
            ctx.fused_path = False
        ctx.save_for_backward(gathered, w16)
        ctx.ctxp = ctxp
        return y

    @staticmethod
    def backward(ctx, dy):
        gathered, w16 = ctx.saved_tensors
        ctxp = ctx.ctxp
        dy = dy.contiguous()
        # dx_shard = reduce_scatter(dy @ W): W is stored [contraction = N_local, K]
        if ctx.fused_path and dy.shape[1] % 64 == 0 and w16.shape[1] % 8 == 0:
            dx = ctxp.tp.gemm_rs(dy, w16, True)
        else:
            full = dy @ w16
            dx = _reduce_scatter_rows(full, ctxp) if ctxp.world > 1 else full
        dw = _wgrad(dy, gathered, ctx.fused_path)
        return dx, dw, None


class _RowParallelFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, ctxp: TensorParallelContext):
        w16 = _w16(weight)
        rows_local = x.shape[0] // max(ctxp.world, 1)
        if ctxp.fused and rows_local % 128 == 0 and x.shape[1] % 64 == 0 and w16.shape[0] % 8 == 0:
            y = ctxp.tp.gemm_rs(x.contiguous(), w16, False)
            ctx.fused_path = True
        else:
            full = F.linear(x, w16)
            y = _reduce_scatter_rows(full, ctxp) if ctxp.world > 1 else full
            ctx.fused_path = False
        ctx.save_for_backward(x, w16)
        ctx.ctxp = ctxp
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w16 = ctx.saved_tensors
        ctxp = ctx.ctxp
        dy = dy.contiguous()
        rows_local = dy.shape[0]
        # dx = all_gather(dy) @ W: W is stored [contraction = N, K_local]
        if ctx.fused_path and dy.shape[1] % 64 == 0 and w16.shape[1] % 8 == 0:
            sym = ctxp.stage(dy)
            dx, dy_full, _ = ctxp.tp.ag_gemm(sym, 0, rows_local, w16, True)
        else:
            dy_full = _all_gather_rows(dy, ctxp) if ctxp.world > 1 else dy
            dx = dy_full @ w16
        dw = _wgrad(dy_full, x, ctx.fused_path)
        return dx, dw, None


class ColumnParallelLinear(nn.Module):
    """Weight [out_total / world, in]; input rows sharded over the ranks, output rows complete."""

    def __init__(self, d_in: int, d_out_total: int, ctx: TensorParallelContext, std: float = 0.02):
        super().__init__()
        assert d_out_total % ctx.world == 0
        self.ctx = ctx
        self.weight = nn.Parameter(torch.empty(d_out_total // ctx.world, d_in).normal_(0.0, std))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return _ColumnParallelFn.apply(x, self.weight, self.ctx)


class RowParallelLinear(nn.Module):
    """Weight [out, in_total / world]; input rows complete (features sharded), output rows sharded."""

    def __init__(self, d_in_total: int, d_out: int, ctx: TensorParallelContext, std: float = 0.02):
        super().__init__()
        assert d_in_total % ctx.world == 0
        self.ctx = ctx
        self.weight = nn.Parameter(torch.empty(d_out, d_in_total // ctx.world).normal_(0.0, std))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return _RowParallelFn.apply(x, self.weight, self.ctx)


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-5, native: bool = False):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps, self.native = eps, native

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.native and x.is_cuda:
            from .. import ops
            return ops.norm(x, self.weight, None, self.eps)
        return F.rms_norm(x.float(), (x.shape[-1],), self.weight, self.eps).to(x.dtype)


class ParallelAttention(nn.Module):
    """Heads split over the ranks; QKV column-parallel, output projection row-parallel."""

    def __init__(self, d_model: int, n_heads: int, ctx: TensorParallelContext, batch: int, seq: int, n_layers: int = 24):
        super().__init__()
        assert n_heads % ctx.world == 0
        self.ctx, self.batch, self.seq = ctx, batch, seq
        self.heads_local, self.head_dim = n_heads // ctx.world, d_model // n_heads
        self.qkv = ColumnParallelLinear(d_model, 3 * d_model, ctx)
        self.proj = RowParallelLinear(d_model, d_model, ctx, std=0.02 / (2 * n_layers) ** 0.5)

    def forward(self, x: torch.Tensor, rope) -> torch.Tensor:
        from ..models.decoder import apply_rope
        B, S, H, D = self.batch, self.seq, self.heads_local, self.head_dim
        qkv = self.qkv(x).view(B, S, 3, H, D)
        q, k, v = (t.transpose(1, 2) for t in qkv.unbind(2))
        if rope is not None:
            q, k = apply_rope(q, *rope), apply_rope(k, *rope)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        return self.proj(a.transpose(1, 2).reshape(B * S, H * D))


class ParallelMLP(nn.Module):
    """SwiGLU feed-forward: gate and up projections column-parallel, down projection row-parallel."""

    def __init__(self, d_model: int, d_ff: int, ctx: TensorParallelContext, n_layers: int = 24):
        super().__init__()
        # gate and up share their input: one all-gather and one GEMM produce [gate_local | up_local]
        self.gate_up = ColumnParallelLinear(d_model, 2 * d_ff, ctx)
        self.down = RowParallelLinear(d_ff, d_model, ctx, std=0.02 / (2 * n_layers) ** 0.5)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        gate, up = self.gate_up(x).chunk(2, dim=-1)
        return self.down(F.silu(gate) * up)


class TPDecoderLayer(nn.Module):
    def __init__(self, d_model, n_heads, d_ff, ctx, batch, seq, n_layers):
        super().__init__()
        self.n1, self.n2 = RMSNorm(d_model, native=ctx.native), RMSNorm(d_model, native=ctx.native)
        self.attn = ParallelAttention(d_model, n_heads, ctx, batch, seq, n_layers)
        self.mlp = ParallelMLP(d_model, d_ff, ctx, n_layers)

    def forward(self, x, rope):
        x = x + self.attn(self.n1(x), rope)
        return x + self.mlp(self.n2(x))


class TPDecoder(nn.Module):
    """Decoder whose layers are tensor parallel over `ctx`; token rows are sharded between layers.

    The embedding, final norm and LM head are replicated and applied to this rank's rows only, so
    their gradients (like those of the RMSNorm weights) have to be summed over the group:
    ``sync_replicated_grads()``.
    """

    def __init__(self, ctx: TensorParallelContext, vocab=32000, d_model=2048, n_layers=24, n_heads=16, d_ff=8192, batch=8,
                 seq=2048, layers_range=None):
        super().__init__()
        self.ctx, self.batch, self.seq, self.d_model, self.n_heads = ctx, batch, seq, d_model, n_heads
        lo, hi = layers_range or (0, n_layers)
        self.first, self.last = lo == 0, hi == n_layers
        self.tok = nn.Embedding(vocab, d_model) if self.first else None
        if self.tok is not None:
            nn.init.normal_(self.tok.weight, 0.0, 0.02)
        self.layers = nn.ModuleList(TPDecoderLayer(d_model, n_heads, d_ff, ctx, batch, seq, n_layers) for _ in range(lo, hi))
        self.norm = RMSNorm(d_model, native=ctx.native) if self.last else None
        self.head = nn.Parameter(torch.empty(vocab, d_model).normal_(0.0, 0.02)) if self.last else None

    def rows(self):
        total = self.batch * self.seq
        per = total // self.ctx.world
        return self.ctx.rank * per, per

    def forward(self, tokens: Optional[torch.Tensor], targets: Optional[torch.Tensor] = None, hidden: Optional[torch.Tensor] = None):
        from ..models.decoder import _rope_tables
        start, per = self.rows()
        dev = tokens.device if tokens is not None else hidden.device
        rope = _rope_tables(self.seq, self.d_model // self.n_heads, dev)
        if self.first:
            x = self.tok(tokens.reshape(-1)[start:start + per]).to(torch.bfloat16)
        else:
            x = hidden
        for layer in self.layers:
            x = layer(x, rope)
        if not self.last:
            return x
        x = self.norm(x)
        logits = F.linear(x, self.head.to(x.dtype))
        if targets is None:
            return logits
        # mean over ALL tokens of the batch: local sum / total tokens, summed over the group by the caller
        return F.cross_entropy(logits.float(), targets.reshape(-1)[start:start + per], reduction="sum") / (self.batch * self.seq)

    def replicated_parameters(self):
        for name, p in self.named_parameters():
            if ".qkv." in name or ".proj." in name or ".gate_up." in name or ".down." in name:
                continue
            yield p

    def sync_replicated_grads(self) -> None:
        if self.ctx.world == 1:
            return
        grads = [p.grad for p in self.replicated_parameters() if p.grad is not None]
        if not grads:
            return
        flat = torch.cat([g.reshape(-1).float() for g in grads])
        dist.all_reduce(flat, group=self.ctx.group)
        off = 0
        for g in grads:
            g.copy_(flat[off:off + g.numel()].view_as(g))
            off += g.numel()
