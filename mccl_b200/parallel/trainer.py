"""Data-parallel training engine built on the device communicator.

The reference reaches its headline numbers with stock DistributedDataParallel
over its allreduce (README.md:44-54, tests/test_ddp_e2e.py); stock DDP works on
this backend too (see ``mccl_b200.parallel.ddp``).  This engine is the
B200-first form of the same job:

* all parameters live in one flat fp32 buffer and all gradients in one flat
  fp32 buffer allocated from the group's symmetric heap, ordered so that the
  gradients that finish first in backward sit in the first bucket;
* when the last gradient of a bucket has been accumulated, the bucket is
  all-reduced in place on a side stream while backward continues: in-switch
  (``multimem.ld_reduce``) when the fabric offers it, otherwise by direct peer
  loads, or staged through the arena with bf16 on the wire and fp32
  accumulation (``wire="bf16"``), with the 1/world scale fused in every case;
* AdamW is one fused kernel over the flat buffers;
* forward, backward, the bucket collectives and the optimizer are captured
  once into a CUDA graph and replayed, so a step costs one launch on the host.
"""
from __future__ import annotations

import math
import os
from typing import List, Optional

import torch
import torch.distributed as dist

from .. import _C, ops


class _Bucket:
    __slots__ = ("start", "numel", "pending", "total", "late")

    def __init__(self, start: int):
        self.start, self.numel, self.pending, self.total = start, 0, 0, 0
        # True once a gradient of this bucket has arrived through autograd's own accumulation: such a
        # bucket is reduced after backward() has returned (the engine has then joined the stream that
        # accumulated it with the caller's stream), not from inside the hook.
        self.late = False


class DDPTrainer:
    def __init__(self, model: torch.nn.Module, device: torch.device, lr: float = 3e-4, betas=(0.9, 0.999),
                 eps: float = 1e-8, weight_decay: float = 0.01, group=None, wire: str = "bf16",
                 bucket_mb: float = 25.0, overlap: bool = True, use_graph: bool = True, algo: str = "auto"):
        self.model, self.device = model, device
        self.lr, self.betas, self.eps, self.wd = lr, betas, eps, weight_decay
        self.wire, self.overlap, self.use_graph, self.algo = wire, overlap, use_graph, algo
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.comm = None
        self._late: List[_Bucket] = []
        if self.world > 1:
            import mccl_b200
            be = mccl_b200.get_backend(group)
            if be is None:
                raise RuntimeError("DDPTrainer needs a process group created with backend='mccl'")
            self.comm = be.device_comm(device.index)
        self._flatten(bucket_mb)
        self.step_t = torch.zeros((), device=device, dtype=torch.float32)
        self.m = torch.zeros_like(self.flat_p)
        self.v = torch.zeros_like(self.flat_p)
        self.comm_stream = torch.cuda.Stream(device=device, priority=-1) if self.world > 1 else None
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.static_tokens = None
        self.static_targets = None
        self.static_loss = None
        self.launches_per_step = 0
        if self.world > 1:
            self._sync_initial_params(group)

    # ------------------------------------------------------------ buffers --
    def _flatten(self, bucket_mb: float) -> None:
        params = [p for p in self.model.parameters() if p.requires_grad]
        # Backward produces gradients roughly in reverse registration order.
        order = list(reversed(params))
        align = 16 * max(self.world, 1)  # chunk boundaries of the collectives stay 16-element aligned
        bucket_cap = int(bucket_mb * (1 << 20) / 4)
        offsets, total = [], 0
        self.buckets: List[_Bucket] = [_Bucket(0)]
        for p in order:
            b = self.buckets[-1]
            if b.numel > 0 and b.numel + p.numel() > bucket_cap:
                total = (total + align - 1) // align * align
                b.numel = total - b.start
                self.buckets.append(_Bucket(total))
                b = self.buckets[-1]
            offsets.append(total)
            n = (p.numel() + 7) // 8 * 8  # every parameter starts 16-byte aligned in fp32 and in bf16
            total += n
            b.numel = total - b.start
            b.total += 1
        total = (total + align - 1) // align * align
        self.buckets[-1].numel = total - self.buckets[-1].start
        self.total = total
        self.flat_p = torch.zeros(total, device=self.device, dtype=torch.float32)
        if self.comm is not None and self.wire != "bf16":
            # the in-place symmetric allreduce reads the peers' gradient buffers directly
            self.symm = self.comm.symm_alloc(total * 4)
            self.flat_g = self.symm.tensor(self.rank, 0, [total], torch.float32, self.device.index)
        else:
            # the staged (bf16-wire) allreduce copies through the arena, so the gradients stay in ordinary
            # device memory: every weight-gradient GEMM and the optimizer touch this buffer, and plain
            # memory is faster for them than a peer-mapped, multicast-bound allocation
            self.symm = None
            self.flat_g = torch.zeros(total, device=self.device, dtype=torch.float32)
        self.flat_g.zero_()
        self._param_bucket = {}
        bi = 0
        for p, off in zip(order, offsets):
            while off >= self.buckets[bi].start + self.buckets[bi].numel:
                bi += 1
            view = self.flat_p[off:off + p.numel()].view_as(p)
            view.copy_(p.data.to(self.device))
            p.data = view
            p.grad = self.flat_g[off:off + p.numel()].view_as(p)
            self._param_bucket[p] = bi
            # native operators write gradients straight into the flat buffer ...
            p._grad_sink = p.grad
            if self.world > 1:
                # ... and say so; gradients that come back through autograd fire its hook instead
                p._grad_ready = (lambda q=p: self._on_grad_ready(q))
                p.register_post_accumulate_grad_hook(self._on_autograd_grad)
        # bf16 working copies of the parameters, refreshed by the optimizer kernel (the GEMMs
        # read them in either orientation, so no transposed copies are kept).
        self.flat_p16 = None
        if self.device.type == "cuda" and ops.native_ops_available().get("adamw_flat"):
            self.flat_p16 = _C.cast_bf16(self.flat_p)
            for p, off in zip(order, offsets):
                p._bf16 = self.flat_p16[off:off + p.numel()].view_as(p)

    def _sync_initial_params(self, group) -> None:
        dist.broadcast(self.flat_p, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
        if self.flat_p16 is not None:
            _C.cast_bf16(self.flat_p, self.flat_p16)
        torch.cuda.synchronize(self.device)

    # ------------------------------------------------------- communication --
    def _on_grad_ready(self, p: torch.Tensor) -> None:
        b = self.buckets[self._param_bucket[p]]
        b.pending += 1
        if b.pending == b.total:
            b.pending = 0
            if b.late:
                self._late.append(b)
            else:
                self._reduce_bucket(b)

    def _on_autograd_grad(self, p: torch.Tensor) -> None:
        self.buckets[self._param_bucket[p]].late = True
        self._on_grad_ready(p)

    def _reduce_bucket(self, b: _Bucket) -> None:
        main = torch.cuda.current_stream(self.device)
        stream = self.comm_stream if self.overlap else main
        if stream is not main:
            stream.wait_stream(main)
        with torch.cuda.stream(stream):
            if self.wire == "bf16":
                g = self.flat_g[b.start:b.start + b.numel]
                self.comm.allreduce([g], [g], op="avg", algo=("twoshot" if self.algo == "auto" else self.algo),
                                    wire="bf16")
            else:
                self.comm.allreduce_symm(self.symm, b.start * 4, b.numel, torch.float32, "avg")

    # ---------------------------------------------------------------- step --
    def _step_body(self, tokens: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        self.flat_g.zero_()
        loss = self.model(tokens, targets)
        loss.backward()
        for b in self._late:
            self._reduce_bucket(b)
        self._late.clear()
        if self.comm_stream is not None and self.overlap:
            torch.cuda.current_stream(self.device).wait_stream(self.comm_stream)
        self.step_t.add_(1.0)
        ops.adamw_step(self.flat_p, self.flat_g, self.m, self.v, self.lr, self.betas[0], self.betas[1], self.eps,
                       self.wd, self.step_t, p_bf16=self.flat_p16)
        return loss.detach()

    def _capture(self, tokens: torch.Tensor, targets: torch.Tensor) -> None:
        self.static_tokens = tokens.clone()
        self.static_targets = targets.clone()
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            for _ in range(2):  # warm up allocator, autotuners and lazy inits outside the capture
                self._step_body(self.static_tokens, self.static_targets)
        torch.cuda.current_stream(self.device).wait_stream(side)
        torch.cuda.synchronize(self.device)
        before = ops.launch_count() + (self.comm.launches if self.comm is not None else 0)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.static_loss = self._step_body(self.static_tokens, self.static_targets)
        self.launches_per_step = ops.launch_count() + (self.comm.launches if self.comm is not None else 0) - before

    def step(self, tokens: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        """One optimizer step on device-resident tokens; returns the loss (device tensor)."""
        if not self.use_graph:
            before = ops.launch_count() + (self.comm.launches if self.comm is not None else 0)
            loss = self._step_body(tokens, targets)
            self.launches_per_step = ops.launch_count() + (self.comm.launches if self.comm is not None else 0) - before
            return loss
        if self.graph is None:
            self._capture(tokens, targets)
        self.static_tokens.copy_(tokens, non_blocking=True)
        self.static_targets.copy_(targets, non_blocking=True)
        self.graph.replay()
        return self.static_loss

    def step_from_host(self, tokens_pinned: torch.Tensor, targets_pinned: torch.Tensor) -> float:
        """End-to-end step: host→device copy of the batch, the step, device→host read of the loss."""
        if self.use_graph and self.graph is None:
            self._capture(tokens_pinned.to(self.device), targets_pinned.to(self.device))
        if self.use_graph:
            self.static_tokens.copy_(tokens_pinned, non_blocking=True)
            self.static_targets.copy_(targets_pinned, non_blocking=True)
            self.graph.replay()
            return float(self.static_loss.item())
        loss = self._step_body(tokens_pinned.to(self.device, non_blocking=True),
                               targets_pinned.to(self.device, non_blocking=True))
        return float(loss.item())

    def check(self) -> None:
        if self.comm is not None:
            self.comm.check_status()
