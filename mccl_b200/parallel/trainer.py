"""Data-parallel training engine built on the device communicator.

The reference reaches its headline numbers with stock DistributedDataParallel
over its allreduce (README.md:44-54, tests/test_ddp_e2e.py); stock DDP works on
this backend too (see ``mccl_b200.parallel.ddp``).  This engine is the
B200-first form of the same job:

* all parameters live in one flat fp32 buffer and all gradients in one flat
  fp32 buffer, ordered so that the gradients that finish first in backward sit
  in the first bucket; the last bucket is kept small, because it is the one
  whose collective cannot hide behind backward;
* when the last gradient of a bucket has been accumulated, the bucket is
  all-reduced in place on a side stream while backward continues: staged
  through the arena with bf16 on the wire and fp32 accumulation
  (``wire="bf16"``), or in-switch (``multimem.ld_reduce``) / by direct peer
  loads on a gradient buffer in the symmetric heap (``wire="native"``), with
  the 1/world scale fused in every case;
* when backward ends, the fused AdamW kernel (which also clears the gradients
  it has consumed) runs over the buckets that are already reduced while the
  collectives of the tail buckets are still in flight on the side stream, and
  then over the tail, so the last collectives hide behind the optimizer;
* during backward the GEMMs can leave ``comm_sms`` SMs unoccupied for the
  collectives, which then run as that many 512-thread CTAs (a CTA of that size
  only fits on an SM that holds no persistent GEMM CTA);
* forward, backward, the bucket collectives and the optimizer are captured
  once into a CUDA graph and replayed, so a step costs one launch on the host.
"""
from __future__ import annotations

import os
from typing import List, Optional

import torch
import torch.distributed as dist

from .. import _C, ops
from ..ops import native as _native


class _Bucket:
    __slots__ = ("start", "numel", "pending", "total", "late", "tail", "fired", "applied")

    def __init__(self, start: int):
        self.start, self.numel, self.pending, self.total = start, 0, 0, 0
        self.tail = False    # completes when backward ends: nothing is left to share the GPU with
        self.fired = -1      # step in which the bucket was last reduced / updated
        self.applied = -1    # step in which the optimizer already updated the bucket during backward (one GPU)
        # True once a gradient of this bucket has arrived through autograd's own accumulation: such a
        # bucket is reduced after backward() has returned (the engine has then joined the stream that
        # accumulated it with the caller's stream), not from inside the hook.
        self.late = False


class DDPTrainer:
    def __init__(self, model: torch.nn.Module, device: torch.device, lr: float = 3e-4, betas=(0.9, 0.999),
                 eps: float = 1e-8, weight_decay: float = 0.01, group=None, wire: str = "bf16",
                 bucket_mb: float = 25.0, overlap: bool = True, use_graph: bool = True, algo: str = "auto",
                 comm_sms: Optional[int] = None, comm_threads: Optional[int] = None,
                 overlap_optimizer: Optional[bool] = None, last_bucket_mb: float = 4.0):
        self.model, self.device = model, device
        self.lr, self.betas, self.eps, self.wd = lr, betas, eps, weight_decay
        self.wire, self.overlap, self.use_graph, self.algo = wire, overlap, use_graph, algo
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.comm = None
        self._late: List[_Bucket] = []
        self._step_id = 0
        if self.world > 1:
            import mccl_b200
            be = mccl_b200.get_backend(group)
            if be is None:
                raise RuntimeError("DDPTrainer needs a process group created with backend='mccl'")
            self.comm = be.device_comm(device.index)
        # SMs kept free of GEMM CTAs during backward for the bucket collectives (0: none, the collectives
        # then share SMs with the GEMMs as 256-thread CTAs).
        if comm_sms is None:
            comm_sms = int(os.environ.get("MCCL_DDP_COMM_SMS", "40"))
        self.comm_sms = comm_sms if (self.world > 1 and overlap) else 0
        # SMs every backward GEMM leaves free when no collectives need them (one GPU): room for the weight-gradient stream
        self._bwd_free_sms = int(os.environ.get("MCCL_BWD_FREE_SMS", "0")) if device.type == "cuda" else 0
        # CTA caps of the backward GEMMs on the main stream and of the weight-gradient GEMMs on the side stream.  Two
        # GEMMs that each want every SM take turns, set-up and tail included; capped at 88 of 148 CTAs each they mostly
        # run side by side (a second round of tiles costs a CTA about a third more, not twice).  Measured on the 70M
        # decoder: 4.72 -> 4.49 ms per step on one GPU, 4.97 -> 4.68 on two (with 40 SMs kept for the collectives).
        side_on = device.type == "cuda" and os.environ.get("MCCL_SIDE_WGRAD", "1") != "0"
        self._bwd_main_ctas = int(os.environ.get("MCCL_BWD_MAIN_CTAS", "88" if side_on else "0")) if device.type == "cuda" else 0
        self._bwd_side_ctas = int(os.environ.get("MCCL_BWD_SIDE_CTAS", "88" if side_on else "0")) if device.type == "cuda" else 0
        # without an explicit setting the graph is captured with and without the caps and the faster one is kept
        self._tune_caps = "MCCL_BWD_MAIN_CTAS" not in os.environ and "MCCL_BWD_SIDE_CTAS" not in os.environ
        if comm_threads is None:
            comm_threads = int(os.environ.get("MCCL_DDP_COMM_THREADS", "512" if self.comm_sms > 0 else "0"))
        self.comm_threads = comm_threads
        # The optimizer pass over the already reduced buckets runs while the tail buckets' collectives are still
        # in flight.  (Running the optimizer bucket by bucket during backward was measured too: its CTAs delay
        # the GEMMs by as much as the pass saves, 6.71 against 6.64 ms per step of the 70M decoder on one GPU.)
        if overlap_optimizer is None:
            overlap_optimizer = os.environ.get("MCCL_DDP_OVERLAP_OPTIMIZER", "1") != "0"
        self.overlap_optimizer = bool(overlap_optimizer and overlap and self.world > 1 and device.type == "cuda"
                                      and ops.native_ops_available().get("adamw_flat"))
        self._fused_zero = device.type == "cuda" and bool(ops.native_ops_available().get("adamw_flat"))
        # Hooks are needed whenever something happens per bucket.
        # One GPU, MCCL_OVERLAP_ADAMW=1: the optimizer update of a bucket whose gradients are complete runs on the
        # weight-gradient stream while backward continues.  Off by default: measured 4.79 ms per step against 4.72 with
        # one update at the end (AdamW's traffic slows the GEMMs it runs beside by more than it hides).
        self._local_overlap = (self.world == 1 and device.type == "cuda"
                               and os.environ.get("MCCL_SIDE_WGRAD", "1") != "0"
                               and os.environ.get("MCCL_OVERLAP_ADAMW", "0") == "1")
        self._per_bucket = self.world > 1 or self._local_overlap
        self._body_done = None   # event on the side stream: every non-tail bucket has been reduced
        # weight-gradient GEMMs on a stream of their own, beside the input-gradient chain (MCCL_SIDE_WGRAD=0: in line)
        self.wgrad_stream = None
        if device.type == "cuda" and os.environ.get("MCCL_SIDE_WGRAD", "1") != "0":
            self.wgrad_stream = torch.cuda.Stream(device=device)
        self._flatten(bucket_mb, last_bucket_mb)
        self.step_t = torch.zeros((), device=device, dtype=torch.float32)
        self.m = torch.zeros_like(self.flat_p)
        self.v = torch.zeros_like(self.flat_p)
        self.comm_stream = (torch.cuda.Stream(device=device, priority=-1)
                            if (self.world > 1 and device.type == "cuda") else None)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.static_tokens = None
        self.static_targets = None
        self.static_loss = None
        self.launches_per_step = 0
        if self.world > 1:
            self._sync_initial_params(group)

    # ------------------------------------------------------------ buffers --
    def _flatten(self, bucket_mb: float, last_bucket_mb: float) -> None:
        params = [p for p in self.model.parameters() if p.requires_grad]
        # Backward produces gradients roughly in reverse registration order.
        order = list(reversed(params))
        align = 16 * max(self.world, 1)  # chunk boundaries of the collectives stay 16-element aligned
        bucket_cap = int(bucket_mb * (1 << 20) / 4)
        last_cap = int(max(last_bucket_mb, 0.0) * (1 << 20) / 4)
        # The tail: the parameters whose gradients arrive last.  Their collectives (and optimizer slices)
        # run after backward has ended, so they go into buckets of their own: every parameter larger than
        # last_cap alone, the small ones before it together up to last_cap.
        tail_from = len(order)
        if self._per_bucket and last_cap > 0 and len(order) > 1:
            acc = 0
            i = len(order) - 1
            while i >= 0 and order[i].numel() > last_cap:   # large trailing parameters (a tied embedding table)
                i -= 1
            j = i
            while j >= 0 and acc + order[j].numel() <= last_cap:
                acc += order[j].numel()
                j -= 1
            tail_from = j + 1
        offsets, total = [], 0
        self.buckets: List[_Bucket] = [_Bucket(0)]

        def close_bucket():
            nonlocal total
            total = (total + align - 1) // align * align
            self.buckets[-1].numel = total - self.buckets[-1].start
            self.buckets.append(_Bucket(total))

        for k, p in enumerate(order):
            b = self.buckets[-1]
            in_tail = k >= tail_from
            cap = bucket_cap
            new = b.numel > 0 and b.numel + p.numel() > cap
            if in_tail and b.numel > 0 and (k == tail_from or p.numel() > last_cap or order[k - 1].numel() > last_cap):
                new = True
            if new:
                close_bucket()
                b = self.buckets[-1]
            b.tail = in_tail
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
            if self._per_bucket:
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
        # A parameter reports once per step.  (autograd's post-accumulate hook also fires when a native
        # operator returned None for the gradient because it had written it into the sink itself, and
        # that second report must not count: it would mark every bucket as late and reduce it twice.)
        if getattr(p, "_ready_step", -1) == self._step_id:
            return
        p._ready_step = self._step_id
        b = self.buckets[self._param_bucket[p]]
        b.pending += 1
        if b.pending == b.total:
            b.pending = 0
            if b.late:
                self._late.append(b)
            else:
                self._reduce_bucket(b)

    def _on_autograd_grad(self, p: torch.Tensor) -> None:
        if getattr(p, "_ready_step", -1) == self._step_id:
            return   # already reported by the native operator that wrote the gradient
        self.buckets[self._param_bucket[p]].late = True
        self._on_grad_ready(p)

    def _adamw(self, start: int, numel: int) -> None:
        end = start + numel
        ops.adamw_step(self.flat_p[start:end], self.flat_g[start:end], self.m[start:end], self.v[start:end], self.lr,
                       self.betas[0], self.betas[1], self.eps, self.wd, self.step_t,
                       p_bf16=None if self.flat_p16 is None else self.flat_p16[start:end], zero_grad=self._fused_zero)

    def _reduce_bucket(self, b: _Bucket) -> None:
        """Collective (world > 1) and optimizer slice (overlap_optimizer) of one bucket, on the side stream."""
        b.fired = self._step_id
        main = torch.cuda.current_stream(self.device)
        if self.comm is None and self.world == 1:
            if self._local_overlap and self._in_backward and self.wgrad_stream is not None and not b.late:
                # every kernel that reads this bucket's weights in backward is already queued on the main stream
                self.wgrad_stream.wait_stream(main)
                with torch.cuda.stream(self.wgrad_stream):
                    self._adamw(b.start, b.numel)
                _native.mark_wgrad_pending()
                b.applied = self._step_id
            return
        stream = self.comm_stream if (self.overlap and self.comm_stream is not None) else main
        if stream is not main:
            stream.wait_stream(main)
        _native.join_wgrad(stream)   # the bucket's weight gradients may still be running on their own stream
        shaped = self.comm is not None and (self.comm_sms > 0 or self.comm_threads > 0) and self._in_backward and not b.tail
        was_auto = self.comm is not None and self.comm.launch_shape_auto
        if shaped:
            saved = (self.comm.max_ctas, self.comm.launch_threads)
            self.comm.set_launch_shape(self.comm_sms, self.comm_threads)
        elif was_auto:
            # tail buckets run beside the optimizer update: keep the compact default shape (the automatic shape for
            # large messages wants 512 free thread slots on 128 SMs and would wait for the update to finish)
            saved = (self.comm.max_ctas, self.comm.launch_threads)
            self.comm.set_launch_shape(saved[0], 256)
        with torch.cuda.stream(stream):
            if self.comm is not None:
                if self.wire == "bf16":
                    g = self.flat_g[b.start:b.start + b.numel]
                    self.comm.allreduce([g], [g], op="avg", algo=("twoshot" if self.algo == "auto" else self.algo),
                                        wire="bf16")
                else:
                    self.comm.allreduce_symm(self.symm, b.start * 4, b.numel, torch.float32, "avg")
            if self.overlap_optimizer and not b.tail and stream is not main:
                if self._body_done is None:
                    self._body_done = torch.cuda.Event()
                self._body_done.record(stream)
                self._body_recorded = True
        if was_auto:
            self.comm.set_launch_shape(-1, -1)
        elif shaped:
            self.comm.set_launch_shape(saved[0], saved[1] if saved[1] > 0 else -1)

    # ---------------------------------------------------------------- step --
    def _step_body(self, tokens: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        self._step_id += 1
        for b in self.buckets:
            b.pending = 0
        self.step_t.add_(1.0)
        self._body_recorded = False
        if not self._fused_zero:
            self.flat_g.zero_()   # otherwise the optimizer cleared what it consumed
        loss = self.model(tokens, targets)
        free_sms = self.comm_sms if self.comm_sms > 0 else self._bwd_free_sms
        main_ctas = max(_C.gemm_sm_count() - free_sms, 2) if free_sms > 0 else 0
        if self._bwd_main_ctas > 0:
            main_ctas = self._bwd_main_ctas if main_ctas == 0 else min(main_ctas, self._bwd_main_ctas)
        if main_ctas > 0:
            _C.set_gemm_cta_limit(main_ctas)
        self._in_backward = True
        _native.set_wgrad_stream(self.wgrad_stream, main_ctas, self._bwd_side_ctas)
        try:
            loss.backward()
            if self.wgrad_stream is not None:
                _native.join_wgrad(torch.cuda.current_stream(self.device))
        finally:
            _native.set_wgrad_stream(None)
            self._in_backward = False
            if main_ctas > 0 or self._bwd_side_ctas > 0:
                _C.set_gemm_cta_limit(0)
        for b in self._late:
            self._reduce_bucket(b)
        self._late.clear()
        if self._per_bucket:
            for b in self.buckets:   # buckets none of whose parameters took part in this step's graph
                if b.fired != self._step_id and b.pending == 0:
                    self._reduce_bucket(b)
                elif b.fired != self._step_id:   # some parameters of the bucket had no gradient: it is complete now
                    b.pending = 0
                    self._reduce_bucket(b)
        main = torch.cuda.current_stream(self.device) if self.device.type == "cuda" else None
        tail_start = min((b.start for b in self.buckets if b.tail), default=self.total)
        if self.overlap_optimizer and self._body_recorded and 0 < tail_start < self.total:
            # the buckets before the tail are reduced: update them while the tail's collectives run
            main.wait_event(self._body_done)
            self._adamw(0, tail_start)
            main.wait_stream(self.comm_stream)
            self._adamw(tail_start, self.total - tail_start)
        else:
            if self.comm_stream is not None and self.overlap:
                main.wait_stream(self.comm_stream)
            if self._local_overlap:
                # buckets updated during backward are done (the streams were joined after backward); the rest now,
                # neighbouring ranges merged into one launch
                start = None
                for b in self.buckets + [None]:
                    todo = b is not None and b.applied != self._step_id
                    if todo and start is None:
                        start = b.start
                    if not todo and start is not None:
                        end = b.start if b is not None else self.total
                        self._adamw(start, end - start)
                        start = None
            else:
                self._adamw(0, self.total)
        return loss.detach()

    _in_backward = False

    def _capture_one(self) -> "torch.cuda.CUDAGraph":
        graph = torch.cuda.CUDAGraph()
        # the step is captured on a high-priority stream: its kernels are placed before those of the weight-gradient
        # stream (default priority), which then only fills what the main chain leaves free
        capture_stream = torch.cuda.Stream(device=self.device, priority=-1)
        with torch.cuda.graph(graph, stream=capture_stream):
            self.static_loss = self._step_body(self.static_tokens, self.static_targets)
        return graph

    def _capture(self, tokens: torch.Tensor, targets: torch.Tensor) -> None:
        """Warm-up, capture, and a short trial of the candidates for the backward GEMMs' CTA caps.  The optimizer state
        is saved before and put back after, so everything here leaves the model as it found it and the first replay
        is the first update."""
        self.static_tokens = tokens.clone()
        self.static_targets = targets.clone()
        saved = [t.clone() for t in (self.flat_p, self.m, self.v, self.step_t)]
        saved_p16 = None if self.flat_p16 is None else self.flat_p16.clone()
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            for _ in range(2):  # warm up allocator, autotuners and lazy inits outside the capture
                self._step_body(self.static_tokens, self.static_targets)
        torch.cuda.current_stream(self.device).wait_stream(side)
        torch.cuda.synchronize(self.device)
        before = ops.launch_count() + (self.comm.launches if self.comm is not None else 0)
        candidates = [(self._bwd_main_ctas, self._bwd_side_ctas)]
        if self._tune_caps and candidates[0] != (0, 0):
            candidates.append((0, 0))   # the caps pay when a GEMM's tiles fit the capped grid in few rounds; not always
        best = None
        for main_ctas, side_ctas in candidates:
            self._bwd_main_ctas, self._bwd_side_ctas = main_ctas, side_ctas
            graph = self._capture_one()
            if best is None:
                self.launches_per_step = ops.launch_count() + (self.comm.launches if self.comm is not None else 0) - before
            if len(candidates) == 1:
                best = (0.0, graph, main_ctas, side_ctas, self.static_loss)
                break
            graph.replay()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(3):
                graph.replay()
            e1.record()
            torch.cuda.synchronize(self.device)
            t = torch.tensor([e0.elapsed_time(e1)], device=self.device)
            if self.world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)   # every rank takes the same decision
            if best is None or float(t.item()) < best[0]:
                best = (float(t.item()), graph, main_ctas, side_ctas, self.static_loss)
        _, self.graph, self._bwd_main_ctas, self._bwd_side_ctas, self.static_loss = best
        for dst, src in zip((self.flat_p, self.m, self.v, self.step_t), saved):
            dst.copy_(src)
        if saved_p16 is not None:
            self.flat_p16.copy_(saved_p16)
        self.flat_g.zero_()
        torch.cuda.synchronize(self.device)

    def step(self, tokens: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        """One optimizer step on device-resident tokens; returns the loss (device tensor).

        On CUDA the gradient buffer is cleared by the optimizer kernel as it consumes it (that replaces a
        memset at the start of the next step), so ``p.grad`` reads as zero after a step."""
        if not self.use_graph:
            before = ops.launch_count() + (self.comm.launches if self.comm is not None else 0)
            loss = self._step_body(tokens, targets)
            self.launches_per_step = ops.launch_count() + (self.comm.launches if self.comm is not None else 0) - before
            return loss
        if self.graph is None:
            self._capture(tokens, targets)
        self.check()   # a wait that ran out in an earlier step raises here, before its gradients are used again
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
            loss = float(self.static_loss.item())
            self.check()
            return loss
        loss = self._step_body(tokens_pinned.to(self.device, non_blocking=True),
                               targets_pinned.to(self.device, non_blocking=True))
        return float(loss.item())

    def check(self) -> None:
        """Raises TimeoutError when a device-side wait of this trainer's collectives ran out."""
        if self.comm is not None and self.comm.status() != 0:
            self.comm.check_status()
