"""Pipeline parallelism over point-to-point send / recv.

The reference verifies ``dist.send`` / ``dist.recv`` between stages and names
pipeline parallelism as something its primitives carry, with a sketch of a
stage runtime that was never connected (README.md:75, tests/collectives/test_p2p.py,
mccl/distributed/sharding.py:71-89 ``pipeline_parallel_split``,
csrc/runtime/DistributedMetalRuntime.cpp ``dispatch_pipeline``).  This module is
the working form: a one-forward-one-backward (1F1B) schedule over micro-batches,
each stage a ``torch.nn.Module`` on its own rank (or its own tensor-parallel
group), activations and their gradients exchanged with the stage's neighbours.

On CUDA the backend hands ``send`` / ``recv`` to NCCL point-to-point (NVLink);
on CPU they travel over the TCP mesh, which is what the tests use.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence

import torch
import torch.distributed as dist


def split_layers(n_layers: int, n_stages: int) -> List[range]:
    """Contiguous, near-equal layer ranges, earlier stages taking the remainder
    (the rule of ``pipeline_parallel_split``, mccl/distributed/sharding.py:71-89)."""
    base, extra = divmod(n_layers, n_stages)
    out, start = [], 0
    for s in range(n_stages):
        n = base + (1 if s < extra else 0)
        out.append(range(start, start + n))
        start += n
    return out


class PipelineStage:
    """One stage of a pipeline.

    stage_fn(x_or_None, microbatch_index) -> tensor: the stage's forward.  The first stage receives
    ``None`` and reads its own input for that micro-batch; the last stage returns the scalar loss
    of the micro-batch (already divided by the number of micro-batches if a mean is wanted).
    prev_rank / next_rank: global ranks of the neighbouring stages (None at the ends).
    act_shape / act_dtype: shape and dtype of the activation this stage RECEIVES (ignored on the
    first stage); out_shape of what it sends is taken from the produced tensor.
    """

    def __init__(self, stage_fn: Callable[[Optional[torch.Tensor], int], torch.Tensor], stage: int, n_stages: int,
                 prev_rank: Optional[int], next_rank: Optional[int], act_shape: Sequence[int], act_dtype: torch.dtype,
                 device: torch.device, group=None):
        self.fn, self.stage, self.n_stages = stage_fn, stage, n_stages
        self.prev, self.next = prev_rank, next_rank
        self.act_shape, self.act_dtype, self.device, self.group = tuple(act_shape), act_dtype, device, group
        self.first, self.last = stage == 0, stage == n_stages - 1

    # -------------------------------------------------------------- plumbing --
    # Every transfer is a blocking send or recv.  Where a stage has one of each with the same neighbour
    # back to back, the order is fixed so that the two sides never both wait to send: after a forward a
    # stage first RECEIVES the gradient of an earlier micro-batch from the next stage and then sends its
    # activation; after a backward it first SENDS its input gradient to the previous stage and then
    # receives the next activation.
    def _recv_forward(self) -> Optional[torch.Tensor]:
        if self.first:
            return None
        x = torch.empty(self.act_shape, dtype=self.act_dtype, device=self.device)
        dist.recv(x, src=self.prev, group=self.group)
        return x.requires_grad_(True)

    def _send_forward(self, y: torch.Tensor) -> None:
        if not self.last:
            dist.send(y.detach().contiguous(), dst=self.next, group=self.group)

    def _recv_backward(self, y: torch.Tensor) -> Optional[torch.Tensor]:
        if self.last:
            return None
        g = torch.empty_like(y)
        dist.recv(g, src=self.next, group=self.group)
        return g

    def _send_backward(self, x: Optional[torch.Tensor]) -> None:
        if not self.first:
            dist.send(x.grad.contiguous(), dst=self.prev, group=self.group)

    @staticmethod
    def _backward(y: torch.Tensor, g: Optional[torch.Tensor]) -> None:
        if g is None:
            y.backward()
        else:
            y.backward(g)

    # -------------------------------------------------------------- schedule --
    def run(self, n_microbatches: int) -> Optional[torch.Tensor]:
        """Runs forward and backward of all micro-batches in 1F1B order.  Returns the summed loss on the
        last stage, None elsewhere.  Gradients accumulate in the stage's parameters."""
        warm = min(self.n_stages - self.stage - 1, n_microbatches)
        steady = n_microbatches - warm
        live: list = []          # (input, output) of forwards whose backward is still to come
        total = None
        mb = 0

        def forward(x):
            nonlocal mb, total
            y = self.fn(x, mb)
            mb += 1
            live.append((x, y))
            if self.last:
                total = y.detach() if total is None else total + y.detach()
            return y

        for _ in range(warm):
            self._send_forward(forward(self._recv_forward()))
        x = self._recv_forward() if steady > 0 else None
        for i in range(steady):
            y = forward(x)
            g = self._recv_backward(y)          # gradient of the oldest live micro-batch ...
            self._send_forward(y)               # ... then this activation
            xb, yb = live.pop(0)
            self._backward(yb, g)
            self._send_backward(xb)
            if i + 1 < steady:
                x = self._recv_forward()
        for _ in range(warm):
            xb, yb = live.pop(0)
            g = self._recv_backward(yb)
            self._backward(yb, g)
            self._send_backward(xb)
        return total
