"""One tiny training step of the flagship decoder through the native operators."""
from __future__ import annotations

import torch


def run_smoke(device: torch.device) -> float:
    from .. import ops
    from ..parallel import DDPTrainer
    from .decoder import build_decoder

    torch.manual_seed(0)
    # two heads of 64 and a sequence of 128, so that attention runs on this package's kernels too
    model = build_decoder("tiny", native=True, n_heads=2, max_seq=128).to(device)
    trainer = DDPTrainer(model, device, use_graph=False)
    tokens = torch.randint(0, model.cfg.vocab, (4, 129), device=device)
    before = ops.launch_count()
    l0 = float(trainer.step(tokens[:, :-1].contiguous(), tokens[:, 1:].contiguous()).item())
    for _ in range(3):
        loss = trainer.step(tokens[:, :-1].contiguous(), tokens[:, 1:].contiguous())
    l1 = float(loss.item())
    torch.cuda.synchronize(device)
    launched = ops.launch_count() - before
    print(f"smoke: loss {l0:.4f} -> {l1:.4f}; native operator launches: {launched}; available: {ops.native_ops_available()}")
    assert l1 == l1 and l1 < l0 + 1e-3, "loss did not go down"
    return l1
