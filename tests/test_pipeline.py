"""1F1B pipeline schedule over send / recv against a single-process reference (CPU ranks)."""
import pytest
import torch
import torch.distributed as dist
import torch.nn as nn

from tests.common import spawn


def _make_layers(n):
    torch.manual_seed(11)
    return [nn.Sequential(nn.Linear(16, 16), nn.Tanh()) for _ in range(n)]


def _pipeline(rank, world, n_mb):
    from mccl_b200.parallel.pp import PipelineStage, split_layers
    layers = _make_layers(6)
    mine = nn.Sequential(*[layers[i] for i in split_layers(6, world)[rank]])
    torch.manual_seed(5)
    data = torch.randn(n_mb, 4, 16)
    target = torch.randn(n_mb, 4, 16)

    def fn(x, mb):
        h = mine(data[mb] if x is None else x)
        if rank == world - 1:
            return ((h - target[mb]) ** 2).mean() / n_mb
        return h

    stage = PipelineStage(fn, rank, world, rank - 1 if rank > 0 else None, rank + 1 if rank < world - 1 else None,
                          (4, 16), torch.float32, torch.device("cpu"))
    loss = stage.run(n_mb)
    grads = torch.cat([p.grad.reshape(-1) for p in mine.parameters()])
    # reference: the whole model on this rank
    ref_layers = _make_layers(6)
    full = nn.Sequential(*ref_layers)
    ref_loss = sum(((full(data[m]) - target[m]) ** 2).mean() / n_mb for m in range(n_mb))
    ref_loss.backward()
    ref = torch.cat([p.grad.reshape(-1) for i in split_layers(6, world)[rank] for p in ref_layers[i].parameters()])
    assert torch.allclose(grads, ref, atol=1e-6), (grads - ref).abs().max()
    if rank == world - 1:
        assert torch.allclose(loss, ref_loss.detach(), atol=1e-6)
    return True


@pytest.mark.parametrize("world,n_mb", [(2, 1), (2, 4), (3, 4), (3, 2)])
def test_1f1b_matches_single_process(world, n_mb):
    assert all(spawn(_pipeline, world, timeout=120, n_mb=n_mb))


def test_split_layers_gives_remainder_to_early_stages():
    from mccl_b200.parallel.pp import split_layers
    assert [list(r) for r in split_layers(7, 3)] == [[0, 1, 2], [3, 4], [5, 6]]
    assert [len(r) for r in split_layers(24, 2)] == [12, 12]
