"""Python-side pieces that need no GPU: CLI helpers, environment checks, tuning
table, sharding helpers, distributed tensors on CPU process groups."""
import json
import os

import pytest
import torch
import torch.distributed as dist

from tests.common import spawn


def test_parse_memory_and_cli_jobs(tmp_path, monkeypatch):
    from mccl_b200 import cli
    assert cli.parse_memory("16GB") == 16 << 30 and cli.parse_memory("512mb") == 512 << 20 and cli.parse_memory("100") == 100
    monkeypatch.setenv("MCCL_STATE_FILE", str(tmp_path / "jobs.json"))
    assert cli.main(["submit", "--name", "train", "--priority", "high", "--nodes", "2", "--memory", "40GB", "python", "x.py"]) == 0
    jobs = json.load(open(tmp_path / "jobs.json"))
    assert jobs[0]["name"] == "train" and jobs[0]["priority"] == "HIGH" and jobs[0]["memory_per_node"] == 40 << 30
    assert cli.main(["jobs"]) == 0
    assert cli.main(["cancel", "1"]) == 0
    assert cli.main(["cancel", "1"]) == 1


def test_check_runs_and_required_checks_pass(capsys):
    from mccl_b200 import check
    rc = check.run_all()
    out = capsys.readouterr().out
    assert rc == 0 and "backend 'mccl' registered" in out


def test_tuning_table_crossover(tmp_path, monkeypatch):
    from mccl_b200 import tuning
    rows = [{"bytes": 1024, "algo": "oneshot", "us": 10}, {"bytes": 1024, "algo": "twoshot", "us": 17},
            {"bytes": 1 << 20, "algo": "oneshot", "us": 26}, {"bytes": 1 << 20, "algo": "twoshot", "us": 37},
            {"bytes": 4 << 20, "algo": "oneshot", "us": 70}, {"bytes": 4 << 20, "algo": "twoshot", "us": 42}]
    assert tuning.crossover_from_sweep(rows) == 1 << 20
    path = tuning.save_tuning_table(rows, 8, str(tmp_path / "t.json"))
    assert tuning.load_tuning_table(path)["tree_below"] == 1 << 20
    monkeypatch.setenv("MCCL_TUNING_FILE", path)
    monkeypatch.delenv("MCCL_TREE_BELOW", raising=False)
    applied = tuning.apply_nvlink_production_defaults(training_defaults=True)
    try:
        assert applied["MCCL_TREE_BELOW"] == str(1 << 20) and os.environ["DDP_BUCKET_MB"] == "25"
    finally:
        for k in applied:      # set directly in os.environ by the call above: remove them the same way
            os.environ.pop(k, None)


def test_model_parallel_plan_splits():
    from mccl_b200.distributed import ModelParallelPlan as P
    b = torch.arange(10).reshape(10, 1)
    assert [P.data_parallel_split(b, 3, r).shape[0] for r in range(3)] == [3, 3, 4]
    w = torch.zeros(8, 6)
    assert [t.shape for t in P.tensor_parallel_split(w, 0, 4)] == [torch.Size([2, 6])] * 4
    assert P.pipeline_parallel_split(list(range(7)), 3) == [[0, 1], [2, 3], [4, 5, 6]]


def _dist_tensor(rank, world):
    from mccl_b200.distributed import DistributedModel, DistributedTensor, ShardingSpec
    t = DistributedTensor(torch.full((6,), float(rank + 1)), ShardingSpec.DATA_PARALLEL)
    assert torch.equal(t.all_gather(), torch.cat([torch.full((6,), float(r + 1)) for r in range(world)]))
    assert torch.equal(t.reduce_scatter("sum"), torch.full((6 // world,), float(sum(range(1, world + 1)))))
    assert torch.allclose(t.sync_gradient(), torch.full((6,), sum(range(1, world + 1)) / world))
    torch.manual_seed(rank)
    model = torch.nn.Linear(4, 3)
    dm = DistributedModel(model)
    dm.register_parameters()
    x = torch.full((2, 4), float(rank + 1))
    dm(x).sum().backward()
    dm.sync_gradients()
    g = model.weight.grad.clone()
    gs = [torch.empty_like(g) for _ in range(world)]
    dist.all_gather(gs, g)
    assert all(torch.equal(a, gs[0]) for a in gs)
    assert torch.allclose(g, torch.full_like(g, 2 * sum(range(1, world + 1)) / world))
    return True


def test_distributed_tensor_and_model_on_cpu_group():
    assert all(spawn(_dist_tensor, 2))
