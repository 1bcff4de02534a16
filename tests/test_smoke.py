"""Import, registration and world==1 fast paths (no network, no GPU).

Mirrors the reference's smoke test (tests/test_smoke.py:1-41) and its build
test's version checks (tests/test_build.py:27-46).
"""
import torch
import torch.distributed as dist


def test_import_and_versions():
    import mccl
    import mccl_b200
    assert mccl.__version__ == mccl_b200.__version__ == mccl._C.__version__ == "0.4.0"
    assert mccl._C.__protocol_version__ == 1
    assert "features" in mccl.COMPATIBILITY_MATRIX


def test_backend_registered():
    import mccl  # noqa: F401
    assert "mccl" in dist.Backend.backend_list
    mccl.register()  # idempotent


def test_iface_priority_roundtrip():
    import os
    import mccl
    mccl.set_iface_priority(["10.1.", "10.2."])
    assert os.environ["MCCL_IFACE_PRIORITY"] == "10.1.,10.2."
    mccl.set_iface_priority([])
    assert "MCCL_IFACE_PRIORITY" not in os.environ


def test_config_roundtrip(monkeypatch):
    from mccl import DistroConfig
    monkeypatch.setenv("DISTRO_NODE_ID", "3")
    monkeypatch.setenv("MCCL_ALLREDUCE_ALGO", "butterfly")
    monkeypatch.setenv("DISTRO_FAST_MATH", "0")
    cfg = DistroConfig.from_env()
    assert cfg.node_id == 3 and cfg.allreduce_algo == "butterfly" and cfg.fast_math is False
    d = cfg.to_dict()
    assert DistroConfig.from_dict(d).to_dict() == d
    import pytest
    with pytest.raises(ValueError):
        DistroConfig(node_id=-1)
    with pytest.raises(ValueError):
        DistroConfig(allreduce_algo="bogus")


def test_world1_collectives_are_noops():
    import mccl  # noqa: F401
    store = dist.HashStore()
    dist.init_process_group("mccl", store=store, rank=0, world_size=1)
    try:
        t = torch.arange(8, dtype=torch.float32)
        dist.all_reduce(t)
        assert torch.equal(t, torch.arange(8, dtype=torch.float32))
        dist.broadcast(t, 0)
        out = torch.empty(8)
        dist.all_gather_into_tensor(out, t)
        assert torch.equal(out, t)
        outs = [torch.empty(8)]
        dist.all_gather(outs, t)
        assert torch.equal(outs[0], t)
        rs = torch.empty(8)
        dist.reduce_scatter_tensor(rs, t)
        assert torch.equal(rs, t)
        a2a = torch.empty(8)
        dist.all_to_all_single(a2a, t)
        assert torch.equal(a2a, t)
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_metrics_object_shape():
    import mccl
    m = mccl.get_metrics()
    for field in ("total_ops", "avg_latency_ms", "avg_sync_ms", "avg_network_ms", "avg_reduce_ms"):
        assert hasattr(m, field)


def test_host_kernels_match_torch():
    """Host restatement of the element-wise kernels (same bindings the GPU tests call)."""
    import mccl
    C = mccl._C
    for dt in (torch.float32, torch.float16, torch.bfloat16, torch.int32):
        for n in (1, 3, 7, 13, 97, 997):
            a = (torch.arange(n) % 7 + 1).to(dt)
            b = (torch.arange(n) % 3 + 1).to(dt)
            assert torch.equal(C._mccl_accumulate_chunk(a.clone(), b), a + b)
            assert torch.equal(C._metal_elementwise_min(a.clone(), b), torch.minimum(a, b))
            assert torch.equal(C._mccl_elementwise_max(a.clone(), b), torch.maximum(a, b))
            assert torch.equal(C._mccl_elementwise_product(a.clone(), b), a * b)
    x = torch.full((5,), 6.0)
    assert torch.allclose(C._mccl_scale_inplace(x.clone(), 0.5), x * 0.5)
    assert torch.allclose(C._mccl_accumulate_and_scale(x.clone(), x, 0.25), (x + x) * 0.25)
