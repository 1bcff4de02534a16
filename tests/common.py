"""Shared harness for the multi-process tests.

Follows the reference's strategy (tests/common.py:25-185): real processes over
real sockets on one host, a per-rank result handed back to the parent, fp64
golden results computed on the CPU, and tolerances of 1e-2 for half / bf16,
1e-4 for fp32 and exact equality for integers.
"""
from __future__ import annotations

import os
import socket
import traceback
from typing import Any, Callable, Dict, List

import torch
import torch.multiprocessing as mp

WORLD = int(os.environ.get("MCCL_TEST_WORLD", "2"))

FLOAT_DTYPES = [torch.float32, torch.float16, torch.bfloat16, torch.float64]
INT_DTYPES = [torch.int8, torch.int16, torch.int32, torch.int64, torch.uint8]
DTYPES = FLOAT_DTYPES + INT_DTYPES + [torch.bool]
REDUCE_OPS = ["sum", "min", "max", "product", "avg"]


def tol(dtype: torch.dtype) -> float:
    if dtype in (torch.float16, torch.bfloat16):
        return 1e-2
    if dtype == torch.float32:
        return 1e-4
    if dtype == torch.float64:
        return 1e-10
    return 0.0


def free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, fn: Callable, kwargs: Dict[str, Any], env: Dict[str, str], queue) -> None:
    try:
        # a rank that is still running shortly before the harness gives up prints where it is (shown with the failure)
        dump_after = kwargs.pop("_dump_after", 0.0)
        if dump_after > 0:
            import faulthandler
            faulthandler.enable()
            faulthandler.dump_traceback_later(dump_after, exit=False)
        os.environ.update(env)
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        import torch.distributed as dist
        import mccl_b200  # noqa: F401  (registers the backend)
        use_cuda = kwargs.pop("_cuda", False)
        device_id = None
        if use_cuda:
            torch.cuda.set_device(rank % torch.cuda.device_count())
            device_id = torch.device("cuda", rank % torch.cuda.device_count())
        dist.init_process_group(
            backend="mccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
            timeout=__import__("datetime").timedelta(seconds=kwargs.pop("_timeout", 60)),
        )
        skip_barrier = kwargs.pop("_skip_final_barrier", False)
        result = fn(rank, world, **kwargs)
        if use_cuda:
            torch.cuda.synchronize()
        if not skip_barrier:
            dist.barrier()
            dist.destroy_process_group()
        queue.put((rank, "ok", result))
    except BaseException as e:  # noqa: BLE001
        queue.put((rank, "error", f"{type(e).__name__}: {e}\n{traceback.format_exc()}"))


def spawn(fn: Callable, world: int = WORLD, timeout: float = 120.0, env: Dict[str, str] | None = None, **kwargs) -> List[Any]:
    """Runs ``fn(rank, world, **kwargs)`` in `world` processes joined by backend "mccl".

    Returns the per-rank results ordered by rank; raises if any rank failed or
    the group did not finish in time.  ``fn`` must be a module-level function.
    """
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = free_port()
    kwargs.setdefault("_dump_after", max(5.0, timeout - 10.0))
    procs = [ctx.Process(target=_worker, args=(r, world, port, fn, dict(kwargs), env or {}, queue), daemon=True)
             for r in range(world)]
    for p in procs:
        p.start()
    results: Dict[int, Any] = {}
    errors: List[str] = []
    import queue as pyqueue
    import time
    deadline = time.time() + timeout
    while len(results) + len(errors) < world and time.time() < deadline:
        try:
            rank, status, payload = queue.get(timeout=0.5)
        except pyqueue.Empty:
            if errors and all(not p.is_alive() for p in procs):
                break
            # a rank that died without a word (a signal, os._exit) is a failure now, not a timeout later
            dead = [(r, p.exitcode) for r, p in enumerate(procs) if not p.is_alive() and p.exitcode not in (0, None) and r not in results]
            if dead and not errors:
                errors.extend(f"[rank {r}] process died with exit code {code}" for r, code in dead)
                deadline = min(deadline, time.time() + 10)
            continue
        if status == "ok":
            results[rank] = payload
        else:
            errors.append(f"[rank {rank}] {payload}")
            deadline = min(deadline, time.time() + 10)  # peers will time out; do not wait long
    for p in procs:
        p.join(timeout=5)
        if p.is_alive():
            p.terminate()
    if errors:
        raise AssertionError("worker failure:\n" + "\n".join(errors))
    if len(results) < world:
        raise AssertionError(f"only {len(results)}/{world} ranks finished within {timeout}s")
    return [results[r] for r in range(world)]


# ---- inputs and fp64 goldens ------------------------------------------------
def rank_tensor(rank: int, numel: int, dtype: torch.dtype, device="cpu") -> torch.Tensor:
    """Deterministic per-rank input that is exact in every dtype."""
    if dtype == torch.bool:
        return ((torch.arange(numel) + rank) % 2 == 0).to(device)
    base = (torch.arange(numel, dtype=torch.float64) % 5) + rank + 1
    return base.to(dtype).to(device)


def randn_tensor(rank: int, numel: int, dtype=torch.float32, device="cpu") -> torch.Tensor:
    g = torch.Generator().manual_seed(rank)
    return torch.randn(numel, generator=g, dtype=torch.float32).to(dtype).to(device)


def golden_allreduce(inputs: List[torch.Tensor], op: str) -> torch.Tensor:
    dt = inputs[0].dtype
    if dt == torch.bool:
        st = torch.stack([t.to(torch.int64) for t in inputs])
        return {"sum": st.sum(0) > 0, "max": st.max(0).values > 0, "min": st.min(0).values > 0,
                "product": st.prod(0) > 0, "avg": st.sum(0) > 0}[op]
    wide = torch.int64 if not dt.is_floating_point else torch.float64
    st = torch.stack([t.to(wide) for t in inputs])
    if op == "sum":
        return st.sum(0)
    if op == "avg":
        s = st.sum(0)
        return s / len(inputs) if dt.is_floating_point else torch.div(s, len(inputs), rounding_mode="trunc")
    if op == "min":
        return st.min(0).values
    if op == "max":
        return st.max(0).values
    if op == "product":
        return st.prod(0)
    raise ValueError(op)


def assert_close(actual: torch.Tensor, golden: torch.Tensor, dtype: torch.dtype, what: str = "") -> None:
    t = tol(dtype)
    a = actual.detach().cpu()
    if dtype == torch.bool:
        assert torch.equal(a, golden.to(torch.bool)), what
        return
    if t == 0.0:
        assert torch.equal(a.to(torch.int64), golden.to(torch.int64).to(dtype).to(torch.int64)), what
        return
    a64, g64 = a.to(torch.float64), golden.to(torch.float64)
    denom = g64.abs().clamp_min(1.0)
    err = ((a64 - g64).abs() / denom).max().item() if a64.numel() else 0.0
    assert err <= t, f"{what}: max rel err {err:.3e} > {t:.1e}"


def reduce_op(name: str):
    import torch.distributed as dist
    return {"sum": dist.ReduceOp.SUM, "min": dist.ReduceOp.MIN, "max": dist.ReduceOp.MAX,
            "product": dist.ReduceOp.PRODUCT, "avg": dist.ReduceOp.AVG}[name]
