"""The allocation-free column-sum entry point, called the way an embedder would:
through its exported C symbol, with raw device pointers.

Some callers of this library may not allocate device memory (plugins running
inside another framework's stream-ordered region, loops with a no-allocation
rule, runtimes that own all memory).  For them the library exports
``mccl_colsum_bf16_noalloc``, whose scratch space is a fixed array inside the
library image.  The test checks it against the regular entry point
(``_C.colsum_bf16``, scratch from torch's allocator) on two calls in a row,
since the second call reuses the array the first one left behind, and checks
that an oversized problem is refused rather than run.

This file sorts last on purpose: a run that stops at the first failure has
already been through every other test.
"""
import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    import mccl_b200
    lib = ctypes.CDLL(os.path.join(os.path.dirname(mccl_b200.__file__), "_C.so"))
    lib.mccl_colsum_bf16_noalloc.restype = ctypes.c_int
    lib.mccl_colsum_bf16_noalloc.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    lib.mccl_noalloc_last_error.restype = ctypes.c_char_p
    return lib, mccl_b200._C


def test_noalloc_colsum_matches_regular_entry_point_twice():
    lib, C = _lib()
    torch.cuda.set_device(0)
    stream = torch.cuda.current_stream().cuda_stream
    for (rows, dim), seed in (((4096, 512), 1), ((1000, 2048), 2)):   # second call reuses the shared array
        torch.manual_seed(seed)
        x = torch.randn(rows, dim, device="cuda").bfloat16()
        out = torch.full((dim,), float("nan"), device="cuda")
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        free_before, _ = torch.cuda.mem_get_info()      # the driver's own count: sees a cudaMalloc made inside the library too
        rc = lib.mccl_colsum_bf16_noalloc(x.data_ptr(), out.data_ptr(), rows, dim, stream)
        assert rc == 0, lib.mccl_noalloc_last_error()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        free_after, _ = torch.cuda.mem_get_info()
        assert free_after >= free_before, (free_before, free_after)   # nothing was taken from the device
        ref = C.colsum_bf16(x)
        torch.cuda.synchronize()
        err = ((out - ref).abs().max() / ref.abs().max().clamp_min(1e-6)).item()
        assert err < 1e-5, err   # same reduction order as the regular path: expect equality up to fp32 rounding
        gold = x.float().sum(0)
        assert ((out - gold).abs().max() / gold.abs().max()).item() < 1e-4


def test_noalloc_colsum_refuses_what_does_not_fit():
    lib, _ = _lib()
    torch.cuda.set_device(0)
    x = torch.zeros(8, 8, device="cuda", dtype=torch.bfloat16)
    out = torch.zeros(8, device="cuda")
    # ceil(rows / 64) * dim = 2^21 floats > 2^20: refused from the sizes alone, nothing is launched
    rc = lib.mccl_colsum_bf16_noalloc(x.data_ptr(), out.data_ptr(), 64 * 1024, 2048, None)
    assert rc == -2 and b"too large" in lib.mccl_noalloc_last_error()
    # many rows of a narrow matrix: the partial sums would fit (78125 * 8 floats) but the slab count exceeds the
    # grid-dimension limit; this, too, is refused up front with TOO_LARGE instead of failing at launch
    rc = lib.mccl_colsum_bf16_noalloc(x.data_ptr(), out.data_ptr(), 5_000_000, 8, None)
    assert rc == -2 and b"too large" in lib.mccl_noalloc_last_error()
    rc = lib.mccl_colsum_bf16_noalloc(x.data_ptr(), out.data_ptr(), 8, 12, None)
    assert rc == -1
    # pinned host memory is not device memory of the current device
    host = torch.zeros(8, 8, dtype=torch.bfloat16).pin_memory()
    rc = lib.mccl_colsum_bf16_noalloc(host.data_ptr(), out.data_ptr(), 8, 8, None)
    assert rc == -1 and b"current device" in lib.mccl_noalloc_last_error()
    torch.cuda.synchronize()
