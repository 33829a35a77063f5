"""The allocation-free sum-of-squares entry point, called through its exported C symbol, against the regular entry
point (which takes caller-provided scratch). It is meant for callers that may not allocate device memory: code inside a
CUDA-graph capture, plug-ins with a fixed memory budget, services that forbid allocation after start-up. Collected last
so that a run stopping at the first failure has already run every other test."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_no_alloc_sumsq_matches_regular_entry_point_twice():
    from popxl_addons_b200.ops import native as nat

    fn = nat.LIB.xl_grad_sumsq_noalloc
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p]
    fn.restype = ctypes.c_int
    torch.manual_seed(0)
    stream = torch.cuda.current_stream().cuda_stream
    scale = torch.tensor(0.25, device="cuda")
    out = torch.zeros((), device="cuda")
    # the first call on a device looks the scratch array's address up (and may load the kernels' module): warm it up,
    # so that the free-memory readings below see only what a steady-state call does
    warm = torch.ones(16, device="cuda")
    assert fn(warm.data_ptr(), 0, None, out.data_ptr(), 16, stream) == 0
    torch.cuda.synchronize()
    for dtype, n in ((torch.bfloat16, (1 << 22) + 3), (torch.float32, 1000)):  # two calls in a row, shared scratch
        x = torch.randn(n, device="cuda", dtype=dtype)
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        free_before, _ = torch.cuda.mem_get_info()  # the driver's view: also sees a cudaMalloc made inside the library
        rc = fn(x.data_ptr(), nat._CODE[dtype], scale.data_ptr(), out.data_ptr(), n, stream)
        assert rc == 0
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        assert torch.cuda.memory_allocated() == before
        assert free_after >= free_before, (free_before, free_after)
        expected = nat.grad_sumsq_cuda(x, scale)
        torch.cuda.synchronize()
        torch.testing.assert_close(out, expected, rtol=1e-4, atol=1e-2)
        torch.testing.assert_close(out, (x.float() ** 2).sum() * 0.25, rtol=1e-4, atol=1e-2)
    # no scale pointer, and refusal of sizes beyond the stated maximum
    x = torch.ones(4096, device="cuda")
    assert fn(x.data_ptr(), 0, None, out.data_ptr(), 4096, stream) == 0
    torch.cuda.synchronize()
    assert float(out) == 4096.0
    assert fn(x.data_ptr(), 0, None, out.data_ptr(), (1 << 32) + 1, stream) == -2
    assert fn(None, 0, None, out.data_ptr(), 16, stream) == -1
