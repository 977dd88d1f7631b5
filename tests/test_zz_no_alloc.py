"""The matrix product that allocates nothing (zinfer_b200/csrc/gemm_static_scratch.h).

Some users of the kernel library cannot call cudaMalloc: a plug-in invoked while
its host application captures a CUDA graph, a real-time loop that forbids
allocation, a C program that links the library without torch (which otherwise
hands the split-K workspace to the kernel).  For them the library exports
``zi_gemm_tcgen05_static_scratch``: the same tensor-core product, with its split-K
partial sums in a fixed 8 MiB array inside the library's device image.

This test calls that function through its exported C symbol, as such a user would,
twice in a row with different shapes (the second, smaller product must not be
disturbed by what the first left in the shared array), and compares each result
with the ordinary entry point's.  It also checks that the calls leave the amount of
free device memory unchanged (they allocate nothing), that the library's own status
word can be read by a caller who passes none, and that an oversized product is
refused with a clear message instead of overrunning the array.  The file sorts
last, so a run that stops at the first failure has run every other test before it.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _call(lib, x, w, out, status=None):
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    M, K = x.shape
    N = w.shape[0]
    return lib.zi_gemm_tcgen05_static_scratch(
        ctypes.c_void_p(out.data_ptr()), 1 if out.dtype == torch.bfloat16 else 0, ctypes.c_void_p(x.data_ptr()),
        ctypes.c_void_p(w.data_ptr()), M, N, K, x.stride(0), w.stride(0), out.stride(0), sms,
        ctypes.c_void_p(status.data_ptr() if status is not None else 0),
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


def test_static_scratch_product_matches_the_ordinary_entry_point():
    from zinfer_b200 import ops

    lib = ops.lib()
    lib.zi_gemm_static_scratch_capacity_bytes.restype = ctypes.c_longlong
    assert lib.zi_gemm_static_scratch_capacity_bytes() == 8 * 1024 * 1024
    g = torch.Generator().manual_seed(7)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    # two calls in a row: both split K (8 tokens x 12288 and 3 tokens x 4096), different sizes of partial sums
    for M, N, K, odt in ((8, 4096, 12288, torch.bfloat16), (3, 1024, 4096, torch.float32)):
        x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
        w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
        plan = (ctypes.c_int * 3)()
        need = lib.zi_gemm_tcgen05_plan(M, N, K, torch.cuda.get_device_properties(0).multi_processor_count, plan)
        assert plan[2] > 1 and need > 0, "the case is meant to use the scratch"
        want = ops.linear(x, w, out_dtype=odt)                 # the existing entry point, workspace from torch
        out = torch.full((M, N), float("nan"), dtype=odt, device=DEV)
        rc = _call(lib, x, w, out, status)
        assert rc == 0, lib.zi_last_error().decode()
        torch.cuda.synchronize()
        assert int(status.item()) == 0, "a bounded wait inside the kernel ran out"
        # same kernels, same split, same order of additions: the results agree to the last bit
        tol = dict(rtol=1.6e-2, atol=1e-3) if odt == torch.bfloat16 else dict(rtol=2e-5, atol=2e-6)
        torch.testing.assert_close(out.float(), want.float(), **tol)
        ref = x.float() @ w.float().T
        torch.testing.assert_close(out.float(), ref, rtol=1.6e-2, atol=2e-2)
    # without a status word of the caller's, the library's own is used, and can be read
    out2 = torch.empty((M, N), dtype=odt, device=DEV)
    out3 = torch.empty((M, N), dtype=odt, device=DEV)
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    assert _call(lib, x, w, out2) == 0
    assert _call(lib, x, w, out3) == 0
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, "the entry point that allocates nothing changed the free device memory"
    assert lib.zi_gemm_static_scratch_status() == 0
    assert torch.equal(out2, out) and torch.equal(out3, out)


def test_static_scratch_refuses_what_does_not_fit():
    from zinfer_b200 import ops

    lib = ops.lib()
    M, N, K = 64, 8320, 16384           # 4 splits x 64 x 8320 x 4 bytes > 8 MiB
    plan = (ctypes.c_int * 3)()
    need = lib.zi_gemm_tcgen05_plan(M, N, K, torch.cuda.get_device_properties(0).multi_processor_count, plan)
    if need <= 8 * 1024 * 1024:
        pytest.skip("this GPU's plan does not split the product far enough to exceed the scratch")
    x = torch.zeros(M, K, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(N, K, dtype=torch.bfloat16, device=DEV)
    out = torch.zeros(M, N, dtype=torch.bfloat16, device=DEV)
    assert _call(lib, x, w, out) == -1
    msg = lib.zi_last_error().decode()
    assert "scratch" in msg and str(need) in msg
