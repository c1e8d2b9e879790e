"""The allocation-free 3xTF32 entry point, for hosts that forbid plug-ins to allocate device memory
(all of it belongs to the host's own pool) or that cannot afford the device-wide synchronisation
hidden in cudaMalloc / cudaFree inside a latency-bound loop.

`b200_gemm_f32_3xtf32_static` keeps its split operands in a fixed array inside the library
instead of a cudaMalloc'ed workspace.  It is called here through the C ABI, twice in a row on
different problems (the second one smaller, so stale contents of the shared array would show),
and must agree with the allocating entry point `b200_gemm_f32(..., B200_F32_3XTF32)`.

This file is named so that pytest collects it last.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

TOL_F32 = 1e-5  # relative Frobenius error, the tolerance of the fp32 tests


def rel_fro(got, want):
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    return float(np.linalg.norm(got - want) / np.linalg.norm(want))


def call_static(capi, a, b, out, M, N, K, layout):
    import torch

    st = capi.lib.b200_gemm_f32_3xtf32_static(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, 0, 0, 0, layout,
                                              C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert st == 0, capi.lib.b200_last_error().decode()


def test_static_scratch_entry_point_matches_allocating_one(cb, oracle, device):
    import torch

    from cudaintro_b200 import capi

    g = torch.Generator(device=device).manual_seed(2024)
    # two calls in a row: a larger row-major problem, then a smaller column-major one
    for (M, N, K, layout) in ((640, 520, 1001, cb.ROW_MAJOR), (136, 72, 333, cb.COL_MAJOR_NN)):
        if layout == cb.ROW_MAJOR:
            a = torch.rand((M, K), device=device, generator=g) * 2 - 1
            b = torch.rand((K, N), device=device, generator=g) * 2 - 1
            out = torch.full((M, N), float("nan"), device=device)
        else:  # column-major storage: A is [K, M], B is [N, K], C is [N, M]
            a = torch.rand((K, M), device=device, generator=g) * 2 - 1
            b = torch.rand((N, K), device=device, generator=g) * 2 - 1
            out = torch.full((N, M), float("nan"), device=device)
        call_static(capi, a, b, out, M, N, K, layout)
        cb.check_device()
        want = cb.gemm_f32(a, b, layout, mode=cb.F32_3XTF32)
        cb.check_device()
        assert rel_fro(out.cpu().numpy(), want.cpu().numpy()) <= TOL_F32
        # and both sit within the stated tolerance of the fp64-accumulated product
        truth = oracle.gemm_f32(a.cpu().numpy(), b.cpu().numpy(), M, N, K, layout, acc64=True)
        assert rel_fro(out.cpu().numpy(), truth) <= TOL_F32


def test_static_scratch_entry_point_takes_no_device_memory_after_its_first_call(cb, device):
    """After one warm-up call on the device (which loads the library's code and the 32 MiB array
    with it), further calls must leave the amount of free device memory exactly where it was:
    nothing on their path allocates, not even from a pool.  Operands and results are created
    before the measurement; the calls go through the C ABI only."""
    import torch

    from cudaintro_b200 import capi

    M, N, K = 384, 264, 520
    g = torch.Generator(device=device).manual_seed(7)
    a = torch.rand((M, K), device=device, generator=g)
    b = torch.rand((K, N), device=device, generator=g)
    out = torch.empty((M, N), device=device)
    call_static(capi, a, b, out, M, N, K, cb.ROW_MAJOR)  # first call: set-up
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info(device)
    for _ in range(5):
        call_static(capi, a, b, out, M, N, K, cb.ROW_MAJOR)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info(device)
    assert free_after == free_before


def test_static_scratch_entry_point_refuses_what_does_not_fit(cb, device):
    import torch

    from cudaintro_b200 import capi

    t = torch.zeros(16, device=device)
    # 4096 x 4096 x 4096 needs 64 Mi floats of split planes, the built-in array holds 8 Mi
    st = capi.lib.b200_gemm_f32_3xtf32_static(t.data_ptr(), t.data_ptr(), t.data_ptr(), 4096, 4096, 4096, 0, 0, 0,
                                              cb.ROW_MAJOR, None)
    assert st == 5
    assert b"built-in scratch" in capi.lib.b200_last_error()
