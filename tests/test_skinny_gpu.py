"""GPU parity tests of the K-split cluster kernel for skinny products (at most 128 rows of A): forced
through tile policy 3 at every tile width, both layouts of B, ragged N and K, then as chosen
automatically for the decode-shape linear layer.  int8 -> int32 and W8A8 -> bf16 are bit-exact (which
checks the exchange of partial sums between the CTAs of a cluster to the last bit); fp16 <= 2e-3 and
bf16 <= 1e-2 relative Frobenius error against the unrounded fp32 sums of the one-thread-per-element kernel."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture
def policy(cb):
    yield cb.set_tile_policy
    cb.set_tile_policy(0, 0, 0)


def rel(a, b):
    return float((a.float() - b.float()).norm() / b.float().norm())


SHAPES = [(16, 11008, 4096), (1, 4096, 4096), (32, 1000, 2176), (7, 264, 64), (32, 520, 200), (5, 1004, 512),
          (31, 37000, 256), (16, 2048, 16384), (33, 1000, 2176), (64, 4096, 4096), (100, 11008, 1024),
          (128, 11008, 4096), (128, 520, 200), (96, 1004, 512)]


@pytest.mark.parametrize("bn", [0, 128, 192, 256])
@pytest.mark.parametrize("b_is_nk", [False, True])
@pytest.mark.parametrize("shape", SHAPES)
def test_skinny_kernel_forced(cb, device, policy, shape, b_is_nk, bn):
    import torch
    from cudaintro_b200 import capi

    M, N, K = shape
    if not b_is_nk and N % 8:
        pytest.skip("rows of an [K, N] matrix must be 16-byte multiples")
    layout = cb.ROW_MAJOR_BT if b_is_nk else cb.ROW_MAJOR
    g = torch.Generator(device=device).manual_seed(M * 31 + N + K + bn)
    for dt, fn, tol in ((torch.float16, cb.gemm_f16, 2e-3), (torch.bfloat16, cb.gemm_bf16, 1e-2)):
        a = torch.randn((M, K), device=device, generator=g).to(dt)
        b = (torch.randn((N, K) if b_is_nk else (K, N), device=device, generator=g) * 0.05).to(dt)
        ref = cb.gemm_naive(a, b, layout)
        policy(3, bn, 0)
        if N > 148 * (bn or 256):  # more tiles than SMs at this width: refused, not silently rerouted
            c = torch.empty((M, N), dtype=dt, device=device)
            st = capi.lib.b200_gemm_f16(a.data_ptr(), b.data_ptr(), c.data_ptr(), M, N, K, 0, 0, 0, layout, None)
            assert st == 2
            continue
        if M > 64 and bn == 256:  # 256 columns x 96 or 128 rows of exchange area leave no room for a ring
            c = torch.empty((M, N), dtype=dt, device=device)
            st = capi.lib.b200_gemm_f16(a.data_ptr(), b.data_ptr(), c.data_ptr(), M, N, K, 0, 0, 0, layout, None)
            assert st == 2
            continue
        c1 = fn(a, b, layout)
        c2 = fn(a, b, layout)
        cb.check_device()
        assert torch.equal(c1.view(torch.int16), c2.view(torch.int16))  # ranges are added in a fixed order
        assert rel(c1, ref) <= tol, (dt, rel(c1, ref))
        policy(1, 128, 0)
        general = fn(a, b, layout)
        cb.check_device()
        assert rel(c1, general) <= tol / 2


@pytest.mark.parametrize("bn", [0, 128, 192, 256])
@pytest.mark.parametrize("b_is_nk", [False, True])
@pytest.mark.parametrize("shape", [(16, 11008, 4096), (1, 4096, 4096), (32, 1008, 2176), (7, 272, 128), (33, 1040, 8192),
                                   (64, 4096, 4096), (128, 11008, 1024), (128, 528, 208), (96, 1004, 512)])
def test_skinny_kernel_forced_int8_and_w8a8_bit_exact(cb, device, policy, shape, b_is_nk, bn):
    import torch
    from cudaintro_b200 import capi

    M, N, K = shape
    if not b_is_nk and N % 16:
        pytest.skip("rows of an int8 [K, N] matrix must be 16-byte multiples")
    layout = cb.ROW_MAJOR_BT if b_is_nk else cb.ROW_MAJOR
    g = torch.Generator(device=device).manual_seed(M * 17 + N + K + bn)
    a = torch.randint(-127, 128, (M, K), dtype=torch.int8, device=device, generator=g)
    b = torch.randint(-127, 128, (N, K) if b_is_nk else (K, N), dtype=torch.int8, device=device, generator=g)
    want = cb.gemm_naive(a, b, layout)
    policy(3, bn, 0)
    feasible = not (M > 64 and bn == 256) and not (not b_is_nk and bn == 192)  # int8 spans of N are 128 columns wide
    if not feasible:
        c = torch.empty((M, N), dtype=torch.int32, device=device)
        assert capi.lib.b200_gemm_i8_i32(a.data_ptr(), b.data_ptr(), c.data_ptr(), M, N, K, 0, 0, 0, layout, None) == 2
        return
    for _ in range(2):
        c = cb.gemm_i8_i32(a, b, layout)
        cb.check_device()
        assert torch.equal(c, want)
    if not b_is_nk:
        rs = torch.rand(M, device=device, generator=g) * 0.01 + 0.001
        cs = torch.rand(N, device=device, generator=g) * 0.01 + 0.001
        cw = cb.gemm_w8a8_bf16(a, b, rs, cs)
        cb.check_device()
        want_w = ((want.float() * rs[:, None]) * cs[None, :]).to(torch.bfloat16)
        assert torch.equal(cw.view(torch.int16), want_w.view(torch.int16))


def test_skinny_kernel_refuses_what_it_was_not_built_for(cb, device, policy):
    import torch
    from cudaintro_b200 import capi

    policy(3, 0, 0)
    a = torch.zeros((129, 256), dtype=torch.float16, device=device)
    b = torch.zeros((256, 512), dtype=torch.float16, device=device)
    c = torch.zeros((129, 512), dtype=torch.float16, device=device)
    lib = capi.lib
    assert lib.b200_gemm_f16(a.data_ptr(), b.data_ptr(), c.data_ptr(), 129, 512, 256, 0, 0, 0, 0, None) == 2
    a32 = torch.zeros((16, 256), dtype=torch.float32, device=device)
    b32 = torch.zeros((256, 512), dtype=torch.float32, device=device)
    c32 = torch.zeros((16, 512), dtype=torch.float32, device=device)
    args32 = (a32.data_ptr(), b32.data_ptr(), c32.data_ptr(), 16, 512, 256, 0, 0, 0, 0, cb.F32_TF32, None)
    assert lib.b200_gemm_f32(*args32) == 2  # no tf32 variant of the skinny kernel
    policy(0, 0, 0)
    assert lib.b200_gemm_f32(*args32) == 0
    torch.cuda.synchronize()


@pytest.mark.parametrize("M", [1, 16, 32, 64])
def test_decode_shape_linear_layer_takes_the_skinny_kernel_by_itself(cb, oracle, device, policy, M):
    """[4096 -> 11008] on a decode batch with nothing forced: the result must be the forced kernel's,
    bit for bit (the general kernel sums K in one piece and rounds differently somewhere in 11008 x M
    outputs), with and without the bias / ReLU tail, which is checked against the CPU oracle."""
    import torch

    K, N = 4096, 11008
    g = torch.Generator(device=device).manual_seed(90 + M)
    x = torch.randn((M, K), device=device, generator=g).to(torch.float16)
    w = (torch.randn((K, N), device=device, generator=g) * 0.02).to(torch.float16)
    bias = torch.rand(N, device=device, generator=g) - 0.5
    auto = cb.gemm_f16(x, w)
    policy(3, 0, 0)
    forced = cb.gemm_f16(x, w)
    policy(1, 128, 0)
    general = cb.gemm_f16(x, w)
    policy(0, 0, 0)
    cb.check_device()
    assert torch.equal(auto.view(torch.int16), forced.view(torch.int16))
    assert rel(auto, general) <= 1e-3
    y = cb.linear(x, w, bias, cb.ROW_MAJOR, relu=True)
    cb.check_device()
    _, want32 = oracle.linear_h16(x.view(torch.int16).cpu().numpy().view(np.uint16),
                                  w.view(torch.int16).cpu().numpy().view(np.uint16), bias.cpu().numpy(), False,
                                  w_is_out_in=False, relu=True)
    got = y.float().cpu().numpy()
    assert float(np.linalg.norm(got - want32) / np.linalg.norm(want32)) <= 2e-3
    assert (got >= 0).all() and (got == 0).any()
