"""GPU parity tests of the fused fully connected layer (b200_linear) against the CPU restatement of
the reference's MNIST layers: fullyConnectedForwardKernel + reluActivationKernel
(MNIST/mnist_kernels.cu:78-102, MNIST/mnist_cnn_kernels.cu:136-149) and the two layers of
MNIST/mnist_nn.cu:10-48.  Sizes are the reference's: 784 -> 512 -> 10 (mnist_nn.h:12-14) and
2048 -> 1024 -> 10 (mnist_cnn.h:55-56), on batches small enough for the CPU loop.

* fp32, FFMA mode: bit-exact (same fused multiply-adds in the same order, either bias order)
* fp32, 3xTF32: relative Frobenius error <= 1e-5;  single-pass TF32: <= 2e-3
* fp16: <= 2e-3;  bf16: <= 1e-2 (against the fp32 sums of the 16-bit inputs)
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def rel_fro(got, want):
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    return float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30))


def dev(x, device):
    import torch

    return torch.from_numpy(np.ascontiguousarray(x)).to(device)


# (batch, in, out, weights stored [out, in]?, bias first?, relu?)
REFERENCE_LAYERS = [
    (257, 784, 512, False, True, True),     # mnist_nn.cu hidden layer + ReLU
    (257, 512, 10, False, True, False),     # mnist_nn.cu output layer (rows of W are 40 bytes)
    (100, 2048, 1024, True, False, True),   # mnist_kernels.cu FC + ReLU
    (100, 2048, 1024, True, True, True),    # mnist_cnn_kernels.cu FC (sum starts from the bias)
    (33, 1024, 10, True, False, False),     # output layer of the CNN
    (1, 7, 3, True, False, True),
]


@pytest.mark.parametrize("layer", REFERENCE_LAYERS)
def test_linear_fp32_ffma_reproduces_the_reference_loops_bit_for_bit(cb, oracle, device, layer):
    batch, in_f, out_f, out_in, bias_first, relu = layer
    rng = np.random.default_rng(batch * 7 + in_f + out_f)
    x = rng.uniform(-1, 1, (batch, in_f)).astype(np.float32)
    w = (rng.standard_normal((out_f, in_f) if out_in else (in_f, out_f)) * 0.05).astype(np.float32)
    b = rng.uniform(-0.5, 0.5, out_f).astype(np.float32)
    want = oracle.linear_f32(x, w, b, out_in, relu, bias_first, fused=True)
    got = cb.linear(dev(x, device), dev(w, device), dev(b, device), cb.ROW_MAJOR_BT if out_in else cb.ROW_MAJOR,
                    relu=relu, bias_first=bias_first, mode=cb.F32_FFMA)
    cb.check_device()
    assert np.array_equal(got.cpu().numpy(), want)
    if relu:
        assert (got >= 0).all() and (got == 0).any()
    # without a bias the layer is the plain product (then ReLU)
    got0 = cb.linear(dev(x, device), dev(w, device), None, cb.ROW_MAJOR_BT if out_in else cb.ROW_MAJOR, relu=relu)
    assert np.array_equal(got0.cpu().numpy(), oracle.linear_f32(x, w, None, out_in, relu, False, fused=True))


@pytest.fixture
def tile_policy(cb):
    yield cb.set_tile_policy
    cb.set_tile_policy(0, 0, 0)


@pytest.mark.parametrize("tiles", [(0, 0), (4, 256)])  # automatic; CTA pairs with two row blocks (eight-warp epilogue)
@pytest.mark.parametrize("out_in", [True, False])
@pytest.mark.parametrize("shape", [(257, 784, 512), (100, 2048, 1024), (520, 1032, 264)])
def test_linear_tensor_core_modes_within_tolerance(cb, oracle, device, tile_policy, shape, out_in, tiles):
    import torch

    tile_policy(tiles[0], tiles[1], 0)
    batch, in_f, out_f = shape
    rng = np.random.default_rng(in_f + out_f + int(out_in))
    x = rng.standard_normal((batch, in_f)).astype(np.float32)
    w = (rng.standard_normal((out_f, in_f) if out_in else (in_f, out_f)) * 0.05).astype(np.float32)
    b = rng.uniform(-0.5, 0.5, out_f).astype(np.float32)
    layout = cb.ROW_MAJOR_BT if out_in else cb.ROW_MAJOR
    want = oracle.linear_f32(x, w, b, out_in, True, False, fused=False)
    for mode, tol in ((cb.F32_3XTF32, 1e-5), (cb.F32_TF32, 2e-3)):
        got = cb.linear(dev(x, device), dev(w, device), dev(b, device), layout, relu=True, mode=mode)
        cb.check_device()
        assert rel_fro(got.cpu().numpy(), want) <= tol, mode
        assert (got >= 0).all()
    for is_bf16, tol in ((True, 1e-2), (False, 2e-3)):
        if is_bf16:
            xb, wb, dt = oracle.f32_to_bf16_bits(x), oracle.f32_to_bf16_bits(w), torch.bfloat16
        else:
            xb, wb, dt = x.astype(np.float16).view(np.uint16), w.astype(np.float16).view(np.uint16), torch.float16
        _, want32 = oracle.linear_h16(xb, wb, b, is_bf16, out_in, relu=True)
        got = cb.linear(dev(xb.view(np.int16), device).view(dt), dev(wb.view(np.int16), device).view(dt),
                        dev(b, device), layout, relu=True)
        cb.check_device()
        assert rel_fro(got.float().cpu().numpy(), want32) <= tol, is_bf16
        # bias only, no activation: negative outputs survive
        _, lin32 = oracle.linear_h16(xb, wb, b, is_bf16, out_in, relu=False)
        got = cb.linear(dev(xb.view(np.int16), device).view(dt), dev(wb.view(np.int16), device).view(dt),
                        dev(b, device), layout, relu=False)
        assert rel_fro(got.float().cpu().numpy(), lin32) <= tol, is_bf16
        assert (got < 0).any()


def test_linear_equals_product_then_bias_then_relu_as_separate_steps(cb, device):
    """The fused layer against the unfused sequence on the device (GEMM entry point, then torch for
    bias and ReLU): identical bits for fp32 FFMA with the bias added last, and for bf16."""
    import torch

    g = torch.Generator(device=device).manual_seed(5)
    x = torch.randn((300, 1024), device=device, generator=g)
    w = torch.randn((640, 1024), device=device, generator=g) * 0.05
    b = torch.rand(640, device=device, generator=g) - 0.5
    from cudaintro_b200 import capi

    fused = cb.linear(x, w, b, cb.ROW_MAJOR_BT, relu=True)
    capi.lib.b200_set_ffma_k_ranges(0)  # the layer keeps one ascending sum per output; make the plain product do so too
    try:
        steps = torch.relu(cb.gemm_f32(x, w, cb.ROW_MAJOR_BT, mode=cb.F32_FFMA) + b)
    finally:
        capi.lib.b200_set_ffma_k_ranges(-1)
    assert torch.equal(fused, steps)
    xb, wb = x.bfloat16(), w.bfloat16()
    fused = cb.linear(xb, wb, b, cb.ROW_MAJOR_BT, relu=True)
    sums = cb.gemm_naive(xb, wb, cb.ROW_MAJOR_BT)  # unrounded fp32 sums, k ascending
    steps = torch.relu(sums + b).bfloat16()
    assert float((fused.float() - steps.float()).norm() / steps.float().norm()) <= 4e-3
    cb.check_device()


def test_linear_refuses_what_it_cannot_do(cb, device):
    import torch
    from cudaintro_b200 import capi

    x = torch.zeros((4, 16), device=device)
    w = torch.zeros((8, 16), device=device)
    y = torch.zeros((4, 8), device=device)
    lib = capi.lib
    args = (x.data_ptr(), w.data_ptr(), 0, y.data_ptr(), 4, 16, 8)
    assert lib.b200_linear(capi.F32, *args, cb.COL_MAJOR_NN, 0, 0, None) == 1
    assert lib.b200_linear(capi.F32, *args, cb.ROW_MAJOR_BT, 4, 0, None) == 1      # unknown flag
    assert lib.b200_linear(capi.I8, *args, cb.ROW_MAJOR_BT, 0, 0, None) == 1       # integer layer
    assert lib.b200_linear(capi.F32, *args, cb.ROW_MAJOR_BT, 0, 9, None) == 1      # unknown fp32 mode
    assert lib.b200_linear(capi.F32, x.data_ptr(), w.data_ptr(), 0, y.data_ptr(), 0, 16, 8, cb.ROW_MAJOR_BT, 0, 0,
                           None) == 1
    # the [in, out] = [512, 10] output layer has 40-byte rows: fine for FFMA, refused by the tensor cores
    w10 = torch.zeros((512, 10), device=device)
    x512 = torch.zeros((4, 512), device=device)
    y10 = torch.zeros((4, 10), device=device)
    assert lib.b200_linear(capi.F32, x512.data_ptr(), w10.data_ptr(), 0, y10.data_ptr(), 4, 512, 10, cb.ROW_MAJOR, 0,
                           cb.F32_FFMA, None) == 0
    assert lib.b200_linear(capi.F32, x512.data_ptr(), w10.data_ptr(), 0, y10.data_ptr(), 4, 512, 10, cb.ROW_MAJOR, 0,
                           cb.F32_TF32, None) == 2
    torch.cuda.synchronize()
