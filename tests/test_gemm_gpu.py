"""GPU parity tests: every case calls the CUDA kernels through the C ABI (ctypes) and checks the
result against the CPU oracle, the golden fixtures written by the reference's own matrixMulCPU,
or a size-independent property.  Tolerances are the stated ones:

* int8 -> int32 and W8A8 -> bf16 : bit-exact
* bf16  : relative Frobenius error <= 1e-2 against the fp32 reference sums
* fp16  : <= 2e-3
* fp32  : <= 1e-5 against the fp64-accumulated reference (both FFMA and 3xTF32)
"""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

TOL_BF16 = 1e-2
TOL_F16 = 2e-3
TOL_F32 = 1e-5


def golden(name):
    return np.load(os.path.join(GOLDEN, name))


def to_dev(x, device, dtype=None):
    import torch

    t = torch.from_numpy(np.ascontiguousarray(x)).to(device)
    return t.view(dtype) if dtype is not None else t


def rel_fro(got, want):
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    return float(np.linalg.norm(got - want) / np.linalg.norm(want))


def storage_shapes(cb, M, N, K, layout):
    if layout == cb.ROW_MAJOR:
        return (M, K), (K, N)
    if layout == cb.ROW_MAJOR_BT:
        return (M, K), (N, K)
    return (K, M), (N, K)


def oracle_i8(oracle, cb, a, b, M, N, K, layout, rows=None):
    """Oracle result in the storage shape of the layout ([N,M] for column-major)."""
    if layout == cb.ROW_MAJOR_BT:
        return oracle.gemm_i8_i32(a, np.ascontiguousarray(b.T), M, N, K, oracle.ROW_MAJOR, rows)
    return oracle.gemm_i8_i32(a, b, M, N, K, layout, rows)


# ------------------------------------------------------------------ fills (suite generators)

def test_device_fills_match_oracle_bit_for_bit(cb, oracle, device):
    import torch

    n = 1 << 18
    t = cb.fill(torch.empty(n, dtype=torch.int8, device=device), 0x4234)
    assert np.array_equal(t.cpu().numpy(), oracle.fill_int8(n, 0x4234))
    t = cb.fill(torch.empty(n, dtype=torch.float32, device=device), 0x3234)
    assert np.array_equal(t.cpu().numpy().view(np.uint32), oracle.fill_f32(n, 0x3234).view(np.uint32))
    t = cb.fill(torch.empty(n, dtype=torch.float16, device=device), 0x2234)
    assert np.array_equal(t.view(torch.int16).cpu().numpy().view(np.uint16), oracle.fill_f16(n, 0x2234))
    t = cb.fill(torch.empty(n, dtype=torch.bfloat16, device=device), 0x1234)
    assert np.array_equal(t.view(torch.int16).cpu().numpy().view(np.uint16), oracle.fill_bf16(n, 0x1234))


# ------------------------------------------------------------------ int8 -> int32

@pytest.mark.parametrize("name", ["ref_i8_128.npz", "ref_i8_suitefill_64.npz"])
def test_int8_against_reference_fixture(cb, device, name):
    g = golden(name)
    c = cb.gemm_i8_i32(to_dev(g["a"], device), to_dev(g["b"], device))
    cb.check_device()
    assert np.array_equal(c.cpu().numpy(), g["c"])


I8_SHAPES = [(128, 128, 128), (256, 512, 1024), (208, 336, 1008), (1, 16, 16), (129, 144, 48), (16, 4096, 64),
             (384, 272, 4112)]


@pytest.mark.parametrize("layout_name", ["ROW_MAJOR", "COL_MAJOR_NN", "ROW_MAJOR_BT"])
@pytest.mark.parametrize("shape", I8_SHAPES)
def test_int8_bit_exact_vs_oracle(cb, oracle, device, shape, layout_name):
    layout = getattr(cb, layout_name)
    M, N, K = shape
    if layout == cb.COL_MAJOR_NN and M % 16:
        M = (M + 15) // 16 * 16  # column-major needs lda = M in whole 16-byte rows
    rng = np.random.default_rng(hash((M, N, K, layout)) & 0xFFFF)
    sa, sb = storage_shapes(cb, M, N, K, layout)
    a = rng.integers(-127, 128, sa).astype(np.int8)
    b = rng.integers(-127, 128, sb).astype(np.int8)
    c = cb.gemm_i8_i32(to_dev(a, device), to_dev(b, device), layout)
    cb.check_device()
    assert np.array_equal(c.cpu().numpy(), oracle_i8(oracle, cb, a, b, M, N, K, layout))


def test_int8_extreme_values_full_k(cb, device):
    import torch

    K = 8192
    a = torch.full((128, K), -127, dtype=torch.int8, device=device)
    b = torch.full((K, 256), -127, dtype=torch.int8, device=device)
    c = cb.gemm_i8_i32(a, b)
    assert int(c.min()) == int(c.max()) == K * 127 * 127


def test_int8_config_4096_suite_fill_column_major(cb, oracle, device):
    """The suite's own int8 problem (quantization/GEMM_int8.cu:21-56): 4096^3, hash fill, column-major NN.
    Sampled rows against the oracle, the whole matrix against the one-thread-per-element kernel."""
    import torch

    n = 4096
    a = cb.fill(torch.empty((n, n), dtype=torch.int8, device=device), 0x4234)
    b = cb.fill(torch.empty((n, n), dtype=torch.int8, device=device), 0x6676)
    c = cb.gemm_i8_i32(a, b, cb.COL_MAJOR_NN)
    cb.check_device()
    full = cb.gemm_naive(a, b, cb.COL_MAJOR_NN)
    assert torch.equal(c, full)
    rows = [0, 1, 127, 128, 2047, 4095] + list(range(1000, 1016))
    want = oracle.gemm_i8_i32(oracle.fill_int8(n * n, 0x4234), oracle.fill_int8(n * n, 0x6676), n, n, n,
                              oracle.COL_MAJOR_NN, rows)
    got = c.cpu().numpy().T[rows]  # storage is [N, M]; row m of C is column m of the storage
    assert np.array_equal(got, want)


def test_int8_config_4096_row_major_uniform(cb, oracle, device):
    """int8 4096^3 row-major, i.i.d. uniform integers in [-127, 127]; also cross-checked against
    the vendor library's int8 GEMM (a second opinion: exact integer arithmetic must agree)."""
    import torch

    n = 4096
    g = torch.Generator(device=device).manual_seed(42)
    a = torch.randint(-127, 128, (n, n), dtype=torch.int8, device=device, generator=g)
    b = torch.randint(-127, 128, (n, n), dtype=torch.int8, device=device, generator=g)
    c = cb.gemm_i8_i32(a, b)
    c2 = cb.gemm_i8_i32(a, b)  # a pipeline with a race is rarely reproducible
    cb.check_device()
    assert torch.equal(c, c2)
    rows = [0, 127, 128, 4095] + list(range(2040, 2060))
    want = oracle.gemm_i8_i32(a.cpu().numpy(), b.cpu().numpy(), n, n, n, oracle.ROW_MAJOR, rows)
    assert np.array_equal(c[rows].cpu().numpy(), want)
    assert torch.equal(c, cb.gemm_naive(a, b))
    try:
        lib_c = torch._int_mm(a, b)
    except Exception:  # not every torch build exposes it
        lib_c = None
    if lib_c is not None:
        assert torch.equal(c, lib_c)


def test_int8_8192_checksums_and_linearity(cb, device):
    """Full-size properties at 8192^3: column sums of C equal (column sums of A) * B, and the
    product is linear in B: A*(B1+B2) = A*B1 + A*B2 exactly."""
    import torch

    n = 8192
    g = torch.Generator(device=device).manual_seed(7)
    a = torch.randint(-127, 128, (n, n), dtype=torch.int8, device=device, generator=g)
    b1 = torch.randint(-63, 64, (n, n), dtype=torch.int8, device=device, generator=g)
    b2 = torch.randint(-63, 64, (n, n), dtype=torch.int8, device=device, generator=g)
    c1 = cb.gemm_i8_i32(a, b1)
    c2 = cb.gemm_i8_i32(a, b2)
    c12 = cb.gemm_i8_i32(a, b1 + b2)
    cb.check_device()
    assert torch.equal(c12, c1 + c2)
    col_sum_a = a.sum(dim=0, dtype=torch.int64).double()        # [K], exact in fp64
    want = col_sum_a @ b1.double()                               # [N], |value| < 2^53
    assert torch.equal(c1.sum(dim=0, dtype=torch.int64).double(), want)
    row_sum_b = b1.sum(dim=1, dtype=torch.int64).double()
    assert torch.equal(c1.sum(dim=1, dtype=torch.int64).double(), a.double() @ row_sum_b)


def test_int8_8192_sampled_rows_vs_oracle(cb, oracle, device):
    """int8 8192^3 (the shape the int8 metric is quoted on), uniform [-127, 127]: rows from the first,
    an inner and the last tile rows of C, bit for bit against the oracle; the first 512 rows against
    the one-thread-per-element kernel."""
    import torch

    n = 8192
    g = torch.Generator(device=device).manual_seed(11)
    a = torch.randint(-127, 128, (n, n), dtype=torch.int8, device=device, generator=g)
    b = torch.randint(-127, 128, (n, n), dtype=torch.int8, device=device, generator=g)
    c = cb.gemm_i8_i32(a, b)
    cb.check_device()
    rows = [0, 1, 127, 128, 255, 256, 4095, 4096, 6001, 8063, 8064, 8191]
    want = oracle.gemm_i8_i32(a.cpu().numpy(), b.cpu().numpy(), n, n, n, oracle.ROW_MAJOR, rows)
    assert np.array_equal(c[rows].cpu().numpy(), want)
    assert torch.equal(c[:512], cb.gemm_naive(a[:512], b))


def test_fp16_8192_normal_inputs_sampled_rows_vs_oracle(cb, oracle, device):
    """fp16 8192^3 (the shape the fp16 metric is quoted on), N(0,1) inputs, fp32 accumulate, fp16 out:
    relative Frobenius error <= 2e-3 against the oracle's fp32 sums on sampled rows, the first 1024
    rows against the validation kernel, and two runs bit-identical."""
    import torch

    n = 8192
    g = torch.Generator(device=device).manual_seed(12)
    a = torch.randn((n, n), device=device, generator=g).to(torch.float16)
    b = torch.randn((n, n), device=device, generator=g).to(torch.float16)
    c = cb.gemm_f16(a, b)
    c2 = cb.gemm_f16(a, b)
    cb.check_device()
    assert torch.equal(c.view(torch.int16), c2.view(torch.int16))
    rows = [0, 127, 128, 255, 256, 4097, 8064, 8191] + list(range(5000, 5008))
    _, o32 = oracle.gemm_h16(a.view(torch.int16).cpu().numpy().view(np.uint16),
                             b.view(torch.int16).cpu().numpy().view(np.uint16), n, n, n, False, oracle.ROW_MAJOR, rows)
    assert rel_fro(c[rows].float().cpu().numpy(), o32) <= TOL_F16
    ref = cb.gemm_naive(a[:1024], b)
    assert float((c[:1024].float() - ref).norm() / ref.norm()) <= TOL_F16


def test_padding_of_c_is_left_untouched(cb, device):
    """ldc > N: the columns between N and ldc (and rows past M) must keep their canary value."""
    import torch
    from cudaintro_b200 import capi

    M, N, K, ldc = 200, 300, 256, 320
    g = torch.Generator(device=device).manual_seed(3)
    a = torch.randint(-127, 128, (M, K), dtype=torch.int8, device=device, generator=g)
    b = torch.randint(-127, 128, (K, N), dtype=torch.int8, device=device, generator=g)
    out = torch.full((M + 8, ldc), 0x5A5A5A5A, dtype=torch.int32, device=device)
    b_pad = torch.zeros((K, 304), dtype=torch.int8, device=device)
    b_pad[:, :N] = b
    st = capi.lib.b200_gemm_i8_i32(a.data_ptr(), b_pad.data_ptr(), out.data_ptr(), M, N, K, K, 304, ldc, cb.ROW_MAJOR,
                                   None)
    assert st == 0, capi.lib.b200_last_error()
    torch.cuda.synchronize()
    assert torch.equal(out[:M, :N], (a.double() @ b.double()).to(torch.int32))
    assert bool((out[:M, N:] == 0x5A5A5A5A).all()) and bool((out[M:] == 0x5A5A5A5A).all())


def test_unaligned_leading_dimension_is_refused(cb, device):
    import torch

    a = torch.zeros((64, 100), dtype=torch.int8, device=device)
    b = torch.zeros((100, 64), dtype=torch.int8, device=device)
    with pytest.raises(cb.B200Error) as e:
        cb.gemm_i8_i32(a, b)
    assert e.value.status == 2


# ------------------------------------------------------------------ bf16 / fp16

@pytest.mark.parametrize("name,is_bf16", [("ref_bf16_96.npz", True), ("ref_f16_96.npz", False)])
def test_16bit_against_reference_fixture(cb, device, name, is_bf16):
    import torch

    g = golden(name)
    dt = torch.bfloat16 if is_bf16 else torch.float16
    fn = cb.gemm_bf16 if is_bf16 else cb.gemm_f16
    # 96 columns of 16-bit elements = 192 bytes per row: a whole number of 16-byte units
    c = fn(to_dev(g["a"].view(np.int16), device, dt), to_dev(g["b"].view(np.int16), device, dt))
    cb.check_device()
    assert rel_fro(c.float().cpu().numpy(), g["c32"]) <= (TOL_BF16 if is_bf16 else TOL_F16)


H16_SHAPES = [(128, 64, 64), (264, 520, 1000), (16, 512, 256), (1, 8, 8), (520, 264, 2056)]


@pytest.mark.parametrize("is_bf16", [True, False])
@pytest.mark.parametrize("layout_name", ["ROW_MAJOR", "COL_MAJOR_NN", "ROW_MAJOR_BT"])
@pytest.mark.parametrize("shape", H16_SHAPES)
def test_16bit_vs_oracle(cb, oracle, device, shape, layout_name, is_bf16):
    import torch

    layout = getattr(cb, layout_name)
    M, N, K = shape
    if layout == cb.COL_MAJOR_NN and M % 8:
        M = (M + 7) // 8 * 8
    rng = np.random.default_rng(hash((M, N, K, layout, is_bf16)) & 0xFFFF)
    sa, sb = storage_shapes(cb, M, N, K, layout)
    af = rng.standard_normal(sa).astype(np.float32)
    bf = rng.standard_normal(sb).astype(np.float32)
    if is_bf16:
        a, b, dt, fn = oracle.f32_to_bf16_bits(af), oracle.f32_to_bf16_bits(bf), torch.bfloat16, cb.gemm_bf16
    else:
        a, b = af.astype(np.float16).view(np.uint16), bf.astype(np.float16).view(np.uint16)
        dt, fn = torch.float16, cb.gemm_f16
    c = fn(to_dev(a.view(np.int16), device, dt), to_dev(b.view(np.int16), device, dt), layout)
    cb.check_device()
    if layout == cb.ROW_MAJOR_BT:
        o16, o32 = oracle.gemm_h16(a, np.ascontiguousarray(b.T), M, N, K, is_bf16)
    else:
        o16, o32 = oracle.gemm_h16(a, b, M, N, K, is_bf16, layout)
    got = c.float().cpu().numpy()
    assert rel_fro(got, o32) <= (TOL_BF16 if is_bf16 else TOL_F16)
    # and element-wise the rounded output is within 2 units in the last place of the oracle's
    widen = oracle.bf16_bits_to_f32 if is_bf16 else oracle.f16_bits_to_f32
    ulp = np.maximum(np.abs(o32), 1e-3) * (2.0 ** -7 if is_bf16 else 2.0 ** -10)
    assert np.all(np.abs(got - widen(o16)) <= 2 * ulp + 1e-3)


@pytest.mark.parametrize("is_bf16", [True, False])
@pytest.mark.parametrize("layout_name", ["ROW_MAJOR", "COL_MAJOR_NN", "ROW_MAJOR_BT"])
@pytest.mark.parametrize("shape", [(128, 256, 512), (200, 328, 1000), (1024, 1024, 1024), (16, 72, 64)])
def test_16bit_operands_fp32_result(cb, oracle, device, shape, layout_name, is_bf16):
    """b200_gemm_16_f32: 16-bit operands, the fp32 sums stored unrounded.  Products of two 16-bit
    floats are exact in fp32, so the result differs from the oracle's fp32 sums only by the order of
    the fp32 additions (and the tensor cores' alignment of addends): relative Frobenius error <= 2e-5."""
    import torch

    layout = getattr(cb, layout_name)
    M, N, K = shape
    if layout == cb.COL_MAJOR_NN:
        M = (M + 7) // 8 * 8
    else:
        N = (N + 7) // 8 * 8 if layout == cb.ROW_MAJOR else N
    K = (K + 7) // 8 * 8
    rng = np.random.default_rng(M * 7 + N * 3 + K + int(is_bf16))
    sa, sb = storage_shapes(cb, M, N, K, layout)
    af = rng.standard_normal(sa).astype(np.float32)
    bf = rng.standard_normal(sb).astype(np.float32)
    if is_bf16:
        a16, b16, dt = oracle.f32_to_bf16_bits(af), oracle.f32_to_bf16_bits(bf), torch.bfloat16
    else:
        a16, b16, dt = af.astype(np.float16).view(np.uint16), bf.astype(np.float16).view(np.uint16), torch.float16
    c = cb.gemm_16_f32(to_dev(a16.view(np.int16), device, dt), to_dev(b16.view(np.int16), device, dt), layout)
    cb.check_device()
    assert c.dtype == torch.float32
    if layout == cb.ROW_MAJOR_BT:
        _, o32 = oracle.gemm_h16(a16, np.ascontiguousarray(b16.T), M, N, K, is_bf16, oracle.ROW_MAJOR)
    else:
        _, o32 = oracle.gemm_h16(a16, b16, M, N, K, is_bf16, layout)
    assert rel_fro(c.cpu().numpy(), o32) <= 2e-5


def test_bf16_config_8192_normal_inputs(cb, oracle, device):
    """bf16 8192^3, N(0,1) inputs, fp32 accumulate, bf16 out; relative Frobenius error <= 1e-2
    against the fp32 reference on sampled rows; whole matrix against the validation kernel."""
    import torch

    n = 8192
    g = torch.Generator(device=device).manual_seed(1)
    a = torch.randn((n, n), device=device, generator=g).to(torch.bfloat16)
    b = torch.randn((n, n), device=device, generator=g).to(torch.bfloat16)
    c = cb.gemm_bf16(a, b)
    c2 = cb.gemm_bf16(a, b)
    cb.check_device()
    assert torch.equal(c.view(torch.int16), c2.view(torch.int16))
    rows = [0, 127, 128, 4097, 8191] + list(range(3000, 3011))
    _, o32 = oracle.gemm_h16(a.view(torch.int16).cpu().numpy().view(np.uint16),
                             b.view(torch.int16).cpu().numpy().view(np.uint16), n, n, n, True, oracle.ROW_MAJOR, rows)
    assert rel_fro(c[rows].float().cpu().numpy(), o32) <= TOL_BF16
    ref = cb.gemm_naive(a[:1024], b)  # 1024 full rows on the device
    err = (c[:1024].float() - ref).norm() / ref.norm()
    assert float(err) <= TOL_BF16


@pytest.mark.parametrize("M", [16, 128, 1024, 4096])
def test_fp16_llm_linear_sweep(cb, oracle, device, M):
    """fp16 activations [M,4096] ~ N(0,1) times weights [4096,11008] ~ N(0,0.02), fp32 accumulate,
    fp16 out (decode-to-prefill shapes)."""
    import torch

    K, N = 4096, 11008
    g = torch.Generator(device=device).manual_seed(100 + M)
    x = torch.randn((M, K), device=device, generator=g).to(torch.float16)
    w = (torch.randn((K, N), device=device, generator=g) * 0.02).to(torch.float16)
    y = cb.gemm_f16(x, w)
    cb.check_device()
    rows = sorted(set([0, M - 1, M // 2] + list(range(0, M, max(1, M // 13)))))[:16]
    _, o32 = oracle.gemm_h16(x.view(torch.int16).cpu().numpy().view(np.uint16),
                             w.view(torch.int16).cpu().numpy().view(np.uint16), M, N, K, False, oracle.ROW_MAJOR, rows)
    assert rel_fro(y[rows].float().cpu().numpy(), o32) <= TOL_F16
    full = cb.gemm_naive(x, w)
    assert float((y.float() - full).norm() / full.norm()) <= TOL_F16


# ------------------------------------------------------------------ fp32

@pytest.mark.parametrize("name", ["ref_f32_32.npz", "ref_f32_96.npz", "ref_f32_unit_64.npz"])
@pytest.mark.parametrize("mode_name", ["F32_FFMA", "F32_3XTF32"])
def test_fp32_against_reference_fixture(cb, device, name, mode_name):
    g = golden(name)
    c = cb.gemm_f32(to_dev(g["a"], device), to_dev(g["b"], device), mode=getattr(cb, mode_name))
    cb.check_device()
    assert rel_fro(c.cpu().numpy(), g["c"]) <= TOL_F32


def test_fp32_config_1024_suite_fill(cb, oracle, device):
    """fp32 1024^3 row-major, uniform[-1,1] from the suite's generator: the case the reference's
    own driver checks against matrixMulCPU (TileProgramming/kernel.cu:119-159)."""
    import torch

    n = 1024
    a = cb.fill(torch.empty((n, n), dtype=torch.float32, device=device), 0x3234)
    b = cb.fill(torch.empty((n, n), dtype=torch.float32, device=device), 0x7776)
    ah, bh = oracle.fill_f32(n * n, 0x3234).reshape(n, n), oracle.fill_f32(n * n, 0x7776).reshape(n, n)
    assert np.array_equal(a.cpu().numpy(), ah)
    cpu_loop = oracle.gemm_f32(ah, bh, n, n, n)            # == matrixMulCPU bit for bit
    truth = oracle.gemm_f32(ah, bh, n, n, n, acc64=True)
    cpu_err = rel_fro(cpu_loop, truth)
    for mode in (cb.F32_FFMA, cb.F32_3XTF32):
        c = cb.gemm_f32(a, b, mode=mode).cpu().numpy()
        cb.check_device()
        err = rel_fro(c, truth)
        assert err <= TOL_F32
        if mode == cb.F32_FFMA:
            assert err <= 2 * cpu_err  # no further from the truth than the reference loop itself
            # the reference's own check is |gpu - cpu| <= 1e-5 absolute; report how it fares
            print(f"fp32 FFMA: relfro vs fp64 {err:.2e} (cpu loop {cpu_err:.2e}); max |gpu-cpu| {np.abs(c - cpu_loop).max():.2e}")


F32_SHAPES = [(64, 64, 64), (333, 517, 1001), (1, 1, 1), (130, 70, 17), (257, 1024, 96)]


@pytest.mark.parametrize("layout_name", ["ROW_MAJOR", "COL_MAJOR_NN", "ROW_MAJOR_BT"])
@pytest.mark.parametrize("shape", F32_SHAPES)
def test_fp32_ffma_any_shape(cb, oracle, device, shape, layout_name):
    layout = getattr(cb, layout_name)
    M, N, K = shape
    rng = np.random.default_rng(hash((M, N, K, layout)) & 0xFFFF)
    sa, sb = storage_shapes(cb, M, N, K, layout)
    a = rng.uniform(-1, 1, sa).astype(np.float32)
    b = rng.uniform(-1, 1, sb).astype(np.float32)
    c = cb.gemm_f32(to_dev(a, device), to_dev(b, device), layout).cpu().numpy()
    if layout == cb.ROW_MAJOR_BT:
        truth = oracle.gemm_f32(a, np.ascontiguousarray(b.T), M, N, K, acc64=True)
    else:
        truth = oracle.gemm_f32(a, b, M, N, K, layout, acc64=True)
    assert rel_fro(c, truth) <= TOL_F32


@pytest.mark.parametrize("layout_name", ["ROW_MAJOR", "COL_MAJOR_NN", "ROW_MAJOR_BT"])
@pytest.mark.parametrize("shape", [(64, 64, 64), (333, 517, 1001), (1024, 1024, 1024), (130, 70, 17)])
def test_fp32_3xtf32_any_shape(cb, oracle, device, shape, layout_name):
    layout = getattr(cb, layout_name)
    M, N, K = shape
    rng = np.random.default_rng(hash((M, N, K, layout, 3)) & 0xFFFF)
    sa, sb = storage_shapes(cb, M, N, K, layout)
    a = rng.uniform(-1, 1, sa).astype(np.float32)
    b = rng.uniform(-1, 1, sb).astype(np.float32)
    c = cb.gemm_f32(to_dev(a, device), to_dev(b, device), layout, mode=cb.F32_3XTF32).cpu().numpy()
    cb.check_device()
    if layout == cb.ROW_MAJOR_BT:
        truth = oracle.gemm_f32(a, np.ascontiguousarray(b.T), M, N, K, acc64=True)
    else:
        truth = oracle.gemm_f32(a, b, M, N, K, layout, acc64=True)
    assert rel_fro(c, truth) <= TOL_F32


TOL_TF32 = 2e-3  # one tf32 product per term: operands cut to 10 mantissa bits


@pytest.fixture
def f32_paths(cb):
    from cudaintro_b200 import capi

    yield capi.lib.b200_set_3xtf32_path, capi.lib.b200_set_ffma_k_ranges
    capi.lib.b200_set_3xtf32_path(0)
    capi.lib.b200_set_ffma_k_ranges(-1)


@pytest.mark.parametrize("path", [1, 2])
@pytest.mark.parametrize("layout_name", ["ROW_MAJOR", "COL_MAJOR_NN", "ROW_MAJOR_BT"])
@pytest.mark.parametrize("shape", [(64, 64, 64), (332, 516, 1000), (1024, 1024, 1024), (128, 72, 36), (2048, 1100, 520)])
def test_fp32_3xtf32_both_kernels(cb, oracle, device, f32_paths, shape, layout_name, path):
    """The two 3xTF32 kernels (1 = split planes in a scratch buffer, 2 = operands split on chip),
    each forced, on aligned shapes in all layouts: relative Frobenius error <= 1e-5 against the
    fp64-accumulated product, and a second launch reproduces the first bit for bit."""
    import torch

    set_path, _ = f32_paths
    layout = getattr(cb, layout_name)
    M, N, K = shape
    rng = np.random.default_rng(M + 3 * N + 7 * K + layout)
    sa, sb = storage_shapes(cb, M, N, K, layout)
    a = rng.uniform(-1, 1, sa).astype(np.float32)
    b = rng.uniform(-1, 1, sb).astype(np.float32)
    assert set_path(path) == 0
    ad, bd = to_dev(a, device), to_dev(b, device)
    c = cb.gemm_f32(ad, bd, layout, mode=cb.F32_3XTF32)
    c2 = cb.gemm_f32(ad, bd, layout, mode=cb.F32_3XTF32)
    cb.check_device()
    assert torch.equal(c, c2)
    bt = np.ascontiguousarray(b.T) if layout == cb.ROW_MAJOR_BT else b
    truth = oracle.gemm_f32(a, bt, M, N, K, oracle.ROW_MAJOR if layout == cb.ROW_MAJOR_BT else layout, acc64=True)
    assert rel_fro(c.cpu().numpy(), truth) <= TOL_F32


@pytest.mark.parametrize("path", [1, 2])
def test_fp32_3xtf32_calls_on_two_streams_do_not_share_scratch(cb, oracle, device, f32_paths, path):
    """Two 3xTF32 products with different operands, enqueued alternately on two streams so that their
    kernels overlap on the GPU: each result must be its own product (the split-plane kernel takes its
    scratch per call from a stream-ordered pool on the call's stream; the on-chip kernel has none)."""
    import torch

    set_path, _ = f32_paths
    assert set_path(path) == 0
    rng = np.random.default_rng(77 + path)
    shapes = [(512, 384, 1024), (384, 640, 768)]
    hosts = [(rng.uniform(-1, 1, (M, K)).astype(np.float32), rng.uniform(-1, 1, (K, N)).astype(np.float32))
             for M, N, K in shapes]
    devs = [(to_dev(a, device), to_dev(b, device)) for a, b in hosts]
    outs = [torch.empty((M, N), device=device) for M, N, K in shapes]
    streams = [torch.cuda.Stream(device=device), torch.cuda.Stream(device=device)]
    torch.cuda.synchronize()
    for _ in range(8):
        for i in (0, 1):
            with torch.cuda.stream(streams[i]):
                cb.gemm_f32(devs[i][0], devs[i][1], mode=cb.F32_3XTF32, out=outs[i])
    for st in streams:
        st.synchronize()
    cb.check_device()
    for (M, N, K), (a, b), out in zip(shapes, hosts, outs):
        assert rel_fro(out.cpu().numpy(), oracle.gemm_f32(a, b, M, N, K, acc64=True)) <= TOL_F32


@pytest.mark.parametrize("ranges", [0, 2, 4])
@pytest.mark.parametrize("layout_name", ["ROW_MAJOR", "COL_MAJOR_NN", "ROW_MAJOR_BT"])
@pytest.mark.parametrize("shape", [(1024, 1024, 1024), (250, 130, 515), (64, 64, 64), (70, 3, 97)])
def test_fp32_ffma_k_ranges(cb, oracle, device, f32_paths, shape, layout_name, ranges):
    """FFMA with K cut into 0 (never), 2 or 4 ranges inside a cluster: <= 1e-5 against the
    fp64-accumulated product and no further from it than twice the reference loop's own distance;
    with K uncut the result is the single ascending sum (the oracle's bits when the oracle fuses
    nothing: compared to 1e-6 here); two launches agree bit for bit."""
    import torch

    _, set_ranges = f32_paths
    layout = getattr(cb, layout_name)
    M, N, K = shape
    rng = np.random.default_rng(M + 3 * N + 7 * K + layout + ranges)
    sa, sb = storage_shapes(cb, M, N, K, layout)
    a = rng.uniform(-1, 1, sa).astype(np.float32)
    b = rng.uniform(-1, 1, sb).astype(np.float32)
    assert set_ranges(ranges) == 0
    ad, bd = to_dev(a, device), to_dev(b, device)
    c = cb.gemm_f32(ad, bd, layout, mode=cb.F32_FFMA)
    c2 = cb.gemm_f32(ad, bd, layout, mode=cb.F32_FFMA)
    cb.check_device()
    assert torch.equal(c, c2)
    bt = np.ascontiguousarray(b.T) if layout == cb.ROW_MAJOR_BT else b
    lay = oracle.ROW_MAJOR if layout == cb.ROW_MAJOR_BT else layout
    truth = oracle.gemm_f32(a, bt, M, N, K, lay, acc64=True)
    loop = oracle.gemm_f32(a, bt, M, N, K, lay)
    err = rel_fro(c.cpu().numpy(), truth)
    assert err <= TOL_F32
    assert err <= 2 * rel_fro(loop, truth) + 1e-7


@pytest.mark.parametrize("layout_name", ["ROW_MAJOR", "COL_MAJOR_NN", "ROW_MAJOR_BT"])
@pytest.mark.parametrize("shape", [(64, 64, 64), (332, 516, 1000), (1024, 1024, 1024), (4096, 512, 256)])
def test_fp32_single_pass_tf32(cb, oracle, device, shape, layout_name):
    layout = getattr(cb, layout_name)
    M, N, K = shape
    rng = np.random.default_rng(hash((M, N, K, layout, 1)) & 0xFFFF)
    sa, sb = storage_shapes(cb, M, N, K, layout)
    a = rng.uniform(-1, 1, sa).astype(np.float32)
    b = rng.uniform(-1, 1, sb).astype(np.float32)
    c = cb.gemm_f32(to_dev(a, device), to_dev(b, device), layout, mode=cb.F32_TF32).cpu().numpy()
    cb.check_device()
    if layout == cb.ROW_MAJOR_BT:
        truth = oracle.gemm_f32(a, np.ascontiguousarray(b.T), M, N, K, acc64=True)
    else:
        truth = oracle.gemm_f32(a, b, M, N, K, layout, acc64=True)
    err = rel_fro(c, truth)
    assert err <= TOL_TF32
    assert err > 1e-6  # it really is the reduced-precision path


def test_fp32_single_pass_tf32_needs_aligned_rows(cb, device):
    import torch

    a = torch.zeros((64, 30), device=device)
    b = torch.zeros((30, 64), device=device)
    with pytest.raises(cb.B200Error) as e:
        cb.gemm_f32(a, b, mode=cb.F32_TF32)
    assert e.value.status == 2


# ------------------------------------------------------------------ W8A8 and the quantiser

@pytest.mark.parametrize("shape", [(33, 80, 64), (300, 520, 1024), (128, 4096, 2048), (17, 70, 0), (5, 9000, 0),
                                   (2048, 12288, 0), (1, 1, 0)])
def test_quantiser_bit_exact_vs_oracle(cb, oracle, device, shape):
    R, C, _ = shape
    rng = np.random.default_rng(R * C)
    x = rng.standard_normal((R, C)).astype(np.float32)
    x[R // 2] = 0.0       # an all-zero row and an all-zero column take scale 1
    x[:, C // 3] = 0.0
    xd = to_dev(x, device)
    for along in (0, 1):
        q, s = cb.quantize_absmax(xd, along)
        want_q, want_s = oracle.quantize_absmax(x, along)
        assert np.array_equal(s.cpu().numpy(), want_s)
        assert np.array_equal(q.cpu().numpy(), want_q)


def test_quantiser_rounding_ties_match_the_division(cb, oracle, device):
    """Values whose quotient by the scale sits on (or a few ulps beside) a rounding tie k + 0.5:
    the kernels' fast quotient must give the same integers as the IEEE division of the oracle."""
    rng = np.random.default_rng(4)
    R, C = 64, 4096
    scale = rng.uniform(0.003, 0.05, R).astype(np.float32)
    k = rng.integers(-126, 126, (R, C)).astype(np.float32) + 0.5
    x = (k * scale[:, None]).astype(np.float32)
    ulps = rng.integers(-3, 4, (R, C)).astype(np.int32)
    x = (x.view(np.int32) + ulps).view(np.float32)
    assert np.isfinite(x).all()
    x[:, 0] = 127.0 * scale            # pins the row maximum, hence the scale
    xd = to_dev(x, device)
    for along, xx in ((0, x), (1, np.ascontiguousarray(x.T))):
        q, s = cb.quantize_absmax(to_dev(xx, device), along)
        want_q, want_s = oracle.quantize_absmax(xx, along)
        assert np.array_equal(s.cpu().numpy(), want_s)
        assert np.array_equal(q.cpu().numpy(), want_q)


@pytest.mark.parametrize("shape", [(128, 256, 256), (300, 528, 1024), (17, 128, 8192)])
def test_w8a8_bit_exact_vs_oracle(cb, oracle, device, shape):
    M, N, K = shape
    rng = np.random.default_rng(M + N + K)
    x = rng.standard_normal((M, K)).astype(np.float32)
    w = rng.standard_normal((K, N)).astype(np.float32)
    qx, sx = oracle.quantize_absmax(x, 0)
    qw, sw = oracle.quantize_absmax(w, 1)
    c = cb.gemm_w8a8_bf16(to_dev(qx, device), to_dev(qw, device), to_dev(sx, device), to_dev(sw, device))
    cb.check_device()
    want = oracle.gemm_w8a8_bf16(qx, qw, sx, sw, M, N, K)
    import torch

    assert np.array_equal(c.view(torch.int16).cpu().numpy().view(np.uint16), want)


def test_w8a8_config_8192x28672x8192_sampled_rows(cb, oracle, device):
    """The sharded-linear shape on one GPU: quantise N(0,1) sources on the device, run the fused
    dequantising GEMM, and compare sampled rows bit for bit with the oracle."""
    import torch

    M, N, K = 8192, 28672, 8192
    g = torch.Generator(device=device).manual_seed(5)
    x = torch.randn((M, K), device=device, generator=g)
    w = torch.randn((K, N), device=device, generator=g)
    qx, sx = cb.quantize_absmax(x, 0)
    qw, sw = cb.quantize_absmax(w, 1)
    del x, w
    c = cb.gemm_w8a8_bf16(qx, qw, sx, sw)
    cb.check_device()
    rows = [0, 127, 128, 5000, 8191, 4096, 1023, 6001]
    want = oracle.gemm_w8a8_bf16(qx.cpu().numpy(), qw.cpu().numpy(), sx.cpu().numpy(), sw.cpu().numpy(), M, N, K, rows)
    got = c[rows].view(torch.int16).cpu().numpy().view(np.uint16)
    assert np.array_equal(got, want)
    # per-tensor scales are the same entry point with constant scale vectors
    one_r = torch.full((M,), 0.5, device=device)
    one_c = torch.full((N,), 0.25, device=device)
    c2 = cb.gemm_w8a8_bf16(qx[:256], qw, one_r[:256], one_c)
    acc = cb.gemm_i8_i32(qx[:256], qw)
    assert torch.equal(c2, ((acc.float() * 0.5) * 0.25).to(torch.bfloat16))


# ------------------------------------------------------------------ host-buffer entry point and the suite bodies

def test_host_buffer_entry_point(cb, oracle):
    from cudaintro_b200 import capi

    rng = np.random.default_rng(21)
    M, N, K = 256, 384, 512
    a = rng.integers(-127, 128, (M, K)).astype(np.int8)
    b = rng.integers(-127, 128, (K, N)).astype(np.int8)
    c = np.zeros((M, N), dtype=np.int32)
    cb.gemm_host(capi.I8, a, b, c, M, N, K)
    assert np.array_equal(c, oracle.gemm_i8_i32(a, b, M, N, K))
    af = rng.uniform(-1, 1, (M, K)).astype(np.float32)
    bf = rng.uniform(-1, 1, (K, N)).astype(np.float32)
    cf = np.zeros((M, N), dtype=np.float32)
    cb.gemm_host(capi.F32, af, bf, cf, M, N, K)
    assert rel_fro(cf, oracle.gemm_f32(af, bf, M, N, K, acc64=True)) <= TOL_F32
    capi.lib.b200_host_release()


@pytest.mark.parametrize("layout_name", ["ROW_MAJOR", "COL_MAJOR_NN", "ROW_MAJOR_BT"])
def test_host_buffer_entry_point_in_several_slabs(cb, oracle, device, layout_name):
    """2000 lines of the slab dimension: four slabs of 512 (the last one ragged) travel up, through
    the kernels and down again on three streams.  int8 bit-exact against the oracle; bf16 equal to
    the device-buffer call to rounding.
    Called twice: the second call reuses the workspace while nothing of the first is in flight."""
    import torch
    from cudaintro_b200 import capi

    layout = getattr(cb, layout_name)
    M, N, K = (2000, 656, 768) if layout != cb.COL_MAJOR_NN else (656, 2000, 768)
    if layout == cb.COL_MAJOR_NN:
        M = 656 // 16 * 16 + 16
    rng = np.random.default_rng(7 + layout)
    sa, sb = storage_shapes(cb, M, N, K, layout)
    sc = (N, M) if layout == cb.COL_MAJOR_NN else (M, N)
    a = rng.integers(-127, 128, sa).astype(np.int8)
    b = rng.integers(-127, 128, sb).astype(np.int8)
    want = oracle_i8(oracle, cb, a, b, M, N, K, layout)
    for _ in range(2):
        c = np.full(sc, -7, dtype=np.int32)
        cb.gemm_host(capi.I8, a, b, c, M, N, K, layout)
        assert np.array_equal(c, want)
    a16 = oracle.f32_to_bf16_bits(rng.standard_normal(sa).astype(np.float32))
    b16 = oracle.f32_to_bf16_bits(rng.standard_normal(sb).astype(np.float32))
    want16 = cb.gemm_bf16(to_dev(a16.view(np.int16), device, torch.bfloat16),
                          to_dev(b16.view(np.int16), device, torch.bfloat16), layout)
    c16 = np.zeros(sc, dtype=np.uint16)
    cb.gemm_host(capi.BF16, a16, b16, c16, M, N, K, layout)
    got = torch.from_numpy(c16.view(np.int16)).view(torch.bfloat16).float().numpy()
    assert rel_fro(got, want16.float().cpu().numpy()) <= 1e-3
    capi.lib.b200_host_release()


def test_host_buffers_against_weights_kept_on_the_device(cb, oracle, device):
    """b200_host_weights_upload / b200_gemm_host_weights: B goes up once, then several A of different
    heights (one slab, several slabs with a ragged last one) are multiplied from host buffers.  int8
    bit-exact against the oracle; the handle is refused once freed."""
    from cudaintro_b200 import capi

    rng = np.random.default_rng(33)
    N, K = 400, 640
    b = rng.integers(-127, 128, (K, N)).astype(np.int8)
    w = capi.HostWeights(capi.I8, b, K, N)
    for M in (48, 1300, 512):
        a = rng.integers(-127, 128, (M, K)).astype(np.int8)
        c = np.full((M, N), -3, dtype=np.int32)
        w.matmul(a, c, M)
        assert np.array_equal(c, oracle.gemm_i8_i32(a, b, M, N, K)), M
    w.close()
    capi.lib.b200_host_release()
    assert capi.lib.b200_gemm_host_weights(None, a.ctypes.data, c.ctypes.data, 8) == 1


def test_host_buffer_calls_keep_one_workspace_per_device(cb, oracle):
    """With two GPUs visible, a host-buffer product on device 1 after one on device 0 must use
    streams and buffers of device 1 (each device has a workspace of its own)."""
    import torch
    from cudaintro_b200 import capi

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    rng = np.random.default_rng(34)
    M, N, K = 640, 256, 384
    a = rng.integers(-127, 128, (M, K)).astype(np.int8)
    b = rng.integers(-127, 128, (K, N)).astype(np.int8)
    want = oracle.gemm_i8_i32(a, b, M, N, K)
    for dev in (0, 1, 0):
        with torch.cuda.device(dev):
            c = np.zeros((M, N), dtype=np.int32)
            cb.gemm_host(capi.I8, a, b, c, M, N, K)
            assert np.array_equal(c, want), dev
    for dev in (0, 1):
        with torch.cuda.device(dev):
            capi.lib.b200_host_release()


def test_suite_entry_points_keep_the_reference_protocol(cb, device, monkeypatch):
    """run_gemm_* (quantization/gemm_common.h:64-67) through their C++ symbols: name, iteration
    count in multiples of 256, and the reference's TFLOP/s formula (GEMM_int8.cu:80-84)."""
    import ctypes as C

    from cudaintro_b200 import capi

    class GemmResult(C.Structure):
        _fields_ = [("name", C.c_char_p), ("iters", C.c_uint64), ("secs", C.c_double), ("tflops", C.c_double)]

    monkeypatch.setenv("GEMM_SUITE_SECONDS", "0.2")
    handle = C.CDLL(capi.LIB_PATH)
    for sym, name in (("_Z13run_gemm_int8P13cublasContext", b"INT8"), ("_Z13run_gemm_bf16P13cublasContext", b"BF16"),
                      ("_Z13run_gemm_fp16P13cublasContext", b"FP16"), ("_Z13run_gemm_fp32P13cublasContext", b"FP32")):
        fn = getattr(handle, sym)
        fn.restype = GemmResult
        fn.argtypes = [C.c_void_p]
        r = fn(None)
        assert r.name == name
        assert r.iters >= 256 and r.iters % 256 == 0
        assert r.secs >= 0.2
        assert abs(r.tflops - 2.0 * 4096 ** 3 * r.iters / (r.secs * 1e12)) <= 1e-9 * r.tflops


def test_reference_driver_binary_runs_on_this_library(cb, device):
    """The reference's own host driver (quantization/main.cu:8-31), compiled unchanged against
    include/gemm_common.h and linked with libb200gemm by `make -C oracle suite`: it must exit 0 and
    print its four result lines (main.cu:24-26) in the driver's order BF16, FP16, FP32, INT8."""
    import re
    import subprocess

    exe = os.path.join(os.path.dirname(GOLDEN), os.pardir, "oracle", "_ref", "gemm_suite_b200")
    exe = os.path.normpath(exe)
    if not os.path.exists(exe):
        pytest.skip("oracle/_ref/gemm_suite_b200 was not built on a machine with the reference tree")
    env = dict(os.environ, GEMM_SUITE_SECONDS="0.2")
    res = subprocess.run([exe], capture_output=True, text=True, timeout=300, env=env)
    assert res.returncode == 0, res.stdout + res.stderr
    lines = [ln for ln in res.stdout.splitlines() if ln.startswith("Ran ")]
    assert len(lines) == 4, res.stdout
    for ln, name in zip(lines, ("BF16", "FP16", "FP32", "INT8")):
        m = re.fullmatch(r"Ran (\d+) (\w+) GEMMs in ([0-9.eE+-]+) s \(([0-9.eE+-]+) TFLOP/s\)", ln)
        assert m and m.group(2) == name, ln
        iters, secs, tflops = int(m.group(1)), float(m.group(3)), float(m.group(4))
        assert iters >= 256 and iters % 256 == 0 and secs >= 0.2
        assert abs(tflops - 2.0 * 4096 ** 3 * iters / (secs * 1e12)) <= 2e-3 * tflops  # printed with 6 digits
    for name in ("BF16", "FP16", "FP32", "INT8"):
        assert f"Running {name}..." in res.stdout


# ------------------------------------------------------------------ tile policies (single CTAs vs CTA pairs)

@pytest.fixture
def policy(cb):
    yield cb.set_tile_policy
    cb.set_tile_policy(0, 0)


POLICY_SHAPES = [(256, 256, 128), (208, 336, 1008), (16, 512, 4112), (1024, 768, 2048), (257, 272, 64)]


def test_l2_eviction_hints_do_not_change_results(cb, device):
    """b200_set_l2_hints only changes the cache policy words that travel with the TMA loads and stores:
    every setting must give the bits of the default (int8 exact, bf16 identical)."""
    import torch
    from cudaintro_b200 import capi

    g = torch.Generator(device=device).manual_seed(3)
    a = torch.randint(-127, 128, (1024, 768), dtype=torch.int8, device=device, generator=g)
    b = torch.randint(-127, 128, (768, 1280), dtype=torch.int8, device=device, generator=g)
    ah, bh = a.bfloat16(), b.bfloat16()
    want_i, want_h = cb.gemm_i8_i32(a, b), cb.gemm_bf16(ah, bh)
    assert torch.equal(want_i, cb.gemm_naive(a, b))
    try:
        for hints in range(8):
            assert capi.lib.b200_set_l2_hints(hints) == 0
            assert torch.equal(cb.gemm_i8_i32(a, b), want_i), hints
            assert torch.equal(cb.gemm_bf16(ah, bh), want_h), hints
        cb.check_device()
        assert capi.lib.b200_set_l2_hints(8) == 1
    finally:
        capi.lib.b200_set_l2_hints(-1)


@pytest.mark.parametrize("cg,M", [(1, 128), (2, 256), (4, 512)])
def test_kernel_gives_up_a_wait_that_cannot_end_and_the_device_stays_usable(cb, oracle, device, policy, cg, M):
    """Failure handling of the tensor-core kernel itself, without any fault: the producer of a
    one-tile launch (a single CTA, a CTA pair, a pair with two row blocks per CTA) leaves out the
    loads of one k-block in CTA 0 (b200_test_lose_arrival), so the MMA lane's bounded wait for that
    stage runs out after the 50 ms budget given here; every role of every CTA gives up its own wait,
    the kernel returns, b200_check_device reports B200_ERR_DEVICE_WAIT, and the next product on the
    same context is bit-exact again."""
    import time

    import torch
    from cudaintro_b200 import capi

    rng = np.random.default_rng(5)
    N, K = 256, 512
    a = rng.integers(-127, 128, (M, K)).astype(np.int8)
    b = rng.integers(-127, 128, (K, N)).astype(np.int8)
    ad, bd = to_dev(a, device), to_dev(b, device)
    want = oracle.gemm_i8_i32(a, b, M, N, K)
    policy(cg, 256)  # the general kernel, one tile
    assert np.array_equal(cb.gemm_i8_i32(ad, bd).cpu().numpy(), want)
    cb.check_device()
    try:
        capi._check(capi.lib.b200_test_lose_arrival(1, 50_000_000))
        t0 = time.perf_counter()
        cb.gemm_i8_i32(ad, bd)
        with pytest.raises(cb.B200Error) as info:
            cb.check_device()
        waited = time.perf_counter() - t0
        assert info.value.status == 4  # B200_ERR_DEVICE_WAIT
        assert 0.04 <= waited < 2.0, waited
    finally:
        capi._check(capi.lib.b200_test_lose_arrival(-1, 0))
    cb.check_device()  # the record was cleared by the failing check
    for _ in range(2):
        assert np.array_equal(cb.gemm_i8_i32(ad, bd).cpu().numpy(), want)
    cb.check_device()
    torch.cuda.synchronize()


@pytest.mark.parametrize("cg,bn", [(1, 256), (1, 128), (2, 256), (4, 256)])
@pytest.mark.parametrize("layout_name", ["ROW_MAJOR", "COL_MAJOR_NN", "ROW_MAJOR_BT"])
@pytest.mark.parametrize("shape", POLICY_SHAPES)
def test_int8_every_tile_policy_is_bit_exact(cb, oracle, device, policy, shape, layout_name, cg, bn):
    layout = getattr(cb, layout_name)
    M, N, K = shape
    if layout == cb.COL_MAJOR_NN and M % 16:
        M = (M + 15) // 16 * 16
    rng = np.random.default_rng(hash((M, N, K, layout, cg, bn)) & 0xFFFF)
    sa, sb = storage_shapes(cb, M, N, K, layout)
    a = rng.integers(-127, 128, sa).astype(np.int8)
    b = rng.integers(-127, 128, sb).astype(np.int8)
    policy(cg, bn)
    c = cb.gemm_i8_i32(to_dev(a, device), to_dev(b, device), layout)
    cb.check_device()
    assert np.array_equal(c.cpu().numpy(), oracle_i8(oracle, cb, a, b, M, N, K, layout))


@pytest.mark.parametrize("cg,bn", [(1, 256), (1, 64), (2, 256), (4, 256)])
@pytest.mark.parametrize("layout_name", ["ROW_MAJOR", "ROW_MAJOR_BT"])
def test_16bit_and_tf32_every_tile_policy(cb, oracle, device, policy, layout_name, cg, bn):
    import torch

    layout = getattr(cb, layout_name)
    M, N, K = 392, 520, 1032
    rng = np.random.default_rng(cg * 1000 + bn + layout)
    sa, sb = storage_shapes(cb, M, N, K, layout)
    af = rng.standard_normal(sa).astype(np.float32)
    bf = rng.standard_normal(sb).astype(np.float32)
    policy(cg, bn)
    a16, b16 = oracle.f32_to_bf16_bits(af), oracle.f32_to_bf16_bits(bf)
    c = cb.gemm_bf16(to_dev(a16.view(np.int16), device, torch.bfloat16), to_dev(b16.view(np.int16), device, torch.bfloat16),
                     layout)
    cb.check_device()
    b_kn = b16 if layout == cb.ROW_MAJOR else np.ascontiguousarray(b16.T)
    _, o32 = oracle.gemm_h16(a16, b_kn, M, N, K, True)
    assert rel_fro(c.float().cpu().numpy(), o32) <= TOL_BF16
    c32 = cb.gemm_f32(to_dev(af, device), to_dev(bf, device), layout, mode=cb.F32_3XTF32)
    cb.check_device()
    bf_kn = bf if layout == cb.ROW_MAJOR else np.ascontiguousarray(bf.T)
    assert rel_fro(c32.cpu().numpy(), oracle.gemm_f32(af, bf_kn, M, N, K, acc64=True)) <= TOL_F32


def test_w8a8_tile_policies_agree_bit_for_bit(cb, oracle, device, policy):
    import torch

    M, N, K = 520, 784, 2048
    rng = np.random.default_rng(77)
    qx, sx = oracle.quantize_absmax(rng.standard_normal((M, K)).astype(np.float32), 0)
    qw, sw = oracle.quantize_absmax(rng.standard_normal((K, N)).astype(np.float32), 1)
    want = oracle.gemm_w8a8_bf16(qx, qw, sx, sw, M, N, K)
    for cg, bn in ((1, 256), (1, 128), (2, 256)):
        policy(cg, bn)
        c = cb.gemm_w8a8_bf16(to_dev(qx, device), to_dev(qw, device), to_dev(sx, device), to_dev(sw, device))
        cb.check_device()
        assert np.array_equal(c.view(torch.int16).cpu().numpy().view(np.uint16), want), (cg, bn)


@pytest.mark.parametrize("M", [1, 16, 32, 33, 64, 65])
def test_skinny_products_on_wide_tiles(cb, oracle, device, policy, M):
    """A handful of rows against a wide weight matrix on 128-wide tiles (the decode-shape path): most
    of the 128 accumulator rows of every tile are padding; nothing of them may reach C, and the rows
    that count must still be exact.  K is long enough for the stage ring to wrap several times."""
    import torch

    N, K = 528, 2176  # 17 / 34 k-blocks
    rng = np.random.default_rng(4000 + M)
    policy(1, 128)
    # int8, both B layouts, bit-exact
    a = rng.integers(-127, 128, (M, K)).astype(np.int8)
    b = rng.integers(-127, 128, (K, N)).astype(np.int8)
    want = oracle.gemm_i8_i32(a, b, M, N, K, oracle.ROW_MAJOR)
    for layout, bb in ((cb.ROW_MAJOR, b), (cb.ROW_MAJOR_BT, np.ascontiguousarray(b.T))):
        c = cb.gemm_i8_i32(to_dev(a, device), to_dev(bb, device), layout)
        cb.check_device()
        assert np.array_equal(c.cpu().numpy(), want), layout
    # W8A8 -> bf16, bit-exact
    qx, sx = oracle.quantize_absmax(rng.standard_normal((M, K)).astype(np.float32), 0)
    qw, sw = oracle.quantize_absmax(rng.standard_normal((K, N)).astype(np.float32), 1)
    c = cb.gemm_w8a8_bf16(to_dev(qx, device), to_dev(qw, device), to_dev(sx, device), to_dev(sw, device))
    cb.check_device()
    assert np.array_equal(c.view(torch.int16).cpu().numpy().view(np.uint16),
                          oracle.gemm_w8a8_bf16(qx, qw, sx, sw, M, N, K))
    # fp16 and bf16 within their tolerances, and finite everywhere
    af = rng.standard_normal((M, K)).astype(np.float32)
    bf = (rng.standard_normal((K, N)) * 0.02).astype(np.float32)
    for is_bf16, tol in ((True, TOL_BF16), (False, TOL_F16)):
        conv = oracle.f32_to_bf16_bits if is_bf16 else (lambda x: x.astype(np.float16).view(np.uint16))
        dt = torch.bfloat16 if is_bf16 else torch.float16
        a16, b16 = conv(af), conv(bf)
        fn = cb.gemm_bf16 if is_bf16 else cb.gemm_f16
        c = fn(to_dev(a16.view(np.int16), device, dt), to_dev(b16.view(np.int16), device, dt), cb.ROW_MAJOR)
        cb.check_device()
        _, o32 = oracle.gemm_h16(a16, b16, M, N, K, is_bf16)
        got = c.float().cpu().numpy()
        assert np.isfinite(got).all()
        assert rel_fro(got, o32) <= tol, is_bf16
