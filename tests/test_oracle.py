"""CPU tests of the oracle itself: known answers, golden fixtures made by the reference's own
matrixMulCPU, and (where the reference loop was compiled) a live comparison against it."""
import glob
import os

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load(name):
    return np.load(os.path.join(GOLDEN, name))


# ---- known answers of the suite's generators (quantization/GEMM_int8.cu:8-19, GEMM_fp32.cu:7-17)

def test_fill_int8_known_answers(oracle):
    assert oracle.fill_int8(16, 0x4234).tolist() == [22, 34, 46, 58, -27, -15, -3, 9, 119, -123, -111, -99, 70, 82, 94, 106]
    assert oracle.fill_int8(16, 0x6676).tolist() == [-53, -41, -77, -65, -102, -89, -127, -114, 44, 56, 20, 32, -4, 8, -29, -16]


def test_fill_int8_range_and_formula(oracle):
    v = oracle.fill_int8(1 << 16, 0x4234)
    assert v.min() >= -127 and v.max() <= 127
    idx = np.arange(1 << 16, dtype=np.uint64)
    x = (idx ^ np.uint64(0x4234)) * np.uint64(2862933555777941757) + np.uint64(3037000493)
    r = ((x >> np.uint64(11)) & np.uint64(0xFFFF)).astype(np.int64)
    assert np.array_equal(v.astype(np.int64), -127 + r % 255)


def test_fill_f32_known_answers(oracle):
    bits = oracle.fill_f32(3, 0x3234).view(np.uint32).tolist()
    assert bits == [0x3E477A58, 0xBE30D4FC, 0xBF0A4914]
    v = oracle.fill_f32(1 << 16, 0x7776)
    assert v.min() >= -1.0 and v.max() <= 1.0


def test_fill_16bit_is_rounded_f32_fill(oracle):
    f = oracle.fill_f32(4096, 0x1234)
    assert np.array_equal(oracle.fill_bf16(4096, 0x1234), oracle.f32_to_bf16_bits(f))
    assert np.array_equal(oracle.fill_f16(4096, 0x1234), f.astype(np.float16).view(np.uint16))


def test_suite_int8_4x4x4_column_major_known_answer(oracle):
    a = oracle.fill_int8(16, 0x4234)
    b = oracle.fill_int8(16, 0x6676)
    c = oracle.gemm_i8_i32(a, b, 4, 4, 4, layout=oracle.COL_MAJOR_NN)
    assert c.ravel().tolist() == [-13772, 2954, 122, -2710, -22934, 4140, -1044, -6228, 4076, 820, 2644, 4468,
                                  -4875, 1999, 1507, 1015]


# ---- 16-bit conversions

def test_f16_conversions_match_numpy(oracle):
    lib = oracle.load()
    rng = np.random.default_rng(3)
    xs = np.concatenate([rng.standard_normal(3000).astype(np.float32) * s for s in (1e-8, 1e-6, 1e-4, 1, 300, 7e4)])
    with np.errstate(over="ignore"):
        want = xs.astype(np.float16).view(np.uint16)
    got = np.array([lib.oracle_f32_to_f16(float(v)) for v in xs], dtype=np.uint16)
    assert np.array_equal(got, want)
    h = np.arange(0, 1 << 16, 7, dtype=np.uint16)
    back = np.array([lib.oracle_f16_to_f32(int(v)) for v in h], dtype=np.float32)
    want32 = h.view(np.float16).astype(np.float32)
    ok = ~np.isnan(want32)
    assert np.array_equal(back.view(np.uint32)[ok], want32.view(np.uint32)[ok])


def test_bf16_rounding_is_nearest_even(oracle):
    lib = oracle.load()
    # 1 + 2^-8 is a tie between 1.0 and 1 + 2^-7: goes to the even mantissa (1.0)
    assert lib.oracle_f32_to_bf16(1.0 + 2.0 ** -8) == 0x3F80
    assert lib.oracle_f32_to_bf16(1.0 + 3 * 2.0 ** -8) == 0x3F82
    x = np.random.default_rng(5).standard_normal(5000).astype(np.float32)
    got = np.array([lib.oracle_f32_to_bf16(float(v)) for v in x], dtype=np.uint16)
    assert np.array_equal(got, oracle.f32_to_bf16_bits(x))
    err = np.abs(oracle.bf16_bits_to_f32(got) - x)
    assert np.all(err <= np.abs(x) * 2.0 ** -8)


# ---- golden fixtures written by the reference's own matrixMulCPU

@pytest.mark.parametrize("name", ["ref_f32_32.npz", "ref_f32_96.npz", "ref_f32_unit_64.npz"])
def test_f32_loop_matches_reference_output(oracle, name):
    g = load(name)
    w = g["a"].shape[0]
    got = oracle.gemm_f32(g["a"], g["b"], w, w, w)
    assert np.array_equal(got.view(np.uint32), g["c"].view(np.uint32))
    # the column-major call on transposed storage is the same product
    got_cm = oracle.gemm_f32(g["a"].T.copy(), g["b"].T.copy(), w, w, w, layout=oracle.COL_MAJOR_NN)
    assert np.array_equal(got_cm.T.view(np.uint32), g["c"].view(np.uint32))


@pytest.mark.parametrize("name", ["ref_i8_128.npz", "ref_i8_suitefill_64.npz"])
def test_int8_loop_matches_reference_output(oracle, name):
    g = load(name)
    w = g["a"].shape[0]
    assert np.array_equal(oracle.gemm_i8_i32(g["a"], g["b"], w, w, w), g["c"])
    cm = oracle.gemm_i8_i32(g["a"].T.copy(), g["b"].T.copy(), w, w, w, layout=oracle.COL_MAJOR_NN)
    assert np.array_equal(cm.T, g["c"])


@pytest.mark.parametrize("name,is_bf16", [("ref_bf16_96.npz", True), ("ref_f16_96.npz", False)])
def test_16bit_loop_matches_reference_output(oracle, name, is_bf16):
    g = load(name)
    w = g["a"].shape[0]
    o16, o32 = oracle.gemm_h16(g["a"], g["b"], w, w, w, is_bf16)
    assert np.array_equal(o32.view(np.uint32), g["c32"].view(np.uint32))
    if is_bf16:
        assert np.array_equal(o16, oracle.f32_to_bf16_bits(g["c32"]))
    else:
        assert np.array_equal(o16, g["c32"].astype(np.float16).view(np.uint16))


def test_live_reference_loop_if_built(oracle):
    if oracle.load_ref() is None:
        pytest.skip("oracle/_ref/libref_matmulcpu.so not built on this machine")
    rng = np.random.default_rng(11)
    w = 160
    a = rng.uniform(-1, 1, (w, w)).astype(np.float32)
    b = rng.uniform(-1, 1, (w, w)).astype(np.float32)
    assert np.array_equal(oracle.ref_matrix_mul_cpu(a, b, w).view(np.uint32), oracle.gemm_f32(a, b, w, w, w).view(np.uint32))


# ---- shapes, row subsets, edge cases

def test_rectangular_and_row_subset(oracle):
    rng = np.random.default_rng(7)
    M, N, K = 37, 53, 129
    a = rng.integers(-127, 128, (M, K)).astype(np.int8)
    b = rng.integers(-127, 128, (K, N)).astype(np.int8)
    want = a.astype(np.int64) @ b.astype(np.int64)
    assert np.array_equal(oracle.gemm_i8_i32(a, b, M, N, K), want)
    rows = [0, 5, 36]
    assert np.array_equal(oracle.gemm_i8_i32(a, b, M, N, K, rows=rows), want[rows])
    af = rng.standard_normal((M, K)).astype(np.float32)
    bf = rng.standard_normal((K, N)).astype(np.float32)
    full = oracle.gemm_f32(af, bf, M, N, K)
    assert np.array_equal(oracle.gemm_f32(af, bf, M, N, K, rows=rows), full[rows])
    acc64 = oracle.gemm_f32(af, bf, M, N, K, acc64=True)
    assert np.allclose(acc64, af.astype(np.float64) @ bf.astype(np.float64), rtol=1e-12, atol=1e-12)


def test_int8_extremes_do_not_overflow(oracle):
    K = 8192
    a = np.full((2, K), -127, dtype=np.int8)
    b = np.full((K, 3), -127, dtype=np.int8)
    assert np.all(oracle.gemm_i8_i32(a, b, 2, 3, K) == K * 127 * 127)


def test_single_element_and_k1(oracle):
    a = np.array([[3]], dtype=np.int8)
    b = np.array([[-5]], dtype=np.int8)
    assert oracle.gemm_i8_i32(a, b, 1, 1, 1).tolist() == [[-15]]
    x = np.array([[0.5], [2.0]], dtype=np.float32)
    y = np.array([[4.0, -1.0]], dtype=np.float32)
    assert oracle.gemm_f32(x, y, 2, 2, 1).tolist() == [[2.0, -0.5], [8.0, -2.0]]


# ---- W8A8 and the quantiser (defined by this project; no reference counterpart)

def test_quantiser_definition(oracle):
    rng = np.random.default_rng(9)
    x = rng.standard_normal((33, 70)).astype(np.float32)
    x[4] = 0.0
    x[:, 9] = 0.0
    for along in (0, 1):
        q, s = oracle.quantize_absmax(x, along)
        amax = np.abs(x).max(axis=1 - along)
        want_s = np.where(amax > 0, amax / np.float32(127.0), np.float32(1.0)).astype(np.float32)
        assert np.array_equal(s, want_s)
        sb = s[:, None] if along == 0 else s[None, :]
        want_q = np.clip(np.rint(x / sb), -127, 127).astype(np.int8)
        assert np.array_equal(q, want_q)
        assert np.abs(q).max() == 127


def test_quantiser_ties_go_to_even(oracle):
    x = np.array([[127.0, 0.5, 1.5, 2.5, -0.5, -1.5]], dtype=np.float32)  # scale = 1
    q, s = oracle.quantize_absmax(x, 0)
    assert s.tolist() == [1.0]
    assert q.tolist() == [[127, 0, 2, 2, 0, -2]]


def test_w8a8_definition(oracle):
    rng = np.random.default_rng(13)
    M, N, K = 19, 40, 96
    a = rng.integers(-127, 128, (M, K)).astype(np.int8)
    b = rng.integers(-127, 128, (K, N)).astype(np.int8)
    sa = rng.uniform(0.001, 0.05, M).astype(np.float32)
    sw = rng.uniform(0.001, 0.05, N).astype(np.float32)
    acc = (a.astype(np.int64) @ b.astype(np.int64)).astype(np.float32)
    want = oracle.f32_to_bf16_bits((acc * sa[:, None]) * sw[None, :])
    assert np.array_equal(oracle.gemm_w8a8_bf16(a, b, sa, sw, M, N, K), want)
    assert np.array_equal(oracle.gemm_w8a8_bf16(a, b, sa, sw, M, N, K, rows=[3, 18]), want[[3, 18]])


def test_fixture_directory_is_complete():
    names = {os.path.basename(p) for p in glob.glob(os.path.join(GOLDEN, "*.npz"))}
    assert {"ref_f32_32.npz", "ref_f32_96.npz", "ref_f32_unit_64.npz", "ref_i8_128.npz",
            "ref_i8_suitefill_64.npz", "ref_bf16_96.npz", "ref_f16_96.npz"} <= names


# ------------------------------------------------------------------ fully connected layer

def test_linear_known_answers_tell_the_rounding_orders_apart(oracle):
    """Two hand-made cases.  (1) x*w = 1 + 2^-11 + 2^-24 needs 25 bits: rounded on its own it loses
    the last one, fused into the sum with bias -(1 + 2^-11) it leaves exactly 2^-24.  (2) bias 1 and
    products +2^24, -2^24: starting from the bias loses it (2^24 + 1 rounds to 2^24), adding it to
    the finished sum keeps it."""
    x = np.array([[1 + 2.0 ** -12]], dtype=np.float32)
    w = np.array([[1 + 2.0 ** -12]], dtype=np.float32)
    b = np.array([-(1 + 2.0 ** -11)], dtype=np.float32)
    assert oracle.linear_f32(x, w, b, True, False, True, fused=True)[0, 0] == np.float32(2.0 ** -24)
    assert oracle.linear_f32(x, w, b, True, False, True, fused=False)[0, 0] == 0.0
    x = np.array([[4096.0, 4096.0]], dtype=np.float32)
    w = np.array([[4096.0, -4096.0]], dtype=np.float32)
    b = np.array([1.0], dtype=np.float32)
    for fused in (True, False):
        assert oracle.linear_f32(x, w, b, True, False, True, fused=fused)[0, 0] == 0.0   # bias first
        assert oracle.linear_f32(x, w, b, True, False, False, fused=fused)[0, 0] == 1.0  # bias last
    # ReLU and the two weight layouts
    assert oracle.linear_f32(x, -w, -b, True, True, False)[0, 0] == 0.0
    rng = np.random.default_rng(3)
    xs = rng.standard_normal((9, 31)).astype(np.float32)
    ws = rng.standard_normal((13, 31)).astype(np.float32)
    bs = rng.standard_normal(13).astype(np.float32)
    y = oracle.linear_f32(xs, ws, bs, True, True, False)
    assert np.array_equal(y, oracle.linear_f32(xs, np.ascontiguousarray(ws.T), bs, False, True, False))
    want = np.maximum(xs.astype(np.float64) @ ws.T.astype(np.float64) + bs, 0)
    assert np.abs(y - want).max() < 1e-4 and (y == 0).any()


def test_linear_16bit_is_the_fp32_sum_rounded_once(oracle):
    rng = np.random.default_rng(4)
    xs = rng.standard_normal((6, 40)).astype(np.float32)
    ws = rng.standard_normal((10, 40)).astype(np.float32)
    bs = rng.standard_normal(10).astype(np.float32)
    xb, wb = oracle.f32_to_bf16_bits(xs), oracle.f32_to_bf16_bits(ws)
    y16, y32 = oracle.linear_h16(xb, wb, bs, True, True, relu=False)
    sums = oracle.linear_f32(oracle.bf16_bits_to_f32(xb), oracle.bf16_bits_to_f32(wb), bs, True, False, False, fused=False)
    assert np.array_equal(y32, sums)
    assert np.array_equal(y16, oracle.f32_to_bf16_bits(sums))
    xh, wh = xs.astype(np.float16).view(np.uint16), ws.astype(np.float16).view(np.uint16)
    y16, y32 = oracle.linear_h16(xh, wh, None, False, True, relu=True)
    assert (y32 >= 0).all() and np.array_equal(y16.view(np.float16), y32.astype(np.float16))
