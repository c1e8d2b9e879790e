"""ctypes front end of the CPU oracle (``gemm_oracle.c``).  TEST INFRASTRUCTURE ONLY.

Only the tests, the smoke check and the bench's CPU-baseline legs may import this package;
the shipped library never does.  The product path has no CPU route at all.

``load()`` returns the compiled oracle, building it with ``make -C oracle oracle`` when the
shared object is missing.  ``load_ref()`` returns the reference's own ``matrixMulCPU``
(TileProgramming/tensor_utils.cu:35-45), compiled unmodified from the reference tree by
``make -C oracle ref`` into ``oracle/_ref/``; it returns ``None`` when that file was never
built (the reference tree is not present on every machine).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROW_MAJOR = 0
COL_MAJOR_NN = 1

_lib = None
_ref = None

_i64 = C.c_int64
_p = C.c_void_p


def build(ref_tree: str | None = None) -> None:
    """Compile the oracle and, if ``ref_tree`` exists, the reference's own pieces."""
    subprocess.run(["make", "-s", "-C", HERE, "oracle"], check=True)
    if ref_tree and os.path.isdir(os.path.join(ref_tree, "TileProgramming")):
        subprocess.run(["make", "-s", "-C", HERE, "ref", f"REF={ref_tree}"], check=True)
        if os.path.exists(os.path.join(os.path.dirname(HERE), "cudaintro_b200", "libb200gemm.so")):
            subprocess.run(["make", "-s", "-C", HERE, "suite", f"REF={ref_tree}"], check=True)


def load() -> C.CDLL:
    global _lib
    if _lib is None:
        so = os.path.join(HERE, "liboracle.so")
        if not os.path.exists(so):
            build()
        lib = C.CDLL(so)
        lib.oracle_num_threads.restype = C.c_int
        lib.oracle_bf16_to_f32.restype = C.c_float
        lib.oracle_bf16_to_f32.argtypes = [C.c_uint16]
        lib.oracle_f16_to_f32.restype = C.c_float
        lib.oracle_f16_to_f32.argtypes = [C.c_uint16]
        lib.oracle_f32_to_bf16.restype = C.c_uint16
        lib.oracle_f32_to_bf16.argtypes = [C.c_float]
        lib.oracle_f32_to_f16.restype = C.c_uint16
        lib.oracle_f32_to_f16.argtypes = [C.c_float]
        for name in ("int8",):
            getattr(lib, f"oracle_fill_{name}").argtypes = [_p, _i64, C.c_uint64, C.c_int, C.c_int]
        for name in ("f32", "f16", "bf16"):
            getattr(lib, f"oracle_fill_{name}").argtypes = [_p, _i64, C.c_uint64, C.c_float, C.c_float]
        lib.oracle_gemm_f32.argtypes = [_p, _p, _p, _i64, _i64, _i64, C.c_int, _p, _i64]
        lib.oracle_gemm_f32_acc64.argtypes = [_p, _p, _p, _i64, _i64, _i64, C.c_int, _p, _i64]
        lib.oracle_gemm_i8_i32.argtypes = [_p, _p, _p, _i64, _i64, _i64, C.c_int, _p, _i64]
        lib.oracle_gemm_h16.argtypes = [_p, _p, _p, _p, _i64, _i64, _i64, C.c_int, C.c_int, _p, _i64]
        lib.oracle_gemm_w8a8_bf16.argtypes = [_p, _p, _p, _p, _p, _i64, _i64, _i64, _p, _i64]
        lib.oracle_quantize_absmax.argtypes = [_p, _p, _p, _i64, _i64, C.c_int]
        lib.oracle_linear_f32.argtypes = [_p, _p, _p, _p, _i64, _i64, _i64, C.c_int, C.c_int, C.c_int]
        lib.oracle_linear_h16.argtypes = [_p, _p, _p, _p, _p, _i64, _i64, _i64, C.c_int, C.c_int, C.c_int]
        _lib = lib
    return _lib


def load_ref():
    """The reference's matrixMulCPU(float* C, float* A, float* B, int width), or None."""
    global _ref
    if _ref is None:
        so = os.path.join(HERE, "_ref", "libref_matmulcpu.so")
        if not os.path.exists(so):
            return None
        lib = C.CDLL(so)
        fn = lib._Z12matrixMulCPUPfS_S_i
        fn.argtypes = [_p, _p, _p, C.c_int]
        fn.restype = None
        _ref = fn
    return _ref


def _ptr(a: np.ndarray):
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(_p)


def _rows(rows):
    if rows is None:
        return None, None, 0
    r = np.ascontiguousarray(np.asarray(rows, dtype=np.int64))
    return r, _ptr(r), r.size


def num_threads() -> int:
    return int(load().oracle_num_threads())


# ---------------------------------------------------------------- conversions (numpy, vectorised)

def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round to nearest even (finite inputs), the rule of oracle_f32_to_bf16."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def f16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return b.view(np.float16).astype(np.float32)


# ---------------------------------------------------------------- fills (reference hash RNG)

def fill_int8(count: int, seed: int, lo: int = -127, hi: int = 127) -> np.ndarray:
    out = np.empty(count, dtype=np.int8)
    load().oracle_fill_int8(_ptr(out), count, seed, lo, hi)
    return out


def fill_f32(count: int, seed: int, lo: float = -1.0, hi: float = 1.0) -> np.ndarray:
    out = np.empty(count, dtype=np.float32)
    load().oracle_fill_f32(_ptr(out), count, seed, lo, hi)
    return out


def fill_f16(count: int, seed: int, lo: float = -1.0, hi: float = 1.0) -> np.ndarray:
    out = np.empty(count, dtype=np.uint16)
    load().oracle_fill_f16(_ptr(out), count, seed, lo, hi)
    return out


def fill_bf16(count: int, seed: int, lo: float = -1.0, hi: float = 1.0) -> np.ndarray:
    out = np.empty(count, dtype=np.uint16)
    load().oracle_fill_bf16(_ptr(out), count, seed, lo, hi)
    return out


# ---------------------------------------------------------------- product loops

def _out_shape(M, N, layout, rows):
    if rows is not None:
        return (len(rows), N)
    return (M, N) if layout == ROW_MAJOR else (N, M)  # col-major [M,N] == row-major [N,M] storage


def gemm_f32(A, B, M, N, K, layout=ROW_MAJOR, rows=None, acc64=False):
    A = np.ascontiguousarray(A, dtype=np.float32)
    B = np.ascontiguousarray(B, dtype=np.float32)
    keep, rp, nr = _rows(rows)
    out = np.empty(_out_shape(M, N, layout, rows), dtype=np.float64 if acc64 else np.float32)
    fn = load().oracle_gemm_f32_acc64 if acc64 else load().oracle_gemm_f32
    fn(_ptr(out), _ptr(A), _ptr(B), M, N, K, layout, rp, nr)
    return out


def gemm_i8_i32(A, B, M, N, K, layout=ROW_MAJOR, rows=None):
    A = np.ascontiguousarray(A, dtype=np.int8)
    B = np.ascontiguousarray(B, dtype=np.int8)
    keep, rp, nr = _rows(rows)
    out = np.empty(_out_shape(M, N, layout, rows), dtype=np.int32)
    load().oracle_gemm_i8_i32(_ptr(out), _ptr(A), _ptr(B), M, N, K, layout, rp, nr)
    return out


def gemm_h16(A_bits, B_bits, M, N, K, is_bf16, layout=ROW_MAJOR, rows=None):
    """Returns (out16_bits, out32): the rounded 16-bit result and the fp32 sums before rounding."""
    A = np.ascontiguousarray(A_bits, dtype=np.uint16)
    B = np.ascontiguousarray(B_bits, dtype=np.uint16)
    keep, rp, nr = _rows(rows)
    shape = _out_shape(M, N, layout, rows)
    o16 = np.empty(shape, dtype=np.uint16)
    o32 = np.empty(shape, dtype=np.float32)
    load().oracle_gemm_h16(_ptr(o16), _ptr(o32), _ptr(A), _ptr(B), M, N, K, int(is_bf16), layout, rp, nr)
    return o16, o32


def gemm_w8a8_bf16(A, B, row_scale, col_scale, M, N, K, rows=None):
    A = np.ascontiguousarray(A, dtype=np.int8)
    B = np.ascontiguousarray(B, dtype=np.int8)
    rs = np.ascontiguousarray(row_scale, dtype=np.float32)
    cs = np.ascontiguousarray(col_scale, dtype=np.float32)
    keep, rp, nr = _rows(rows)
    out = np.empty(_out_shape(M, N, ROW_MAJOR, rows), dtype=np.uint16)
    load().oracle_gemm_w8a8_bf16(_ptr(out), _ptr(A), _ptr(B), _ptr(rs), _ptr(cs), M, N, K, rp, nr)
    return out


def quantize_absmax(x, along: int):
    """x: [R, C] fp32 row-major; along=0 per-row scales, along=1 per-column scales."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    R, Cc = x.shape
    q = np.empty((R, Cc), dtype=np.int8)
    scale = np.empty(R if along == 0 else Cc, dtype=np.float32)
    load().oracle_quantize_absmax(_ptr(q), _ptr(scale), _ptr(x), R, Cc, along)
    return q, scale


LINEAR_RELU, LINEAR_BIAS_FIRST = 1, 2


def linear_f32(x, w, bias, w_is_out_in=True, relu=False, bias_first=False, fused=True):
    """Fully connected layer of the reference's MNIST networks in fp32 (see oracle_linear_f32).
    x [batch, in]; w [out, in] when w_is_out_in else [in, out]; bias [out] or None."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    w = np.ascontiguousarray(w, dtype=np.float32)
    batch, in_f = x.shape
    out_f = w.shape[0] if w_is_out_in else w.shape[1]
    assert (w.shape[1] if w_is_out_in else w.shape[0]) == in_f
    b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
    y = np.empty((batch, out_f), dtype=np.float32)
    flags = (LINEAR_RELU if relu else 0) | (LINEAR_BIAS_FIRST if bias_first else 0)
    load().oracle_linear_f32(_ptr(y), _ptr(x), _ptr(w), None if b is None else _ptr(b), batch, in_f, out_f,
                             1 if w_is_out_in else 0, flags, 1 if fused else 0)
    return y


def linear_h16(x_bits, w_bits, bias, is_bf16, w_is_out_in=True, relu=False):
    """The same layer on fp16 / bf16 bit patterns; returns (rounded 16-bit bits, fp32 before rounding)."""
    x = np.ascontiguousarray(x_bits, dtype=np.uint16)
    w = np.ascontiguousarray(w_bits, dtype=np.uint16)
    batch, in_f = x.shape
    out_f = w.shape[0] if w_is_out_in else w.shape[1]
    assert (w.shape[1] if w_is_out_in else w.shape[0]) == in_f
    b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
    y16 = np.empty((batch, out_f), dtype=np.uint16)
    y32 = np.empty((batch, out_f), dtype=np.float32)
    load().oracle_linear_h16(_ptr(y16), _ptr(y32), _ptr(x), _ptr(w), None if b is None else _ptr(b), batch, in_f,
                             out_f, 1 if w_is_out_in else 0, LINEAR_RELU if relu else 0, 1 if is_bf16 else 0)
    return y16, y32


def ref_matrix_mul_cpu(A, B, width):
    """The reference's own matrixMulCPU on square row-major fp32 inputs."""
    fn = load_ref()
    if fn is None:
        raise RuntimeError("oracle/_ref/libref_matmulcpu.so was not built (make -C oracle ref)")
    A = np.ascontiguousarray(A, dtype=np.float32)
    B = np.ascontiguousarray(B, dtype=np.float32)
    out = np.empty((width, width), dtype=np.float32)
    fn(_ptr(out), _ptr(A), _ptr(B), width)
    return out
