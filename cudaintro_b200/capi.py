"""ctypes binding of ``libb200gemm.so`` plus torch-tensor wrappers over it.

Every wrapper ends in exactly one call of the C entry point of the same name
(``include/b200gemm.h``).  Nothing here computes: a missing library raises at import time and a
failing call raises :class:`B200Error` with the library's own message.
"""
from __future__ import annotations

import ctypes as C
import os

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "libb200gemm.so")

ROW_MAJOR, COL_MAJOR_NN, ROW_MAJOR_BT = 0, 1, 2
F32_FFMA, F32_3XTF32, F32_TF32 = 0, 1, 2
I8, F16, BF16, F32, W8A8 = 0, 1, 2, 3, 4

STATUS_NAMES = {0: "OK", 1: "BAD_ARGUMENT", 2: "UNSUPPORTED", 3: "CUDA", 4: "DEVICE_WAIT", 5: "TOO_LARGE"}

# name -> (restype, argtypes); must list every symbol include/b200gemm.h declares
_i64, _p, _int = C.c_int64, C.c_void_p, C.c_int
SIGNATURES = {
    "b200_last_error": (C.c_char_p, []),
    "b200_version": (C.c_char_p, []),
    "b200_sm_count": (_int, []),
    "b200_set_tile_policy": (_int, [_int, _int, _int]),
    "b200_check_device": (_int, [_p]),
    "b200_gemm_i8_i32": (_int, [_p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64, _int, _p]),
    "b200_gemm_bf16": (_int, [_p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64, _int, _p]),
    "b200_gemm_f16": (_int, [_p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64, _int, _p]),
    "b200_gemm_16_f32": (_int, [_int, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64, _int, _p]),
    "b200_gemm_f32": (_int, [_p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64, _int, _int, _p]),
    "b200_gemm_f32_3xtf32_static": (_int, [_p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64, _int, _p]),
    "b200_gemm_w8a8_bf16": (_int, [_p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64, _p]),
    "b200_quantize_absmax": (_int, [_p, _p, _p, _i64, _i64, _int, _p]),
    "b200_fill_int8": (_int, [_p, _i64, C.c_uint64, _int, _int, _p]),
    "b200_fill_f16": (_int, [_p, _i64, C.c_uint64, C.c_float, C.c_float, _p]),
    "b200_fill_bf16": (_int, [_p, _i64, C.c_uint64, C.c_float, C.c_float, _p]),
    "b200_fill_f32": (_int, [_p, _i64, C.c_uint64, C.c_float, C.c_float, _p]),
    "b200_gemm_naive": (_int, [_int, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64, _int, _p]),
    "b200_linear": (_int, [_int, _p, _p, _p, _p, _i64, _i64, _i64, _int, _int, _int, _p]),
    "b200_gemm_host": (_int, [_int, _p, _p, _p, _i64, _i64, _i64, _int]),
    "b200_host_release": (_int, []),
    "b200_host_weights_upload": (_int, [_int, _p, _i64, _i64, C.POINTER(C.c_void_p)]),
    "b200_gemm_host_weights": (_int, [_p, _p, _p, _i64]),
    "b200_host_weights_free": (_int, [_p]),
    "b200_set_store_policy": (_int, [_int]),
    "b200_set_dependent_launch": (_int, [_int]),
    "b200_test_lose_arrival": (_int, [_i64, C.c_uint64]),
    "b200_set_l2_hints": (_int, [_int]),
    "b200_set_3xtf32_path": (_int, [_int]),
    "b200_set_ffma_k_ranges": (_int, [_int]),
    "b200_gemm_multi": (_int, [_int, _p, _p, C.POINTER(C.c_void_p), _int, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64,
                               _p]),
    "b200_gemm_multicast": (_int, [_int, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64, _p]),
    "b200_peer_marker": (_int, [C.POINTER(C.c_void_p), _int, _int, C.c_uint32, _p]),
    "b200_peer_alloc": (_int, [C.c_size_t, C.POINTER(C.c_void_p)]),
    "b200_peer_free": (_int, [_p]),
    "b200_ipc_export": (_int, [_p, _p]),
    "b200_ipc_import": (_int, [_p, C.POINTER(C.c_void_p)]),
    "b200_ipc_close": (_int, [_p]),
    "b200_time_gemm": (_int, [_int, _p, _p, _p, _p, _p, _i64, _i64, _i64, _int, _int, _int,
                              C.POINTER(C.c_float), _p]),
}


class B200Error(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"b200gemm status {status} ({STATUS_NAMES.get(status, '?')}): {message}")
        self.status = status


def _load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m cudaintro_b200.build` "
            "(there is no fallback implementation)")
    handle = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(handle, name)  # AttributeError if the library lacks a declared symbol
        fn.restype = res
        fn.argtypes = args
    return handle


lib = _load()


def _check(status: int) -> None:
    if status != 0:
        raise B200Error(status, lib.b200_last_error().decode())


def _stream():
    import torch

    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _dims(a, b, layout):
    """(M, N, K) from the storage shapes of A and B under `layout`."""
    if layout == ROW_MAJOR:      # a [M,K], b [K,N]
        (M, K), (K2, N) = a.shape, b.shape
    elif layout == ROW_MAJOR_BT:  # a [M,K], b [N,K]
        (M, K), (N, K2) = a.shape, b.shape
    elif layout == COL_MAJOR_NN:  # column-major M x K is stored as [K,M]; K x N as [N,K]
        (K, M), (N, K2) = a.shape, b.shape
    else:
        raise ValueError(f"unknown layout {layout}")
    if K != K2:
        raise ValueError(f"inner dimensions differ: {K} vs {K2}")
    return M, N, K


def _out_shape(M, N, layout):
    return (N, M) if layout == COL_MAJOR_NN else (M, N)


def _gemm(fn, a, b, out_dtype, layout, out, extra=()):
    import torch

    assert a.is_cuda and b.is_cuda and a.is_contiguous() and b.is_contiguous()
    M, N, K = _dims(a, b, layout)
    if out is None:
        out = torch.empty(_out_shape(M, N, layout), dtype=out_dtype, device=a.device)
    assert out.is_contiguous() and out.dtype == out_dtype and tuple(out.shape) == _out_shape(M, N, layout)
    with torch.cuda.device(a.device):
        _check(fn(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, 0, 0, 0, layout, *extra, _stream()))
    return out


def gemm_i8_i32(a, b, layout=ROW_MAJOR, out=None):
    import torch

    assert a.dtype == torch.int8 and b.dtype == torch.int8
    return _gemm(lib.b200_gemm_i8_i32, a, b, torch.int32, layout, out)


def gemm_bf16(a, b, layout=ROW_MAJOR, out=None):
    import torch

    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    return _gemm(lib.b200_gemm_bf16, a, b, torch.bfloat16, layout, out)


def gemm_f16(a, b, layout=ROW_MAJOR, out=None):
    import torch

    assert a.dtype == torch.float16 and b.dtype == torch.float16
    return _gemm(lib.b200_gemm_f16, a, b, torch.float16, layout, out)


def gemm_16_f32(a, b, layout=ROW_MAJOR, out=None):
    """fp16 or bf16 operands, fp32 accumulate, fp32 result (the sums, unrounded)."""
    import torch

    assert a.dtype == b.dtype and a.dtype in (torch.float16, torch.bfloat16)
    code = F16 if a.dtype == torch.float16 else BF16
    return _gemm(lambda *args: lib.b200_gemm_16_f32(code, *args), a, b, torch.float32, layout, out)


def gemm_f32(a, b, layout=ROW_MAJOR, mode=F32_FFMA, out=None):
    import torch

    assert a.dtype == torch.float32 and b.dtype == torch.float32
    return _gemm(lib.b200_gemm_f32, a, b, torch.float32, layout, out, extra=(mode,))


def gemm_w8a8_bf16(a, b, row_scale, col_scale, out=None):
    import torch

    assert a.dtype == torch.int8 and b.dtype == torch.int8
    assert row_scale.dtype == torch.float32 and col_scale.dtype == torch.float32
    M, N, K = _dims(a, b, ROW_MAJOR)
    assert row_scale.numel() == M and col_scale.numel() == N
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
    with torch.cuda.device(a.device):
        _check(lib.b200_gemm_w8a8_bf16(a.data_ptr(), b.data_ptr(), row_scale.data_ptr(), col_scale.data_ptr(),
                                       out.data_ptr(), M, N, K, 0, 0, 0, _stream()))
    return out


def quantize_absmax(x, along: int):
    """x: [R, C] fp32 CUDA tensor -> (q int8 [R, C], scale fp32 [R] or [C])."""
    import torch

    assert x.dtype == torch.float32 and x.is_cuda and x.is_contiguous() and x.dim() == 2
    R, Cc = x.shape
    q = torch.empty((R, Cc), dtype=torch.int8, device=x.device)
    scale = torch.empty(R if along == 0 else Cc, dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        _check(lib.b200_quantize_absmax(x.data_ptr(), q.data_ptr(), scale.data_ptr(), R, Cc, along, _stream()))
    return q, scale


_DTYPE_CODE = None


def _code(dtype):
    import torch

    global _DTYPE_CODE
    if _DTYPE_CODE is None:
        _DTYPE_CODE = {torch.int8: I8, torch.float16: F16, torch.bfloat16: BF16, torch.float32: F32}
    return _DTYPE_CODE[dtype]


LINEAR_RELU, LINEAR_BIAS_FIRST = 1, 2


def linear(x, w, bias=None, w_layout=ROW_MAJOR_BT, relu=False, bias_first=False, mode=F32_FFMA, out=None):
    """Fused fully connected layer: act(x @ W^T + bias) for W [out, in] (ROW_MAJOR_BT, the default) or
    act(x @ W + bias) for W [in, out] (ROW_MAJOR).  x, W: fp32, fp16 or bf16 CUDA tensors; bias fp32."""
    import torch

    assert x.dtype == w.dtype and x.dim() == 2 and w.dim() == 2
    batch, in_f = x.shape
    out_f = w.shape[0] if w_layout == ROW_MAJOR_BT else w.shape[1]
    assert (w.shape[1] if w_layout == ROW_MAJOR_BT else w.shape[0]) == in_f
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.numel() == out_f
    if out is None:
        out = torch.empty((batch, out_f), dtype=x.dtype, device=x.device)
    flags = (LINEAR_RELU if relu else 0) | (LINEAR_BIAS_FIRST if bias_first else 0)
    with torch.cuda.device(x.device):
        _check(lib.b200_linear(_code(x.dtype), x.data_ptr(), w.data_ptr(), 0 if bias is None else bias.data_ptr(),
                               out.data_ptr(), batch, in_f, out_f, w_layout, flags, mode, _stream()))
    return out


def gemm_naive(a, b, layout=ROW_MAJOR):
    """One-thread-per-element validation GEMM: int32 for int8 inputs, unrounded fp32 sums otherwise."""
    import torch

    M, N, K = _dims(a, b, layout)
    out = torch.empty(_out_shape(M, N, layout), dtype=torch.int32 if a.dtype == torch.int8 else torch.float32,
                      device=a.device)
    with torch.cuda.device(a.device):
        _check(lib.b200_gemm_naive(_code(a.dtype), a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, 0, 0, 0,
                                   layout, _stream()))
    return out


def fill(t, seed: int, lo=None, hi=None):
    """Fills a CUDA tensor in place with the reference suite's index-hash generator."""
    import torch

    n = t.numel()
    with torch.cuda.device(t.device):
        if t.dtype == torch.int8:
            _check(lib.b200_fill_int8(t.data_ptr(), n, seed, -127 if lo is None else lo, 127 if hi is None else hi,
                                      _stream()))
        else:
            fn = {torch.float16: lib.b200_fill_f16, torch.bfloat16: lib.b200_fill_bf16,
                  torch.float32: lib.b200_fill_f32}[t.dtype]
            _check(fn(t.data_ptr(), n, seed, -1.0 if lo is None else lo, 1.0 if hi is None else hi, _stream()))
    return t


def set_tile_policy(cta_group: int = 0, tile_n: int = 0, group_rows: int = 0) -> None:
    """Forces single CTAs (1), CTA pairs (2), CTA pairs with two row blocks per CTA (4) or the K-split
    cluster kernel for skinny products (3), a tile width and the rows per tile-order group; zeros restore
    the automatic choice."""
    _check(lib.b200_set_tile_policy(cta_group, tile_n, group_rows))


def check_device() -> None:
    """Synchronises the current stream and raises if a kernel gave up a bounded wait."""
    _check(lib.b200_check_device(_stream()))


def time_gemm(what, a, b, out, M, N, K, layout=ROW_MAJOR, iters=1, row_scale=None, col_scale=None,
              f32_mode=F32_FFMA) -> float:
    """Milliseconds for `iters` back-to-back launches (CUDA events inside the library)."""
    ms = C.c_float(0.0)
    _check(lib.b200_time_gemm(what, a.data_ptr(), b.data_ptr(), out.data_ptr(),
                              0 if row_scale is None else row_scale.data_ptr(),
                              0 if col_scale is None else col_scale.data_ptr(), M, N, K, layout, f32_mode, iters,
                              C.byref(ms), _stream()))
    return float(ms.value)


def gemm_host(dtype_code: int, a_np, b_np, c_np, M, N, K, layout=ROW_MAJOR) -> None:
    """Host-buffer entry point: numpy (or any buffer with ctypes data) in, result written to c_np."""
    _check(lib.b200_gemm_host(dtype_code, a_np.ctypes.data, b_np.ctypes.data, c_np.ctypes.data, M, N, K, layout))


class HostWeights:
    """A row-major [K, N] weight matrix uploaded once from host memory (numpy array or pinned torch CPU
    tensor) to the current device; ``matmul(a, out)`` then multiplies host buffers against it."""

    def __init__(self, dtype_code: int, b_host, K: int, N: int):
        self._h = C.c_void_p()
        ptr = b_host.ctypes.data if hasattr(b_host, "ctypes") else b_host.data_ptr()
        _check(lib.b200_host_weights_upload(dtype_code, ptr, K, N, C.byref(self._h)))
        self.K, self.N = K, N

    def matmul(self, a_host, c_host, M: int) -> None:
        pa = a_host.ctypes.data if hasattr(a_host, "ctypes") else a_host.data_ptr()
        pc = c_host.ctypes.data if hasattr(c_host, "ctypes") else c_host.data_ptr()
        _check(lib.b200_gemm_host_weights(self._h, pa, pc, M))

    def close(self) -> None:
        if self._h:
            _check(lib.b200_host_weights_free(self._h))
            self._h = C.c_void_p()


def set_store_policy(register_stores: bool = False) -> None:
    """True: C is written straight from registers; False: automatic (staged TMA stores when aligned)."""
    _check(lib.b200_set_store_policy(1 if register_stores else 0))


def gemm_multicast(what: int, a, b, mc_ptr: int, M: int, N: int, K: int, row_scale=None, col_scale=None) -> None:
    """Row-major GEMM written once to the multicast address `mc_ptr` of the [M, N] slab (every GPU bound
    to the multicast object receives it).  `what` is I8, F16, BF16 or W8A8."""
    import torch

    with torch.cuda.device(a.device):
        _check(lib.b200_gemm_multicast(what, a.data_ptr(), b.data_ptr(), C.c_void_p(int(mc_ptr)),
                                       0 if row_scale is None else row_scale.data_ptr(),
                                       0 if col_scale is None else col_scale.data_ptr(), M, N, K, 0, 0, 0, _stream()))


def gemm_multi(what: int, a, b, dest_ptrs, M: int, N: int, K: int, row_scale=None, col_scale=None) -> None:
    """Row-major GEMM written to every pointer of `dest_ptrs` (device addresses of the [M, N] slab in
    each destination buffer, local or peer).  `what` is I8, F16, BF16 or W8A8."""
    import torch

    arr = (C.c_void_p * len(dest_ptrs))(*[C.c_void_p(int(p)) for p in dest_ptrs])
    with torch.cuda.device(a.device):
        _check(lib.b200_gemm_multi(what, a.data_ptr(), b.data_ptr(), arr, len(dest_ptrs),
                                   0 if row_scale is None else row_scale.data_ptr(),
                                   0 if col_scale is None else col_scale.data_ptr(), M, N, K, 0, 0, 0, _stream()))
