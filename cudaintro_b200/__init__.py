"""cudaintro_b200 — B200 (sm_100a) quantized GEMM suite behind a C ABI.

The product is ``libb200gemm.so`` (``include/b200gemm.h``); this package loads it with ctypes
and offers thin wrappers that take torch CUDA tensors, used by the tests and the bench.  Torch
only provides device memory and streams here.  There is no CPU path: if the library cannot be
loaded, the first use of any wrapper raises, and every call on a machine without a GPU returns
an error status that the wrappers turn into :class:`B200Error`.

The binding (:mod:`cudaintro_b200.capi`) is imported on first attribute access, so that
``python -m cudaintro_b200.build`` can (re)build the library before anything tries to load it.
"""
import importlib

_CAPI_NAMES = (
    "B200Error", "COL_MAJOR_NN", "F32_3XTF32", "F32_FFMA", "F32_TF32", "ROW_MAJOR", "ROW_MAJOR_BT", "check_device", "fill",
    "gemm_16_f32", "gemm_bf16", "gemm_f16", "gemm_f32", "gemm_host", "gemm_i8_i32", "gemm_naive", "gemm_w8a8_bf16", "lib", "linear",
    "quantize_absmax", "set_tile_policy", "time_gemm",
)


def __getattr__(name):
    if name in _CAPI_NAMES:
        return getattr(importlib.import_module(".capi", __name__), name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
