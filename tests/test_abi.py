"""CPU tests of the drop-in boundary: the library builds, loads, and exports every symbol its
headers declare; argument errors are reported as status codes without touching a GPU."""
import ctypes as C
import os
import re
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CUDA_INCLUDE = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "b200gemm.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_all_bound_and_exported(cb):
    from cudaintro_b200 import capi

    names = declared_symbols()
    assert len(names) >= 15
    assert set(names) == set(capi.SIGNATURES), "capi.SIGNATURES must list exactly the header's entry points"
    handle = C.CDLL(capi.LIB_PATH)
    for n in names:
        assert getattr(handle, n) is not None


def test_reference_suite_symbols_are_exported(cb):
    """The mangled names the reference's main.cu links against (quantization/gemm_common.h:64-67)."""
    from cudaintro_b200 import capi

    out = subprocess.run(["nm", "-D", "--defined-only", capi.LIB_PATH], capture_output=True, text=True, check=True).stdout
    for dt in ("bf16", "fp16", "fp32", "int8"):
        assert f"_Z13run_gemm_{dt}P13cublasContext" in out


def test_gemm_result_layout_matches_reference_record(tmp_path):
    """GemmResult is {const char*, uint64_t, double, double}: 32 bytes, fields at 0/8/16/24."""
    src = tmp_path / "t.cpp"
    src.write_text(
        '#include "gemm_common.h"\n#include <cstddef>\n#include <cstdio>\n'
        'int main(){std::printf("%zu %zu %zu %zu %zu",sizeof(GemmResult),offsetof(GemmResult,name),'
        "offsetof(GemmResult,iters),offsetof(GemmResult,secs),offsetof(GemmResult,tflops));}\n")
    exe = tmp_path / "t"
    subprocess.run(["g++", "-std=c++17", "-I", os.path.join(ROOT, "include"), "-I", CUDA_INCLUDE, str(src), "-o",
                    str(exe)], check=True)
    assert subprocess.run([str(exe)], capture_output=True, text=True).stdout.split() == ["32", "0", "8", "16", "24"]


def test_reference_driver_compiles_against_the_stand_in_header_alone(tmp_path, reference_tree):
    """quantization/main.cu:8-31 uses CHECK_CUBLAS, GemmResult and the four run_gemm_* declarations
    of its "gemm_common.h".  A quoted include looks beside the including file first, so the
    reference's file is reached through a symbolic link in an empty directory: the only
    gemm_common.h it can then find is this repository's include/gemm_common.h."""
    link = tmp_path / "main_link.cu"
    os.symlink(os.path.join(reference_tree, "quantization", "main.cu"), link)
    obj = tmp_path / "main.o"
    subprocess.run(["nvcc", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-I",
                    os.path.join(ROOT, "include"), "-c", str(link), "-o", str(obj)], check=True)
    syms = subprocess.run(["nm", "-u", str(obj)], capture_output=True, text=True, check=True).stdout
    for dt in ("bf16", "fp16", "fp32", "int8"):
        assert f"_Z13run_gemm_{dt}P13cublasContext" in syms


def test_error_helpers_print_like_the_reference_and_exit(tmp_path):
    """CHECK_CUDA / CHECK_CUBLAS (quantization/gemm_common.h:37-55): one line
    "<CUDA|cuBLAS> error: <text> at <file>:<line>" on stderr, then exit(EXIT_FAILURE);
    cublas_status_to_string (:10-35) spells the enumerator, unknown codes read CUBLAS_STATUS_UNKNOWN."""
    src = tmp_path / "e.cpp"
    src.write_text(
        '#include "gemm_common.h"\n#include <cstring>\n'
        "int main(int argc, char** argv) {\n"
        '  if (std::strcmp(cublas_status_to_string(CUBLAS_STATUS_ARCH_MISMATCH), "CUBLAS_STATUS_ARCH_MISMATCH")) return 3;\n'
        '  if (std::strcmp(cublas_status_to_string((cublasStatus_t)12345), "CUBLAS_STATUS_UNKNOWN")) return 4;\n'
        "  CHECK_CUBLAS(CUBLAS_STATUS_SUCCESS);\n"
        "  if (argc > 1) CHECK_CUBLAS(CUBLAS_STATUS_NOT_INITIALIZED);\n"
        "  CHECK_CUDA(cudaErrorInvalidValue);\n"
        "  return 0;\n}\n")
    exe = tmp_path / "e"
    cuda_lib = os.path.join(os.path.dirname(CUDA_INCLUDE), "lib64")
    subprocess.run(["g++", "-std=c++17", "-I", os.path.join(ROOT, "include"), "-I", CUDA_INCLUDE, str(src), "-o",
                    str(exe), "-L", cuda_lib, "-lcudart", f"-Wl,-rpath,{cuda_lib}"], check=True)
    r = subprocess.run([str(exe)], capture_output=True, text=True)
    assert r.returncode == 1 and re.fullmatch(r"CUDA error: invalid argument at .*e\.cpp:8\n", r.stderr), r
    r = subprocess.run([str(exe), "x"], capture_output=True, text=True)
    assert r.returncode == 1 and re.fullmatch(r"cuBLAS error: CUBLAS_STATUS_NOT_INITIALIZED at .*e\.cpp:7\n", r.stderr), r


def test_public_header_is_plain_c(tmp_path):
    """include/b200gemm.h is the binding surface for any host language: it must compile as C11 with
    nothing but the standard headers it includes itself."""
    src = tmp_path / "h.c"
    src.write_text('#include "b200gemm.h"\nint main(void) { return (int)B200_OK; }\n')
    subprocess.run(["gcc", "-std=c11", "-Wall", "-Wextra", "-pedantic", "-Werror", "-I", os.path.join(ROOT, "include"),
                    "-fsyntax-only", str(src)], check=True)


def test_bad_arguments_are_status_codes_not_crashes(cb):
    from cudaintro_b200 import capi

    lib = capi.lib
    one = C.c_void_p(16)
    # null pointers / non-positive sizes / unknown enums are rejected before any CUDA call
    assert lib.b200_gemm_i8_i32(None, None, None, 128, 128, 128, 0, 0, 0, 0, None) == 1
    assert b"null" in lib.b200_last_error()
    assert lib.b200_gemm_i8_i32(one, one, one, 0, 128, 128, 0, 0, 0, 0, None) == 1
    assert lib.b200_gemm_bf16(one, one, one, 128, 128, 128, 0, 0, 0, 7, None) == 1
    assert lib.b200_gemm_f32(one, one, one, 8, 8, 8, 0, 0, 0, 0, 9, None) == 1
    assert lib.b200_quantize_absmax(one, one, one, 4, 4, 2, None) == 1
    assert lib.b200_gemm_naive(11, one, one, one, 4, 4, 4, 0, 0, 0, 0, None) == 1
    # fully connected layer: pointers, sizes, weight layout, flags and dtype are checked first
    assert lib.b200_linear(capi.F32, None, one, None, one, 4, 4, 4, 2, 0, 0, None) == 1
    assert lib.b200_linear(capi.F32, one, one, None, one, 4, 0, 4, 2, 0, 0, None) == 1
    assert lib.b200_linear(capi.F32, one, one, None, one, 4, 4, 4, 1, 0, 0, None) == 1   # column-major weights
    assert lib.b200_linear(capi.F32, one, one, None, one, 4, 4, 4, 2, 8, 0, None) == 1   # unknown flag
    assert lib.b200_linear(capi.I8, one, one, None, one, 4, 4, 4, 2, 0, 0, None) == 1
    # alignment rule of the tensor-core entry points: K = 100 int8 elements is not a 16-byte row
    assert lib.b200_gemm_i8_i32(one, one, one, 128, 128, 100, 0, 0, 0, 0, None) == 2
    assert b"16-byte" in lib.b200_last_error()
    assert lib.b200_gemm_bf16(C.c_void_p(8), one, one, 128, 128, 128, 0, 0, 0, 0, None) == 2  # misaligned A
    # leading dimension smaller than the row
    assert lib.b200_gemm_f16(one, one, one, 64, 64, 64, 32, 0, 0, 0, None) == 1


def test_policy_knobs_and_multi_gpu_entry_points_validate_arguments(cb):
    from cudaintro_b200 import capi

    lib = capi.lib
    assert lib.b200_set_tile_policy(5, 0, 0) == 1          # CTA grouping: 0, 1, 2, 3 (the skinny kernel) or 4 (pairs, two row blocks)
    assert lib.b200_set_tile_policy(4, 128, 0) == 1
    assert lib.b200_set_tile_policy(4, 256, 0) == 0
    assert lib.b200_set_tile_policy(3, 64, 0) == 1         # whose tiles are 128, 192 or 256 wide
    assert lib.b200_set_tile_policy(3, 192, 0) == 0
    assert lib.b200_set_tile_policy(2, 128, 0) == 1        # CTA pairs exist for 256-wide tiles only
    assert lib.b200_set_tile_policy(0, 96, 0) == 1
    assert lib.b200_set_tile_policy(0, 0, 100) == 1        # group rows: multiple of 256
    assert lib.b200_set_tile_policy(0, 0, 0) == 0
    one = C.c_void_p(16)
    dests = (C.c_void_p * 9)(*[one] * 9)
    assert lib.b200_gemm_multi(capi.I8, one, one, dests, 9, None, None, 16, 16, 16, 0, 0, 0, None) == 1
    assert lib.b200_gemm_multi(capi.I8, one, one, dests, 0, None, None, 16, 16, 16, 0, 0, 0, None) == 1
    assert lib.b200_gemm_multi(capi.F32, one, one, dests, 1, None, None, 16, 16, 16, 0, 0, 0, None) == 1
    assert lib.b200_gemm_multi(capi.W8A8, one, one, dests, 1, None, None, 16, 16, 16, 0, 0, 0, None) == 1  # no scales
    assert lib.b200_gemm_multicast(capi.I8, one, one, None, None, None, 16, 16, 16, 0, 0, 0, None) == 1
    assert lib.b200_gemm_multicast(capi.F32, one, one, one, None, None, 16, 16, 16, 0, 0, 0, None) == 1
    assert lib.b200_gemm_multicast(capi.BF16, one, one, one, None, None, 16, 20, 16, 0, 0, 0, None) == 2  # ragged rows
    assert lib.b200_peer_marker(dests, 9, 0, 1, None) == 1
    assert lib.b200_peer_marker(dests, 2, 2, 1, None) == 1
    assert lib.b200_peer_marker(None, 2, 0, 1, None) == 1
    assert lib.b200_peer_alloc(0, C.byref(C.c_void_p())) == 1
    assert lib.b200_ipc_export(None, None) == 1 and lib.b200_ipc_import(None, None) == 1
    # host-buffer products against resident weights: pointers, sizes and dtype are checked first
    h = C.c_void_p()
    assert lib.b200_host_weights_upload(capi.I8, None, 16, 16, C.byref(h)) == 1
    assert lib.b200_host_weights_upload(capi.I8, one, 0, 16, C.byref(h)) == 1
    assert lib.b200_host_weights_upload(9, one, 16, 16, C.byref(h)) == 1
    assert lib.b200_gemm_host_weights(None, one, one, 16) == 1
    assert lib.b200_host_weights_free(None) == 0
    # the allocation-free entry point refuses oversized problems before touching the device
    assert lib.b200_gemm_f32_3xtf32_static(one, one, one, 4096, 4096, 4096, 0, 0, 0, 0, None) == 5


def test_no_cpu_fallback_without_device(cb):
    import torch

    if torch.cuda.is_available():
        pytest.skip("this check is for machines without a GPU")
    from cudaintro_b200 import capi

    one = C.c_void_p(16)
    assert capi.lib.b200_sm_count() == 0
    st = capi.lib.b200_gemm_i8_i32(one, one, one, 128, 128, 128, 0, 0, 0, 0, None)
    assert st == 3, "without a device the call must fail with B200_ERR_CUDA, never compute on the CPU"


def test_product_does_not_reference_the_oracle():
    """The shipped package must not import or link the oracle (it is test infrastructure)."""
    pkg = os.path.join(ROOT, "cudaintro_b200")
    for dirpath, _, files in os.walk(pkg):
        if os.path.basename(dirpath) == "build":
            continue
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "liboracle" not in text and "import oracle" not in text and "from oracle" not in text, f
