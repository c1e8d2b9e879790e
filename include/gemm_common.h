/*
 * Stand-in for the reference suite's quantization/gemm_common.h (lines 10-67 there): the result
 * record, the four suite entry points and the error helpers the reference's host driver uses.
 * The reference's quantization/main.cu:8-31 compiles against this header alone, unchanged, and
 * links against libb200gemm, which exports the four entry points under their original C++ names.
 * Include it INSTEAD of the reference's header (both define struct GemmResult, so a translation
 * unit cannot see the two of them).
 *
 * What each entry point does here: fills two 4096 x 4096 matrices with the reference's index-hash
 * generator, runs one warm-up GEMM, then launches GEMMs back to back for about ten seconds (the
 * clock is read every 256 launches, as in quantization/GEMM_int8.cu:59-78) and reports iterations,
 * seconds and 2*M*N*K*iters / secs / 1e12.  The cuBLAS handle is accepted and not used: the
 * products run on this library's own kernels.  Like the reference, a CUDA failure prints the
 * error with its source position to stderr and ends the process with EXIT_FAILURE.
 *
 * Environment: GEMM_SUITE_SECONDS shortens or lengthens the ten-second loop;
 * GEMM_SUITE_FP32_MODE = tf32 (default) | 3xtf32 | ffma picks the arithmetic of the FP32 line.
 */
#pragma once

#include <cublas_v2.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>

/* Name of a cuBLAS status, spelled like the enumerator (quantization/gemm_common.h:10-35 returns
 * the same strings; anything it does not list reads "CUBLAS_STATUS_UNKNOWN" there and here). */
inline const char* cublas_status_to_string(cublasStatus_t status) {
  static const struct { cublasStatus_t code; const char* text; } names[] = {
#define B200_STATUS_NAME(x) {x, #x}
      B200_STATUS_NAME(CUBLAS_STATUS_SUCCESS),          B200_STATUS_NAME(CUBLAS_STATUS_NOT_INITIALIZED),
      B200_STATUS_NAME(CUBLAS_STATUS_ALLOC_FAILED),     B200_STATUS_NAME(CUBLAS_STATUS_INVALID_VALUE),
      B200_STATUS_NAME(CUBLAS_STATUS_ARCH_MISMATCH),    B200_STATUS_NAME(CUBLAS_STATUS_MAPPING_ERROR),
      B200_STATUS_NAME(CUBLAS_STATUS_EXECUTION_FAILED), B200_STATUS_NAME(CUBLAS_STATUS_INTERNAL_ERROR),
      B200_STATUS_NAME(CUBLAS_STATUS_NOT_SUPPORTED),    B200_STATUS_NAME(CUBLAS_STATUS_LICENSE_ERROR),
#undef B200_STATUS_NAME
  };
  for (const auto& n : names)
    if (n.code == status) return n.text;
  return "CUBLAS_STATUS_UNKNOWN";
}

/* The reference's error policy (quantization/gemm_common.h:37-55): one line on stderr,
 * "<library> error: <what> at <file>:<line>", then exit(EXIT_FAILURE).  No status is returned. */
[[noreturn]] inline void b200_suite_die(const char* library, const char* what, const char* file, int line) {
  std::fflush(stdout);
  std::fprintf(stderr, "%s error: %s at %s:%d\n", library, what, file, line);
  std::fflush(stderr);
  std::exit(EXIT_FAILURE);
}

#define CHECK_CUDA(call)                                                                  \
  do {                                                                                    \
    const cudaError_t b200_rc_ = (call);                                                  \
    if (b200_rc_ != cudaSuccess) b200_suite_die("CUDA", cudaGetErrorString(b200_rc_), __FILE__, __LINE__); \
  } while (0)

#define CHECK_CUBLAS(call)                                                                \
  do {                                                                                    \
    const cublasStatus_t b200_rc_ = (call);                                               \
    if (b200_rc_ != CUBLAS_STATUS_SUCCESS)                                                \
      b200_suite_die("cuBLAS", cublas_status_to_string(b200_rc_), __FILE__, __LINE__);   \
  } while (0)

/* quantization/gemm_common.h:57-62.  32 bytes: name@0, iters@8, secs@16, tflops@24. */
struct GemmResult {
  const char* name; /* "BF16", "FP16", "FP32" or "INT8": a string literal, never freed */
  uint64_t iters;
  double secs;
  double tflops;
};

/* quantization/gemm_common.h:64-67, bodies in cudaintro_b200/csrc/legacy_suite.cu. */
GemmResult run_gemm_bf16(cublasHandle_t handle);
GemmResult run_gemm_fp16(cublasHandle_t handle);
GemmResult run_gemm_fp32(cublasHandle_t handle);
GemmResult run_gemm_int8(cublasHandle_t handle);
