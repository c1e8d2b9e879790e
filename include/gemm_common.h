/*
 * The four suite entry points of the reference, kept under their original names and C++
 * linkage so that the reference's host driver (quantization/main.cu:8-31) links against
 * libb200gemm without a change.  Interface replaced: quantization/gemm_common.h:57-67.
 *
 * Each call fills two 4096 x 4096 matrices with the reference's index-hash generator, runs one
 * warm-up GEMM, then launches GEMMs back to back for about ten seconds (the clock is read every
 * 256 launches, as in quantization/GEMM_int8.cu:59-78) and reports iterations, seconds and
 * 2*M*N*K*iters / secs / 1e12.  The cuBLAS handle is accepted and not used: the products run on
 * this library's own kernels.  Like the reference, a CUDA failure prints the error with its
 * source position to stderr and ends the process with EXIT_FAILURE.
 *
 * The environment variable GEMM_SUITE_SECONDS shortens or lengthens the ten-second loop.
 *
 * This header can be included instead of, or after, the reference's own gemm_common.h.
 */
#pragma once

#include <stdint.h>

struct cublasContext;
typedef struct cublasContext* cublasHandle_t;

#ifndef B200_GEMM_RESULT_DEFINED
#define B200_GEMM_RESULT_DEFINED
struct GemmResult {
  const char* name; /* "BF16", "FP16", "FP32" or "INT8": a string literal, never freed */
  uint64_t iters;
  double secs;
  double tflops;
};
#endif

GemmResult run_gemm_bf16(cublasHandle_t handle);
GemmResult run_gemm_fp16(cublasHandle_t handle);
GemmResult run_gemm_fp32(cublasHandle_t handle);
GemmResult run_gemm_int8(cublasHandle_t handle);
