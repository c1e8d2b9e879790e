/*
 * C++ shims with the names and signatures of the reference's matrix-multiply launch wrappers
 * (TileProgramming/matmulTensor.cu:71-87 and :128-135), implemented on libb200gemm.  A caller
 * written against the reference's wrappers (its thrustensor / thrustTensorBfloat16 /
 * thrustcudacore demos, matmulTensor.cu:140-228) compiles against this header unchanged and runs
 * the tcgen05 kernels instead of the WMMA and shared-memory-tiled ones.
 *
 * Semantics: C = A * B for row-major width x width matrices on the device, fp32 result, enqueued
 * on `stream`.  The `grid` and `block` arguments are accepted and ignored (the library sizes its
 * own launches).  One deliberate difference: the reference's WMMA kernels load B as a
 * column-major fragment from row-major storage (matmulTensor.cu:43, :63), so they multiply by a
 * block-transposed B and fail the demos' own comparison with matrixMulCPU; these shims compute the
 * product that comparison expects.
 *
 * Errors follow the reference's wrappers, which return nothing: a failing call prints the
 * library's message to stderr and leaves C untouched.  `width` times the element size must be a
 * multiple of 16 bytes for the two tensor-core wrappers (the TMA rule of the library).
 */
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdio>

#include "b200gemm.h"

#ifndef MATRIX_SIZE
#define MATRIX_SIZE 1024 /* TileProgramming/matmulTensor.cu:16 */
#endif

namespace b200_tile_detail {
inline void report(int status, const char* who) {
  if (status != B200_OK) std::fprintf(stderr, "%s: b200gemm status %d: %s\n", who, status, b200_last_error());
}
}  // namespace b200_tile_detail

/* TileProgramming/matmulTensor.cu:71-78: half in, float out. */
inline void launchMatrixMulTensorCores(half* A, half* B, float* C, int width = MATRIX_SIZE, dim3 grid = dim3(),
                                       dim3 block = dim3(), cudaStream_t stream = 0) {
  (void)grid;
  (void)block;
  b200_tile_detail::report(
      b200_gemm_16_f32(B200_F16, A, B, C, width, width, width, 0, 0, 0, B200_ROW_MAJOR, stream),
      "launchMatrixMulTensorCores");
}

/* TileProgramming/matmulTensor.cu:80-87: __nv_bfloat16 in, float out. */
inline void launchMatrixMulTensorCoresBfloat16(__nv_bfloat16* A, __nv_bfloat16* B, float* C, int width = MATRIX_SIZE,
                                               dim3 grid = dim3(), dim3 block = dim3(), cudaStream_t stream = 0) {
  (void)grid;
  (void)block;
  b200_tile_detail::report(
      b200_gemm_16_f32(B200_BF16, A, B, C, width, width, width, 0, 0, 0, B200_ROW_MAJOR, stream),
      "launchMatrixMulTensorCoresBfloat16");
}

/* TileProgramming/matmulTensor.cu:128-135: fp32 on the CUDA cores; note the output comes first.
 * Runs the exact-arithmetic FFMA kernel (k ascending, one accumulator), like the kernel it replaces. */
inline void launchMatrixMulCudaCores(float* C, float* A, float* B, int width = MATRIX_SIZE, dim3 grid = dim3(),
                                     dim3 block = dim3(), cudaStream_t stream = 0) {
  (void)grid;
  (void)block;
  b200_tile_detail::report(
      b200_gemm_f32(A, B, C, width, width, width, 0, 0, 0, B200_ROW_MAJOR, B200_F32_FFMA, stream),
      "launchMatrixMulCudaCores");
}
