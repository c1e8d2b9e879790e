// C++ caller of the C ABI in the style of the reference's own check (TileProgramming/kernel.cu:117-159):
// fill two width x width fp32 matrices on the host, multiply them on the GPU, multiply them with the CPU
// oracle's restatement of matrixMulCPU, and compare element by element.  Where the reference launches its
// matrixMulTiled kernel (kernel.cu:145-147) this program calls b200_gemm_f32.
//
// The reference's threshold is an absolute 1e-5 on sums of ~width products, which fp32 arithmetic cannot
// meet in either order of rounding (one ulp of a sum near 256 is 3e-5); this program prints how many
// elements pass it and decides on the relative error instead (<= 1e-5 of the Frobenius norm).
//
// usage: tile_check [width=1024] [mode=0 (FFMA) | 1 (3xTF32) | 2 (TF32)]
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "b200gemm.h"

extern "C" void oracle_gemm_f32(float* out, const float* A, const float* B, int64_t M, int64_t N, int64_t K,
                                int layout, const int64_t* rows, int64_t nrows);

#define CHECK_CUDA(call)                                                                        \
  do {                                                                                          \
    cudaError_t s_ = (call);                                                                    \
    if (s_ != cudaSuccess) {                                                                    \
      std::fprintf(stderr, "CUDA error: %s at %s:%d\n", cudaGetErrorString(s_), __FILE__, __LINE__); \
      return 2;                                                                                 \
    }                                                                                           \
  } while (0)

int main(int argc, char** argv) {
  const int width = argc > 1 ? std::atoi(argv[1]) : 1024;
  const int mode = argc > 2 ? std::atoi(argv[2]) : B200_F32_FFMA;
  const size_t n = size_t(width) * width;
  std::vector<float> a(n), b(n), c_gpu(n), c_cpu(n);
  std::srand(1234);  // the reference seeds its tensor-core demos the same way (matmulTensor.cu:148)
  for (size_t i = 0; i < n; ++i) a[i] = std::rand() / static_cast<float>(RAND_MAX);
  for (size_t i = 0; i < n; ++i) b[i] = std::rand() / static_cast<float>(RAND_MAX);

  float *da = nullptr, *db = nullptr, *dc = nullptr;
  CHECK_CUDA(cudaMalloc(&da, n * sizeof(float)));
  CHECK_CUDA(cudaMalloc(&db, n * sizeof(float)));
  CHECK_CUDA(cudaMalloc(&dc, n * sizeof(float)));
  CHECK_CUDA(cudaMemcpy(da, a.data(), n * sizeof(float), cudaMemcpyHostToDevice));
  CHECK_CUDA(cudaMemcpy(db, b.data(), n * sizeof(float), cudaMemcpyHostToDevice));

  int st = b200_gemm_f32(da, db, dc, width, width, width, 0, 0, 0, B200_ROW_MAJOR, mode, nullptr);
  if (st != B200_OK) {
    std::fprintf(stderr, "b200_gemm_f32 failed (%d): %s\n", st, b200_last_error());
    return 2;
  }
  st = b200_check_device(nullptr);
  if (st != B200_OK) {
    std::fprintf(stderr, "device check failed (%d): %s\n", st, b200_last_error());
    return 2;
  }
  CHECK_CUDA(cudaMemcpy(c_gpu.data(), dc, n * sizeof(float), cudaMemcpyDeviceToHost));

  oracle_gemm_f32(c_cpu.data(), a.data(), b.data(), width, width, width, 0, nullptr, 0);

  double num = 0.0, den = 0.0, max_abs = 0.0;
  size_t within_ref_eps = 0;
  for (size_t i = 0; i < n; ++i) {
    const double d = double(c_gpu[i]) - double(c_cpu[i]);
    num += d * d;
    den += double(c_cpu[i]) * double(c_cpu[i]);
    if (std::fabs(d) > max_abs) max_abs = std::fabs(d);
    if (std::fabs(d) <= 1e-5) ++within_ref_eps;
  }
  const double rel = std::sqrt(num / den);
  const double tol = mode == B200_F32_TF32 ? 2e-3 : 1e-5;
  std::printf("width %d mode %d: relative Frobenius error %.3e (tolerance %.0e), max |gpu-cpu| %.3e, "
              "%zu of %zu elements within the reference's absolute 1e-5\n",
              width, mode, rel, tol, max_abs, within_ref_eps, n);
  cudaFree(da);
  cudaFree(db);
  cudaFree(dc);
  if (rel <= tol) {
    std::printf("Matrix multiplication successful! (GPU matches CPU)\n");
    return 0;
  }
  std::printf("Error: Results do not match!\n");
  return 1;
}
