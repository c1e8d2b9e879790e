// The reference suite's four benchmark bodies (quantization/GEMM_{bf16,fp16,fp32,int8}.cu),
// rebuilt on this library's kernels.  Same symbols, same protocol, same result record; the
// cublasGemmEx call in the middle is replaced by the matching b200_gemm_* entry point with the
// column-major NN layout the reference passes to cuBLAS (lda = M, ldb = K, ldc = M).
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "../../include/gemm_common.h"
#include "internal.h"

namespace {

// Print-and-exit error policy of the reference (quantization/gemm_common.h:37-55).
#define SUITE_CUDA(call)                                                                         \
  do {                                                                                           \
    cudaError_t s__ = (call);                                                                    \
    if (s__ != cudaSuccess) {                                                                    \
      std::fprintf(stderr, "CUDA error: %s at %s:%d\n", cudaGetErrorString(s__), __FILE__, __LINE__); \
      std::exit(EXIT_FAILURE);                                                                   \
    }                                                                                            \
  } while (0)
#define SUITE_B200(call)                                                                         \
  do {                                                                                           \
    int s__ = (call);                                                                            \
    if (s__ != B200_OK) {                                                                        \
      std::fprintf(stderr, "b200gemm error %d: %s at %s:%d\n", s__, b200_last_error(), __FILE__, __LINE__); \
      std::exit(EXIT_FAILURE);                                                                   \
    }                                                                                            \
  } while (0)

double suite_seconds() {
  const char* s = std::getenv("GEMM_SUITE_SECONDS");
  if (s && *s) {
    double v = std::atof(s);
    if (v > 0.0) return v;
  }
  return 10.0;
}

constexpr int64_t kDim = 4096;  // M = N = K in all four bodies

// GEMM_SUITE_FP32_MODE = ffma | 3xtf32 | tf32.  The reference asks cuBLAS for tensor-op math on fp32
// data (quantization/GEMM_fp32.cu:49-54 with the handle in CUBLAS_TENSOR_OP_MATH, main.cu:11), which
// on this hardware runs at tf32 precision; "tf32" is therefore the like-for-like default, "3xtf32"
// keeps fp32 accuracy on the tensor cores, "ffma" is exact fp32 arithmetic on the CUDA cores.
int suite_fp32_mode() {
  const char* s = std::getenv("GEMM_SUITE_FP32_MODE");
  if (s && std::strcmp(s, "ffma") == 0) return B200_F32_FFMA;
  if (s && std::strcmp(s, "3xtf32") == 0) return B200_F32_3XTF32;
  return B200_F32_TF32;
}

GemmResult run_suite(const char* name, int dtype, size_t in_elem, size_t out_elem, uint64_t seed_a,
                     uint64_t seed_b) {
  const int64_t M = kDim, N = kDim, K = kDim;
  void *a = nullptr, *b = nullptr, *c = nullptr;
  SUITE_CUDA(cudaMalloc(&a, size_t(M * K) * in_elem));
  SUITE_CUDA(cudaMalloc(&b, size_t(K * N) * in_elem));
  SUITE_CUDA(cudaMalloc(&c, size_t(M * N) * out_elem));

  switch (dtype) {
    case B200_I8:
      SUITE_B200(b200_fill_int8(static_cast<int8_t*>(a), M * K, seed_a, -127, 127, nullptr));
      SUITE_B200(b200_fill_int8(static_cast<int8_t*>(b), K * N, seed_b, -127, 127, nullptr));
      break;
    case B200_F16:
      SUITE_B200(b200_fill_f16(a, M * K, seed_a, -1.0f, 1.0f, nullptr));
      SUITE_B200(b200_fill_f16(b, K * N, seed_b, -1.0f, 1.0f, nullptr));
      break;
    case B200_BF16:
      SUITE_B200(b200_fill_bf16(a, M * K, seed_a, -1.0f, 1.0f, nullptr));
      SUITE_B200(b200_fill_bf16(b, K * N, seed_b, -1.0f, 1.0f, nullptr));
      break;
    default:
      SUITE_B200(b200_fill_f32(static_cast<float*>(a), M * K, seed_a, -1.0f, 1.0f, nullptr));
      SUITE_B200(b200_fill_f32(static_cast<float*>(b), K * N, seed_b, -1.0f, 1.0f, nullptr));
      break;
  }

  const int fp32_mode = suite_fp32_mode();
  auto gemm = [&]() {
    switch (dtype) {
      case B200_I8:
        return b200_gemm_i8_i32(static_cast<const int8_t*>(a), static_cast<const int8_t*>(b),
                                static_cast<int32_t*>(c), M, N, K, M, K, M, B200_COL_MAJOR_NN, nullptr);
      case B200_F16: return b200_gemm_f16(a, b, c, M, N, K, M, K, M, B200_COL_MAJOR_NN, nullptr);
      case B200_BF16: return b200_gemm_bf16(a, b, c, M, N, K, M, K, M, B200_COL_MAJOR_NN, nullptr);
      default:
        return b200_gemm_f32(static_cast<const float*>(a), static_cast<const float*>(b), static_cast<float*>(c),
                             M, N, K, M, K, M, B200_COL_MAJOR_NN, fp32_mode, nullptr);
    }
  };

  SUITE_B200(gemm());  // warm-up
  SUITE_CUDA(cudaDeviceSynchronize());

  const double budget = suite_seconds();
  auto start = std::chrono::steady_clock::now();
  auto now = start;
  uint64_t iters = 0;
  while (std::chrono::duration<double>(now - start).count() < budget) {
    SUITE_B200(gemm());
    ++iters;
    if ((iters & 0xFF) == 0) {
      SUITE_CUDA(cudaDeviceSynchronize());
      now = std::chrono::steady_clock::now();
    }
  }
  SUITE_CUDA(cudaDeviceSynchronize());
  auto end = std::chrono::steady_clock::now();
  SUITE_B200(b200_check_device(nullptr));
  const double secs = std::chrono::duration<double>(end - start).count();
  const double per_iter = 2.0 * double(M) * double(N) * double(K);
  const double tflops = per_iter * double(iters) / (secs * 1.0e12);

  SUITE_CUDA(cudaFree(c));
  SUITE_CUDA(cudaFree(a));
  SUITE_CUDA(cudaFree(b));
  return {name, iters, secs, tflops};
}

}  // namespace

// Seeds: quantization/GEMM_bf16.cu:44-45, GEMM_fp16.cu:44-45, GEMM_fp32.cu:42-43, GEMM_int8.cu:44-45.
GemmResult run_gemm_bf16(cublasHandle_t) { return run_suite("BF16", B200_BF16, 2, 2, 0x1234U, 0x9876U); }
GemmResult run_gemm_fp16(cublasHandle_t) { return run_suite("FP16", B200_F16, 2, 2, 0x2234U, 0x8876U); }
GemmResult run_gemm_fp32(cublasHandle_t) { return run_suite("FP32", B200_F32, 4, 4, 0x3234U, 0x7776U); }
GemmResult run_gemm_int8(cublasHandle_t) { return run_suite("INT8", B200_I8, 1, 4, 0x4234U, 0x6676U); }
