// The reference's tensor-core demos (TileProgramming/matmulTensor.cu:140-228: thrustTensorBfloat16,
// thrustensor, thrustcudacore) restated as one C++ caller of the launch wrappers in
// include/tile_programming.h: srand(1234), inputs rand()/RAND_MAX in [0, 1] as fp32 and rounded to
// the 16-bit type, width 1024 by default, GPU product through the wrapper, CPU product of the
// UNROUNDED fp32 inputs through the oracle's restatement of matrixMulCPU, element-wise comparison.
//
// The reference's thresholds are absolute (1e-5 for fp16 and fp32, 2e-3 for bf16) on sums near
// width / 4, which 16-bit inputs cannot meet (rounding an input to fp16 alone moves a sum of 1024
// products by about 1e-2); this program reports how many elements meet them and decides on the
// relative Frobenius error instead: <= 1e-3 for fp16 inputs, <= 1e-2 for bf16 inputs (the input
// rounding, 2^-11 and 2^-8 per element, dominates), <= 1e-5 for the fp32 wrapper.
//
// usage: tensor_wrappers_check half|bf16|f32 [width=1024]
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "tile_programming.h"

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

template <typename T>
int upload(const std::vector<T>& h, T** d) {
  CHECK_CUDA(cudaMalloc(reinterpret_cast<void**>(d), h.size() * sizeof(T)));
  CHECK_CUDA(cudaMemcpy(*d, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice));
  return 0;
}

int main(int argc, char** argv) {
  const char* kind = argc > 1 ? argv[1] : "half";
  const int width = argc > 2 ? std::atoi(argv[2]) : MATRIX_SIZE;
  const size_t n = size_t(width) * width;
  std::vector<float> a(n), b(n), c_gpu(n), c_cpu(n);
  std::srand(1234);
  for (size_t i = 0; i < n; ++i) a[i] = std::rand() / static_cast<float>(RAND_MAX);
  for (size_t i = 0; i < n; ++i) b[i] = std::rand() / static_cast<float>(RAND_MAX);

  float* dc = nullptr;
  CHECK_CUDA(cudaMalloc(reinterpret_cast<void**>(&dc), n * sizeof(float)));
  CHECK_CUDA(cudaMemset(dc, 0xff, n * sizeof(float)));
  double tol = 1e-5, ref_eps = 1e-5;
  const char* label = "CUDA Cores";
  if (std::strcmp(kind, "half") == 0) {
    std::vector<half> ah(n), bh(n);
    for (size_t i = 0; i < n; ++i) { ah[i] = __float2half(a[i]); bh[i] = __float2half(b[i]); }
    half *da = nullptr, *db = nullptr;
    if (upload(ah, &da) || upload(bh, &db)) return 2;
    launchMatrixMulTensorCores(da, db, dc, width);
    tol = 1e-3; label = "Tensor Cores";
  } else if (std::strcmp(kind, "bf16") == 0) {
    std::vector<__nv_bfloat16> ah(n), bh(n);
    for (size_t i = 0; i < n; ++i) { ah[i] = __float2bfloat16(a[i]); bh[i] = __float2bfloat16(b[i]); }
    __nv_bfloat16 *da = nullptr, *db = nullptr;
    if (upload(ah, &da) || upload(bh, &db)) return 2;
    launchMatrixMulTensorCoresBfloat16(da, db, dc, width);
    tol = 1e-2; ref_eps = 2e-3; label = "bfloat16 Tensor Cores";
  } else {
    float *da = nullptr, *db = nullptr;
    if (upload(a, &da) || upload(b, &db)) return 2;
    launchMatrixMulCudaCores(dc, da, db, width);
  }
  if (b200_check_device(nullptr) != B200_OK) {
    std::fprintf(stderr, "device check failed: %s\n", b200_last_error());
    return 2;
  }
  CHECK_CUDA(cudaMemcpy(c_gpu.data(), dc, n * sizeof(float), cudaMemcpyDeviceToHost));
  oracle_gemm_f32(c_cpu.data(), a.data(), b.data(), width, width, width, 0, nullptr, 0);

  double num = 0.0, den = 0.0;
  size_t within = 0;
  for (size_t i = 0; i < n; ++i) {
    const double d = double(c_gpu[i]) - double(c_cpu[i]);
    num += d * d;
    den += double(c_cpu[i]) * double(c_cpu[i]);
    if (std::fabs(d) <= ref_eps) ++within;
  }
  const double rel = std::sqrt(num / den);
  std::printf("%s, width %d: relative Frobenius error %.3e (tolerance %.0e); %zu of %zu elements within the "
              "reference's absolute %.0e\n", label, width, rel, tol, within, n, ref_eps);
  if (rel <= tol) {
    std::printf("%s: Matrix multiplication successful!\n", label);
    return 0;
  }
  std::printf("%s: Results do not match!\n", label);
  return 1;
}
