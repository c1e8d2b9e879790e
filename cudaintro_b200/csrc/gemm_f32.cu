// fp32 GEMM on the CUDA cores: C[M,N] = A[M,K] * B with B as [K,N] (N contiguous) or [N,K]
// (K contiguous).  Register-tiled FFMA: a 256-thread CTA owns a TBM x TBN tile of C, each thread a
// (TBM/16) x (TBN/16) patch held in registers; A and B tiles of 16 k-values are staged through
// double-buffered shared memory (A transposed on the way in so that both operands are read as
// float4 along the thread's patch).  Every element of C accumulates its products in ascending k
// into one fp32 accumulator, the order of the reference's CPU loop
// (TileProgramming/tensor_utils.cu:35-45); the only difference is that the GPU fuses each
// multiply-add.  No alignment requirement: edges and unaligned rows take a scalar, bounds-checked
// load path.
#include "internal.h"

namespace b200 {
namespace {

constexpr int BKF = 16;
constexpr int kSgemmThreads = 256;
constexpr int kPad = 4;  // floats of padding per shared-memory row: keeps float4 alignment, spreads banks

// Loads 4 consecutive k-values of row `r` of a [rows, K] K-contiguous matrix (zero outside).
template <bool VEC>
__device__ __forceinline__ float4 load_k4(const float* __restrict__ base, int64_t ld, int r, int rows,
                                          int k, int K) {
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
  if (r < rows) {
    const float* p = base + int64_t(r) * ld + k;
    if (VEC && k + 4 <= K) {
      v = __ldg(reinterpret_cast<const float4*>(p));
    } else {
      if (k + 0 < K) v.x = __ldg(p + 0);
      if (k + 1 < K) v.y = __ldg(p + 1);
      if (k + 2 < K) v.z = __ldg(p + 2);
      if (k + 3 < K) v.w = __ldg(p + 3);
    }
  }
  return v;
}

// Loads 4 consecutive n-values of k-row `k` of a [K, N] N-contiguous matrix (zero outside).
template <bool VEC>
__device__ __forceinline__ float4 load_n4(const float* __restrict__ base, int64_t ld, int k, int K,
                                          int n, int N) {
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
  if (k < K) {
    const float* p = base + int64_t(k) * ld + n;
    if (VEC && n + 4 <= N) {
      v = __ldg(reinterpret_cast<const float4*>(p));
    } else {
      if (n + 0 < N) v.x = __ldg(p + 0);
      if (n + 1 < N) v.y = __ldg(p + 1);
      if (n + 2 < N) v.z = __ldg(p + 2);
      if (n + 3 < N) v.w = __ldg(p + 3);
    }
  }
  return v;
}

template <int TBM, int TBN, bool B_NK, bool VEC>
__global__ void __launch_bounds__(kSgemmThreads, 2)
sgemm_ffma_kernel(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ C, int M,
                  int N, int K, int64_t lda, int64_t ldb, int64_t ldc, const float* __restrict__ bias, int flags) {
  constexpr int TM = TBM / 16, TN = TBN / 16;  // patch per thread (8 or 4 on each side)
  constexpr int GM = TM / 4, GN = TN / 4;      // float4 groups per side, 64 rows / columns apart
  constexpr int A_LOADS = TBM * 4 / kSgemmThreads;  // float4 loads of a K-contiguous operand per thread
  constexpr int BT_LOADS = TBN * 4 / kSgemmThreads;
  constexpr int B_LOADS = BKF * (TBN / 4) / kSgemmThreads;

  __shared__ __align__(16) float As[2][BKF][TBM + kPad];
  __shared__ __align__(16) float Bs[2][BKF][TBN + kPad];

  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * TBM, n0 = blockIdx.x * TBN;

  // Fully connected layer: the sum of column n either starts from bias[n] or gets it added at the
  // end; both orders exist in the reference and round differently.
  const bool bias_first = bias != nullptr && (flags & B200_LINEAR_BIAS_FIRST) != 0;
  const bool bias_last = bias != nullptr && !bias_first;
  const bool relu = (flags & B200_LINEAR_RELU) != 0;
  float acc[TM][TN];
#pragma unroll
  for (int j = 0; j < TN; ++j) {
    const int n = n0 + (j / 4) * 64 + tx * 4 + (j % 4);
    const float start = (bias_first && n < N) ? __ldg(bias + n) : 0.f;
#pragma unroll
    for (int i = 0; i < TM; ++i) acc[i][j] = start;
  }

  float4 ra[A_LOADS];
  float4 rb[B_NK ? BT_LOADS : B_LOADS];

  auto fetch = [&](int k0) {
#pragma unroll
    for (int l = 0; l < A_LOADS; ++l) {
      int idx = tid + l * kSgemmThreads;  // row = idx / 4, k-quad = idx % 4
      ra[l] = load_k4<VEC>(A, lda, m0 + (idx >> 2), M, k0 + (idx & 3) * 4, K);
    }
    if constexpr (B_NK) {
#pragma unroll
      for (int l = 0; l < BT_LOADS; ++l) {
        int idx = tid + l * kSgemmThreads;
        rb[l] = load_k4<VEC>(B, ldb, n0 + (idx >> 2), N, k0 + (idx & 3) * 4, K);
      }
    } else {
#pragma unroll
      for (int l = 0; l < B_LOADS; ++l) {
        int idx = tid + l * kSgemmThreads;  // k-row = idx / (TBN/4), n-quad = idx % (TBN/4)
        rb[l] = load_n4<VEC>(B, ldb, k0 + idx / (TBN / 4), K, n0 + (idx % (TBN / 4)) * 4, N);
      }
    }
  };
  auto stash = [&](int buf) {
#pragma unroll
    for (int l = 0; l < A_LOADS; ++l) {
      int idx = tid + l * kSgemmThreads;
      int r = idx >> 2, kq = (idx & 3) * 4;
      As[buf][kq + 0][r] = ra[l].x;
      As[buf][kq + 1][r] = ra[l].y;
      As[buf][kq + 2][r] = ra[l].z;
      As[buf][kq + 3][r] = ra[l].w;
    }
    if constexpr (B_NK) {
#pragma unroll
      for (int l = 0; l < BT_LOADS; ++l) {
        int idx = tid + l * kSgemmThreads;
        int r = idx >> 2, kq = (idx & 3) * 4;
        Bs[buf][kq + 0][r] = rb[l].x;
        Bs[buf][kq + 1][r] = rb[l].y;
        Bs[buf][kq + 2][r] = rb[l].z;
        Bs[buf][kq + 3][r] = rb[l].w;
      }
    } else {
#pragma unroll
      for (int l = 0; l < B_LOADS; ++l) {
        int idx = tid + l * kSgemmThreads;
        *reinterpret_cast<float4*>(&Bs[buf][idx / (TBN / 4)][(idx % (TBN / 4)) * 4]) = rb[l];
      }
    }
  };

  const int num_kb = (K + BKF - 1) / BKF;
  fetch(0);
  stash(0);
  __syncthreads();

  for (int kb = 0; kb < num_kb; ++kb) {
    const int buf = kb & 1;
    if (kb + 1 < num_kb) fetch((kb + 1) * BKF);
#pragma unroll
    for (int k = 0; k < BKF; ++k) {
      float a[TM], b[TN];
#pragma unroll
      for (int g = 0; g < GM; ++g) {
        float4 va = *reinterpret_cast<const float4*>(&As[buf][k][g * 64 + ty * 4]);
        a[g * 4 + 0] = va.x; a[g * 4 + 1] = va.y; a[g * 4 + 2] = va.z; a[g * 4 + 3] = va.w;
      }
#pragma unroll
      for (int g = 0; g < GN; ++g) {
        float4 vb = *reinterpret_cast<const float4*>(&Bs[buf][k][g * 64 + tx * 4]);
        b[g * 4 + 0] = vb.x; b[g * 4 + 1] = vb.y; b[g * 4 + 2] = vb.z; b[g * 4 + 3] = vb.w;
      }
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    if (kb + 1 < num_kb) {
      stash(buf ^ 1);
      __syncthreads();
    }
  }

  if (bias_last || relu) {
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + (j / 4) * 64 + tx * 4 + (j % 4);
      const float add = (bias_last && n < N) ? __ldg(bias + n) : 0.f;
#pragma unroll
      for (int i = 0; i < TM; ++i) {
        float v = bias_last ? acc[i][j] + add : acc[i][j];
        acc[i][j] = relu ? fmaxf(0.0f, v) : v;
      }
    }
  }
  const bool vec_out = VEC && (ldc % 4 == 0) && (reinterpret_cast<uintptr_t>(C) % 16 == 0);
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    int m = m0 + (i / 4) * 64 + ty * 4 + (i % 4);
    if (m >= M) continue;
#pragma unroll
    for (int g = 0; g < GN; ++g) {
      int n = n0 + g * 64 + tx * 4;
      float* dst = C + int64_t(m) * ldc + n;
      if (vec_out && n + 4 <= N) {
        *reinterpret_cast<float4*>(dst) =
            make_float4(acc[i][g * 4], acc[i][g * 4 + 1], acc[i][g * 4 + 2], acc[i][g * 4 + 3]);
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (n + j < N) dst[j] = acc[i][g * 4 + j];
      }
    }
  }
}

template <int TBM, int TBN, bool B_NK>
int launch_tb(bool vec, const float* A, const float* B, float* C, int M, int N, int K, int64_t lda,
              int64_t ldb, int64_t ldc, cudaStream_t stream, const Tail& tail) {
  dim3 grid((N + TBN - 1) / TBN, (M + TBM - 1) / TBM);
  if (grid.y > 65535) return fail(B200_ERR_TOO_LARGE, "fp32 GEMM: too many row tiles");
  if (vec)
    sgemm_ffma_kernel<TBM, TBN, B_NK, true><<<grid, kSgemmThreads, 0, stream>>>(A, B, C, M, N, K, lda, ldb, ldc,
                                                                                tail.bias, tail.flags);
  else
    sgemm_ffma_kernel<TBM, TBN, B_NK, false><<<grid, kSgemmThreads, 0, stream>>>(A, B, C, M, N, K, lda, ldb, ldc,
                                                                                 tail.bias, tail.flags);
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}

template <bool B_NK>
int launch_shape(bool vec, const float* A, const float* B, float* C, int M, int N, int K, int64_t lda, int64_t ldb,
                 int64_t ldc, cudaStream_t stream, const Tail& tail) {
  // Largest tile whose grid still covers the machine (two CTAs fit on an SM): 128x128 once there
  // are at least 148 of them, else 128x64, else 64x64.
  auto tiles = [&](int tbm, int tbn) { return int64_t((M + tbm - 1) / tbm) * ((N + tbn - 1) / tbn); };
  if (tiles(128, 128) >= 148) return launch_tb<128, 128, B_NK>(vec, A, B, C, M, N, K, lda, ldb, ldc, stream, tail);
  if (tiles(128, 64) >= 120) return launch_tb<128, 64, B_NK>(vec, A, B, C, M, N, K, lda, ldb, ldc, stream, tail);
  return launch_tb<64, 64, B_NK>(vec, A, B, C, M, N, K, lda, ldb, ldc, stream, tail);
}

}  // namespace

int launch_sgemm_ffma(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K,
                      int64_t lda, int64_t ldb, int64_t ldc, bool b_is_nk, cudaStream_t stream, const Tail& tail) {
  if (!A || !B || !C) return fail(B200_ERR_BAD_ARGUMENT, "null matrix pointer");
  if (M <= 0 || N <= 0 || K <= 0) return fail(B200_ERR_BAD_ARGUMENT, "M, N and K must be positive");
  if (M > (1 << 30) || N > (1 << 30) || K > (1 << 30))
    return fail(B200_ERR_TOO_LARGE, "a dimension exceeds 2^30");
  if (lda < K || ldb < (b_is_nk ? K : N) || ldc < N)
    return fail(B200_ERR_BAD_ARGUMENT, "a leading dimension is smaller than the row it spans");
  const bool vec = lda % 4 == 0 && ldb % 4 == 0 && reinterpret_cast<uintptr_t>(A) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(B) % 16 == 0;
  return b_is_nk ? launch_shape<true>(vec, A, B, C, int(M), int(N), int(K), lda, ldb, ldc, stream, tail)
                 : launch_shape<false>(vec, A, B, C, int(M), int(N), int(K), lda, ldb, ldc, stream, tail);
}

}  // namespace b200
