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
  // Accumulators in pairs along n: the inner loop issues packed fp32 FMAs (two per instruction, each an
  // ordinary IEEE fused multiply-add), which halves the issue slots the FMAs take.
  float2 acc2[TM][TN / 2];
  auto acc = [&](int i, int j) -> float& { return (j & 1) ? acc2[i][j >> 1].y : acc2[i][j >> 1].x; };
#pragma unroll
  for (int j = 0; j < TN; ++j) {
    const int n = n0 + (j / 4) * 64 + tx * 4 + (j % 4);
    const float start = (bias_first && n < N) ? __ldg(bias + n) : 0.f;
#pragma unroll
    for (int i = 0; i < TM; ++i) acc(i, j) = start;
  }

  float4 ra[A_LOADS];
  float4 rb[B_NK ? BT_LOADS : B_LOADS];

  // A tile inside the matrices with K in whole slices loads through pointers worked out once, unchecked.
  const bool interior = VEC && m0 + TBM <= M && n0 + TBN <= N && K % BKF == 0;
  const float* pa0 = A + int64_t(m0 + (tid >> 2)) * lda + (tid & 3) * 4;  // load l: 64 rows below load l - 1
  const float* pb0 = B_NK ? B + int64_t(n0 + (tid >> 2)) * ldb + (tid & 3) * 4
                          : B + int64_t(tid / (TBN / 4)) * ldb + n0 + (tid % (TBN / 4)) * 4;
  const int64_t pa_step = 64 * lda, pb_step = (B_NK ? 64 : kSgemmThreads / (TBN / 4)) * ldb;
  auto fetch = [&](int k0) {
    if (interior) {
#pragma unroll
      for (int l = 0; l < A_LOADS; ++l) ra[l] = __ldg(reinterpret_cast<const float4*>(pa0 + l * pa_step + k0));
      if constexpr (B_NK) {
#pragma unroll
        for (int l = 0; l < BT_LOADS; ++l) rb[l] = __ldg(reinterpret_cast<const float4*>(pb0 + l * pb_step + k0));
      } else {
#pragma unroll
        for (int l = 0; l < B_LOADS; ++l)
          rb[l] = __ldg(reinterpret_cast<const float4*>(pb0 + l * pb_step + int64_t(k0) * ldb));
      }
      return;
    }
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
      for (int i = 0; i < TM; ++i) {
        const float2 a2 = make_float2(a[i], a[i]);
#pragma unroll
        for (int j = 0; j < TN / 2; ++j) acc2[i][j] = __ffma2_rn(a2, make_float2(b[2 * j], b[2 * j + 1]), acc2[i][j]);
      }
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
        float v = bias_last ? acc(i, j) + add : acc(i, j);
        acc(i, j) = relu ? fmaxf(0.0f, v) : v;
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
            make_float4(acc(i, g * 4), acc(i, g * 4 + 1), acc(i, g * 4 + 2), acc(i, g * 4 + 3));
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (n + j < N) dst[j] = acc(i, g * 4 + j);
      }
    }
  }
}

// ---------------------------------------------------------------------------- small products: K cut inside a cluster
//
// A product with few tiles cannot fill the machine with whole-K tiles (1024^3 is 128 tiles of
// 128 x 64 for 148 SMs, one 8-warp CTA each).  Here a 64 x 64 tile belongs to a cluster of KS CTAs
// of 64 threads (8 x 8 patch per thread), each summing one range of K in ascending k; the ranges'
// sums then meet in the first CTA through distributed shared memory and are added in range order:
// ((s0 + s1) + s2) + s3.  The result is deterministic; it differs from the single ascending sum in
// rounding only (fewer, shorter chains).  KS x as many CTAs, about seven per SM at 1024^3, keep
// every SM's FP32 pipe fed.
constexpr int kKsThreads = 64;
constexpr int kKsTile = 64;

__device__ __forceinline__ uint32_t ks_cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void ks_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float4 ks_ld_remote(const float* local_smem_ptr, uint32_t rank) {
  const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(local_smem_ptr));
  uint32_t ra;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(a), "r"(rank));
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"(ra)
               : "memory");
  return v;
}

template <bool B_NK, bool VEC>
__global__ void __launch_bounds__(kKsThreads, 6)
sgemm_ffma_ksplit_kernel(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ C, int M,
                         int N, int K, int64_t lda, int64_t ldb, int64_t ldc, int k_per_cta, int ks) {
  constexpr int T = kKsTile, LD = T + kPad;
  // As[2][BKF][LD] then Bs[2][BKF][LD]; after the main loop the same bytes hold this CTA's partial sums.
  __shared__ __align__(16) float sm[4 * BKF * LD];
  float (*As)[BKF][LD] = reinterpret_cast<float (*)[BKF][LD]>(sm);
  float (*Bs)[BKF][LD] = reinterpret_cast<float (*)[BKF][LD]>(sm + 2 * BKF * LD);

  const int tid = threadIdx.x;
  const int tx = tid & 7, ty = tid >> 3;
  const int m0 = blockIdx.y * T, n0 = blockIdx.x * T;
  const uint32_t rank = ks_cluster_rank();
  const int k_begin = int(rank) * k_per_cta;
  const int k_end = min(K, k_begin + k_per_cta);

  float2 acc2[8][4];  // pairs along n for the packed fp32 FMA
  auto acc = [&](int i, int j) -> float& { return (j & 1) ? acc2[i][j >> 1].y : acc2[i][j >> 1].x; };
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc2[i][j] = make_float2(0.f, 0.f);

  float4 ra[4], rb[4];
  // A tile that lies inside the matrices with a K range of whole slices loads through pointers worked out
  // once, without bounds checks: the staging instructions are a quarter of what this small CTA issues.
  const bool interior = VEC && m0 + T <= M && n0 + T <= N && (k_end - k_begin) % BKF == 0;
  // load l of a thread is 16 rows (K-contiguous operand) or 4 k-rows (N-contiguous B) below load l - 1
  const float* pa0 = A + int64_t(m0 + (tid >> 2)) * lda + (tid & 3) * 4;
  const float* pb0 = B_NK ? B + int64_t(n0 + (tid >> 2)) * ldb + (tid & 3) * 4
                          : B + int64_t(tid >> 4) * ldb + n0 + (tid & 15) * 4;
  const int64_t pa_step = 16 * lda, pb_step = (B_NK ? 16 : 4) * ldb;
  auto fetch = [&](int k0) {
    if (interior) {
#pragma unroll
      for (int l = 0; l < 4; ++l) {
        ra[l] = __ldg(reinterpret_cast<const float4*>(pa0 + l * pa_step + k0));
        if constexpr (B_NK) rb[l] = __ldg(reinterpret_cast<const float4*>(pb0 + l * pb_step + k0));
        else rb[l] = __ldg(reinterpret_cast<const float4*>(pb0 + l * pb_step + int64_t(k0) * ldb));
      }
      return;
    }
#pragma unroll
    for (int l = 0; l < 4; ++l) {
      const int idx = tid + l * kKsThreads;  // row = idx / 4, k-quad = idx % 4
      ra[l] = load_k4<VEC>(A, lda, m0 + (idx >> 2), M, k0 + (idx & 3) * 4, k_end);
      if constexpr (B_NK) rb[l] = load_k4<VEC>(B, ldb, n0 + (idx >> 2), N, k0 + (idx & 3) * 4, k_end);
      else rb[l] = load_n4<VEC>(B, ldb, k0 + (idx >> 4), k_end, n0 + (idx & 15) * 4, N);
    }
  };
  auto stash = [&](int buf) {
#pragma unroll
    for (int l = 0; l < 4; ++l) {
      const int idx = tid + l * kKsThreads;
      const int r = idx >> 2, kq = (idx & 3) * 4;
      As[buf][kq + 0][r] = ra[l].x; As[buf][kq + 1][r] = ra[l].y;
      As[buf][kq + 2][r] = ra[l].z; As[buf][kq + 3][r] = ra[l].w;
      if constexpr (B_NK) {
        Bs[buf][kq + 0][r] = rb[l].x; Bs[buf][kq + 1][r] = rb[l].y;
        Bs[buf][kq + 2][r] = rb[l].z; Bs[buf][kq + 3][r] = rb[l].w;
      } else {
        *reinterpret_cast<float4*>(&Bs[buf][idx >> 4][(idx & 15) * 4]) = rb[l];
      }
    }
  };

  const int num_kb = k_end > k_begin ? (k_end - k_begin + BKF - 1) / BKF : 0;
  if (num_kb > 0) {
    fetch(k_begin);
    stash(0);
  }
  __syncthreads();
  for (int kb = 0; kb < num_kb; ++kb) {
    const int buf = kb & 1;
    if (kb + 1 < num_kb) fetch(k_begin + (kb + 1) * BKF);
#pragma unroll
    for (int k = 0; k < BKF; ++k) {
      float a[8], b[8];
#pragma unroll
      for (int g = 0; g < 2; ++g) {
        const float4 va = *reinterpret_cast<const float4*>(&As[buf][k][g * 32 + ty * 4]);
        a[g * 4 + 0] = va.x; a[g * 4 + 1] = va.y; a[g * 4 + 2] = va.z; a[g * 4 + 3] = va.w;
        const float4 vb = *reinterpret_cast<const float4*>(&Bs[buf][k][g * 32 + tx * 4]);
        b[g * 4 + 0] = vb.x; b[g * 4 + 1] = vb.y; b[g * 4 + 2] = vb.z; b[g * 4 + 3] = vb.w;
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float2 a2 = make_float2(a[i], a[i]);
#pragma unroll
        for (int j = 0; j < 4; ++j) acc2[i][j] = __ffma2_rn(a2, make_float2(b[2 * j], b[2 * j + 1]), acc2[i][j]);
      }
    }
    if (kb + 1 < num_kb) {
      stash(buf ^ 1);
      __syncthreads();
    }
  }

  // Meet in the first CTA of the cluster.  part[q][tid] (float4) is conflict-free for writer and reader.
  __syncthreads();  // every thread is done with the operand tiles these bytes held
  float4* part = reinterpret_cast<float4*>(sm);
  if (rank != 0) {
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int g = 0; g < 2; ++g)
        part[(i * 2 + g) * kKsThreads + tid] = make_float4(acc(i, g * 4), acc(i, g * 4 + 1), acc(i, g * 4 + 2), acc(i, g * 4 + 3));
  }
  ks_cluster_sync();
  if (rank == 0) {
    for (int r = 1; r < ks; ++r) {
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int g = 0; g < 2; ++g) {
          const float4 v = ks_ld_remote(reinterpret_cast<const float*>(&part[(i * 2 + g) * kKsThreads + tid]), uint32_t(r));
          acc(i, g * 4 + 0) += v.x; acc(i, g * 4 + 1) += v.y; acc(i, g * 4 + 2) += v.z; acc(i, g * 4 + 3) += v.w;
        }
    }
  }
  ks_cluster_sync();  // the other CTAs' shared memory must outlive the reads above
  if (rank != 0) return;

  const bool vec_out = VEC && (ldc % 4 == 0) && (reinterpret_cast<uintptr_t>(C) % 16 == 0);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int m = m0 + (i / 4) * 32 + ty * 4 + (i % 4);
    if (m >= M) continue;
#pragma unroll
    for (int g = 0; g < 2; ++g) {
      const int n = n0 + g * 32 + tx * 4;
      float* dst = C + int64_t(m) * ldc + n;
      if (vec_out && n + 4 <= N) {
        *reinterpret_cast<float4*>(dst) = make_float4(acc(i, g * 4), acc(i, g * 4 + 1), acc(i, g * 4 + 2), acc(i, g * 4 + 3));
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (n + j < N) dst[j] = acc(i, g * 4 + j);
      }
    }
  }
}

template <bool B_NK>
int launch_ksplit(bool vec, int ks, const float* A, const float* B, float* C, int M, int N, int K, int64_t lda,
                  int64_t ldb, int64_t ldc, cudaStream_t stream) {
  const int k_per_cta = ((K + ks - 1) / ks + BKF - 1) / BKF * BKF;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(unsigned((N + kKsTile - 1) / kKsTile), unsigned((M + kKsTile - 1) / kKsTile), unsigned(ks));
  cfg.blockDim = dim3(kKsThreads);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = unsigned(ks);
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (vec)
    B200_CUDA_TRY(cudaLaunchKernelEx(&cfg, sgemm_ffma_ksplit_kernel<B_NK, true>, A, B, C, M, N, K, lda, ldb, ldc,
                                     k_per_cta, ks));
  else
    B200_CUDA_TRY(cudaLaunchKernelEx(&cfg, sgemm_ffma_ksplit_kernel<B_NK, false>, A, B, C, M, N, K, lda, ldb, ldc,
                                     k_per_cta, ks));
  return B200_OK;
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

int g_ffma_ksplit = -1;  // -1 = automatic, 0 = never, 2 / 4 = that many K ranges whenever the shape allows

template <bool B_NK>
int launch_shape(bool vec, const float* A, const float* B, float* C, int M, int N, int K, int64_t lda, int64_t ldb,
                 int64_t ldc, cudaStream_t stream, const Tail& tail, bool may_split_k) {
  // Few tiles and a long K: cut K inside clusters (plain products only: the fully connected layers
  // keep the single ascending sum that reproduces the reference loops bit for bit).
  if (may_split_k && tail.bias == nullptr && tail.flags == 0 && g_ffma_ksplit != 0 && M <= 65535 * kKsTile) {
    const int64_t tiles64 = int64_t((M + 63) / 64) * ((N + 63) / 64);
    int ks = 0;
    if (g_ffma_ksplit > 0) ks = g_ffma_ksplit;
    else if (tiles64 < 148 && K >= 1024) ks = 4;       // fewer tiles than SMs: four ranges each
    else if (tiles64 <= 2 * 148 && K >= 512) ks = 2;   // 1024^3: 256 tiles x 2 = 512 CTAs of 64 threads: 54.3 us (four ranges: 56.0)
    else if (tiles64 <= 8 * 148 && K >= 512) ks = 2;   // 2048^3: 344 us against 395 us for whole-K 128 x 128 tiles
    if (ks > 1 && K >= ks * BKF) return launch_ksplit<B_NK>(vec, ks, A, B, C, M, N, K, lda, ldb, ldc, stream);
  }
  // Largest tile whose grid still covers the machine (two CTAs fit on an SM): 128x128 once there
  // are at least 148 of them, else 128x64, else 64x64.
  auto tiles = [&](int tbm, int tbn) { return int64_t((M + tbm - 1) / tbm) * ((N + tbn - 1) / tbn); };
  if (tiles(128, 128) >= 148) return launch_tb<128, 128, B_NK>(vec, A, B, C, M, N, K, lda, ldb, ldc, stream, tail);
  if (tiles(128, 64) >= 120) return launch_tb<128, 64, B_NK>(vec, A, B, C, M, N, K, lda, ldb, ldc, stream, tail);
  return launch_tb<64, 64, B_NK>(vec, A, B, C, M, N, K, lda, ldb, ldc, stream, tail);
}

}  // namespace

int set_ffma_ksplit(int ks) {
  if (ks != -1 && ks != 0 && ks != 2 && ks != 4) return fail(B200_ERR_BAD_ARGUMENT, "FFMA K ranges: -1, 0, 2 or 4");
  g_ffma_ksplit = ks;
  return B200_OK;
}

int launch_sgemm_ffma(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K,
                      int64_t lda, int64_t ldb, int64_t ldc, bool b_is_nk, cudaStream_t stream, const Tail& tail,
                      bool may_split_k) {
  if (!A || !B || !C) return fail(B200_ERR_BAD_ARGUMENT, "null matrix pointer");
  if (M <= 0 || N <= 0 || K <= 0) return fail(B200_ERR_BAD_ARGUMENT, "M, N and K must be positive");
  if (M > (1 << 30) || N > (1 << 30) || K > (1 << 30))
    return fail(B200_ERR_TOO_LARGE, "a dimension exceeds 2^30");
  if (lda < K || ldb < (b_is_nk ? K : N) || ldc < N)
    return fail(B200_ERR_BAD_ARGUMENT, "a leading dimension is smaller than the row it spans");
  const bool vec = lda % 4 == 0 && ldb % 4 == 0 && reinterpret_cast<uintptr_t>(A) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(B) % 16 == 0;
  return b_is_nk ? launch_shape<true>(vec, A, B, C, int(M), int(N), int(K), lda, ldb, ldc, stream, tail, may_split_k)
                 : launch_shape<false>(vec, A, B, C, int(M), int(N), int(K), lda, ldb, ldc, stream, tail, may_split_k);
}

}  // namespace b200
