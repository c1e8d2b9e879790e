// Small SIMT kernels around the GEMMs: the reference's input fills, the validation ("naive")
// GEMM, and the absmax int8 quantiser.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "internal.h"

namespace b200 {
namespace {

// ------------------------------------------------------------------ fills
// element i = one LCG step of (i ^ seed); quantization/GEMM_int8.cu:8-19 and siblings.
__device__ __forceinline__ uint64_t fill_hash(int64_t idx, uint64_t seed) {
  uint64_t x = static_cast<uint64_t>(idx) ^ seed;
  return x * 2862933555777941757ULL + 3037000493ULL;
}
__device__ __forceinline__ float fill_unit(int64_t idx, uint64_t seed, float lo, float hi) {
  float r = __fdiv_rn(static_cast<float>((fill_hash(idx, seed) >> 11) & 0xFFFFFF), 16777215.0f);
  // `lo + r * (hi - lo)` as nvcc compiles it in the reference: one fused multiply-add
  return fmaf(r, __fsub_rn(hi, lo), lo);
}

__global__ void fill_int8_kernel(int8_t* data, int64_t count, uint64_t seed, int lo, int hi) {
  int64_t stride = int64_t(gridDim.x) * blockDim.x;
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += stride) {
    int r = static_cast<int>((fill_hash(i, seed) >> 11) & 0xFFFF);
    data[i] = static_cast<int8_t>(lo + (r % (hi - lo + 1)));
  }
}
template <typename T>
__global__ void fill_float_kernel(T* data, int64_t count, uint64_t seed, float lo, float hi) {
  int64_t stride = int64_t(gridDim.x) * blockDim.x;
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += stride) {
    float v = fill_unit(i, seed, lo, hi);
    if constexpr (sizeof(T) == 4) data[i] = v;
    else if constexpr (std::is_same<T, __half>::value) data[i] = __float2half_rn(v);
    else data[i] = __float2bfloat16_rn(v);
  }
}

int fill_grid(int64_t count) {
  int64_t blocks = (count + 255) / 256;
  return int(blocks > 148 * 16 ? 148 * 16 : (blocks < 1 ? 1 : blocks));
}

// ------------------------------------------------------------------ validation GEMM
__device__ __forceinline__ float widen(int8_t v) { return float(v); }
__device__ __forceinline__ float widen(__half v) { return __half2float(v); }
__device__ __forceinline__ float widen(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float widen(float v) { return v; }

// One thread per element of C; k ascending; products and sums rounded separately (like the CPU
// loop) for the floating-point types, exact int32 for int8.
template <typename T, typename Acc>
__global__ void naive_gemm_kernel(const T* __restrict__ A, const T* __restrict__ B, Acc* __restrict__ C,
                                  int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc,
                                  int layout) {
  int64_t n = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  int64_t m = int64_t(blockIdx.y) * blockDim.y + threadIdx.y;
  if (layout == B200_COL_MAJOR_NN) {  // make consecutive threads walk the contiguous index of C
    int64_t t = n; n = m; m = t;
  }
  if (m >= M || n >= N) return;
  Acc acc = 0;
  for (int64_t k = 0; k < K; ++k) {
    T a = layout == B200_COL_MAJOR_NN ? A[m + k * lda] : A[m * lda + k];
    T b = layout == B200_ROW_MAJOR ? B[k * ldb + n] : (layout == B200_COL_MAJOR_NN ? B[k + n * ldb] : B[n * ldb + k]);
    if constexpr (std::is_same<Acc, int32_t>::value) acc += int32_t(a) * int32_t(b);
    else acc = __fadd_rn(acc, __fmul_rn(widen(a), widen(b)));
  }
  if (layout == B200_COL_MAJOR_NN) C[m + n * ldc] = acc;
  else C[m * ldc + n] = acc;
}

// ------------------------------------------------------------------ quantiser
// q = clamp(rint(x / scale), -127, 127) with the IEEE quotient.  The quotient is first
// approximated by x * (1 / scale), which is within two units in the last place of it; the
// rounded integer can only differ when that approximation lies next to a rounding tie (k + 0.5),
// and only then is the division carried out.  The result is the same bits as dividing always.
__device__ __forceinline__ int quant_one(float x, float s, float inv_s) {
  float t = x * inv_s;
  float r = rintf(t);
  if (fabsf(fabsf(t - r) - 0.5f) < 1e-3f) r = rintf(__fdiv_rn(x, s));
  r = fminf(fmaxf(r, -127.f), 127.f);
  return static_cast<int>(r);
}
__device__ __forceinline__ uint32_t quant_pack4(float4 v, float4 s, float4 inv) {
  uint32_t a = uint32_t(quant_one(v.x, s.x, inv.x)) & 0xffu, b = uint32_t(quant_one(v.y, s.y, inv.y)) & 0xffu;
  uint32_t c = uint32_t(quant_one(v.z, s.z, inv.z)) & 0xffu, d = uint32_t(quant_one(v.w, s.w, inv.w)) & 0xffu;
  return a | (b << 8) | (c << 16) | (d << 24);
}
__device__ __forceinline__ float absmax4(float m, float4 v) {
  return fmaxf(fmaxf(m, fmaxf(fabsf(v.x), fabsf(v.y))), fmaxf(fabsf(v.z), fabsf(v.w)));
}

constexpr int kQuantThreads = 256;
constexpr int kRowCache = 8;  // float4 per thread kept in registers between the two passes of a row

__device__ __forceinline__ float block_max(float v, float* red) {
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
  if (threadIdx.x < 32)
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  if (threadIdx.x == 0) red[0] = v;
  __syncthreads();
  v = red[0];
  __syncthreads();
  return v;
}

// Per-row scales: one CTA per row.  VEC: the row is read as float4 (C % 4 == 0, 16-byte aligned
// rows); the first kRowCache float4 of every thread stay in registers, so rows of up to
// 256 * 8 * 4 = 8192 elements are read from memory once.  4 B read, 1 B written per element.
template <bool VEC>
__global__ void __launch_bounds__(kQuantThreads, 4)
quantize_rows_kernel(const float* __restrict__ x, int8_t* __restrict__ q, float* __restrict__ scale, int64_t R,
                     int64_t C) {
  __shared__ float red[32];
  for (int64_t r = blockIdx.x; r < R; r += gridDim.x) {
    const float* xr = x + r * C;
    int8_t* qr = q + r * C;
    float amax = 0.f;
    if constexpr (VEC) {
      const float4* x4 = reinterpret_cast<const float4*>(xr);
      const int64_t n4 = C >> 2;
      float4 cache[kRowCache];
#pragma unroll
      for (int i = 0; i < kRowCache; ++i) {
        int64_t j = threadIdx.x + int64_t(i) * kQuantThreads;
        cache[i] = j < n4 ? __ldg(x4 + j) : make_float4(0.f, 0.f, 0.f, 0.f);
        amax = absmax4(amax, cache[i]);
      }
      for (int64_t j = threadIdx.x + int64_t(kRowCache) * kQuantThreads; j < n4; j += kQuantThreads)
        amax = absmax4(amax, __ldg(x4 + j));
      amax = block_max(amax, red);
      const float s = amax > 0.f ? __fdiv_rn(amax, 127.0f) : 1.0f;
      const float inv = __fdiv_rn(1.0f, s);
      if (threadIdx.x == 0) scale[r] = s;
      const float4 s4 = make_float4(s, s, s, s), i4 = make_float4(inv, inv, inv, inv);
      uint32_t* q4 = reinterpret_cast<uint32_t*>(qr);
#pragma unroll
      for (int i = 0; i < kRowCache; ++i) {
        int64_t j = threadIdx.x + int64_t(i) * kQuantThreads;
        if (j < n4) q4[j] = quant_pack4(cache[i], s4, i4);
      }
      for (int64_t j = threadIdx.x + int64_t(kRowCache) * kQuantThreads; j < n4; j += kQuantThreads)
        q4[j] = quant_pack4(__ldg(x4 + j), s4, i4);
    } else {
      for (int64_t c = threadIdx.x; c < C; c += blockDim.x) amax = fmaxf(amax, fabsf(xr[c]));
      amax = block_max(amax, red);
      const float s = amax > 0.f ? __fdiv_rn(amax, 127.0f) : 1.0f;
      const float inv = __fdiv_rn(1.0f, s);
      if (threadIdx.x == 0) scale[r] = s;
      for (int64_t c = threadIdx.x; c < C; c += blockDim.x) qr[c] = static_cast<int8_t>(quant_one(xr[c], s, inv));
    }
  }
}

// Per-column scales.  A CTA covers 256 * VW consecutive columns and a band of rows; each thread
// owns VW columns (a float4 when VW = 4), so a warp reads and writes whole contiguous segments
// and keeps several independent loads in flight.
//   pass 1: partial column maxima folded into `amax` with an integer atomicMax (|x| >= 0, so the
//           bit pattern of a float orders like an unsigned integer); `amax` is zero on entry.
//   pass 2: scale = amax / 127 in place, then a second sweep that quantises.
template <int VW>
__global__ void __launch_bounds__(kQuantThreads)
col_absmax_kernel(const float* __restrict__ x, uint32_t* __restrict__ amax, int64_t R, int64_t C,
                  int64_t rows_per_band) {
  const int64_t c = (int64_t(blockIdx.x) * kQuantThreads + threadIdx.x) * VW;
  if (c >= C) return;
  const int64_t r0 = int64_t(blockIdx.y) * rows_per_band;
  const int64_t r1 = r0 + rows_per_band < R ? r0 + rows_per_band : R;
  if constexpr (VW == 4) {
    float4 m = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
    for (int64_t r = r0; r < r1; ++r) {
      float4 v = __ldg(reinterpret_cast<const float4*>(x + r * C + c));
      m.x = fmaxf(m.x, fabsf(v.x)); m.y = fmaxf(m.y, fabsf(v.y));
      m.z = fmaxf(m.z, fabsf(v.z)); m.w = fmaxf(m.w, fabsf(v.w));
    }
    atomicMax(amax + c + 0, __float_as_uint(m.x));
    atomicMax(amax + c + 1, __float_as_uint(m.y));
    atomicMax(amax + c + 2, __float_as_uint(m.z));
    atomicMax(amax + c + 3, __float_as_uint(m.w));
  } else {
    float m = 0.f;
    for (int64_t r = r0; r < r1; ++r) m = fmaxf(m, fabsf(x[r * C + c]));
    atomicMax(amax + c, __float_as_uint(m));
  }
}
__global__ void col_scale_kernel(float* __restrict__ scale, int64_t C) {
  int64_t c = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float v = scale[c];
  scale[c] = v > 0.f ? __fdiv_rn(v, 127.0f) : 1.0f;
}
template <int VW>
__global__ void __launch_bounds__(kQuantThreads)
quantize_cols_kernel(const float* __restrict__ x, int8_t* __restrict__ q, const float* __restrict__ scale,
                     int64_t R, int64_t C, int64_t rows_per_band) {
  const int64_t c = (int64_t(blockIdx.x) * kQuantThreads + threadIdx.x) * VW;
  if (c >= C) return;
  const int64_t r0 = int64_t(blockIdx.y) * rows_per_band;
  const int64_t r1 = r0 + rows_per_band < R ? r0 + rows_per_band : R;
  if constexpr (VW == 4) {
    const float4 s = *reinterpret_cast<const float4*>(scale + c);
    const float4 inv = make_float4(__fdiv_rn(1.0f, s.x), __fdiv_rn(1.0f, s.y), __fdiv_rn(1.0f, s.z),
                                   __fdiv_rn(1.0f, s.w));
#pragma unroll 4
    for (int64_t r = r0; r < r1; ++r) {
      float4 v = __ldg(reinterpret_cast<const float4*>(x + r * C + c));
      *reinterpret_cast<uint32_t*>(q + r * C + c) = quant_pack4(v, s, inv);
    }
  } else {
    const float s = scale[c];
    const float inv = __fdiv_rn(1.0f, s);
    for (int64_t r = r0; r < r1; ++r) q[r * C + c] = static_cast<int8_t>(quant_one(x[r * C + c], s, inv));
  }
}

}  // namespace

int launch_naive(int dtype, const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K,
                 int64_t lda, int64_t ldb, int64_t ldc, int layout, cudaStream_t stream) {
  if (!A || !B || !C) return fail(B200_ERR_BAD_ARGUMENT, "null matrix pointer");
  if (M <= 0 || N <= 0 || K <= 0) return fail(B200_ERR_BAD_ARGUMENT, "M, N and K must be positive");
  dim3 block(32, 8);
  int64_t fast = layout == B200_COL_MAJOR_NN ? M : N, slow = layout == B200_COL_MAJOR_NN ? N : M;
  dim3 grid(unsigned((fast + 31) / 32), unsigned((slow + 7) / 8));
  if (grid.y > 65535) return fail(B200_ERR_TOO_LARGE, "validation GEMM: too many rows");
  switch (dtype) {
    case B200_I8:
      naive_gemm_kernel<int8_t, int32_t><<<grid, block, 0, stream>>>(
          static_cast<const int8_t*>(A), static_cast<const int8_t*>(B), static_cast<int32_t*>(C), M, N, K,
          lda, ldb, ldc, layout);
      break;
    case B200_F16:
      naive_gemm_kernel<__half, float><<<grid, block, 0, stream>>>(
          static_cast<const __half*>(A), static_cast<const __half*>(B), static_cast<float*>(C), M, N, K, lda,
          ldb, ldc, layout);
      break;
    case B200_BF16:
      naive_gemm_kernel<__nv_bfloat16, float><<<grid, block, 0, stream>>>(
          static_cast<const __nv_bfloat16*>(A), static_cast<const __nv_bfloat16*>(B), static_cast<float*>(C), M,
          N, K, lda, ldb, ldc, layout);
      break;
    case B200_F32:
      naive_gemm_kernel<float, float><<<grid, block, 0, stream>>>(
          static_cast<const float*>(A), static_cast<const float*>(B), static_cast<float*>(C), M, N, K, lda, ldb,
          ldc, layout);
      break;
    default:
      return fail(B200_ERR_BAD_ARGUMENT, "unknown dtype %d", dtype);
  }
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}

}  // namespace b200

using namespace b200;

extern "C" int b200_fill_int8(int8_t* data, int64_t count, uint64_t seed, int lo, int hi, void* stream) {
  if (!data || count < 0 || hi < lo) return fail(B200_ERR_BAD_ARGUMENT, "fill: bad argument");
  if (count == 0) return B200_OK;
  fill_int8_kernel<<<fill_grid(count), 256, 0, static_cast<cudaStream_t>(stream)>>>(data, count, seed, lo, hi);
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}
extern "C" int b200_fill_f16(void* data, int64_t count, uint64_t seed, float lo, float hi, void* stream) {
  if (!data || count < 0) return fail(B200_ERR_BAD_ARGUMENT, "fill: bad argument");
  if (count == 0) return B200_OK;
  fill_float_kernel<__half><<<fill_grid(count), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__half*>(data), count, seed, lo, hi);
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}
extern "C" int b200_fill_bf16(void* data, int64_t count, uint64_t seed, float lo, float hi, void* stream) {
  if (!data || count < 0) return fail(B200_ERR_BAD_ARGUMENT, "fill: bad argument");
  if (count == 0) return B200_OK;
  fill_float_kernel<__nv_bfloat16><<<fill_grid(count), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(data), count, seed, lo, hi);
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}
extern "C" int b200_fill_f32(float* data, int64_t count, uint64_t seed, float lo, float hi, void* stream) {
  if (!data || count < 0) return fail(B200_ERR_BAD_ARGUMENT, "fill: bad argument");
  if (count == 0) return B200_OK;
  fill_float_kernel<float><<<fill_grid(count), 256, 0, static_cast<cudaStream_t>(stream)>>>(data, count, seed,
                                                                                           lo, hi);
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}

extern "C" int b200_quantize_absmax(const float* x, int8_t* q, float* scale, int64_t R, int64_t C, int along,
                                    void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!x || !q || !scale) return fail(B200_ERR_BAD_ARGUMENT, "quantize: null pointer");
  if (R <= 0 || C <= 0) return fail(B200_ERR_BAD_ARGUMENT, "quantize: R and C must be positive");
  const bool vec = C % 4 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0 && reinterpret_cast<uintptr_t>(q) % 4 == 0;
  if (along == 0) {
    int grid = int(R < 148 * 16 ? R : 148 * 16);
    if (vec) quantize_rows_kernel<true><<<grid, kQuantThreads, 0, stream>>>(x, q, scale, R, C);
    else quantize_rows_kernel<false><<<grid, kQuantThreads, 0, stream>>>(x, q, scale, R, C);
  } else if (along == 1) {
    // The scale buffer doubles as the integer amax accumulator of pass 1.
    B200_CUDA_TRY(cudaMemsetAsync(scale, 0, sizeof(float) * C, stream));
    const bool vec_cols = vec && reinterpret_cast<uintptr_t>(scale) % 16 == 0;
    const int vw = vec_cols ? 4 : 1;
    const int64_t col_groups = (C + int64_t(kQuantThreads) * vw - 1) / (int64_t(kQuantThreads) * vw);
    int64_t bands = (148 * 16 + col_groups - 1) / col_groups;  // about 16 CTAs per SM in total
    if (bands > (R + 7) / 8) bands = (R + 7) / 8;
    if (bands < 1) bands = 1;
    if (bands > 65535) bands = 65535;
    const int64_t rows_per_band = (R + bands - 1) / bands;
    dim3 grid(unsigned(col_groups), unsigned((R + rows_per_band - 1) / rows_per_band));
    if (vec_cols) {
      col_absmax_kernel<4><<<grid, kQuantThreads, 0, stream>>>(x, reinterpret_cast<uint32_t*>(scale), R, C, rows_per_band);
      col_scale_kernel<<<unsigned((C + 255) / 256), 256, 0, stream>>>(scale, C);
      quantize_cols_kernel<4><<<grid, kQuantThreads, 0, stream>>>(x, q, scale, R, C, rows_per_band);
    } else {
      col_absmax_kernel<1><<<grid, kQuantThreads, 0, stream>>>(x, reinterpret_cast<uint32_t*>(scale), R, C, rows_per_band);
      col_scale_kernel<<<unsigned((C + 255) / 256), 256, 0, stream>>>(scale, C);
      quantize_cols_kernel<1><<<grid, kQuantThreads, 0, stream>>>(x, q, scale, R, C, rows_per_band);
    }
  } else {
    return fail(B200_ERR_BAD_ARGUMENT, "quantize: along must be 0 (rows) or 1 (columns)");
  }
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}
