/*
 * CPU oracle for the quantized GEMM suite.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the arithmetic the reference defines for its GEMM path so
 * that the CUDA kernels can be checked against it.  Nothing in the shipped library may call
 * it: only the tests, the smoke check and the bench's cpu-baseline leg load it.
 *
 * What it follows in the reference (paths inside the reference project):
 *   - TileProgramming/tensor_utils.cu:35-45  matrixMulCPU: row-major C = A*B, for each (i,j)
 *     `sum = 0; for k: sum += A[i][k]*B[k][j]` in fp32, multiply and add rounded separately.
 *   - quantization/GEMM_int8.cu:8-19, GEMM_fp32.cu:7-17, GEMM_fp16.cu:8-19, GEMM_bf16.cu:8-19
 *     the index-hash fills that make the suite's inputs.
 *   - quantization/GEMM_{int8,fp16,bf16,fp32}.cu:51-56 the cublasGemmEx calls: column-major,
 *     no transposes, alpha = 1, beta = 0; int8 x int8 -> int32, fp16/bf16 with fp32 compute and
 *     16-bit output, fp32.  cuBLAS itself is a closed library that is not part of the reference
 *     tree; what is restated here is the mathematical definition of those calls with the
 *     accumulation order of matrixMulCPU (k ascending, one accumulator).
 *
 * Parity status: the fp32, int8, fp16 and bf16 product loops are pinned against outputs of the
 * reference's own matrixMulCPU (compiled unmodified from the reference file, see
 * oracle/Makefile) through the fixtures under tests/golden/.  The fills are pinned by
 * known-answer vectors computed from the reference formulas.  The per-row / per-column scaled
 * int8 path (W8A8) and the quantiser have no counterpart in the reference: parity unpinned for
 * those two; they are defined here.
 *   - MNIST/mnist_kernels.cu:87-102 (fullyConnectedForwardKernel) and :78-84
 *     (reluActivationKernel); the variants that start the sum from the bias,
 *     MNIST/mnist_cnn_kernels.cu:136-149 and MNIST/mnist_nn.cu:10-48 (weights stored [in][out]
 *     there).  These are device kernels in files that include OpenCV headers (not in the image),
 *     so they can be neither compiled nor run where this oracle is built: parity unpinned for
 *     the fully connected layer; oracle_linear_* restate the loops, with the multiply-add fused
 *     as nvcc's default contraction makes it in device code.
 *
 * Loop order.  The product loops run i, then k, then j over a row of accumulators.  Every
 * output element still receives its products in ascending k into a single accumulator, so the
 * results are bit-identical to the i,j,k order of matrixMulCPU; the inner loop just walks B
 * along a row instead of down a column.  Build with -ffp-contract=off so that no multiply-add
 * is fused: the reference's loop rounds the product and the sum separately.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_ROW_MAJOR 0    /* C[m][n] = sum_k A[m][k] * B[k][n], all row-major            */
#define ORACLE_COL_MAJOR_NN 1 /* C[m+n*M] = sum_k A[m+k*M] * B[k+n*K]  (the cuBLAS NN call)  */

int oracle_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

void oracle_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

/* ------------------------------------------------------------------ 16-bit float conversions */

static inline float bits_to_f32(uint32_t u) {
  float f;
  memcpy(&f, &u, 4);
  return f;
}
static inline uint32_t f32_to_bits(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  return u;
}

float oracle_bf16_to_f32(uint16_t h) { return bits_to_f32((uint32_t)h << 16); }

/* round-to-nearest-even, NaN kept quiet: what __float2bfloat16 does */
uint16_t oracle_f32_to_bf16(float f) {
  uint32_t u = f32_to_bits(f);
  if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fff;
  uint32_t lsb = (u >> 16) & 1u;
  u += 0x7fffu + lsb;
  return (uint16_t)(u >> 16);
}

float oracle_f16_to_f32(uint16_t h) {
  uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1fu;
  uint32_t man = h & 0x3ffu;
  if (exp == 0) {
    if (man == 0) return bits_to_f32(sign);
    /* subnormal: value = man * 2^-24 */
    float v = (float)man * 5.9604644775390625e-08f;
    return sign ? -v : v;
  }
  if (exp == 31) return bits_to_f32(sign | 0x7f800000u | (man << 13));
  return bits_to_f32(sign | ((exp + 112u) << 23) | (man << 13));
}

/* round-to-nearest-even with overflow to infinity and gradual underflow: __float2half_rn */
uint16_t oracle_f32_to_f16(float f) {
  uint32_t u = f32_to_bits(f);
  uint16_t sign = (uint16_t)((u >> 16) & 0x8000u);
  uint32_t a = u & 0x7fffffffu;
  if (a > 0x7f800000u) return (uint16_t)(sign | 0x7fffu);
  if (a >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u); /* >= 65520 rounds to inf */
  if (a < 0x33000000u) return sign;                        /* < 2^-25 rounds to zero */
  int32_t e = (int32_t)(a >> 23) - 127;
  uint32_t m = (a & 0x7fffffu) | 0x800000u;
  int shift;
  uint32_t base;
  if (e < -14) { /* subnormal half: result = round(m * 2^(e-23+24)) */
    shift = 13 + (-14 - e);
    base = 0;
  } else {
    shift = 13;
    base = (uint32_t)(e + 15) << 10;
    m &= 0x7fffffu;
  }
  uint32_t q = m >> shift;
  uint32_t rem = m & ((1u << shift) - 1u);
  uint32_t half = 1u << (shift - 1);
  if (rem > half || (rem == half && (q & 1u))) q += 1; /* a carry walks into the exponent */
  return (uint16_t)(sign | (base + q));
}

/* ------------------------------------------------------------------ the suite's input fills */

static inline uint64_t fill_hash(int64_t idx, uint64_t seed) {
  uint64_t x = (uint64_t)idx ^ seed;
  return x * 2862933555777941757ULL + 3037000493ULL;
}

/* quantization/GEMM_int8.cu:8-19 */
void oracle_fill_int8(int8_t* data, int64_t count, uint64_t seed, int lo, int hi) {
  for (int64_t i = 0; i < count; ++i) {
    int r = (int)((fill_hash(i, seed) >> 11) & 0xFFFF);
    data[i] = (int8_t)(lo + (r % (hi - lo + 1)));
  }
}

static inline float fill_unit(int64_t idx, uint64_t seed, float lo, float hi) {
  float r = (float)((fill_hash(idx, seed) >> 11) & 0xFFFFFF) / 16777215.0f;
  /* the reference evaluates `lo + r * (hi - lo)` on the GPU, where nvcc fuses it into one
   * multiply-add; for the suite's own range [-1, 1] fused and unfused give the same bits */
  return fmaf(r, hi - lo, lo);
}

/* quantization/GEMM_fp32.cu:7-17 */
void oracle_fill_f32(float* data, int64_t count, uint64_t seed, float lo, float hi) {
  for (int64_t i = 0; i < count; ++i) data[i] = fill_unit(i, seed, lo, hi);
}
/* quantization/GEMM_fp16.cu:8-19 */
void oracle_fill_f16(uint16_t* data, int64_t count, uint64_t seed, float lo, float hi) {
  for (int64_t i = 0; i < count; ++i) data[i] = oracle_f32_to_f16(fill_unit(i, seed, lo, hi));
}
/* quantization/GEMM_bf16.cu:8-19 */
void oracle_fill_bf16(uint16_t* data, int64_t count, uint64_t seed, float lo, float hi) {
  for (int64_t i = 0; i < count; ++i) data[i] = oracle_f32_to_bf16(fill_unit(i, seed, lo, hi));
}

/* ------------------------------------------------------------------ product loops
 *
 * Every routine takes an optional list of rows (`rows`, `nrows`): when given, only those rows
 * of C are computed and they are written densely, row r of the list to out row r ([nrows, N],
 * N contiguous).  With rows == NULL all M rows are computed and `out` has the layout's own
 * shape.  "Row" always means an index m of C (a row of A), also for the column-major layout.
 */

#define A_AT(T, A, m, k) ((layout) == ORACLE_ROW_MAJOR ? (A)[(int64_t)(m) * K + (k)] : (A)[(int64_t)(m) + (int64_t)(k) * M])
#define B_AT(T, B, k, n) ((layout) == ORACLE_ROW_MAJOR ? (B)[(int64_t)(k) * N + (n)] : (B)[(int64_t)(k) + (int64_t)(n) * K])

static inline int64_t out_index(int layout, int dense, int64_t r, int64_t m, int64_t n, int64_t M,
                                int64_t N) {
  if (dense) return r * N + n;
  return layout == ORACLE_ROW_MAJOR ? m * N + n : m + n * M;
}

/* fp32: TileProgramming/tensor_utils.cu:35-45 generalised to M x N x K and both layouts */
void oracle_gemm_f32(float* out, const float* A, const float* B, int64_t M, int64_t N, int64_t K,
                     int layout, const int64_t* rows, int64_t nrows) {
  int dense = rows != NULL;
  int64_t R = dense ? nrows : M;
#pragma omp parallel
  {
    float* acc = (float*)malloc(sizeof(float) * (size_t)N);
    float* brow = (float*)malloc(sizeof(float) * (size_t)N);
#pragma omp for schedule(dynamic, 1)
    for (int64_t r = 0; r < R; ++r) {
      int64_t m = dense ? rows[r] : r;
      for (int64_t n = 0; n < N; ++n) acc[n] = 0.0f;
      for (int64_t k = 0; k < K; ++k) {
        float a = A_AT(float, A, m, k);
        const float* bp;
        if (layout == ORACLE_ROW_MAJOR) {
          bp = B + k * N;
        } else {
          for (int64_t n = 0; n < N; ++n) brow[n] = B[k + n * K];
          bp = brow;
        }
        for (int64_t n = 0; n < N; ++n) {
          float p = a * bp[n];
          acc[n] = acc[n] + p;
        }
      }
      for (int64_t n = 0; n < N; ++n) out[out_index(layout, dense, r, m, n, M, N)] = acc[n];
    }
    free(acc);
    free(brow);
  }
}

/* the same sum carried in fp64: the yardstick both fp32 implementations are measured against */
void oracle_gemm_f32_acc64(double* out, const float* A, const float* B, int64_t M, int64_t N,
                           int64_t K, int layout, const int64_t* rows, int64_t nrows) {
  int dense = rows != NULL;
  int64_t R = dense ? nrows : M;
#pragma omp parallel
  {
    double* acc = (double*)malloc(sizeof(double) * (size_t)N);
#pragma omp for schedule(dynamic, 1)
    for (int64_t r = 0; r < R; ++r) {
      int64_t m = dense ? rows[r] : r;
      for (int64_t n = 0; n < N; ++n) acc[n] = 0.0;
      for (int64_t k = 0; k < K; ++k) {
        double a = (double)A_AT(float, A, m, k);
        for (int64_t n = 0; n < N; ++n) acc[n] += a * (double)B_AT(float, B, k, n);
      }
      for (int64_t n = 0; n < N; ++n) out[out_index(layout, dense, r, m, n, M, N)] = acc[n];
    }
    free(acc);
  }
}

/* int8 x int8 -> int32, exact (quantization/GEMM_int8.cu:51-56: CUBLAS_COMPUTE_32I, alpha 1, beta 0) */
void oracle_gemm_i8_i32(int32_t* out, const int8_t* A, const int8_t* B, int64_t M, int64_t N,
                        int64_t K, int layout, const int64_t* rows, int64_t nrows) {
  int dense = rows != NULL;
  int64_t R = dense ? nrows : M;
#pragma omp parallel
  {
    int32_t* acc = (int32_t*)malloc(sizeof(int32_t) * (size_t)N);
    int8_t* brow = (int8_t*)malloc((size_t)N);
#pragma omp for schedule(dynamic, 1)
    for (int64_t r = 0; r < R; ++r) {
      int64_t m = dense ? rows[r] : r;
      for (int64_t n = 0; n < N; ++n) acc[n] = 0;
      for (int64_t k = 0; k < K; ++k) {
        int32_t a = (int32_t)A_AT(int8_t, A, m, k);
        const int8_t* bp;
        if (layout == ORACLE_ROW_MAJOR) {
          bp = B + k * N;
        } else {
          for (int64_t n = 0; n < N; ++n) brow[n] = B[k + n * K];
          bp = brow;
        }
        for (int64_t n = 0; n < N; ++n) acc[n] += a * (int32_t)bp[n];
      }
      for (int64_t n = 0; n < N; ++n) out[out_index(layout, dense, r, m, n, M, N)] = acc[n];
    }
    free(acc);
    free(brow);
  }
}

/* 16-bit inputs (is_bf16 ? bf16 : fp16) widened to fp32, fp32 sequential accumulate; the fp32
 * sums go to out32 (if not NULL) and, rounded to nearest even, to out16 (if not NULL).
 * quantization/GEMM_fp16.cu:51-56 and GEMM_bf16.cu:51-56: CUBLAS_COMPUTE_32F, 16-bit C. */
void oracle_gemm_h16(uint16_t* out16, float* out32, const uint16_t* A, const uint16_t* B,
                     int64_t M, int64_t N, int64_t K, int is_bf16, int layout, const int64_t* rows,
                     int64_t nrows) {
  int dense = rows != NULL;
  int64_t R = dense ? nrows : M;
#pragma omp parallel
  {
    float* acc = (float*)malloc(sizeof(float) * (size_t)N);
    float* brow = (float*)malloc(sizeof(float) * (size_t)N);
#pragma omp for schedule(dynamic, 1)
    for (int64_t r = 0; r < R; ++r) {
      int64_t m = dense ? rows[r] : r;
      for (int64_t n = 0; n < N; ++n) acc[n] = 0.0f;
      for (int64_t k = 0; k < K; ++k) {
        uint16_t ab = A_AT(uint16_t, A, m, k);
        float a = is_bf16 ? oracle_bf16_to_f32(ab) : oracle_f16_to_f32(ab);
        for (int64_t n = 0; n < N; ++n) {
          uint16_t bb = B_AT(uint16_t, B, k, n);
          brow[n] = is_bf16 ? oracle_bf16_to_f32(bb) : oracle_f16_to_f32(bb);
        }
        for (int64_t n = 0; n < N; ++n) {
          float p = a * brow[n];
          acc[n] = acc[n] + p;
        }
      }
      for (int64_t n = 0; n < N; ++n) {
        int64_t o = out_index(layout, dense, r, m, n, M, N);
        if (out32) out32[o] = acc[n];
        if (out16) out16[o] = is_bf16 ? oracle_f32_to_bf16(acc[n]) : oracle_f32_to_f16(acc[n]);
      }
    }
    free(acc);
    free(brow);
  }
}

/* W8A8 linear, row-major only: exact int32 accumulate, then
 *   out[m][n] = bf16_rn( ((float)acc * row_scale[m]) * col_scale[n] )
 * every floating-point step is one correctly rounded operation, so the result is unique. */
void oracle_gemm_w8a8_bf16(uint16_t* out, const int8_t* A, const int8_t* B, const float* row_scale,
                           const float* col_scale, int64_t M, int64_t N, int64_t K,
                           const int64_t* rows, int64_t nrows) {
  int dense = rows != NULL;
  int64_t R = dense ? nrows : M;
#pragma omp parallel
  {
    int32_t* acc = (int32_t*)malloc(sizeof(int32_t) * (size_t)N);
#pragma omp for schedule(dynamic, 1)
    for (int64_t r = 0; r < R; ++r) {
      int64_t m = dense ? rows[r] : r;
      for (int64_t n = 0; n < N; ++n) acc[n] = 0;
      for (int64_t k = 0; k < K; ++k) {
        int32_t a = (int32_t)A[m * K + k];
        const int8_t* bp = B + k * N;
        for (int64_t n = 0; n < N; ++n) acc[n] += a * (int32_t)bp[n];
      }
      float sa = row_scale[m];
      for (int64_t n = 0; n < N; ++n) {
        float t = (float)acc[n] * sa;
        float v = t * col_scale[n];
        out[(dense ? r : m) * N + n] = oracle_f32_to_bf16(v);
      }
    }
    free(acc);
  }
}

/* Symmetric absmax quantiser for a row-major [R, C] fp32 matrix.
 *   along == 0: one scale per row     (activations: scale[r] = max_c |x[r][c]| / 127)
 *   along == 1: one scale per column  (weights:     scale[c] = max_r |x[r][c]| / 127)
 * q = clamp(rintf(x / scale), -127, 127) with rintf rounding half to even; an all-zero row or
 * column gets scale 1 so that the division is defined. */
void oracle_quantize_absmax(int8_t* q, float* scale, const float* x, int64_t R, int64_t C,
                            int along) {
  int64_t S = along == 0 ? R : C;
  for (int64_t s = 0; s < S; ++s) scale[s] = 0.0f;
  for (int64_t r = 0; r < R; ++r)
    for (int64_t c = 0; c < C; ++c) {
      float a = fabsf(x[r * C + c]);
      int64_t s = along == 0 ? r : c;
      if (a > scale[s]) scale[s] = a;
    }
  for (int64_t s = 0; s < S; ++s) scale[s] = scale[s] > 0.0f ? scale[s] / 127.0f : 1.0f;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < R; ++r)
    for (int64_t c = 0; c < C; ++c) {
      float v = rintf(x[r * C + c] / scale[along == 0 ? r : c]);
      if (v > 127.0f) v = 127.0f;
      if (v < -127.0f) v = -127.0f;
      q[r * C + c] = (int8_t)v;
    }
}


/* ------------------------------------------------------------------ fully connected layer */

/* y[b][o] = act(sum_i x[b][i] * w(o,i) + bias[o]) in fp32, i ascending, one accumulator.
 *   w_is_out_in = 1: w[o*in + i] (MNIST/mnist_kernels.cu:96); 0: w[i*out + o] (MNIST/mnist_nn.cu:17).
 *   flags bit 0: ReLU, fmaxf(0, y) (mnist_kernels.cu:82).
 *   flags bit 1: the sum starts from bias[o] (mnist_nn.cu:14, mnist_cnn_kernels.cu:141); otherwise
 *                the bias is added to the finished sum (mnist_kernels.cu:99).
 *   fused = 1: sum = fmaf(x, w, sum), what nvcc's default -fmad=true makes of `sum += x * w` in
 *              the reference's device code; fused = 0: product and sum rounded separately. */
void oracle_linear_f32(float* y, const float* x, const float* w, const float* bias, int64_t batch,
                       int64_t in_f, int64_t out_f, int w_is_out_in, int flags, int fused) {
#pragma omp parallel for schedule(static)
  for (int64_t b = 0; b < batch; ++b) {
    for (int64_t o = 0; o < out_f; ++o) {
      float sum = (bias && (flags & 2)) ? bias[o] : 0.0f;
      for (int64_t i = 0; i < in_f; ++i) {
        const float xv = x[b * in_f + i];
        const float wv = w_is_out_in ? w[o * in_f + i] : w[i * out_f + o];
        if (fused) {
          sum = fmaf(xv, wv, sum);
        } else {
          const float prod = xv * wv;
          sum = sum + prod;
        }
      }
      if (bias && !(flags & 2)) sum = sum + bias[o];
      if (flags & 1) sum = fmaxf(0.0f, sum);
      y[b * out_f + o] = sum;
    }
  }
}

/* The same layer on fp16 / bf16 inputs: products of two 16-bit floats are exact in fp32, the sum
 * runs in fp32 in ascending i, the bias is added in fp32, then ReLU, then one rounding to the
 * 16-bit type.  y32 receives the value before that rounding, y16 the rounded bits (either may be
 * NULL). */
void oracle_linear_h16(uint16_t* y16, float* y32, const uint16_t* x, const uint16_t* w, const float* bias,
                       int64_t batch, int64_t in_f, int64_t out_f, int w_is_out_in, int flags, int is_bf16) {
#pragma omp parallel for schedule(static)
  for (int64_t b = 0; b < batch; ++b) {
    for (int64_t o = 0; o < out_f; ++o) {
      float sum = 0.0f;
      for (int64_t i = 0; i < in_f; ++i) {
        const uint16_t xb = x[b * in_f + i];
        const uint16_t wb = w_is_out_in ? w[o * in_f + i] : w[i * out_f + o];
        const float xv = is_bf16 ? oracle_bf16_to_f32(xb) : oracle_f16_to_f32(xb);
        const float wv = is_bf16 ? oracle_bf16_to_f32(wb) : oracle_f16_to_f32(wb);
        const float prod = xv * wv;
        sum = sum + prod;
      }
      if (bias) sum = sum + bias[o];
      if (flags & 1) sum = fmaxf(0.0f, sum);
      if (y32) y32[b * out_f + o] = sum;
      if (y16) y16[b * out_f + o] = is_bf16 ? oracle_f32_to_bf16(sum) : oracle_f32_to_f16(sum);
    }
  }
}
