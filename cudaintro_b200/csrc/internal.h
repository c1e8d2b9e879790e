// Declarations shared by the translation units of libb200gemm (not part of the public ABI).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/b200gemm.h"

namespace b200 {

// Records the text b200_last_error() returns on this thread and passes `code` through.
int fail(int code, const char* fmt, ...);

#define B200_CUDA_TRY(call)                                                          \
  do {                                                                               \
    cudaError_t e__ = (call);                                                        \
    if (e__ != cudaSuccess)                                                          \
      return ::b200::fail(B200_ERR_CUDA, "%s: %s", #call, cudaGetErrorString(e__)); \
  } while (0)

enum Epilogue { EPI_I32 = 0, EPI_F32 = 1, EPI_BF16 = 2, EPI_F16 = 3, EPI_W8A8_BF16 = 4 };

// Optional tail of a floating-point product (the fully connected layer): out = act(sum + bias[n]).
// `flags` are b200_linear_flags; bias = nullptr and flags = 0 leave the product as it is.
struct Tail {
  const float* bias = nullptr;
  int flags = 0;
};

// A row-major problem C[M,N] = A[M,K] * B with B either [K,N] (b_is_nk = false, N contiguous) or
// [N,K] (b_is_nk = true, K contiguous), on the tensor cores.  `kind` is a b200::MmaKind value.
// force_bn = 0 lets the launcher pick the tile width.
int launch_umma_gemm(int kind, int epi, const void* A, const void* B, void* C, int64_t M, int64_t N,
                     int64_t K, int64_t lda, int64_t ldb, int64_t ldc, bool b_is_nk,
                     const float* row_scale, const float* col_scale, int force_bn,
                     cudaStream_t stream, const Tail& tail = Tail());

// Same product written to n_dest destination buffers at once (this GPU's C and peers' copies).
int launch_umma_gemm_multi(int kind, int epi, const void* A, const void* B, void* const* C_list, int n_dest,
                           int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc, bool b_is_nk,
                           const float* row_scale, const float* col_scale, int force_bn, cudaStream_t stream,
                           const Tail& tail = Tail());

// Same product (row-major B) written once to a multicast address: one store per 16 bytes reaches every
// GPU's copy of C through the NVSwitch.
int launch_umma_gemm_multicast(int kind, int epi, const void* A, const void* B, void* C_multicast, int64_t M, int64_t N,
                               int64_t K, int64_t lda, int64_t ldb, int64_t ldc, const float* row_scale,
                               const float* col_scale, cudaStream_t stream);

// The same kind of product for at most 128 rows of A (fp16, bf16, or int8 with the int32 or the W8A8
// epilogue): tiles shared by clusters that split K and add their partial sums through distributed
// shared memory (gemm_skinny.cu).  *used tells whether the
// kernel took the product; `general_cost` is what one SM would stream in the general kernel
// (tile columns x k-blocks x waves), the yardstick it has to beat unless `force` is set.
int launch_skinny_gemm(int kind, int epi, const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K,
                       int64_t lda, int64_t ldb, int64_t ldc, bool b_is_nk, const float* row_scale,
                       const float* col_scale, const Tail& tail, int force_bn, bool force, int64_t general_cost,
                       cudaStream_t stream, bool* used);
int read_and_clear_skinny_status(uint32_t* out);

// 2-D tensor map over a row-major [rows, cols] matrix of MmaKind `kind` elements with leading
// dimension `ld`: box = box_cols x box_rows, 128-byte swizzle (on 32-byte chunks if `chunks32`),
// zero fill outside the matrix.
int encode_operand_map(CUtensorMap* map, int kind, const void* base, int64_t rows, int64_t cols, int64_t ld,
                       int box_cols, int box_rows, bool chunks32);

// Whether kernels are launched with programmatic stream serialisation (set_dependent_launch).
bool dependent_launch_enabled();

// Test of the give-up path of the tensor-core kernel: lose_kb >= 0 makes the next launches' first CTA
// leave out the loads of that k-block of its first tile; budget_ns (0 = the default four seconds)
// is how long a single device-side wait may last.  lose_kb = -1, budget_ns = 0 restores normal operation.
int set_wait_test(long long lose_kb, unsigned long long budget_ns);

// Which 3xTF32 kernel b200_gemm_f32 / b200_linear take: 0 = automatic, 1 = split planes in global
// memory (scratch from the stream-ordered pool), 2 = operands split on chip.
int set_x3_path(int path);

// L2 eviction hints of the tensor-core kernel's TMA traffic: -1 = automatic, else a bit set
// (1 = keep A's slab, 2 = B streams, 4 = C's stores stream).
int set_l2_hints(int hints);

// 1 (default) = GEMM kernels are launched with programmatic stream serialisation; 0 = plain launches.
int set_dependent_launch(int enabled);

// 1 = write C from registers with 16-byte stores instead of staged TMA stores; 0 = automatic.
int set_store_policy(int register_stores);

// Overrides the automatic choice of CTA grouping (1 or 2 CTAs per tile) and tile width; 0 = automatic.
int set_tile_policy(int cg, int bn, int group_rows);

// Reads and clears the device-side wait record of the tensor-core kernels (0 = clean).
int read_and_clear_umma_status(cudaStream_t stream, uint32_t* out);

// may_split_k: a plain product with few tiles may be cut along K inside clusters (the ranges' sums
// are added in range order); false keeps the single ascending sum whatever the shape.
int launch_sgemm_ffma(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K,
                      int64_t lda, int64_t ldb, int64_t ldc, bool b_is_nk, cudaStream_t stream,
                      const Tail& tail = Tail(), bool may_split_k = false);
// -1 = automatic, 0 = never cut K, 2 or 4 = that many ranges for every plain FFMA product.
int set_ffma_ksplit(int ks);

// 3xTF32: tensor-core fp32 GEMM from split operands (a = hi + lo, three products per term).
int launch_sgemm_3xtf32(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K,
                        int64_t lda, int64_t ldb, int64_t ldc, bool b_is_nk, cudaStream_t stream,
                        const Tail& tail = Tail());

// Single-pass tf32: fp32 operands read directly by the tensor cores (reduced precision, no scratch).
int launch_sgemm_tf32(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K, int64_t lda,
                      int64_t ldb, int64_t ldc, bool b_is_nk, cudaStream_t stream, const Tail& tail = Tail());

int launch_naive(int dtype, const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K,
                 int64_t lda, int64_t ldb, int64_t ldc, int layout, cudaStream_t stream);

}  // namespace b200
