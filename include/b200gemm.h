/*
 * b200gemm — C ABI of the B200 (sm_100a) quantized GEMM suite.
 *
 * These entry points stand where the reference calls cublasGemmEx inside its per-type benchmark
 * bodies; each one cites the call it replaces (paths are inside the reference project).
 * All matrix pointers are DEVICE pointers unless the name ends in _host.  Every call is
 * asynchronous on `stream` (a cudaStream_t passed as void*; NULL = the default stream) and
 * returns a b200_status; nothing here exits the process or traps the GPU.  There is no CPU
 * route: without a usable sm_100 device the calls return B200_ERR_CUDA.
 *
 * Layouts
 *   B200_ROW_MAJOR     C[m*ldc+n] = sum_k A[m*lda+k] * B[k*ldb+n]
 *   B200_COL_MAJOR_NN  C[m+n*ldc] = sum_k A[m+k*lda] * B[k+n*ldb]   (what the reference passes to
 *                      cuBLAS: CUBLAS_OP_N, CUBLAS_OP_N, lda = M, ldb = K, ldc = M)
 *   B200_ROW_MAJOR_BT  C[m*ldc+n] = sum_k A[m*lda+k] * B[n*ldb+k]   (B stored transposed, [N,K])
 * A leading dimension of 0 means "packed" (the natural one for the layout).
 *
 * Tensor-core entry points (int8, fp16, bf16, W8A8) read A and B with TMA: lda and ldb, times
 * the element size, must be multiples of 16 bytes and both base pointers 16-byte aligned;
 * otherwise they return B200_ERR_UNSUPPORTED.  C has no such rule (an unaligned C is written
 * element by element).  M, N and K themselves may be any positive sizes.
 */
#ifndef B200GEMM_H_
#define B200GEMM_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum b200_status {
  B200_OK = 0,
  B200_ERR_BAD_ARGUMENT = 1, /* null pointer, non-positive size, unknown enum value          */
  B200_ERR_UNSUPPORTED = 2,  /* alignment or leading-dimension rule above not met            */
  B200_ERR_CUDA = 3,         /* a CUDA runtime / driver call failed (see b200_last_error)    */
  B200_ERR_DEVICE_WAIT = 4,  /* a kernel gave up a bounded wait; results are not valid       */
  B200_ERR_TOO_LARGE = 5     /* size beyond a stated maximum of the entry point              */
} b200_status;

typedef enum b200_layout {
  B200_ROW_MAJOR = 0,
  B200_COL_MAJOR_NN = 1,
  B200_ROW_MAJOR_BT = 2
} b200_layout;

typedef enum b200_f32_mode {
  B200_F32_FFMA = 0,  /* fp32 FMA on the CUDA cores, k ascending                              */
  B200_F32_3XTF32 = 1, /* three tf32 tensor-core products per term (hi*hi + hi*lo + lo*hi):
                          fp32-level accuracy (relative Frobenius error <= 1e-5)              */
  B200_F32_TF32 = 2    /* one tf32 tensor-core product per term: operands cut to 10 mantissa bits,
                          fp32 accumulate (relative Frobenius error <= 2e-3).  This is the
                          precision class the reference's cublasGemmEx call runs at on this
                          hardware (CUBLAS_GEMM_DEFAULT_TENSOR_OP under CUBLAS_TENSOR_OP_MATH).
                          Needs lda, ldb multiples of 4 and 16-byte aligned A, B                */
} b200_f32_mode;

/* Element types of the operands. */
typedef enum b200_dtype { B200_I8 = 0, B200_F16 = 1, B200_BF16 = 2, B200_F32 = 3 } b200_dtype;

/* Text of the most recent failure on the calling thread ("" if none). */
const char* b200_last_error(void);

/* Library / device facts: version string, SM count of the current device (0 if none). */
const char* b200_version(void);
int b200_sm_count(void);

/* Tuning knob for tests and measurements (process-wide, not thread-safe against running calls):
 * forces the tensor-core kernels to use single CTAs (cta_group = 1) or CTA pairs (2) per tile
 * and a tile width of 64, 128 or 256 columns; `group_rows` (a multiple of 256) is how many rows
 * of C share one sweep across N in the tile order.  0 restores the automatic choice of each.
 * CTA pairs exist for 256-wide tiles only.  cta_group = 4 is a CTA pair in which every CTA owns two
 * 128-row blocks (512 x 256 tiles, eight epilogue warps; chosen by itself for tf32 products and for
 * 16-bit products with K >= 4096 and int8 -> int32 products with K >= 8192 when it costs no extra wave of tiles).  cta_group = 3 sends fp16 / bf16 products of at most
 * 128 rows to the K-split cluster kernel (tile_n 0, 128, 192 or 256) and makes every other product
 * fail with B200_ERR_UNSUPPORTED; without a policy that kernel is chosen by itself when it lets
 * every SM stream clearly less of B.  Integer results do not depend on the policy;
 * floating-point results may differ in the last bits (the order of the K blocks changes). */
int b200_set_tile_policy(int cta_group, int tile_n, int group_rows);

/* Waits for `stream` and reports whether any kernel of this library gave up a device-side wait
 * since the last call (B200_ERR_DEVICE_WAIT), clearing the record. */
int b200_check_device(void* stream);

/* int8 x int8 -> int32, exact.  Replaces cublasGemmEx(CUDA_R_8I, CUDA_R_8I, CUDA_R_32I,
 * CUBLAS_COMPUTE_32I) at quantization/GEMM_int8.cu:51-56 and :64-69. */
int b200_gemm_i8_i32(const int8_t* A, const int8_t* B, int32_t* C, int64_t M, int64_t N, int64_t K,
                     int64_t lda, int64_t ldb, int64_t ldc, int layout, void* stream);

/* bf16 x bf16, fp32 accumulate, bf16 out (round to nearest even).  Replaces
 * cublasGemmEx(CUDA_R_16BF ..., CUBLAS_COMPUTE_32F) at quantization/GEMM_bf16.cu:51-56, :64-69. */
int b200_gemm_bf16(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K,
                   int64_t lda, int64_t ldb, int64_t ldc, int layout, void* stream);

/* fp16 x fp16, fp32 accumulate, fp16 out.  Replaces cublasGemmEx(CUDA_R_16F ...,
 * CUBLAS_COMPUTE_32F) at quantization/GEMM_fp16.cu:51-56, :64-69. */
int b200_gemm_f16(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K,
                  int64_t lda, int64_t ldb, int64_t ldc, int layout, void* stream);

/* fp16 x fp16 or bf16 x bf16 (dtype = B200_F16 / B200_BF16), fp32 accumulate, fp32 out: the sums
 * are stored unrounded.  Replaces the WMMA kernels behind launchMatrixMulTensorCores and
 * launchMatrixMulTensorCoresBfloat16 (TileProgramming/matmulTensor.cu:31-48, :51-68, wrappers
 * :71-87), which take half / __nv_bfloat16 operands and write float; C++ shims with those
 * wrappers' names and signatures are in include/tile_programming.h.  Alignment rules of the
 * 16-bit entry points above. */
int b200_gemm_16_f32(int dtype, const void* A, const void* B, float* C, int64_t M, int64_t N, int64_t K,
                     int64_t lda, int64_t ldb, int64_t ldc, int layout, void* stream);

/* fp32 GEMM.  Replaces cublasGemmEx(CUDA_R_32F ..., CUBLAS_COMPUTE_32F) at
 * quantization/GEMM_fp32.cu:49-54, :62-67, and the tiled kernel launched at
 * TileProgramming/kernel.cu:145-147.  `mode` is a b200_f32_mode. No alignment rule in FFMA mode. */
int b200_gemm_f32(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K,
                  int64_t lda, int64_t ldb, int64_t ldc, int layout, int mode, void* stream);

/* The 3xTF32 product of b200_gemm_f32 for callers that must not allocate device memory.
 * No counterpart in the reference.  b200_gemm_f32 in 3xTF32 mode keeps the split (high / low)
 * copies of A and B in a workspace it obtains with cudaMalloc and grows on demand; this variant
 * keeps them in a fixed 32 MiB array built into the library instead, and calls neither
 * cudaMalloc nor cudaFree nor anything else that allocates.  It is meant for hosts that gave
 * all device memory to a pool of their own and forbid plug-ins to allocate, and for loops with
 * a latency bound that the device-wide synchronisation inside cudaMalloc / cudaFree would break.
 *   - Limit: 2*M*K + 2*K*N floats (each row padded to a multiple of 4 floats) must fit in
 *     8 Mi floats, e.g. up to 1024 x 1024 x 2048; larger products return B200_ERR_TOO_LARGE.
 *   - Every GPU that loads the library holds the 32 MiB until the process exits.
 *   - The first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress, with that device current); make that first call before any stream
 *     capture begins.  With CUDA's lazy module loading that first call may also be the moment the
 *     library's code, and the 32 MiB array with it, is placed on the device, so it can fail for
 *     lack of memory: make it at start-up, before the host claims the rest of the device.  Calls
 *     after the first take no device memory at all.
 *   - All calls on a device share the one array.  Each call rewrites every word it later reads,
 *     so nothing has to be cleared between calls, but two calls whose kernels overlap on the GPU
 *     (different streams, or different host threads) race on it: serialise them.
 * Arguments, layouts, result and error codes are those of b200_gemm_f32. */
int b200_gemm_f32_3xtf32_static(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K,
                                int64_t lda, int64_t ldb, int64_t ldc, int layout, void* stream);

/* W8A8 linear (row-major only): int8 x int8 -> int32 exactly, then
 *   C[m][n] = bf16_rn( ((float)acc * row_scale[m]) * col_scale[n] ).
 * row_scale has M entries, col_scale N entries (fp32, device).  A per-tensor scale is a
 * row_scale/col_scale filled with one value.  No counterpart in the reference (its int8 body,
 * quantization/GEMM_int8.cu:21-91, stops at the int32 result); this is the dequantising
 * epilogue fused onto that same product. */
int b200_gemm_w8a8_bf16(const int8_t* A, const int8_t* B, const float* row_scale,
                        const float* col_scale, void* C, int64_t M, int64_t N, int64_t K,
                        int64_t lda, int64_t ldb, int64_t ldc, void* stream);

/* Row-major GEMM whose result is written to n_dest (1..8) buffers at once: C_list[g] points at
 * the same [M, N] slab (leading dimension ldc) inside destination g.  Destinations may be this
 * GPU's memory or peer GPUs' memory mapped into this process (b200_ipc_import): the epilogue
 * then sends every finished tile over NVLink (peers first, C_list[0] last: pass the local copy
 * there) while later tiles are still being computed, which
 * is how a row-sharded product places its rows in every rank's copy of C without a separate
 * all-gather.  `what` is B200_I8, B200_F16, B200_BF16 or B200_W8A8 (the scales are read only
 * for B200_W8A8).  Remote copies are complete when the kernel has finished on the writing GPU;
 * readers on other GPUs must order themselves after that (any cross-rank barrier).  No
 * counterpart in the reference (it runs on one GPU). */
int b200_gemm_multi(int what, const void* A, const void* B, void* const* C_list, int n_dest,
                    const float* row_scale, const float* col_scale, int64_t M, int64_t N, int64_t K,
                    int64_t lda, int64_t ldb, int64_t ldc, void* stream);

/* The same row-major product written ONCE, to a multicast address: C_multicast points at the [M, N]
 * slab (leading dimension ldc) inside a multicast mapping of C, i.e. a virtual address bound through
 * an NVLink multicast object to the same buffer on every GPU of the group (cuMulticastCreate /
 * cuMulticastBindMem, or a framework's symmetric memory: torch's exposes it as multicast_ptr).  The
 * epilogue stages every tile in shared memory and writes it with multimem.st: each 16 bytes leave
 * this GPU once and the NVSwitch delivers them to all copies, this GPU's included, so a row-sharded
 * product fills every rank's C while sending 1/G of what b200_gemm_multi sends.  Needs N and ldc
 * in whole 16-byte units; the copies are complete when the kernel has finished, and readers on other
 * GPUs must order themselves after that (b200_peer_marker).  Keep it out of runs in which a rank
 * may leave: a process that dies while bound to a multicast object disturbs NVLink for the others.
 * No counterpart in the reference. */
int b200_gemm_multicast(int what, const void* A, const void* B, void* C_multicast, const float* row_scale,
                        const float* col_scale, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb,
                        int64_t ldc, void* stream);

/* Device memory that other processes on the same machine can map: allocate, export a 64-byte
 * handle, import a peer's handle (enables peer access on first use), close, free. */
int b200_peer_alloc(size_t bytes, void** ptr);
int b200_peer_free(void* ptr);
int b200_ipc_export(void* ptr, void* handle64);
int b200_ipc_import(const void* handle64, void** ptr);
int b200_ipc_close(void* ptr);

/* Completion marker for b200_gemm_multi across ranks (one process per GPU, ranks on different
 * GPUs).  flag_arrays[g] is rank g's flag array: 8 zero-initialised 32-bit words in memory from
 * b200_peer_alloc, mapped into this process.  The call enqueues a one-warp kernel on `stream`
 * that writes `value` (use the step number: 1, 2, 3, ...) into slot `rank` of every rank's array
 * and waits until every slot of its own array has reached `value`, i.e. until every rank's
 * kernels enqueued before their marker have finished.  The wait gives up after two seconds and
 * reports through b200_check_device.  No counterpart in the reference. */
int b200_peer_marker(void* const* flag_arrays, int world, int rank, uint32_t value, void* stream);

/* 1 = the tensor-core kernels write C straight from registers (16-byte stores) instead of
 * staging tiles in shared memory for TMA stores; 0 = automatic (TMA stores whenever C and ldc
 * are 16-byte aligned).  For tests and measurements; results do not depend on it. */
int b200_set_store_policy(int register_stores);

/* 1 (default): the tensor-core kernels are launched with programmatic stream serialisation, so
 * that a launch's set-up (barrier initialisation, tensor-memory allocation, descriptor prefetch)
 * overlaps the tail of the kernel before it in the stream; the kernel waits
 * (griddepcontrol.wait) for that predecessor to complete before it touches global memory, so
 * stream order is kept.  0: plain launches.  For measurements; results do not depend on it. */
int b200_set_dependent_launch(int enabled);

/* Which kernel the 3xTF32 mode of b200_gemm_f32 / b200_linear takes (process-wide; for tests and
 * measurements): 0 = automatic (by size), 1 = the operands are first split into high / low planes in
 * a scratch buffer taken from a stream-ordered pool on the call's stream, 2 = the operands are split
 * on chip inside the GEMM kernel (needs 16-byte aligned A, B and row pitches; otherwise 1 is taken).
 * Both meet the mode's tolerance; their results differ in the last bits. */
int b200_set_3xtf32_path(int path);

/* K ranges of the FFMA mode of b200_gemm_f32 (process-wide; for tests and measurements): a plain
 * product with too few 64 x 64 tiles to fill the GPU is cut along K into 2 or 4 ranges, one CTA of a
 * thread-block cluster each; every range is summed in ascending k and the range sums are added in
 * range order, so the result is deterministic and differs from the single ascending sum in rounding
 * only.  -1 = automatic (by shape), 0 = never, 2 or 4 = always that many.  b200_linear never cuts K. */
int b200_set_ffma_k_ranges(int ranges);

/* L2 eviction hints on the tensor-core kernel's TMA traffic (process-wide; for measurements;
 * results do not depend on it): -1 = automatic, else a bit set: 1 = the rows of A that a group of
 * tiles re-reads are kept in L2 in preference to other data (evict last), 2 = B, which streams
 * past, is the first to be evicted, 4 = so are the stores of C. */
int b200_set_l2_hints(int hints);

/* Test hook for the kernels' failure handling (process-wide; not for production use).  Every
 * device-side wait of the tensor-core kernel is bounded: a wait that outlasts its budget makes the
 * CTA give up in an orderly way (all its roles leave, copies in flight land, tensor memory is
 * freed), the kernel returns and b200_check_device reports B200_ERR_DEVICE_WAIT.  This call makes
 * that happen without any fault: with k_block >= 0 the first CTA of every later launch leaves out
 * the loads of that k-block of its first tile, as if their completion had been lost, and
 * wait_budget_ns (0 = the default of four seconds) replaces the budget.  k_block = -1 with
 * wait_budget_ns = 0 restores normal operation.  No counterpart in the reference. */
int b200_test_lose_arrival(int64_t k_block, uint64_t wait_budget_ns);

/* Symmetric absmax quantiser of a row-major fp32 [R, C] matrix to int8 (same shape):
 *   along = 0: scale[r] = max_c |x[r][c]| / 127  (R scales);  along = 1: per column (C scales);
 *   q = clamp(rint(x / scale), -127, 127), ties to even; an all-zero row/column gets scale 1.
 * No counterpart in the reference; it makes the inputs of b200_gemm_w8a8_bf16. */
int b200_quantize_absmax(const float* x, int8_t* q, float* scale, int64_t R, int64_t C, int along,
                         void* stream);

/* The reference's input generators (quantization/GEMM_int8.cu:8-19, GEMM_fp16.cu:8-19,
 * GEMM_bf16.cu:8-19, GEMM_fp32.cu:7-17): element i = hash(i ^ seed) mapped to [lo, hi]. */
int b200_fill_int8(int8_t* data, int64_t count, uint64_t seed, int lo, int hi, void* stream);
int b200_fill_f16(void* data, int64_t count, uint64_t seed, float lo, float hi, void* stream);
int b200_fill_bf16(void* data, int64_t count, uint64_t seed, float lo, float hi, void* stream);
int b200_fill_f32(float* data, int64_t count, uint64_t seed, float lo, float hi, void* stream);

/* Validation kernels: one thread per element of C, k ascending, no tensor cores, no tiling.
 * `dtype` is a b200_dtype; out is int32 for B200_I8, fp32 sums (not rounded) for the others.
 * They exist so that a full-size result of the fast kernels can be compared on the device. */
int b200_gemm_naive(int dtype, const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K,
                    int64_t lda, int64_t ldb, int64_t ldc, int layout, void* stream);

/* Fully connected layer, fused: Y[b][o] = act(sum_i X[b][i] * W(o,i) + bias[o]) in one launch.
 * Replaces fullyConnectedForwardKernel followed by reluActivationKernel
 * (MNIST/mnist_kernels.cu:87-102 and :78-84; the same pair in MNIST/mnist_cnn_kernels.cu:136-149 and
 * the two-layer network's forwardInputToHiddenKernel / forwardHiddenToOutputKernel,
 * MNIST/mnist_nn.cu:10-48), which run one thread per output and a second kernel for the activation.
 *   X [batch, in_features] row-major; Y [batch, out_features] row-major, type of X;
 *   W: B200_ROW_MAJOR_BT = [out_features, in_features] (mnist_kernels.cu, mnist_cnn_kernels.cu),
 *      B200_ROW_MAJOR    = [in_features, out_features] (mnist_nn.cu);
 *   bias: out_features fp32 values, or NULL;
 *   dtype: B200_F32 (f32_mode as in b200_gemm_f32), B200_F16 or B200_BF16 (fp32 sums, bias added in
 *      fp32 before the one rounding to 16 bits; f32_mode ignored);
 *   flags: B200_LINEAR_RELU applies fmaxf(0, .) to the result; B200_LINEAR_BIAS_FIRST starts the
 *      sum from the bias (mnist_nn.cu:14, mnist_cnn_kernels.cu:141) instead of adding it to the
 *      finished sum (mnist_kernels.cu:99).  The order matters to the last bit only in
 *      B200_F32_FFMA mode, which reproduces either reference loop exactly (fused multiply-add in
 *      ascending i, as nvcc compiles them); the tensor-core modes add the bias to the finished sum.
 * Alignment rules are those of the GEMM entry point the dtype and mode select. */
typedef enum b200_linear_flags { B200_LINEAR_RELU = 1, B200_LINEAR_BIAS_FIRST = 2 } b200_linear_flags;
int b200_linear(int dtype, const void* X, const void* W, const float* bias, void* Y, int64_t batch,
                int64_t in_features, int64_t out_features, int w_layout, int flags, int f32_mode, void* stream);

/* Same products with HOST buffers: copies A and B to the device, runs the kernels, copies C
 * back, and returns after the result is in `C`.  `dtype` selects the entry point above
 * (B200_I8 -> int32 out, B200_F16 / B200_BF16 -> 16-bit out, B200_F32 -> FFMA).  The operand
 * every output line needs goes up whole (B; A for the column-major layout); the other one travels
 * in up to 8 slabs of rows (columns), each multiplied as soon as it has arrived and copied back
 * while the next is on its way, so with pinned buffers the call costs about its host-to-device
 * traffic.  Device workspace, three streams and their events are kept per device between calls
 * (the device that is current when the call is made) and grow as needed; b200_host_release()
 * frees those of the current device.  Calls on one device are serialised by a lock.  When the
 * call returns, with or without an error, nothing it issued still touches A, B or C.
 * Stands where the reference's bodies copy nothing (they fill on the device,
 * quantization/GEMM_int8.cu:41-49); it is the host-memory form of the call at :51-56. */
int b200_gemm_host(int dtype, const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K,
                   int layout);
int b200_host_release(void);

/* Host-buffer products against weights that stay on the device: the usual shape of a linear
 * layer, whose weights do not change between calls.  No counterpart in the reference.
 *   b200_host_weights_upload  copies a row-major [K, N] matrix B of `dtype` (b200_dtype) from host
 *                             memory to the current device once and returns a handle;
 *   b200_gemm_host_weights    C[M, N] = A[M, K] * B for host buffers A and C (row-major, packed):
 *                             slabs of A go up, are multiplied and their rows of C come down, all
 *                             three overlapped (uploads and downloads use both directions of the
 *                             host link at once), so a call costs about max(bytes of A, bytes of
 *                             C) over the link.  The device that holds the weights must be current;
 *   b200_host_weights_free    releases the device copy and the handle.
 * Output types and the workspace are those of b200_gemm_host. */
int b200_host_weights_upload(int dtype, const void* B, int64_t K, int64_t N, void** weights);
int b200_gemm_host_weights(const void* weights, const void* A, void* C, int64_t M);
int b200_host_weights_free(void* weights);

/* Timing helper: runs `iters` back-to-back launches of one of the GEMMs above (packed leading
 * dimensions) on `stream` between two CUDA events, waits for them, and returns the elapsed
 * milliseconds in *ms together with the outcome of b200_check_device.  row_scale/col_scale are
 * only read for B200_W8A8. */
#define B200_W8A8 4
int b200_time_gemm(int dtype_or_w8a8, const void* A, const void* B, void* C, const float* row_scale,
                   const float* col_scale, int64_t M, int64_t N, int64_t K, int layout, int f32_mode,
                   int iters, float* ms, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200GEMM_H_ */
