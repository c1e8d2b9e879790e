// The extern "C" surface of libb200gemm: argument checking, layout mapping and dispatch onto the
// kernels.  Declarations and the reference call each entry point replaces: include/b200gemm.h.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "internal.h"
#include "ptx_sm100.cuh"

namespace b200 {

static thread_local char g_last_error[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
  return code;
}

namespace {

int64_t packed_ld(int layout, char which, int64_t M, int64_t N, int64_t K) {
  switch (layout) {
    case B200_ROW_MAJOR: return which == 'a' ? K : N;               // A[M,K] B[K,N] C[M,N]
    case B200_COL_MAJOR_NN: return which == 'a' ? M : (which == 'b' ? K : M);
    case B200_ROW_MAJOR_BT: return which == 'a' ? K : (which == 'b' ? K : N);
  }
  return 0;
}

// Maps a problem in any of the three layouts onto the kernels' native form
//   C'[M',N'] = A'[M',K] * B'   with A' K-contiguous, C' N'-contiguous,
// B' either [K,N'] N'-contiguous or [N',K] K-contiguous.
// Column-major C = A*B is the row-major product C^T = B^T * A^T: B (K contiguous per column)
// becomes A', A (M contiguous per k) becomes B' in its [K,N'] form, and M and N trade places.
struct Native {
  const void* A;
  const void* B;
  int64_t M, N, K, lda, ldb, ldc;
  bool b_is_nk;
};

int to_native(const void* A, const void* B, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb,
              int64_t ldc, int layout, Native* out) {
  if (layout != B200_ROW_MAJOR && layout != B200_COL_MAJOR_NN && layout != B200_ROW_MAJOR_BT)
    return fail(B200_ERR_BAD_ARGUMENT, "unknown layout %d", layout);
  if (M <= 0 || N <= 0 || K <= 0) return fail(B200_ERR_BAD_ARGUMENT, "M, N and K must be positive");
  if (lda == 0) lda = packed_ld(layout, 'a', M, N, K);
  if (ldb == 0) ldb = packed_ld(layout, 'b', M, N, K);
  if (ldc == 0) ldc = packed_ld(layout, 'c', M, N, K);
  if (layout == B200_COL_MAJOR_NN) {
    *out = Native{B, A, N, M, K, ldb, lda, ldc, false};
  } else {
    *out = Native{A, B, M, N, K, lda, ldb, ldc, layout == B200_ROW_MAJOR_BT};
  }
  return B200_OK;
}

int gemm_tensor(int kind, int epi, const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K,
                int64_t lda, int64_t ldb, int64_t ldc, int layout, const float* rs, const float* cs,
                void* stream) {
  Native nv;
  int rc = to_native(A, B, M, N, K, lda, ldb, ldc, layout, &nv);
  if (rc) return rc;
  return launch_umma_gemm(kind, epi, nv.A, nv.B, C, nv.M, nv.N, nv.K, nv.lda, nv.ldb, nv.ldc, nv.b_is_nk, rs,
                          cs, 0, static_cast<cudaStream_t>(stream));
}

// Device workspace of the *_host entry points, one per device (grows on demand): the three
// matrices, one stream per direction of travel plus one for the kernels, and the events that chain
// them chunk by chunk.  Calls on one device are serialised by the workspace's lock; calls on
// different devices do not meet.
constexpr int kHostChunks = 8;
constexpr int kMaxDevices = 64;
struct HostWorkspace {
  std::mutex mu;
  void* dA = nullptr;
  void* dB = nullptr;
  void* dC = nullptr;
  size_t capA = 0, capB = 0, capC = 0;
  cudaStream_t stream = nullptr;      // kernels
  cudaStream_t in_stream = nullptr;   // host -> device copies
  cudaStream_t out_stream = nullptr;  // device -> host copies
  cudaEvent_t whole_in = nullptr;     // the operand that is needed whole has arrived
  cudaEvent_t chunk_in[kHostChunks] = {nullptr};
  cudaEvent_t chunk_done[kHostChunks] = {nullptr};
} g_ws[kMaxDevices];

int current_workspace(HostWorkspace** out) {
  int dev = 0;
  B200_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices)
    return fail(B200_ERR_UNSUPPORTED, "device ordinal %d is beyond the host-workspace table", dev);
  *out = &g_ws[dev];
  return B200_OK;
}

int host_streams_ready(HostWorkspace& ws) {
  if (ws.stream) return B200_OK;
  B200_CUDA_TRY(cudaStreamCreateWithFlags(&ws.stream, cudaStreamNonBlocking));
  B200_CUDA_TRY(cudaStreamCreateWithFlags(&ws.in_stream, cudaStreamNonBlocking));
  B200_CUDA_TRY(cudaStreamCreateWithFlags(&ws.out_stream, cudaStreamNonBlocking));
  B200_CUDA_TRY(cudaEventCreateWithFlags(&ws.whole_in, cudaEventDisableTiming));
  for (int i = 0; i < kHostChunks; ++i) {
    B200_CUDA_TRY(cudaEventCreateWithFlags(&ws.chunk_in[i], cudaEventDisableTiming));
    B200_CUDA_TRY(cudaEventCreateWithFlags(&ws.chunk_done[i], cudaEventDisableTiming));
  }
  return B200_OK;
}

int grow(void** p, size_t* cap, size_t need) {
  if (*cap >= need) return B200_OK;
  if (*p) B200_CUDA_TRY(cudaFree(*p));
  *p = nullptr;
  *cap = 0;
  B200_CUDA_TRY(cudaMalloc(p, need));
  *cap = need;
  return B200_OK;
}

bool host_dtype_sizes(int dtype, size_t* in_elem, size_t* out_elem) {
  switch (dtype) {
    case B200_I8: *in_elem = 1; *out_elem = 4; return true;
    case B200_F16: case B200_BF16: *in_elem = 2; *out_elem = 2; return true;
    case B200_F32: *in_elem = 4; *out_elem = 4; return true;
  }
  return false;
}

// A weight matrix kept on the device between host-buffer calls (b200_host_weights_*).
struct HostWeights {
  uint32_t magic;
  int device;
  int dtype;
  int64_t K, N;
  void* dB;
};
constexpr uint32_t kWeightsMagic = 0xb2005eedu;

}  // namespace

int dispatch_gemm(int what, const void* A, const void* B, void* C, const float* rs, const float* cs, int64_t M,
                  int64_t N, int64_t K, int layout, int f32_mode, void* stream);

namespace {

// The slab pipeline shared by the host-buffer entry points.  `whole_dev` is the operand every line
// of the output needs, already on the device (or on its way: the kernel stream waits for
// `whole_ready` when that is not null).  The other operand travels in up to 16 slabs of `units`
// lines (rows of A; columns of B for the column-major layout); slab i + 1 is on its way up while
// slab i is multiplied and slab i - 1 of the result is on its way down.  Whatever happens, every
// copy and kernel issued here has finished before the function returns: the caller's buffers are
// never touched after an error return.
int run_host_slabs(HostWorkspace& ws, int dtype, int layout, const void* whole_dev, cudaEvent_t whole_ready,
                   const char* slab_src, char* slab_dst, char* c_dev_base, char* c_host, int64_t M, int64_t N,
                   int64_t K, size_t in_elem, size_t out_elem) {
  const bool col = layout == B200_COL_MAJOR_NN;
  const int64_t units = col ? N : M;                       // rows of A / columns of B
  const size_t in_unit = size_t(K) * in_elem;              // bytes of one of them
  const size_t out_unit = size_t(col ? M : N) * out_elem;  // bytes of the matching line of C
  // Slabs of a multiple of 256 units (the tallest tile of a small product), at least 512, at most 8 of them
  // (bf16 8192^3 through b200_gemm_host_weights: 3.49 ms per call with 8 slabs, 3.63-3.71 with 4, 3.80 with 16,
  // 4.19 with 32 of 256 rows; both directions of the host link busy at once move 43.5 GB/s each, 3.09 ms).
  // Nothing goes down while the first slab comes up and nothing comes up while the last goes down, so where
  // there is enough to cut, the first and the last slab are 256 units and the rest is shared by the others.
  int64_t sizes[kHostChunks];
  int n_slabs = 0;
  if (units >= 8 * 512) {
    const int middle = kHostChunks - 2;
    int64_t per = (units - 512 + middle - 1) / middle;
    per = (per + 255) / 256 * 256;
    sizes[n_slabs++] = 256;
    for (int64_t left = units - 512; left > 0 && n_slabs < kHostChunks - 1; left -= per)
      sizes[n_slabs++] = left < per ? left : per;
    sizes[n_slabs++] = 256;
  } else {
    int64_t per = (units + kHostChunks - 1) / kHostChunks;
    per = (per + 255) / 256 * 256;
    if (per < 512) per = 512;
    for (int64_t left = units; left > 0; left -= per) sizes[n_slabs++] = left < per ? left : per;
  }

  int rc = B200_OK;
  cudaError_t ce = cudaSuccess;
  const char* what = "";
#define HOST_STEP(call)                         \
  if (rc == B200_OK && ce == cudaSuccess) {     \
    ce = (call);                                \
    if (ce != cudaSuccess) what = #call;        \
  }
  if (whole_ready) HOST_STEP(cudaStreamWaitEvent(ws.stream, whole_ready, 0));
  int64_t u0 = 0;
  for (int i = 0; i < n_slabs && rc == B200_OK && ce == cudaSuccess; u0 += sizes[i], ++i) {
    const int64_t n_units = sizes[i];
    HOST_STEP(cudaMemcpyAsync(slab_dst + u0 * in_unit, slab_src + u0 * in_unit, size_t(n_units) * in_unit,
                              cudaMemcpyHostToDevice, ws.in_stream));
    HOST_STEP(cudaEventRecord(ws.chunk_in[i], ws.in_stream));
    HOST_STEP(cudaStreamWaitEvent(ws.stream, ws.chunk_in[i], 0));
    if (rc != B200_OK || ce != cudaSuccess) break;
    char* c_dev = c_dev_base + u0 * out_unit;
    if (col)
      rc = dispatch_gemm(dtype, whole_dev, slab_dst + u0 * in_unit, c_dev, nullptr, nullptr, M, n_units, K, layout,
                         B200_F32_FFMA, ws.stream);
    else
      rc = dispatch_gemm(dtype, slab_dst + u0 * in_unit, whole_dev, c_dev, nullptr, nullptr, n_units, N, K, layout,
                         B200_F32_FFMA, ws.stream);
    HOST_STEP(cudaEventRecord(ws.chunk_done[i], ws.stream));
    HOST_STEP(cudaStreamWaitEvent(ws.out_stream, ws.chunk_done[i], 0));
    HOST_STEP(cudaMemcpyAsync(c_host + u0 * out_unit, c_dev, size_t(n_units) * out_unit, cudaMemcpyDeviceToHost,
                              ws.out_stream));
  }
#undef HOST_STEP
  // Common tail, reached on success and on every failure alike: wait for all three streams.
  const cudaError_t e_in = cudaStreamSynchronize(ws.in_stream);
  const cudaError_t e_out = cudaStreamSynchronize(ws.out_stream);
  const int dev_rc = b200_check_device(ws.stream);  // synchronises the kernel stream
  if (rc) return rc;
  if (ce != cudaSuccess) return fail(B200_ERR_CUDA, "%s: %s", what, cudaGetErrorString(ce));
  if (e_in != cudaSuccess) return fail(B200_ERR_CUDA, "host-to-device copies: %s", cudaGetErrorString(e_in));
  if (e_out != cudaSuccess) return fail(B200_ERR_CUDA, "device-to-host copies: %s", cudaGetErrorString(e_out));
  return dev_rc;
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" const char* b200_last_error(void) { return g_last_error; }
extern "C" const char* b200_version(void) { return "b200gemm 0.1 (sm_100a)"; }

extern "C" int b200_sm_count(void) {
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) { cudaGetLastError(); return 0; }
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) { cudaGetLastError(); return 0; }
  return n;
}

extern "C" int b200_set_tile_policy(int cta_group, int tile_n, int group_rows) {
  return set_tile_policy(cta_group, tile_n, group_rows);
}

extern "C" int b200_check_device(void* stream) {
  uint32_t st = 0, st_skinny = 0;
  int rc = read_and_clear_umma_status(static_cast<cudaStream_t>(stream), &st);  // synchronises the stream
  if (rc) return rc;
  rc = read_and_clear_skinny_status(&st_skinny);
  if (rc) return rc;
  st |= st_skinny << 8;
  if (st) return fail(B200_ERR_DEVICE_WAIT, "a tensor-core kernel gave up a bounded wait (status 0x%x)", st);
  return B200_OK;
}

extern "C" int b200_gemm_i8_i32(const int8_t* A, const int8_t* B, int32_t* C, int64_t M, int64_t N, int64_t K,
                                int64_t lda, int64_t ldb, int64_t ldc, int layout, void* stream) {
  return gemm_tensor(KIND_I8, EPI_I32, A, B, C, M, N, K, lda, ldb, ldc, layout, nullptr, nullptr, stream);
}
extern "C" int b200_gemm_bf16(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K,
                              int64_t lda, int64_t ldb, int64_t ldc, int layout, void* stream) {
  return gemm_tensor(KIND_BF16, EPI_BF16, A, B, C, M, N, K, lda, ldb, ldc, layout, nullptr, nullptr, stream);
}
extern "C" int b200_gemm_f16(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K,
                             int64_t lda, int64_t ldb, int64_t ldc, int layout, void* stream) {
  return gemm_tensor(KIND_F16, EPI_F16, A, B, C, M, N, K, lda, ldb, ldc, layout, nullptr, nullptr, stream);
}
extern "C" int b200_gemm_16_f32(int dtype, const void* A, const void* B, float* C, int64_t M, int64_t N, int64_t K,
                                int64_t lda, int64_t ldb, int64_t ldc, int layout, void* stream) {
  if (dtype != B200_F16 && dtype != B200_BF16)
    return fail(B200_ERR_BAD_ARGUMENT, "b200_gemm_16_f32: dtype %d is neither B200_F16 nor B200_BF16", dtype);
  return gemm_tensor(dtype == B200_F16 ? KIND_F16 : KIND_BF16, EPI_F32, A, B, C, M, N, K, lda, ldb, ldc, layout,
                     nullptr, nullptr, stream);
}
extern "C" int b200_gemm_w8a8_bf16(const int8_t* A, const int8_t* B, const float* row_scale,
                                   const float* col_scale, void* C, int64_t M, int64_t N, int64_t K,
                                   int64_t lda, int64_t ldb, int64_t ldc, void* stream) {
  return gemm_tensor(KIND_I8, EPI_W8A8_BF16, A, B, C, M, N, K, lda, ldb, ldc, B200_ROW_MAJOR, row_scale,
                     col_scale, stream);
}

extern "C" int b200_gemm_f32(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K,
                             int64_t lda, int64_t ldb, int64_t ldc, int layout, int mode, void* stream) {
  Native nv;
  int rc = to_native(A, B, M, N, K, lda, ldb, ldc, layout, &nv);
  if (rc) return rc;
  if (mode == B200_F32_FFMA)
    return launch_sgemm_ffma(static_cast<const float*>(nv.A), static_cast<const float*>(nv.B), C, nv.M, nv.N,
                             nv.K, nv.lda, nv.ldb, nv.ldc, nv.b_is_nk, static_cast<cudaStream_t>(stream), Tail(),
                             /*may_split_k=*/true);
  if (mode == B200_F32_3XTF32)
    return launch_sgemm_3xtf32(static_cast<const float*>(nv.A), static_cast<const float*>(nv.B), C, nv.M, nv.N,
                               nv.K, nv.lda, nv.ldb, nv.ldc, nv.b_is_nk, static_cast<cudaStream_t>(stream));
  if (mode == B200_F32_TF32)
    return launch_sgemm_tf32(static_cast<const float*>(nv.A), static_cast<const float*>(nv.B), C, nv.M, nv.N, nv.K,
                             nv.lda, nv.ldb, nv.ldc, nv.b_is_nk, static_cast<cudaStream_t>(stream));
  return fail(B200_ERR_BAD_ARGUMENT, "unknown fp32 mode %d", mode);
}

extern "C" int b200_linear(int dtype, const void* X, const void* W, const float* bias, void* Y, int64_t batch,
                           int64_t in_features, int64_t out_features, int w_layout, int flags, int f32_mode,
                           void* stream_) {
  if (!X || !W || !Y) return fail(B200_ERR_BAD_ARGUMENT, "null matrix pointer");
  if (batch <= 0 || in_features <= 0 || out_features <= 0)
    return fail(B200_ERR_BAD_ARGUMENT, "batch and feature counts must be positive");
  if (w_layout != B200_ROW_MAJOR && w_layout != B200_ROW_MAJOR_BT)
    return fail(B200_ERR_BAD_ARGUMENT, "weights are [in, out] (B200_ROW_MAJOR) or [out, in] (B200_ROW_MAJOR_BT)");
  if (flags & ~(B200_LINEAR_RELU | B200_LINEAR_BIAS_FIRST)) return fail(B200_ERR_BAD_ARGUMENT, "unknown flags 0x%x", flags);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const bool w_is_out_in = w_layout == B200_ROW_MAJOR_BT;
  const int64_t M = batch, N = out_features, K = in_features;
  const int64_t ldw = w_is_out_in ? K : N;
  Tail tail;
  tail.bias = bias;
  tail.flags = flags;
  switch (dtype) {
    case B200_F32: {
      const float* x = static_cast<const float*>(X);
      const float* w = static_cast<const float*>(W);
      float* y = static_cast<float*>(Y);
      if (f32_mode == B200_F32_FFMA) return launch_sgemm_ffma(x, w, y, M, N, K, K, ldw, N, w_is_out_in, stream, tail);
      if (f32_mode == B200_F32_3XTF32) return launch_sgemm_3xtf32(x, w, y, M, N, K, K, ldw, N, w_is_out_in, stream, tail);
      if (f32_mode == B200_F32_TF32) return launch_sgemm_tf32(x, w, y, M, N, K, K, ldw, N, w_is_out_in, stream, tail);
      return fail(B200_ERR_BAD_ARGUMENT, "unknown fp32 mode %d", f32_mode);
    }
    case B200_F16:
      return launch_umma_gemm(KIND_F16, EPI_F16, X, W, Y, M, N, K, K, ldw, N, w_is_out_in, nullptr, nullptr, 0, stream,
                              tail);
    case B200_BF16:
      return launch_umma_gemm(KIND_BF16, EPI_BF16, X, W, Y, M, N, K, K, ldw, N, w_is_out_in, nullptr, nullptr, 0,
                              stream, tail);
  }
  return fail(B200_ERR_BAD_ARGUMENT, "b200_linear: dtype %d is not a floating-point type", dtype);
}

extern "C" int b200_gemm_naive(int dtype, const void* A, const void* B, void* C, int64_t M, int64_t N,
                               int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int layout, void* stream) {
  if (layout != B200_ROW_MAJOR && layout != B200_COL_MAJOR_NN && layout != B200_ROW_MAJOR_BT)
    return fail(B200_ERR_BAD_ARGUMENT, "unknown layout %d", layout);
  if (lda == 0) lda = packed_ld(layout, 'a', M, N, K);
  if (ldb == 0) ldb = packed_ld(layout, 'b', M, N, K);
  if (ldc == 0) ldc = packed_ld(layout, 'c', M, N, K);
  return launch_naive(dtype, A, B, C, M, N, K, lda, ldb, ldc, layout, static_cast<cudaStream_t>(stream));
}

int b200::dispatch_gemm(int what, const void* A, const void* B, void* C, const float* rs, const float* cs, int64_t M,
                        int64_t N, int64_t K, int layout, int f32_mode, void* stream) {
  switch (what) {
    case B200_I8:
      return b200_gemm_i8_i32(static_cast<const int8_t*>(A), static_cast<const int8_t*>(B),
                              static_cast<int32_t*>(C), M, N, K, 0, 0, 0, layout, stream);
    case B200_F16: return b200_gemm_f16(A, B, C, M, N, K, 0, 0, 0, layout, stream);
    case B200_BF16: return b200_gemm_bf16(A, B, C, M, N, K, 0, 0, 0, layout, stream);
    case B200_F32:
      return b200_gemm_f32(static_cast<const float*>(A), static_cast<const float*>(B), static_cast<float*>(C), M,
                           N, K, 0, 0, 0, layout, f32_mode, stream);
    case B200_W8A8:
      if (layout != B200_ROW_MAJOR) return fail(B200_ERR_BAD_ARGUMENT, "W8A8 is row-major only");
      return b200_gemm_w8a8_bf16(static_cast<const int8_t*>(A), static_cast<const int8_t*>(B), rs, cs, C, M, N, K,
                                 0, 0, 0, stream);
  }
  return fail(B200_ERR_BAD_ARGUMENT, "unknown dtype %d", what);
}

extern "C" int b200_time_gemm(int what, const void* A, const void* B, void* C, const float* row_scale,
                              const float* col_scale, int64_t M, int64_t N, int64_t K, int layout, int f32_mode,
                              int iters, float* ms, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!ms || iters <= 0) return fail(B200_ERR_BAD_ARGUMENT, "time_gemm: bad argument");
  cudaEvent_t e0, e1;
  B200_CUDA_TRY(cudaEventCreate(&e0));
  B200_CUDA_TRY(cudaEventCreate(&e1));
  int rc = B200_OK;
  cudaEventRecord(e0, stream);
  for (int i = 0; i < iters && rc == B200_OK; ++i)
    rc = dispatch_gemm(what, A, B, C, row_scale, col_scale, M, N, K, layout, f32_mode, stream_);
  cudaEventRecord(e1, stream);
  cudaError_t se = cudaEventSynchronize(e1);
  if (rc == B200_OK && se != cudaSuccess) rc = fail(B200_ERR_CUDA, "cudaEventSynchronize: %s", cudaGetErrorString(se));
  if (rc == B200_OK) {
    se = cudaEventElapsedTime(ms, e0, e1);
    if (se != cudaSuccess) rc = fail(B200_ERR_CUDA, "cudaEventElapsedTime: %s", cudaGetErrorString(se));
  }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  if (rc == B200_OK) rc = b200_check_device(stream_);
  return rc;
}

// Host buffers in, host buffers out.  The product is cut into up to 16 slabs along the dimension in
// which both an input and the output are contiguous (rows of A and C for the row-major layouts,
// columns of B and C for the column-major one).  The other operand goes up whole; then slab i + 1 is
// on its way up while slab i is multiplied and slab i - 1 of the result is on its way down, so the
// call takes about as long as its host-to-device traffic alone.
extern "C" int b200_gemm_host(int dtype, const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K,
                              int layout) {
  if (!A || !B || !C) return fail(B200_ERR_BAD_ARGUMENT, "null matrix pointer");
  if (M <= 0 || N <= 0 || K <= 0) return fail(B200_ERR_BAD_ARGUMENT, "M, N and K must be positive");
  if (layout != B200_ROW_MAJOR && layout != B200_COL_MAJOR_NN && layout != B200_ROW_MAJOR_BT)
    return fail(B200_ERR_BAD_ARGUMENT, "unknown layout %d", layout);
  size_t in_elem, out_elem;
  if (!host_dtype_sizes(dtype, &in_elem, &out_elem)) return fail(B200_ERR_BAD_ARGUMENT, "unknown dtype %d", dtype);
  HostWorkspace* wsp = nullptr;
  int rc = current_workspace(&wsp);
  if (rc) return rc;
  HostWorkspace& ws = *wsp;
  std::lock_guard<std::mutex> lock(ws.mu);
  if ((rc = host_streams_ready(ws))) return rc;
  const size_t bytesA = size_t(M) * K * in_elem, bytesB = size_t(K) * N * in_elem, bytesC = size_t(M) * N * out_elem;
  if ((rc = grow(&ws.dA, &ws.capA, bytesA))) return rc;
  if ((rc = grow(&ws.dB, &ws.capB, bytesB))) return rc;
  if ((rc = grow(&ws.dC, &ws.capC, bytesC))) return rc;

  const bool col = layout == B200_COL_MAJOR_NN;
  const char* whole_src = static_cast<const char*>(col ? A : B);
  char* whole_dst = static_cast<char*>(col ? ws.dA : ws.dB);
  const size_t whole_bytes = col ? bytesA : bytesB;
  // Nothing else is in flight yet, so a failure of these two calls may return at once.
  B200_CUDA_TRY(cudaMemcpyAsync(whole_dst, whole_src, whole_bytes, cudaMemcpyHostToDevice, ws.in_stream));
  cudaError_t ev = cudaEventRecord(ws.whole_in, ws.in_stream);
  if (ev != cudaSuccess) {
    cudaStreamSynchronize(ws.in_stream);
    return fail(B200_ERR_CUDA, "cudaEventRecord: %s", cudaGetErrorString(ev));
  }
  return run_host_slabs(ws, dtype, layout, whole_dst, ws.whole_in, static_cast<const char*>(col ? B : A),
                        static_cast<char*>(col ? ws.dB : ws.dA), static_cast<char*>(ws.dC), static_cast<char*>(C),
                        M, N, K, in_elem, out_elem);
}

// Frees the host-buffer workspace of the CURRENT device (weights uploaded with
// b200_host_weights_upload are separate objects and stay).
extern "C" int b200_host_release(void) {
  HostWorkspace* wsp = nullptr;
  int rc = current_workspace(&wsp);
  if (rc) return rc;
  HostWorkspace& ws = *wsp;
  std::lock_guard<std::mutex> lock(ws.mu);
  if (ws.dA) cudaFree(ws.dA);
  if (ws.dB) cudaFree(ws.dB);
  if (ws.dC) cudaFree(ws.dC);
  ws.dA = ws.dB = ws.dC = nullptr;
  ws.capA = ws.capB = ws.capC = 0;
  if (ws.stream) {
    cudaStreamDestroy(ws.stream);
    cudaStreamDestroy(ws.in_stream);
    cudaStreamDestroy(ws.out_stream);
    cudaEventDestroy(ws.whole_in);
    for (int i = 0; i < kHostChunks; ++i) {
      cudaEventDestroy(ws.chunk_in[i]);
      cudaEventDestroy(ws.chunk_done[i]);
    }
  }
  ws.stream = ws.in_stream = ws.out_stream = nullptr;
  return B200_OK;
}

// ------------------------------------------------------------------ host buffers, weights kept on the device

extern "C" int b200_host_weights_upload(int dtype, const void* B, int64_t K, int64_t N, void** weights) {
  if (!B || !weights) return fail(B200_ERR_BAD_ARGUMENT, "null pointer");
  if (K <= 0 || N <= 0) return fail(B200_ERR_BAD_ARGUMENT, "K and N must be positive");
  size_t in_elem, out_elem;
  if (!host_dtype_sizes(dtype, &in_elem, &out_elem)) return fail(B200_ERR_BAD_ARGUMENT, "unknown dtype %d", dtype);
  int dev = 0;
  B200_CUDA_TRY(cudaGetDevice(&dev));
  void* dB = nullptr;
  B200_CUDA_TRY(cudaMalloc(&dB, size_t(K) * N * in_elem));
  cudaError_t e = cudaMemcpy(dB, B, size_t(K) * N * in_elem, cudaMemcpyHostToDevice);
  if (e != cudaSuccess) {
    cudaFree(dB);
    return fail(B200_ERR_CUDA, "upload of the weights: %s", cudaGetErrorString(e));
  }
  *weights = new HostWeights{kWeightsMagic, dev, dtype, K, N, dB};
  return B200_OK;
}

extern "C" int b200_host_weights_free(void* weights) {
  if (!weights) return B200_OK;
  HostWeights* w = static_cast<HostWeights*>(weights);
  if (w->magic != kWeightsMagic) return fail(B200_ERR_BAD_ARGUMENT, "not a weights handle");
  int dev = 0;
  B200_CUDA_TRY(cudaGetDevice(&dev));
  if (dev != w->device) B200_CUDA_TRY(cudaSetDevice(w->device));
  cudaError_t e = cudaFree(w->dB);
  if (dev != w->device) cudaSetDevice(dev);
  w->magic = 0;
  delete w;
  if (e != cudaSuccess) return fail(B200_ERR_CUDA, "cudaFree(weights): %s", cudaGetErrorString(e));
  return B200_OK;
}

extern "C" int b200_gemm_host_weights(const void* weights, const void* A, void* C, int64_t M) {
  if (!weights || !A || !C) return fail(B200_ERR_BAD_ARGUMENT, "null pointer");
  const HostWeights* w = static_cast<const HostWeights*>(weights);
  if (w->magic != kWeightsMagic) return fail(B200_ERR_BAD_ARGUMENT, "not a weights handle");
  if (M <= 0) return fail(B200_ERR_BAD_ARGUMENT, "M must be positive");
  int dev = 0;
  B200_CUDA_TRY(cudaGetDevice(&dev));
  if (dev != w->device)
    return fail(B200_ERR_UNSUPPORTED, "the weights live on device %d but device %d is current", w->device, dev);
  size_t in_elem = 0, out_elem = 0;
  host_dtype_sizes(w->dtype, &in_elem, &out_elem);
  HostWorkspace* wsp = nullptr;
  int rc = current_workspace(&wsp);
  if (rc) return rc;
  HostWorkspace& ws = *wsp;
  std::lock_guard<std::mutex> lock(ws.mu);
  if ((rc = host_streams_ready(ws))) return rc;
  if ((rc = grow(&ws.dA, &ws.capA, size_t(M) * w->K * in_elem))) return rc;
  if ((rc = grow(&ws.dC, &ws.capC, size_t(M) * w->N * out_elem))) return rc;
  return run_host_slabs(ws, w->dtype, B200_ROW_MAJOR, w->dB, nullptr, static_cast<const char*>(A),
                        static_cast<char*>(ws.dA), static_cast<char*>(ws.dC), static_cast<char*>(C), M, w->N, w->K,
                        in_elem, out_elem);
}

// ------------------------------------------------------------------ several destinations, peer memory

extern "C" int b200_set_store_policy(int register_stores) { return set_store_policy(register_stores); }
extern "C" int b200_set_dependent_launch(int enabled) { return set_dependent_launch(enabled); }
extern "C" int b200_set_l2_hints(int hints) { return set_l2_hints(hints); }
extern "C" int b200_set_3xtf32_path(int path) { return set_x3_path(path); }
extern "C" int b200_set_ffma_k_ranges(int ranges) { return set_ffma_ksplit(ranges); }
extern "C" int b200_test_lose_arrival(int64_t k_block, uint64_t wait_budget_ns) {
  return set_wait_test(k_block, wait_budget_ns);
}

extern "C" int b200_gemm_multi(int what, const void* A, const void* B, void* const* C_list, int n_dest,
                               const float* row_scale, const float* col_scale, int64_t M, int64_t N, int64_t K,
                               int64_t lda, int64_t ldb, int64_t ldc, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return fail(B200_ERR_BAD_ARGUMENT, "M, N and K must be positive");
  if (lda == 0) lda = K;
  if (ldb == 0) ldb = N;
  if (ldc == 0) ldc = N;
  int kind, epi;
  switch (what) {
    case B200_I8: kind = KIND_I8; epi = EPI_I32; break;
    case B200_F16: kind = KIND_F16; epi = EPI_F16; break;
    case B200_BF16: kind = KIND_BF16; epi = EPI_BF16; break;
    case B200_W8A8: kind = KIND_I8; epi = EPI_W8A8_BF16; break;
    default: return fail(B200_ERR_BAD_ARGUMENT, "b200_gemm_multi: unsupported type %d", what);
  }
  return launch_umma_gemm_multi(kind, epi, A, B, C_list, n_dest, M, N, K, lda, ldb, ldc, false, row_scale,
                                col_scale, 0, static_cast<cudaStream_t>(stream));
}

extern "C" int b200_gemm_multicast(int what, const void* A, const void* B, void* C_multicast, const float* row_scale,
                                   const float* col_scale, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb,
                                   int64_t ldc, void* stream) {
  if (!C_multicast) return fail(B200_ERR_BAD_ARGUMENT, "null multicast pointer");
  if (M <= 0 || N <= 0 || K <= 0) return fail(B200_ERR_BAD_ARGUMENT, "M, N and K must be positive");
  if (lda == 0) lda = K;
  if (ldb == 0) ldb = N;
  if (ldc == 0) ldc = N;
  int kind, epi;
  switch (what) {
    case B200_I8: kind = KIND_I8; epi = EPI_I32; break;
    case B200_F16: kind = KIND_F16; epi = EPI_F16; break;
    case B200_BF16: kind = KIND_BF16; epi = EPI_BF16; break;
    case B200_W8A8: kind = KIND_I8; epi = EPI_W8A8_BF16; break;
    default: return fail(B200_ERR_BAD_ARGUMENT, "b200_gemm_multicast: unsupported type %d", what);
  }
  return launch_umma_gemm_multicast(kind, epi, A, B, C_multicast, M, N, K, lda, ldb, ldc, row_scale, col_scale,
                                    static_cast<cudaStream_t>(stream));
}

extern "C" int b200_peer_alloc(size_t bytes, void** ptr) {
  if (!ptr || bytes == 0) return fail(B200_ERR_BAD_ARGUMENT, "peer_alloc: bad argument");
  B200_CUDA_TRY(cudaMalloc(ptr, bytes));
  return B200_OK;
}
extern "C" int b200_peer_free(void* ptr) {
  if (ptr) B200_CUDA_TRY(cudaFree(ptr));
  return B200_OK;
}
extern "C" int b200_ipc_export(void* ptr, void* handle64) {
  if (!ptr || !handle64) return fail(B200_ERR_BAD_ARGUMENT, "ipc_export: null pointer");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  cudaIpcMemHandle_t h;
  B200_CUDA_TRY(cudaIpcGetMemHandle(&h, ptr));
  memcpy(handle64, &h, sizeof(h));
  return B200_OK;
}
extern "C" int b200_ipc_import(const void* handle64, void** ptr) {
  if (!ptr || !handle64) return fail(B200_ERR_BAD_ARGUMENT, "ipc_import: null pointer");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  B200_CUDA_TRY(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return B200_OK;
}
extern "C" int b200_ipc_close(void* ptr) {
  if (ptr) B200_CUDA_TRY(cudaIpcCloseMemHandle(ptr));
  return B200_OK;
}
