// Skinny tensor-core products for sm_100a: C[M,N] = A[M,K] * B with M <= 128 rows (a decode or
// small-prefill batch against a wide weight matrix): fp16 / bf16 in and out with fp32 accumulation,
// or int8 in with int32 accumulation and either int32 out or the per-row x per-column scaled bf16
// output of the W8A8 product.
//
// Such a product streams B from HBM once and does little arithmetic, so what counts is that every
// SM streams an equal share of B.  A CTA of this kind completes one k-block (128 bytes of K per row)
// about every 0.36 us whether its tile is 128 or 192 columns wide and however deep its ring is (the
// pace of the serial TMA-issue and MMA-issue loops), i.e. 45-70 GB/s per SM: a [4096 -> 11008] layer
// cut into 86 column tiles of 128 therefore runs at the speed of 86 SMs, 3.6 TB/s, while 116 CTAs of
// 192 columns reach the 7 TB/s HBM gives.  Here a tile of BN columns (128, 192 or 256)
// is shared by a thread-block cluster of S CTAs (1, 2, 4 or 8) that each stream one K range of it;
// tiles x S is chosen close to the SM count.  The partial sums meet on chip, reduce-scatter fashion:
//
//   1. every CTA runs the usual ring (TMA producer -> tcgen05.mma into tensor memory) over its K range;
//   2. the columns of the tile are dealt out to the CTAs of the cluster, BN / S each.  Every CTA moves
//      its accumulator out of tensor memory, each 32-column chunk into the exchange area of the CTA that
//      owns those columns (its own included; the others' through distributed shared memory), 16 bytes
//      per lane and store, into the slot of its K range;
//   3. cluster barrier: the slots are complete and visible to their owners;
//   4. every CTA adds the slots of its columns in K order (so the result does not depend on timing),
//      applies the optional bias / ReLU tail, rounds once to the 16-bit type and stores the rows
//      below M.  All four warps share this work whatever M is; only step 2 is tied to the warp that
//      may read a given quarter of tensor memory (a single warp needs about 0.5 us per 32 columns
//      for the arithmetic of step 4, which is why the two steps are separate).
//
// Only R = 32, 64, 96 or 128 rows of A are staged per k-block (M rounded up to 32).  The MMA is
// always 128 rows tall and reads its other operand rows from the bytes that follow in the stage (the
// B tile); an accumulator row depends on its own row of A only, so rows R..127 hold garbage that
// is never read back.
//
// CTA = four warps.  Lane 0 of warp 0 issues the TMA loads, lane 0 of warp 1 the MMAs (warp 1 owns
// the TMEM allocation); warp q < R / 32 then does step 2 for rows 32q..32q+31 and all warps step 4.
// Every mbarrier wait is bounded; the barriers are reached by every thread on every path, including
// the one where a wait was given up.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstring>
#include <mutex>

#include "internal.h"
#include "ptx_sm100.cuh"

namespace b200 {

namespace {

__device__ uint32_t g_skinny_status = 0;  // bit 0: a bounded wait ran out somewhere

// Timeline instrumentation, compiled in only with -DB200_SKINNY_STAMPS (a measurement build; the
// shipped library has none of it).  Every CTA records %globaltimer for its first 64 k-blocks at four
// points: the producer lane after its wait for a free stage and after issuing the stage's loads,
// the MMA lane after its wait for the full stage and after issuing the stage's MMAs; plus one stamp
// right after the dependency wait (row 4, word 0); row 5 holds the tail: word 0 = accumulator complete,
// 1 = tensor memory moved to the exchange slots, 2 = past the barrier, 3 = sums stored (thread 0 each).
// Layout: stamps[cta][6][64] 64-bit words.
#ifdef B200_SKINNY_STAMPS
__device__ unsigned long long* g_sk_stamps = nullptr;
#define SK_STAMP(which, i)                                                                     \
  do {                                                                                         \
    if (g_sk_stamps != nullptr && (i) < 64)                                                    \
      g_sk_stamps[(size_t(blockIdx.x) * 6 + (which)) * 64 + (i)] = global_timer_ns();          \
  } while (0)
#else
#define SK_STAMP(which, i) do { } while (0)
#endif

constexpr int kSkThreads = 128;
constexpr int kSkMaxRows = 128;          // rows of C one launch can produce
constexpr int kSkMaxStages = 8;
constexpr int kSkSmemBudget = 227 * 1024;
constexpr int kSkTailBytes = 256;        // barriers, TMEM slot, abort flag

struct SkinnyArgs {
  void* C;
  int64_t ldc;
  int M, N, K;
  int rows;          // R: rows of A staged = M rounded up to a multiple of 32
  int bn;            // tile width: 128, 192 or 256
  int splits;        // S: CTAs per cluster = K ranges per tile; divides bn / 32
  int kb_per_split;  // k-blocks per range (the last range may be shorter, never empty)
  int stages;
  int kind;          // KIND_F16, KIND_BF16 or KIND_I8
  int esz;           // bytes per element of A and B (2 or 1); a stage holds 128 bytes of K per row
  int epi;           // Epilogue: EPI_F16, EPI_BF16, EPI_I32 or EPI_W8A8_BF16
  int b_is_nk;       // B is [N,K] (K contiguous) instead of [K,N]
  int vec_store;     // rows of C are 16-byte aligned
  const float* bias;
  int tail_flags;    // b200_linear_flags (floating-point products)
  const float* row_scale;  // W8A8
  const float* col_scale;
};

__device__ __forceinline__ void st_cluster_v4(uint32_t cluster_addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared::cluster.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(cluster_addr), "r"(a), "r"(b), "r"(c), "r"(d)
               : "memory");
}

// Step 4 of the kernel below for one epilogue kind: add the K ranges' slots in range order, apply the tail,
// convert and store.  A thread takes (block of 32 rows, group of 8 columns) pairs: its lane is the row
// inside the block, so reads of a slot are conflict-free (consecutive lanes, 16 bytes each).  Only four
// warps run here, one per scheduler, so nothing hides an instruction's latency but the warp's own
// independent work: four pairs are processed together (their loads, sums and conversions interleave).
// Taken one at a time, a pair cost 0.87 us (about 1650 clocks of one dependent chain), 2.9 us of a
// 20 us launch at 16 rows and 11 us at 128.
template <int EPI>
__device__ __forceinline__ void skinny_finish(const SkinnyArgs& p, const uint4* __restrict__ slots, int R, int S,
                                              int own_units, int own_chunks, int row_blocks, int col0, int warp,
                                              int lane) {
  constexpr bool kInteger = EPI == EPI_I32 || EPI == EPI_W8A8_BF16;
  constexpr int kOutBytes = EPI == EPI_I32 ? 4 : 2;
  constexpr int UNR = 4;
  const bool relu = (p.tail_flags & B200_LINEAR_RELU) != 0;
  const int total = row_blocks * own_chunks * 4;
  const int range_stride = own_units * R;  // uint4 words between the slots of successive K ranges
  for (int u0 = warp; u0 < total; u0 += 4 * UNR) {
    uint32_t acc[UNR][8];
    int row[UNR], nc[UNR], ofs[UNR];
    bool live[UNR];
#pragma unroll
    for (int b = 0; b < UNR; ++b) {
      const int u = u0 + 4 * b;
      live[b] = u < total;
      const int uu = live[b] ? u : u0;  // a dead pair re-reads a live one's slots and stores nothing
      const int rb = uu % row_blocks, g = uu / row_blocks;
      row[b] = rb * 32 + lane;
      nc[b] = col0 + g * 8;
      ofs[b] = g * 2 * R + row[b];
      live[b] = live[b] && nc[b] < p.N;
    }
#pragma unroll
    for (int b = 0; b < UNR; ++b) {
      const uint4 t0 = slots[ofs[b]], t1 = slots[ofs[b] + R];
      acc[b][0] = t0.x; acc[b][1] = t0.y; acc[b][2] = t0.z; acc[b][3] = t0.w;
      acc[b][4] = t1.x; acc[b][5] = t1.y; acc[b][6] = t1.z; acc[b][7] = t1.w;
    }
    for (int r = 1; r < S; ++r) {
#pragma unroll
      for (int b = 0; b < UNR; ++b) {
        const uint4 t0 = slots[r * range_stride + ofs[b]], t1 = slots[r * range_stride + ofs[b] + R];
        const uint32_t in[8] = {t0.x, t0.y, t0.z, t0.w, t1.x, t1.y, t1.z, t1.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if constexpr (kInteger) acc[b][j] += in[j];
          else acc[b][j] = __float_as_uint(__uint_as_float(acc[b][j]) + __uint_as_float(in[j]));
        }
      }
    }
#pragma unroll
    for (int b = 0; b < UNR; ++b) {
      uint32_t w[8];  // 8 outputs: 8 words of int32, or 4 words of two 16-bit values
      if constexpr (EPI == EPI_I32) {
#pragma unroll
        for (int j = 0; j < 8; ++j) w[j] = acc[b][j];
      } else {
        float rs = 0.0f;
        if constexpr (EPI == EPI_W8A8_BF16) rs = (live[b] && row[b] < p.M) ? __ldg(p.row_scale + row[b]) : 0.0f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float x0, x1;
          if constexpr (EPI == EPI_W8A8_BF16) {
            // (float(acc) * row_scale) * col_scale, each step rounded once, then to bf16
            const float c0 = __ldg(p.col_scale + min(max(nc[b], 0) + 2 * j, p.N - 1));
            const float c1 = __ldg(p.col_scale + min(max(nc[b], 0) + 2 * j + 1, p.N - 1));
            x0 = __fmul_rn(__fmul_rn(__int2float_rn(int(acc[b][2 * j])), rs), c0);
            x1 = __fmul_rn(__fmul_rn(__int2float_rn(int(acc[b][2 * j + 1])), rs), c1);
          } else {
            x0 = __uint_as_float(acc[b][2 * j]);
            x1 = __uint_as_float(acc[b][2 * j + 1]);
            if (p.bias != nullptr) {
              x0 += __ldg(p.bias + min(nc[b] + 2 * j, p.N - 1));
              x1 += __ldg(p.bias + min(nc[b] + 2 * j + 1, p.N - 1));
            }
            if (relu) {
              x0 = fmaxf(0.0f, x0);
              x1 = fmaxf(0.0f, x1);
            }
          }
          if constexpr (EPI == EPI_F16) {
            __half2 h = __floats2half2_rn(x0, x1);
            w[j] = *reinterpret_cast<uint32_t*>(&h);
          } else {
            __nv_bfloat162 h = __floats2bfloat162_rn(x0, x1);
            w[j] = *reinterpret_cast<uint32_t*>(&h);
          }
        }
      }
      if (live[b] && row[b] < p.M) {
        char* dst = static_cast<char*>(p.C) + (int64_t(row[b]) * p.ldc + nc[b]) * kOutBytes;
        if (p.vec_store && nc[b] + 8 <= p.N) {
          *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
          if constexpr (kOutBytes == 4) *reinterpret_cast<uint4*>(dst + 16) = make_uint4(w[4], w[5], w[6], w[7]);
        } else if constexpr (kOutBytes == 4) {
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (nc[b] + j < p.N) reinterpret_cast<uint32_t*>(dst)[j] = w[j];
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (nc[b] + j < p.N) reinterpret_cast<uint16_t*>(dst)[j] = uint16_t(w[j >> 1] >> ((j & 1) * 16));
        }
      }
    }
  }
}

// ESZ (bytes per element of A and B) and B_NK (B given as [N,K]) are template parameters although the
// code would run with them as arguments: the TMA-issuing lane and the MMA-issuing lane each execute a
// short serial loop per k-block that paces the whole CTA, and every instruction in those loops shows in
// the result (an integer division per iteration doubled the time of the kernel; run-time strides and
// a run-time choice of the MMA kind cost another 10 %).
template <int ESZ, bool B_NK>
__global__ void __launch_bounds__(kSkThreads, 1)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                   const SkinnyArgs p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int R = p.rows;
  const int S = p.splits;
  const int a_bytes = R * 128;
  const int stage_bytes = a_bytes + p.bn * 128;
  // ring of stages | exchange area (written by every CTA of the cluster) | barriers
  // Exchange area: [K range][16-byte unit of this CTA's columns][row][4 floats]; S * (bn / S) * R * 4 bytes.
  float* exch = reinterpret_cast<float*>(smem + p.stages * stage_bytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + p.stages * stage_bytes + p.bn * R * 4);
  uint64_t* full_bar = bars;                    // [stages] producer -> MMA
  uint64_t* empty_bar = bars + kSkMaxStages;    // [stages] MMA -> producer
  uint64_t* acc_full = bars + 2 * kSkMaxStages; // MMA -> the warps that read tensor memory
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = S > 1 ? cluster_cta_rank() : 0u;
  const int tile = int(blockIdx.x) / S;
  const int n0 = tile * p.bn;
  constexpr int bk = 128 / ESZ;          // elements of K per stage (one 128-byte swizzle row)
  constexpr int span_cols = 128 / ESZ;   // columns in one 128-byte span of an N-contiguous B
  constexpr int span_bytes = bk * 128;   // one span: bk k-rows of 128 bytes
  const int nspans = p.bn / span_cols;   // spans of an N-contiguous B tile
  const int num_kb = (p.K + bk - 1) / bk;
  const int kb0 = int(rank) * p.kb_per_split;
  const int kb_count = min(p.kb_per_split, num_kb - kb0);  // >= 1 by construction of the launch
  const uint32_t tmem_cols = p.bn <= 128 ? 128u : 256u;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  // In a cluster this is also the point after which every CTA of it is known to be running, which
  // writing into another CTA's shared memory requires; it costs nothing at the tail that way.
  __syncwarp();
  if (S > 1) cluster_sync_all(); else __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  // Nothing above touched global memory.  Wait for the kernel this launch was serialised behind (a
  // no-op without a programmatic dependency) and let the next kernel begin its own set-up.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (threadIdx.x == 0) SK_STAMP(4, 0);

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int i = 0; i < kb_count; ++i) {
        if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1u, abort_flag)) break;
        SK_STAMP(0, i);
        uint8_t* sa = smem + stage * stage_bytes;
        uint8_t* sb = sa + a_bytes;
        const int k = (kb0 + i) * bk;
        mbar_arrive_expect_tx(&full_bar[stage], uint32_t(stage_bytes));
        tma_load_2d(sa, &tmap_a, &full_bar[stage], k, 0);
        if constexpr (B_NK) {
          tma_load_2d(sb, &tmap_b, &full_bar[stage], k, n0);
        } else {
          for (int s = 0; s < nspans; ++s)
            tma_load_2d(sb + s * span_bytes, &tmap_b, &full_bar[stage], n0 + s * span_cols, k);
        }
        SK_STAMP(1, i);
        if (++stage == p.stages) { stage = 0; phase ^= 1u; }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = make_instr_desc(p.kind, 128, p.bn, 0, B_NK ? 0 : 1);
      // descriptors of stage 0, stepped per k-block (the address field is in units of 16 bytes)
      const uint32_t ring = smem_u32(smem);
      const uint64_t a_desc0 = make_smem_desc_sw128(ring, 16, 1024);
      const uint64_t b_desc0 = B_NK ? make_smem_desc_sw128(ring + uint32_t(a_bytes), 16, 1024)
                                    : make_smem_desc_sw128(ring + uint32_t(a_bytes), uint32_t(span_bytes), 1024);
      const uint64_t stage_step = uint64_t(stage_bytes >> 4);
      uint64_t a_desc = a_desc0, b_desc = b_desc0;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int i = 0; i < kb_count; ++i) {
        if (!mbar_wait_bounded(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
        SK_STAMP(2, i);
        tc_fence_after_sync();
#pragma unroll
        for (int j = 0; j < 4; ++j) {  // 32 bytes of K per instruction
          const uint64_t a_adv = uint64_t((j * 32) >> 4);
          // 32 bytes along a K-contiguous row, or the k-rows of an N-contiguous span that hold 32 bytes of K
          const uint64_t b_adv = B_NK ? uint64_t((j * 32) >> 4) : uint64_t((j * (32 / ESZ) * 128) >> 4);
          umma<(ESZ == 1 ? KIND_I8 : KIND_F16)>(tmem_base, a_desc + a_adv, b_desc + b_adv, idesc,
                                                (i | j) != 0 ? 1u : 0u);
        }
        umma_commit(&empty_bar[stage]);
        SK_STAMP(3, i);
        a_desc += stage_step;
        b_desc += stage_step;
        if (++stage == p.stages) { stage = 0; phase ^= 1u; a_desc = a_desc0; b_desc = b_desc0; }
      }
      if (ok) umma_commit(acc_full);
    }
    __syncwarp();
  }

  const int chunks = min(p.bn / 32, (p.N - n0 + 31) / 32);  // 32-column chunks with a column inside C
  const int own_chunks = p.bn / 32 / S;                     // chunks whose columns one CTA finishes
  const int own_units = own_chunks * 8;                     // 16-byte units (4 columns) of those
  if (warp < R / 32) {
    // ---------------------------------------------------------------- step 2: tensor memory -> slots
    bool acc_ready = mbar_wait_bounded(acc_full, 0u, abort_flag);
    acc_ready = __all_sync(0xffffffffu, acc_ready) != 0;  // the warp acts as one from here on
    if (threadIdx.x == 0) SK_STAMP(5, 0);
    tc_fence_after_sync();
    if (acc_ready) {
      const uint32_t quarter = tmem_base + (uint32_t(warp * 32) << 16);  // rows 32 * warp + lane
      // byte offset of (slot of this K range, unit 0, this thread's row) inside an exchange area
      const uint32_t mine = uint32_t(((int(rank) * own_units) * R + warp * 32 + lane) * 16);
      const uint32_t exch_addr = smem_u32(exch);
      for (int c0 = 0; c0 < chunks; c0 += 4) {  // up to four chunks fetched before the one wait
        uint32_t v[4][32];
#pragma unroll
        for (int g = 0; g < 4; ++g)
          if (c0 + g < chunks) tmem_ld_32x32(quarter + uint32_t((c0 + g) * 32), v[g]);
        tmem_ld_wait();
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          if (c0 + g < chunks) {
            const int c = c0 + g;
            const int owner = c / own_chunks;
            const uint32_t dst = map_to_cta(exch_addr, uint32_t(owner)) + mine +
                                 uint32_t((c - owner * own_chunks) * 8 * R * 16);
#pragma unroll
            for (int q = 0; q < 8; ++q)
              st_cluster_v4(dst + uint32_t(q * R * 16), v[g][4 * q], v[g][4 * q + 1], v[g][4 * q + 2], v[g][4 * q + 3]);
          }
        }
      }
    }
  }
  // Step 3: every slot is complete and visible to its owner.
  __syncwarp();
  if (threadIdx.x == 0) SK_STAMP(5, 1);
  if (S > 1) cluster_sync_all(); else __syncthreads();
  if (threadIdx.x == 0) SK_STAMP(5, 2);

  if (*abort_flag == 0u) {
    // ---------------------------------------------------------------- step 4: add, finish, store
    const int row_blocks = R / 32;
    const int col0 = n0 + int(rank) * own_chunks * 32;  // first column this CTA finishes
    const uint4* slots = reinterpret_cast<const uint4*>(exch);
    switch (p.epi) {
      case EPI_F16: skinny_finish<EPI_F16>(p, slots, R, S, own_units, own_chunks, row_blocks, col0, warp, lane); break;
      case EPI_BF16: skinny_finish<EPI_BF16>(p, slots, R, S, own_units, own_chunks, row_blocks, col0, warp, lane); break;
      case EPI_I32: skinny_finish<EPI_I32>(p, slots, R, S, own_units, own_chunks, row_blocks, col0, warp, lane); break;
      default: skinny_finish<EPI_W8A8_BF16>(p, slots, R, S, own_units, own_chunks, row_blocks, col0, warp, lane); break;
    }
  }

  // Every role gets here: its loop ended or its wait was given up.
  __syncwarp();
  if (threadIdx.x == 0) SK_STAMP(5, 3);
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0) atomicOr(&g_skinny_status, 1u);
    // Give copies and MMAs still in flight time to land before shared and tensor memory go away.
    uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 2000000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, tmem_cols);
  }
}

using SkinnyKernel = void (*)(const CUtensorMap, const CUtensorMap, const SkinnyArgs);
SkinnyKernel skinny_kernel_for(int esz, bool b_is_nk) {
  if (esz == 1) return b_is_nk ? gemm_skinny_kernel<1, true> : gemm_skinny_kernel<1, false>;
  return b_is_nk ? gemm_skinny_kernel<2, true> : gemm_skinny_kernel<2, false>;
}

// Clusters of `splits` CTAs the device can hold at once.  Every configuration takes more than half
// of an SM's shared memory, so one CTA per SM it is; the query is made with the largest footprint.
int max_resident_clusters(int splits, int* out) {
  static std::mutex mu;
  static int cache[64][9];  // [device][splits]: 0 = unknown
  int dev = 0;
  B200_CUDA_TRY(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lock(mu);
  if (dev < 64 && cache[dev][splits]) { *out = cache[dev][splits] > 0 ? cache[dev][splits] : 0; return B200_OK; }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(unsigned(splits));
  cfg.blockDim = dim3(kSkThreads);
  cfg.dynamicSmemBytes = size_t(kSkSmemBudget);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = unsigned(splits);
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  // the four instantiations have the same footprint (one CTA per SM): ask for one of them
  SkinnyKernel probe = skinny_kernel_for(2, false);
  B200_CUDA_TRY(cudaFuncSetAttribute(probe, cudaFuncAttributeMaxDynamicSharedMemorySize, kSkSmemBudget));
  B200_CUDA_TRY(cudaOccupancyMaxActiveClusters(&n, probe, &cfg));
  if (dev < 64) cache[dev][splits] = n > 0 ? n : -1;
  *out = n;
  return B200_OK;
}

}  // namespace

#ifdef B200_SKINNY_STAMPS
}  // namespace b200
// Measurement build only: where the skinny kernel writes its timeline (device memory, 5 * 64 words per CTA), or null.
extern "C" int b200_debug_set_skinny_stamps(void* device_buffer) {
  unsigned long long* p = static_cast<unsigned long long*>(device_buffer);
  return cudaMemcpyToSymbol(b200::g_sk_stamps, &p, sizeof(p)) == cudaSuccess ? 0 : 3;
}
namespace b200 {
#endif

int read_and_clear_skinny_status(uint32_t* out) {
  uint32_t zero = 0;
  B200_CUDA_TRY(cudaMemcpyFromSymbol(out, g_skinny_status, sizeof(uint32_t)));
  if (*out) B200_CUDA_TRY(cudaMemcpyToSymbol(g_skinny_status, &zero, sizeof(uint32_t)));
  return B200_OK;
}

// Decides whether the product is one this kernel should take and, if so, launches it.
//   *used = false and B200_OK: not taken (the caller runs the general kernel).
//   force = true: the caller insists (tile policy 3); a product that does not qualify is an error.
// Costs are what one SM has to pull through its TMA unit, in 128-byte rows: per k-block the columns
// of B (from DRAM) plus 0.3 x the rows of A (from L2, which was measured to weigh about that much).
int launch_skinny_gemm(int kind, int epi, const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K,
                       int64_t lda, int64_t ldb, int64_t ldc, bool b_is_nk, const float* row_scale,
                       const float* col_scale, const Tail& tail, int force_bn, bool force, int64_t general_cost,
                       cudaStream_t stream, bool* used) {
  *used = false;
  const bool known = (kind == KIND_F16 && epi == EPI_F16) || (kind == KIND_BF16 && epi == EPI_BF16) ||
                     (kind == KIND_I8 && (epi == EPI_I32 || epi == EPI_W8A8_BF16));
  if (!known || M > kSkMaxRows) {
    if (force)
      return fail(B200_ERR_UNSUPPORTED, "the skinny kernel takes fp16, bf16 and int8 products of at most %d rows",
                  kSkMaxRows);
    return B200_OK;
  }
  const int esz = kind == KIND_I8 ? 1 : 2;
  const int out_esz = epi == EPI_I32 ? 4 : 2;
  const int bk = 128 / esz;
  int sms = 0;
  int dev = 0;
  B200_CUDA_TRY(cudaGetDevice(&dev));
  B200_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const int num_kb = int((K + bk - 1) / bk);
  const int rows = int((M + 31) / 32) * 32;

  // Tile width and cluster size: the smallest cost per CTA among the configurations that run in one
  // wave, with a charge per split product for the exchange (about 1 us of streaming).
  int best_bn = 0, best_s = 0, best_per = 0, best_stages = 0;
  int64_t best_cost = 0;
  for (int bn = 128; bn <= 256; bn += 64) {
    if (force_bn && bn != force_bn) continue;
    if (!b_is_nk && bn % (128 / esz)) continue;  // an N-contiguous B is staged in whole 128-byte spans
    const int stage_bytes = rows * 128 + bn * 128;
    const int64_t tiles = (N + bn - 1) / bn;
    if (tiles > sms) continue;
    int s_max = int(sms / tiles);
    if (s_max > 8) s_max = 8;
    if (s_max > num_kb) s_max = num_kb;
    // Cluster sizes 1, 2, 4, 8 only: clusters of 3 did not all become resident together on a B200
    // (whatever the occupancy query said) and the product then took a second wave.
    for (int s = s_max >= 8 ? 8 : (s_max >= 4 ? 4 : (s_max >= 2 ? 2 : 1)); s >= 1; s >>= 1) {
      if ((bn / 32) % s) continue;  // the 32-column chunks are dealt out evenly
      if (s == 1 && !force) continue;  // without a split this kernel has nothing over the general one
      const int per = (num_kb + s - 1) / s;
      if ((num_kb + per - 1) / per != s) continue;  // a range would be empty
      // shared memory: ring, then rows x bn fp32 of exchange area; at least three stages
      int stages = (kSkSmemBudget - 1024 - kSkTailBytes - bn * rows * 4) / stage_bytes;
      if (stages > kSkMaxStages) stages = kSkMaxStages;
      if (stages < 3) continue;
      if (s > 1) {
        int resident = 0;
        int rc = max_resident_clusters(s, &resident);
        if (rc) return rc;
        if (resident < tiles) continue;  // a second wave of clusters would cost more than it saves
      }
      const int64_t cost = (int64_t(bn) * 10 + rows * 3) * per / 10 + (s > 1 ? 384 : 0);
      if (best_bn == 0 || cost < best_cost) {
        best_bn = bn; best_s = s; best_per = per; best_stages = stages; best_cost = cost;
      }
      break;  // smaller clusters of this width only stream more per CTA
    }
  }
  if (best_bn == 0) {
    if (force) return fail(B200_ERR_UNSUPPORTED, "no one-wave configuration of the skinny kernel fits N = %lld", (long long)N);
    return B200_OK;
  }
  // Not worth a different kernel unless every SM streams clearly (10 %) less than it would in the general
  // one.  Measured on [4096 -> 11008] fp16, this kernel / the general one: 16 rows 19.0 / 25 us, 64 rows
  // 20.2 / 26 us, 96 rows 22.4 / 26.5 us, 128 rows 25.7 / 26.5 us (there the exchange area leaves a ring of
  // three stages and A is as large as in the general kernel, so little is left of the advantage).
  if (!force && best_cost * 10 > general_cost * 9) return B200_OK;

  if ((lda * esz) % 16 || (ldb * esz) % 16 || reinterpret_cast<uintptr_t>(A) % 16 || reinterpret_cast<uintptr_t>(B) % 16) {
    if (force) return fail(B200_ERR_UNSUPPORTED, "tensor-core GEMM needs 16-byte aligned A and B pointers and leading dimensions");
    return B200_OK;  // the general path reports it
  }
  if (reinterpret_cast<uintptr_t>(C) % out_esz) return fail(B200_ERR_UNSUPPORTED, "C is not aligned to its element size");
  if (epi == EPI_W8A8_BF16 && (!row_scale || !col_scale)) return fail(B200_ERR_BAD_ARGUMENT, "null scale pointer");

  const int smem_bytes = best_stages * (rows * 128 + best_bn * 128) + best_bn * rows * 4 + 1024 + kSkTailBytes;
  SkinnyKernel kernel = skinny_kernel_for(esz, b_is_nk);
  // The shared-memory attribute is per device and per instantiation.
  static thread_local int attr_dev[4] = {-1, -1, -1, -1};
  const int which = (esz == 1 ? 2 : 0) + (b_is_nk ? 1 : 0);
  if (dev != attr_dev[which]) {
    B200_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSkSmemBudget));
    attr_dev[which] = dev;
  }
  CUtensorMap ma, mb;
  int rc = encode_operand_map(&ma, kind, A, M, K, lda, bk, rows, false);
  if (rc) return rc;
  rc = b_is_nk ? encode_operand_map(&mb, kind, B, N, K, ldb, bk, best_bn, false)
               : encode_operand_map(&mb, kind, B, K, N, ldb, 128 / esz, bk, false);
  if (rc) return rc;

  SkinnyArgs args;
  memset(&args, 0, sizeof(args));
  args.C = C;
  args.ldc = ldc;
  args.M = int(M);
  args.N = int(N);
  args.K = int(K);
  args.rows = rows;
  args.bn = best_bn;
  args.splits = best_s;
  args.kb_per_split = best_per;
  args.stages = best_stages;
  args.kind = kind;
  args.esz = esz;
  args.epi = epi;
  args.b_is_nk = b_is_nk ? 1 : 0;
  args.vec_store = ((ldc * out_esz) % 16 == 0 && reinterpret_cast<uintptr_t>(C) % 16 == 0) ? 1 : 0;
  args.bias = tail.bias;
  args.tail_flags = tail.flags;
  args.row_scale = row_scale;
  args.col_scale = col_scale;

  const int tiles = int((N + best_bn - 1) / best_bn);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(unsigned(tiles * best_s));
  cfg.blockDim = dim3(kSkThreads);
  cfg.dynamicSmemBytes = size_t(smem_bytes);
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int nattr = 0;
  if (dependent_launch_enabled()) {
    attr[nattr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[nattr].val.programmaticStreamSerializationAllowed = 1;
    ++nattr;
  }
  if (best_s > 1) {
    attr[nattr].id = cudaLaunchAttributeClusterDimension;
    attr[nattr].val.clusterDim.x = unsigned(best_s);
    attr[nattr].val.clusterDim.y = 1;
    attr[nattr].val.clusterDim.z = 1;
    ++nattr;
  }
  cfg.attrs = attr;
  cfg.numAttrs = unsigned(nattr);
  B200_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, ma, mb, args));
  *used = true;
  return B200_OK;
}

}  // namespace b200
