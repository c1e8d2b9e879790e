// Tensor-core GEMM for sm_100a: C[M,N] = A[M,K] * B, row-major, for int8 (int32 accumulate),
// fp16 / bf16 and tf32 (fp32 accumulate).
//
// Persistent CTAs, one per SM, walk over output tiles.  Inside a CTA the work is split by warp role:
//   warp 0      TMA producer: one lane issues cp.async.bulk.tensor loads of the A tile
//               (128 rows x 128 bytes of K) and the B tile into a ring of shared-memory stages,
//               both with the 128-byte swizzle the MMA descriptors expect.
//   warp 1      MMA issuer: one lane issues tcgen05.mma (32 bytes of K per instruction) from
//               shared memory into an accumulator in tensor memory, and commits each stage back
//               to the producer.  It also owns the TMEM allocation.
//   warps 2-5   epilogue: tcgen05.ld the finished accumulator (one output row per thread),
//               convert / dequantise, and write C either through 128-row x 128-byte tiles staged
//               in shared memory and stored by TMA (one store per destination buffer: the local
//               C and, for the sharded product, every peer GPU's copy), or straight from registers.
// The accumulator is double buffered in TMEM (2 x BN columns), so the epilogue of tile i
// overlaps the main loop of tile i+1.
//
// Two groupings (template parameter CG):
//   CG = 1  a CTA owns a 128 x BN tile (BN = 256, 128 or 64).
//   CG = 2  a pair of CTAs (cluster of 2, the two SMs of a TPC) owns a 256 x 256 tile.  Each CTA
//           stages its own 128 rows of A and its own 128 columns of B; the even-ranked CTA issues
//           tcgen05.mma.cta_group::2 for both and signals both with multicast commits; each CTA
//           drains its own 128 accumulator rows.  Loads carry no multicast.
//
// B may be given either as [K,N] with N contiguous (the row-major product; also what the
// reference's column-major cuBLAS call turns into once both sides are transposed) or as [N,K]
// with K contiguous.  The first form is fed to the tensor cores as an "MN-major" operand: the
// tile is loaded as column spans of 128 bytes, each BK rows tall.
//
// Every mbarrier wait is bounded; a wait that runs out raises a CTA-wide abort flag, all roles
// drain, tensor memory is freed, and a status word tells the host that the result is invalid.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstring>
#include <mutex>

#include "internal.h"
#include "ptx_sm100.cuh"

namespace b200 {

__device__ uint32_t g_umma_status = 0;  // bit 0: a bounded wait ran out somewhere

// Wait accounting, compiled in only with -DB200_SKINNY_STAMPS (the measurement build; the shipped
// library has none of it).  Every CTA adds up SM cycles into waits[cta][8]: 0 = MMA lane waiting for
// full stages, 1 = MMA lane waiting for a free accumulator, 2 = MMA lane's whole loop, 3 = producer
// lane waiting for free stages, 4 = producer lane's whole loop, 5 = epilogue (warp 2) waiting for
// accumulators, 6 = epilogue's whole loop, 7 = k-blocks whose stage was not yet full when asked for,
// 8 = epilogue from "accumulator complete" to "accumulator handed back", 9 = the storing thread
// waiting for the previous tile store to have read its buffer, 10 = the same thread at the barrier.
// Eight-warp epilogue (warp 2): 9 = that wait, 11 = tensor-memory loads, 12 = convert and stage,
// 13 = fence and store issue.
#ifdef B200_SKINNY_STAMPS
__device__ unsigned long long* g_umma_waits = nullptr;
#define UW_DECL(name) long long name = 0
#define UW_BEGIN(name) name -= clock64()
#define UW_END(name) name += clock64()
#define UW_PUT(slot, value)                                                                        \
  do {                                                                                             \
    if (g_umma_waits != nullptr) g_umma_waits[size_t(blockIdx.x) * 16 + (slot)] = (unsigned long long)(value); \
  } while (0)
#else
#define UW_DECL(name) do { } while (0)
#define UW_BEGIN(name) do { } while (0)
#define UW_END(name) do { } while (0)
#define UW_PUT(slot, value) do { } while (0)
#endif

namespace {

constexpr int BM = 128;          // rows of C per tile = TMEM lanes
constexpr int kThreads = 192;    // producer warp, MMA warp, four epilogue warps
constexpr int kThreadsRB2 = 320; // two row blocks per CTA: eight epilogue warps, each storing on its own
constexpr int kSmemBudget = 227 * 1024;

bool g_use_pdl = true;  // launch the GEMM kernel with programmatic stream serialisation

// CG = 1: one CTA owns a 128 x BN tile.  CG = 2: a pair of CTAs (cluster of 2) owns a 256 x BN tile;
// each CTA stages its own 128 rows of A and its own BN/2 columns of B, and the even-ranked CTA
// issues tcgen05.mma.cta_group::2 for both.  RB = 2 (pairs only): every CTA owns two 128-row blocks
// of A, so the pair's tile is 512 x BN.  A k-block of B then feeds twice the arithmetic, which cuts
// the bytes an SM pulls from L2 per flop by a quarter; the price is that the two accumulators
// (2 x BN columns) fill tensor memory, so a tile's epilogue no longer overlaps the next tile's MMAs.
template <int KIND, int BN_, int CG_ = 1, int RB_ = 1>
struct Tile {
  static constexpr int ELEM = KIND == KIND_I8 ? 1 : (KIND == KIND_TF32 ? 4 : 2);
  static constexpr int BN = BN_;
  static constexpr int CG = CG_;
  static constexpr int RB = RB_;
  static constexpr int ACC_BUFS = RB_ == 2 ? 1 : 2;  // accumulator sets in tensor memory (two = epilogue overlaps the next tile)
  static constexpr int EPI_WARPS = RB_ == 2 ? 8 : 4;
  static constexpr int THREADS = 64 + 32 * EPI_WARPS;
  static constexpr int C_BOX_ROWS = RB_ == 2 ? 32 : BM;  // rows of one TMA store: a warp's own rows, or the tile's
  static constexpr int BN_CTA = BN / CG;     // B columns staged by one CTA
  static constexpr int BK = 128 / ELEM;      // elements of K per stage (one 128-byte swizzle row)
  static constexpr int UMMA_K = 32 / ELEM;   // elements of K per tcgen05.mma
  static constexpr int SPAN = 128 / ELEM;    // elements of N in one 128-byte span (MN-major B)
  static constexpr int NSPANS = BN_CTA / SPAN;
  static constexpr int A_BYTES = RB * BM * 128;
  static constexpr int B_BYTES = BN_CTA * 128;
  static constexpr int SPAN_BYTES = BK * 128;  // one span of B: BK k-rows of 128 bytes
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int NSTG = 2;
  static constexpr int STAGING_BYTES = NSTG * BM * 128;  // two 128-row x 128-byte output tiles for the TMA stores
  static constexpr int STAGES_FIT = (kSmemBudget - 2048 - STAGING_BYTES) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_FIT > 8 ? 8 : STAGES_FIT;
  static constexpr int TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;  // BN is a power of two here; RB * ACC_BUFS = 2 always
  static_assert(RB == 1 || (RB == 2 && CG == 2 && BN == 256), "two row blocks per CTA: pairs with 256-wide tiles only");
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + STAGING_BYTES + 1024 /*alignment*/ + 256 /*barriers*/;
};

constexpr int kMaxDest = 8;  // copies of C one launch can write (this GPU's and up to 7 peers')

// STORE_MULTIMEM: tiles are staged like for STORE_TMA, then written with multimem.st to a multicast
// address (one store reaches every GPU bound to the multicast object, replicated in the NVSwitch).
enum StoreMode { STORE_SCALAR = 0, STORE_VECTOR = 1, STORE_TMA = 2, STORE_MULTIMEM = 3 };

struct CMaps {
  CUtensorMap m[kMaxDest];
};

struct GemmArgs {
  void* C[kMaxDest];  // same slab of C in every destination buffer
  int n_dest;
  int64_t ldc;
  int M, N, K;
  int tiles_m, tiles_n;
  int group_m;  // m-tiles per group of the tile order
  int store_mode;  // StoreMode: how the epilogue writes C
  // Bounded waits: how long one wait may last, and (for the test of the give-up path only) the
  // k-block of CTA 0's first tile whose loads the producer leaves out, so that its "stage full"
  // arrival never comes; -1 = none.
  unsigned long long wait_budget_ns;
  int lose_kb;
  // L2 eviction hints, a bit set: 1 = the operand whose slab a group of tiles re-reads (A) is kept
  // (evict last), 2 = the operand that streams past (B) goes first, 4 = so do the stores of C.
  int l2_hints;
  int single_pass;  // tf32 kind only: 1 = plain fp32 operands, one pass (no split planes)
  const float* row_scale;
  const float* col_scale;
  // Fully connected layer (floating-point outputs): out = act(sum + bias[n]), both optional.
  const float* bias;
  int tail_flags;  // b200_linear_flags
};

constexpr int kDefaultGroupRows = 4096;  // rows of C that share a sweep over n (keeps their A slab hot in L2)

// Tile order: groups of kGroupRows rows; inside a group m runs fastest, then n.  A wave of
// concurrently running tiles is then a near-square patch of C, which needs the fewest operand bytes,
// and successive waves of a group re-use the group's slab of A.
__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int kGroupM, int& mb, int& nb) {
  int per_group = kGroupM * tiles_n;
  int g = t / per_group;
  int first_m = g * kGroupM;
  int gm = min(tiles_m - first_m, kGroupM);
  int r = t - g * per_group;
  mb = first_m + r % gm;
  nb = r / gm;
}

// Converts W accumulator columns of one row into output words: W words for 4-byte outputs,
// W/2 words (two elements each) for 2-byte outputs.
template <int EPI, int W = 32>
__device__ __forceinline__ void pack_chunk(const GemmArgs& p, int n0, const uint32_t (&v)[W], float rs,
                                           uint32_t (&w)[W]) {
  [[maybe_unused]] const bool relu = (p.tail_flags & B200_LINEAR_RELU) != 0;
  if constexpr (EPI == EPI_I32) {
#pragma unroll
    for (int i = 0; i < W; ++i) w[i] = v[i];
  } else if constexpr (EPI == EPI_F32) {
    if (p.bias == nullptr && !relu) {
#pragma unroll
      for (int i = 0; i < W; ++i) w[i] = v[i];
    } else {
#pragma unroll
      for (int i = 0; i < W; ++i) {
        float x = __uint_as_float(v[i]);
        if (p.bias != nullptr) x += __ldg(p.bias + min(n0 + i, p.N - 1));
        w[i] = __float_as_uint(relu ? fmaxf(0.0f, x) : x);
      }
    }
  } else {
    if constexpr (EPI == EPI_F16 || EPI == EPI_BF16) {
      if (p.bias == nullptr && !relu) {  // the plain product: one packed conversion per pair, nothing else
#pragma unroll
        for (int i = 0; i < W / 2; ++i) {
          if constexpr (EPI == EPI_F16) {
            __half2 h = __floats2half2_rn(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
            w[i] = *reinterpret_cast<uint32_t*>(&h);
          } else {
            __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
            w[i] = *reinterpret_cast<uint32_t*>(&h);
          }
        }
        return;
      }
    }
    // W8A8: the chunk's column scales, four per load where the chunk lies inside C and the scales
    // are 16-byte aligned (every thread of the warp reads the same addresses: one broadcast each).
    [[maybe_unused]] float cs[W];
    if constexpr (EPI == EPI_W8A8_BF16) {
      if (n0 + W <= p.N && (reinterpret_cast<uintptr_t>(p.col_scale + n0) & 15) == 0) {
#pragma unroll
        for (int i = 0; i < W / 4; ++i) {
          const float4 c4 = __ldg(reinterpret_cast<const float4*>(p.col_scale + n0) + i);
          cs[4 * i] = c4.x; cs[4 * i + 1] = c4.y; cs[4 * i + 2] = c4.z; cs[4 * i + 3] = c4.w;
        }
      } else {
#pragma unroll
        for (int i = 0; i < W; ++i) cs[i] = __ldg(p.col_scale + min(n0 + i, p.N - 1));
      }
    }
#pragma unroll
    for (int i = 0; i < W / 2; ++i) {
      float x0, x1;
      if constexpr (EPI == EPI_W8A8_BF16) {
        // (float(acc) * row_scale) * col_scale, each step rounded once, then to bf16
        const float c0 = cs[2 * i], c1 = cs[2 * i + 1];
        x0 = __fmul_rn(__fmul_rn(__int2float_rn(int(v[2 * i])), rs), c0);
        x1 = __fmul_rn(__fmul_rn(__int2float_rn(int(v[2 * i + 1])), rs), c1);
      } else {
        x0 = __uint_as_float(v[2 * i]);
        x1 = __uint_as_float(v[2 * i + 1]);
        if (p.bias != nullptr) {
          x0 += __ldg(p.bias + min(n0 + 2 * i, p.N - 1));
          x1 += __ldg(p.bias + min(n0 + 2 * i + 1, p.N - 1));
        }
        if (relu) {
          x0 = fmaxf(0.0f, x0);
          x1 = fmaxf(0.0f, x1);
        }
      }
      if constexpr (EPI == EPI_F16) {
        __half2 h = __floats2half2_rn(x0, x1);
        w[i] = *reinterpret_cast<uint32_t*>(&h);
      } else {
        __nv_bfloat162 h = __floats2bfloat162_rn(x0, x1);
        w[i] = *reinterpret_cast<uint32_t*>(&h);
      }
    }
  }
}

// Register path of the epilogue: one thread owns row `row`, columns [n0, n0 + W), and writes
// them to every destination with 16-byte stores (or element by element when C is not aligned).
template <int EPI, int W = 32>
__device__ __forceinline__ void store_chunk(const GemmArgs& p, int row, int n0, const uint32_t (&w)[W]) {
  constexpr int OUT_BYTES = (EPI == EPI_I32 || EPI == EPI_F32) ? 4 : 2;
  constexpr int WORDS = W * OUT_BYTES / 4;
  const bool full = p.store_mode != STORE_SCALAR && n0 + W <= p.N;
  for (int g = 0; g < p.n_dest; ++g) {
    char* crow = static_cast<char*>(p.C[g]) + (int64_t(row) * p.ldc + n0) * OUT_BYTES;
    if (full) {
      uint4* dst = reinterpret_cast<uint4*>(crow);
#pragma unroll
      for (int i = 0; i < WORDS / 4; ++i) dst[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
    } else if constexpr (OUT_BYTES == 4) {
      uint32_t* dst = reinterpret_cast<uint32_t*>(crow);
#pragma unroll
      for (int i = 0; i < W; ++i)
        if (n0 + i < p.N) dst[i] = w[i];
    } else {
      uint16_t* dst = reinterpret_cast<uint16_t*>(crow);
#pragma unroll
      for (int i = 0; i < W; ++i)
        if (n0 + i < p.N) dst[i] = uint16_t(w[i >> 1] >> ((i & 1) * 16));
    }
  }
}

template <int KIND, int BN, bool B_NK, int EPI, int CG, int RB = 1>
__global__ void __launch_bounds__(RB == 2 ? kThreadsRB2 : kThreads, 1)
gemm_umma_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CMaps tmap_c, const GemmArgs p) {
  using T = Tile<KIND, BN, CG, RB>;
  constexpr int TILE_M = BM * CG * RB;
  constexpr int CTA_M = BM * RB;  // rows of the tile this CTA stages and stores
  constexpr int NSTG = T::NSTG;
  extern __shared__ uint8_t smem_raw[];
  // 128-byte swizzle atoms are 1024 bytes: align the stage ring to that.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* staging = smem + T::STAGES * T::STAGE_BYTES;  // two output tiles, 128 rows x 128 bytes each
  uint64_t* bars = reinterpret_cast<uint64_t*>(staging + T::STAGING_BYTES);
  uint64_t* full_bar = bars;                   // [STAGES] producer(s) -> MMA   (pair: the leader's is used)
  uint64_t* empty_bar = bars + T::STAGES;      // [STAGES] MMA -> producer      (pair: one in each CTA)
  uint64_t* acc_full = bars + 2 * T::STAGES;   // [2] MMA -> epilogue           (pair: one in each CTA)
  uint64_t* acc_empty = acc_full + 2;          // [2] epilogue -> MMA           (pair: the leader's is used)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  // Epilogue warps: "this tile's accumulator arrived".  Two words used in turn, so that the warp that
  // posts the word for tile i + 1 never overwrites the one a slower warp is still reading for tile i.
  volatile uint32_t* epi_go_pair = tmem_slot + 2;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = CG == 2 ? cluster_cta_rank() : 0u;  // 0 = leader of the pair
  const int first_tile = CG == 2 ? int(blockIdx.x >> 1) : int(blockIdx.x);
  const int tile_step = CG == 2 ? int(gridDim.x >> 1) : int(gridDim.x);
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int num_kb = (p.K + T::BK - 1) / T::BK;
  // Split-operand fp32 (3xTF32): A and B each arrive as two stacked planes, low parts on top of
  // high parts, and K is walked three times: lo*hi, then hi*lo, then hi*hi (small terms first).
  // With `single_pass` the fp32 operands are read as they are (tf32 keeps the top 19 bits): one walk.
  const bool X3 = KIND == KIND_TF32 && !p.single_pass;
  const int total_kb = X3 ? 3 * num_kb : num_kb;

  if (threadIdx.x == 0) {
    for (int s = 0; s < T::STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], T::EPI_WARPS * CG);  // one arrival per epilogue warp (of both CTAs of a pair)
    }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    if constexpr (CG == 2) {
      tmem_alloc_pair(tmem_slot, T::TMEM_COLS);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(tmem_slot, T::TMEM_COLS);
      tmem_relinquish();
    }
  }
  tc_fence_before_sync();
  if constexpr (CG == 2) cluster_sync_all(); else __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  // Everything above touched only this CTA's shared and tensor memory.  From here on global memory
  // is read and written: wait for the kernel this launch was serialised behind (a no-op when the
  // launch carried no programmatic dependency), and let the next kernel in the stream start its
  // own set-up as soon as SMs become free.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int it = 0;
      const uint64_t pol_a = (p.l2_hints & 1) ? l2_policy_evict_last() : l2_policy_evict_normal();
      const uint64_t pol_b = (p.l2_hints & 2) ? l2_policy_evict_first() : l2_policy_evict_normal();
      UW_DECL(w_empty); UW_DECL(w_all);
      UW_BEGIN(w_all);
      for (int t = first_tile; t < num_tiles && ok; t += tile_step, ++it) {
        int mb, nb;
        tile_coords(t, p.tiles_m, p.tiles_n, p.group_m, mb, nb);
        // Every other tile walks K backwards: a tile then starts on the k-blocks its predecessor
        // touched last, which are the ones still in L2 (a forward-only sweep over a slab larger
        // than the cache would evict each block just before it is needed again).
        const bool k_reversed = (it & 1) != 0;
        const int m0 = mb * TILE_M + int(cta_rank) * CTA_M;
        const int n0 = nb * BN + int(cta_rank) * T::BN_CTA;
        // (pass, kin) = (kbt / num_kb, kbt % num_kb), counted rather than divided: this lane's loop paces
        // the CTA and an integer division per k-block is not free in it.
        int pass = 0, kin = 0;
        for (int kbt = 0; kbt < total_kb; ++kbt) {
          const int kb = k_reversed ? num_kb - 1 - kin : kin;
          const int a_row0 = (X3 && pass != 0) ? p.M : 0;                       // plane 1 = high parts
          const int b_row0 = (X3 && pass != 1) ? (B_NK ? p.N : p.K) : 0;
          UW_BEGIN(w_empty);
          const bool stage_free = mbar_wait_bounded(&empty_bar[stage], phase ^ 1u, abort_flag, p.wait_budget_ns);
          UW_END(w_empty);
          if (!stage_free) { ok = false; break; }
          if (kbt == p.lose_kb && it == 0 && blockIdx.x == 0) {
            // Test of the give-up path: this stage is never filled and never announced, as if its
            // arrival had been lost.  The MMA lane's wait for it runs out and the CTA drains.
            if (++stage == T::STAGES) { stage = 0; phase ^= 1u; }
            if (++kin == num_kb) { kin = 0; ++pass; }
            continue;
          }
          uint8_t* sa = smem + stage * T::STAGE_BYTES;
          uint8_t* sb = sa + T::A_BYTES;
          if constexpr (CG == 2) {
            // Both CTAs' bytes are credited to the leader's barrier; only the leader arms it.
            const uint32_t bar = map_to_cta(smem_u32(&full_bar[stage]), 0);
            if (cta_rank == 0) mbar_arrive_expect_tx(&full_bar[stage], 2 * T::STAGE_BYTES);
            tma_load_2d_pair_hint(sa, &tmap_a, bar, kb * T::BK, a_row0 + m0, pol_a);
            if constexpr (B_NK) {
              tma_load_2d_pair_hint(sb, &tmap_b, bar, kb * T::BK, b_row0 + n0, pol_b);
            } else {
#pragma unroll
              for (int s = 0; s < T::NSPANS; ++s)
                tma_load_2d_pair_hint(sb + s * T::SPAN_BYTES, &tmap_b, bar, n0 + s * T::SPAN, b_row0 + kb * T::BK,
                                      pol_b);
            }
          } else {
            mbar_arrive_expect_tx(&full_bar[stage], T::STAGE_BYTES);
            tma_load_2d_hint(sa, &tmap_a, &full_bar[stage], kb * T::BK, a_row0 + m0, pol_a);
            if constexpr (B_NK) {
              tma_load_2d_hint(sb, &tmap_b, &full_bar[stage], kb * T::BK, b_row0 + n0, pol_b);
            } else {
#pragma unroll
              for (int s = 0; s < T::NSPANS; ++s)
                tma_load_2d_hint(sb + s * T::SPAN_BYTES, &tmap_b, &full_bar[stage], n0 + s * T::SPAN,
                                 b_row0 + kb * T::BK, pol_b);
            }
          }
          if (++stage == T::STAGES) { stage = 0; phase ^= 1u; }
          if (++kin == num_kb) { kin = 0; ++pass; }
        }
      }
      UW_END(w_all);
      UW_PUT(3, w_empty);
      UW_PUT(4, w_all);
      if constexpr (CG == 2) {
        // Stay until every stage this CTA filled has been released: the releases are arrivals sent
        // by the leader's MMA commits into this CTA's shared memory, which must still exist.
        for (int i = 0; i < T::STAGES && ok; ++i) {
          ok = mbar_wait_bounded(&empty_bar[stage], phase ^ 1u, abort_flag, p.wait_budget_ns);
          if (++stage == T::STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && cta_rank == 0) {
      constexpr uint32_t idesc = make_instr_desc(KIND, BM * CG, BN, 0, B_NK ? 0 : 1);
      // Operand descriptors of stage 0; a later stage's differ in the address field only, which is in
      // units of 16 bytes and cannot carry out of its 14 bits for addresses inside shared memory.  This
      // lane's loop feeds the tensor pipe, so the descriptors are stepped, not rebuilt, per k-block.
      const uint32_t ring = smem_u32(smem);
      const uint64_t a_desc0 = make_smem_desc_sw128(ring, 16, 1024);
      // An N-contiguous operand of 32-bit elements only exists in the "128-byte swizzle on
      // 32-byte chunks" form: atoms of 128 bytes of N by 4 k-rows (512 bytes).
      const uint64_t b_desc0 = B_NK ? make_smem_desc_sw128(ring + T::A_BYTES, 16, 1024)
                               : (KIND == KIND_TF32 ? make_smem_desc(ring + T::A_BYTES, T::SPAN_BYTES, 512, 1)
                                                    : make_smem_desc_sw128(ring + T::A_BYTES, T::SPAN_BYTES, 1024));
      constexpr uint64_t kStageStep = uint64_t(T::STAGE_BYTES >> 4);
      uint64_t a_desc = a_desc0, b_desc = b_desc0;
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      UW_DECL(w_full); UW_DECL(w_acc); UW_DECL(w_all); UW_DECL(late);
      UW_BEGIN(w_all);
      for (int t = first_tile; t < num_tiles && ok; t += tile_step, ++it) {
        const int ab = it % T::ACC_BUFS;
        const uint32_t acc_phase = (it / T::ACC_BUFS) & 1;
        UW_BEGIN(w_acc);
        const bool acc_free = mbar_wait_bounded(&acc_empty[ab], acc_phase ^ 1u, abort_flag, p.wait_budget_ns);
        UW_END(w_acc);
        if (!acc_free) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + uint32_t(ab * BN);  // with two row blocks: block 1 at + BN
        for (int kb = 0; kb < total_kb; ++kb) {
#ifdef B200_SKINNY_STAMPS
          if (!mbar_try_wait(&full_bar[stage], phase)) ++late;
#endif
          UW_BEGIN(w_full);
          const bool stage_full = mbar_wait_bounded(&full_bar[stage], phase, abort_flag, p.wait_budget_ns);
          UW_END(w_full);
          if (!stage_full) { ok = false; break; }
          tc_fence_after_sync();
#pragma unroll
          for (int j = 0; j < T::BK / T::UMMA_K; ++j) {
            // A (and a K-contiguous B) advance 32 bytes inside the swizzle row; an N-contiguous
            // B advances UMMA_K whole k-rows of 128 bytes.
            const uint64_t a_adv = uint64_t((j * 32) >> 4);
            const uint64_t b_adv = B_NK ? uint64_t((j * 32) >> 4) : uint64_t((j * T::UMMA_K * 128) >> 4);
            if constexpr (CG == 2) {
#pragma unroll
              for (int rb = 0; rb < RB; ++rb)  // both row blocks take the same slice of B
                umma_pair<KIND>(d_tmem + uint32_t(rb * BN), a_desc + uint64_t((rb * BM * 128) >> 4) + a_adv,
                                b_desc + b_adv, idesc, (kb | j) != 0 ? 1u : 0u);
            } else {
              umma<KIND>(d_tmem, a_desc + a_adv, b_desc + b_adv, idesc, (kb | j) != 0 ? 1u : 0u);
            }
          }
          // the stage is free (in both CTAs of a pair) once these MMAs have read it
          if constexpr (CG == 2) umma_commit_pair(&empty_bar[stage], 3); else umma_commit(&empty_bar[stage]);
          a_desc += kStageStep;
          b_desc += kStageStep;
          if (++stage == T::STAGES) { stage = 0; phase ^= 1u; a_desc = a_desc0; b_desc = b_desc0; }
        }
        if (ok) {
          if constexpr (CG == 2) umma_commit_pair(&acc_full[ab], 3); else umma_commit(&acc_full[ab]);
        }
      }
      UW_END(w_all);
      UW_PUT(0, w_full);
      UW_PUT(1, w_acc);
      UW_PUT(2, w_all);
      UW_PUT(7, late);
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps
    constexpr int OUT_BYTES = (EPI == EPI_I32 || EPI == EPI_F32) ? 4 : 2;
    constexpr int BOX_COLS = 128 / OUT_BYTES;     // columns of C in one 128-byte row of an output tile
    constexpr int CHUNKS_PER_BOX = BOX_COLS / 32;  // 32-column TMEM loads per output tile
    constexpr int UNITS = 8 / CHUNKS_PER_BOX;      // 16-byte units one load contributes to its row
    constexpr int kEpiThreads = 128;
    const int quarter = warp & 3;  // TMEM lanes this warp may read: [32*quarter, 32*quarter + 32)
    const int r_in_tile = quarter * 32 + lane;
    const bool store_thread = warp == 2 && lane == 0;
    uint32_t boxes = 0;
    int it = 0;
    const uint64_t pol_c = (p.l2_hints & 4) ? l2_policy_evict_first() : l2_policy_evict_normal();
    UW_DECL(w_accfull); UW_DECL(w_all); UW_DECL(w_drain); UW_DECL(w_rd); UW_DECL(w_bar);
    UW_BEGIN(w_all);
    if constexpr (RB == 2) {
      // Eight warps, two per 32-lane quarter of tensor memory; warps 2-5 drain row block 0, warps 6-9
      // row block 1.  Nothing here overlaps the next tile's MMAs (the accumulators fill tensor memory), so
      // the drain is what the tensor pipe waits for: once a tile's accumulators are there, every warp works
      // alone, without a barrier shared with the others.  It stages its own 32 rows x 128 bytes, stores them with a TMA request of its
      // own, and hands the accumulators back as soon as its last values are in registers.
      const int group = (warp - 2) >> 2;  // = row block
      UW_DECL(w_ld); UW_DECL(w_cv); UW_DECL(w_st);
      uint8_t* buf = staging + (warp - 2) * (32 * 128);
      uint32_t stores = 0;
      for (int t = first_tile; t < num_tiles; t += tile_step, ++it) {
        int mb, nb;
        tile_coords(t, p.tiles_m, p.tiles_n, p.group_m, mb, nb);
        const uint32_t acc_phase = it & 1;
        volatile uint32_t* epi_go = epi_go_pair + (it & 1);
        // One warp polls the barrier; the other seven sleep at a hardware barrier meanwhile (a main
        // loop lasts tens of microseconds, and 256 polling threads are power the tensor pipe could use).
        UW_BEGIN(w_accfull);
        if (warp == 2) {
          const bool ok = mbar_wait_bounded(&acc_full[0], acc_phase, abort_flag, p.wait_budget_ns);
          if (lane == 0) *epi_go = ok ? 1u : 0u;
        }
        named_barrier_sync(2, 32 * T::EPI_WARPS);
        UW_END(w_accfull);
        if (*epi_go == 0u) break;
        tc_fence_after_sync();
        UW_BEGIN(w_drain);
        const int row0 = mb * TILE_M + int(cta_rank) * CTA_M + group * BM + quarter * 32;  // this warp's first row of C
        const int row = row0 + lane;
        float rs = 0.f;
        if constexpr (EPI == EPI_W8A8_BF16) rs = row < p.M ? __ldg(p.row_scale + row) : 0.f;
        const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + uint32_t(group * BN);
        const int cols_left = p.N - nb * BN;
        const int nboxes = min(BN / BOX_COLS, (cols_left + BOX_COLS - 1) / BOX_COLS);
        if (p.store_mode == STORE_TMA) {
          // A box is 32 rows x 128 bytes: 32 words a thread, whatever the element size (4 boxes of 64 columns
          // for 2-byte outputs, 8 of 32 columns for 4-byte ones).  The accumulators can go back to the MMA
          // lane once every value has left tensor memory, so as many boxes as fit wait converted in registers
          // (three: 96 words) and one more in the staging buffer; only the boxes before those (none for 2-byte
          // outputs, four for 4-byte ones) are converted, staged and stored one after the other while the MMA
          // lane waits.
          constexpr int NB = BN / BOX_COLS;
          constexpr int KEEP = 3;
          constexpr int FRONT = NB - 1 - KEEP;
          uint32_t held[KEEP][32];
          auto buffer_free = [&]() {  // this warp's previous store has read the buffer
            if (lane == 0) tma_store_wait_read<0>();
            __syncwarp();
          };
          // tensor memory -> converted words of box bx; `for_buffer`: the words go to the staging buffer next,
          // so the wait for the buffer is spent while the tensor-memory load is in flight
          auto load_box = [&](int bx, uint32_t (&words)[32], bool for_buffer) {
            uint32_t v[CHUNKS_PER_BOX][32];
#pragma unroll
            for (int h = 0; h < CHUNKS_PER_BOX; ++h) tmem_ld_32x32(taddr + uint32_t(bx * BOX_COLS + h * 32), v[h]);
            if (for_buffer) buffer_free();
            tmem_ld_wait();
#pragma unroll
            for (int h = 0; h < CHUNKS_PER_BOX; ++h) {
              uint32_t w[32];
              pack_chunk<EPI>(p, nb * BN + bx * BOX_COLS + h * 32, v[h], rs, w);
#pragma unroll
              for (int i = 0; i < 32 / CHUNKS_PER_BOX; ++i) words[h * (32 / CHUNKS_PER_BOX) + i] = w[i];
            }
          };
          auto stage_box = [&](const uint32_t (&words)[32]) {  // words -> this warp's buffer, swizzled for the store
#pragma unroll
            for (int unit = 0; unit < 8; ++unit)
              *reinterpret_cast<uint4*>(buf + lane * 128 + ((unit ^ (lane & 7)) << 4)) =
                  make_uint4(words[4 * unit], words[4 * unit + 1], words[4 * unit + 2], words[4 * unit + 3]);
          };
          auto store_box = [&](int bx) {
            const int n0 = nb * BN + bx * BOX_COLS;
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0 && row0 < p.M) {
              if (p.n_dest > 1) {  // peers first, from a start that rotates; the local copy last
                const int peers = p.n_dest - 1;
                int g = 1 + int((uint32_t(first_tile) + stores) % uint32_t(peers));
                for (int i = 0; i < peers; ++i) {
                  tma_store_2d_hint(&tmap_c.m[g], buf, n0, row0, pol_c);
                  if (++g == p.n_dest) g = 1;
                }
              }
              tma_store_2d_hint(&tmap_c.m[0], buf, n0, row0, pol_c);
              tma_store_commit();
            }
            ++stores;
          };
          UW_BEGIN(w_ld);
#pragma unroll
          for (int bx = 0; bx < FRONT; ++bx) {
            if (bx < nboxes) {
              uint32_t words[32];
              load_box(bx, words, true);
              stage_box(words);
              store_box(bx);
            }
          }
          if (FRONT < nboxes) {
            uint32_t words[32];
            load_box(FRONT, words, true);
            stage_box(words);
          }
#pragma unroll
          for (int k = 0; k < KEEP; ++k)
            if (FRONT + 1 + k < nboxes) load_box(FRONT + 1 + k, held[k], false);
          UW_END(w_ld);
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty[0]), 0));
          UW_END(w_drain);
          UW_BEGIN(w_st);
          if (FRONT < nboxes) store_box(FRONT);
#pragma unroll
          for (int k = 0; k < KEEP; ++k) {
            if (FRONT + 1 + k < nboxes) {
              buffer_free();
              stage_box(held[k]);
              store_box(FRONT + 1 + k);
            }
          }
          UW_END(w_st);
          continue;
        }
#pragma unroll 1
        for (int bx = 0; bx < nboxes; ++bx) {
          const int n0 = nb * BN + bx * BOX_COLS;
          uint32_t v[CHUNKS_PER_BOX][32];
          UW_BEGIN(w_ld);
#pragma unroll
          for (int h = 0; h < CHUNKS_PER_BOX; ++h) tmem_ld_32x32(taddr + uint32_t(bx * BOX_COLS + h * 32), v[h]);
          tmem_ld_wait();
          UW_END(w_ld);
          if (bx + 1 == nboxes) {
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty[0]), 0));
            UW_END(w_drain);
          }
          {  // register stores (C not aligned for TMA, or the store policy asks for them)
#pragma unroll
            for (int h = 0; h < CHUNKS_PER_BOX; ++h) {
              uint32_t w[32];
              pack_chunk<EPI>(p, n0 + h * 32, v[h], rs, w);
              if (row < p.M && n0 + h * 32 < p.N) store_chunk<EPI>(p, row, n0 + h * 32, w);
            }
          }
        }
      }
      UW_END(w_all);
      if (store_thread) {
        UW_PUT(5, w_accfull);
        UW_PUT(6, w_all);
        UW_PUT(8, w_drain);
        UW_PUT(9, w_rd);
        UW_PUT(11, w_ld);
        UW_PUT(12, w_cv);
        UW_PUT(13, w_st);
      }
      if (lane == 0 && p.store_mode == STORE_TMA) tma_store_wait_all<0>();
    } else {
    for (int t = first_tile; t < num_tiles; t += tile_step, ++it) {
      int mb, nb;
      tile_coords(t, p.tiles_m, p.tiles_n, p.group_m, mb, nb);
      const int ab = it % T::ACC_BUFS;
      const uint32_t acc_phase = (it / T::ACC_BUFS) & 1;
      volatile uint32_t* epi_go = epi_go_pair + (it & 1);
      // One warp polls the barrier; all four then agree on the outcome, so that they always meet at
      // the same hardware barriers below even when the wait had to be given up.
      if (warp == 2) {
        UW_BEGIN(w_accfull);
        const bool ok = mbar_wait_bounded(&acc_full[ab], acc_phase, abort_flag, p.wait_budget_ns);
        UW_END(w_accfull);
        if (lane == 0) *epi_go = ok ? 1u : 0u;
      }
      named_barrier_sync(2, kEpiThreads);
      if (*epi_go == 0u) break;
      tc_fence_after_sync();
      UW_BEGIN(w_drain);
      bool released = false;  // this warp has handed the accumulators back to the MMA lane
#pragma unroll 1
      for (int rb = 0; rb < RB; ++rb) {
      const int tile_row0 = mb * TILE_M + int(cta_rank) * CTA_M + rb * BM;
      const int row = tile_row0 + r_in_tile;
      float rs = 0.f;
      if constexpr (EPI == EPI_W8A8_BF16) rs = row < p.M ? __ldg(p.row_scale + row) : 0.f;
      const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + uint32_t(ab * BN + rb * BN);
      if (p.store_mode >= STORE_TMA) {
        // Stage 128 x 128-byte output tiles ("boxes") in shared memory, swizzled like the tensor map
        // expects, and let TMA write them: whole rows per request, clipped at the edges of C, one
        // request per destination buffer.  Four warps on four schedulers hide no latency for one
        // another, so the tensor-memory load of box i + 1 is in flight while box i is converted and
        // staged, and a box costs one barrier: the thread that issues the stores waits, before it
        // arrives there, until the store of the box before has read its buffer, which is the buffer
        // the next box will be staged in.
        const int cols_left = p.N - nb * BN;
        const int nboxes = min(BN / BOX_COLS, (cols_left + BOX_COLS - 1) / BOX_COLS);
        uint32_t vn[CHUNKS_PER_BOX][32];
#pragma unroll
        for (int h = 0; h < CHUNKS_PER_BOX; ++h) tmem_ld_32x32(taddr + uint32_t(h * 32), vn[h]);
#pragma unroll 1
        for (int bx = 0; bx < nboxes; ++bx) {
          const int n0 = nb * BN + bx * BOX_COLS;
          uint8_t* buf = staging + (boxes & 1u) * (BM * 128);
          uint32_t v[CHUNKS_PER_BOX][32];
          tmem_ld_wait();
#pragma unroll
          for (int h = 0; h < CHUNKS_PER_BOX; ++h)
#pragma unroll
            for (int i = 0; i < 32; ++i) v[h][i] = vn[h][i];
          if (bx + 1 < nboxes) {
#pragma unroll
            for (int h = 0; h < CHUNKS_PER_BOX; ++h)
              tmem_ld_32x32(taddr + uint32_t((bx + 1) * BOX_COLS + h * 32), vn[h]);
          } else if (rb + 1 == RB) {
            // The tile's last values are in registers: the MMA lane may have the accumulators back
            // while this box is converted and stored.
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
              if constexpr (CG == 2) mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty[ab]), 0));
              else mbar_arrive(&acc_empty[ab]);
            }
            released = true;
            UW_END(w_drain);
          }
#pragma unroll
          for (int h = 0; h < CHUNKS_PER_BOX; ++h) {
            uint32_t w[32];
            pack_chunk<EPI>(p, n0 + h * 32, v[h], rs, w);
#pragma unroll
            for (int i = 0; i < UNITS; ++i) {
              const int unit = h * UNITS + i;
              *reinterpret_cast<uint4*>(buf + r_in_tile * 128 + ((unit ^ (r_in_tile & 7)) << 4)) =
                  make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
            }
          }
          if (p.store_mode == STORE_MULTIMEM) {
            // All four warps write the staged tile to the multicast address: eight consecutive lanes
            // take the eight 16-byte units of one row (128 contiguous bytes per row in every copy).
            // The box after this one is staged in the other buffer, and the one after that in this
            // buffer again only by threads that have passed the next box's barrier, i.e. after every
            // thread has finished the reads below.
            named_barrier_sync(1, kEpiThreads);
            constexpr int ELEMS_PER_UNIT = 16 / OUT_BYTES;
            char* mc = static_cast<char*>(p.C[0]);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int u = i * kEpiThreads + (quarter * 32 + lane);
              const int r = u >> 3, unit = u & 7;
              const uint4 val = *reinterpret_cast<const uint4*>(buf + r * 128 + ((unit ^ (r & 7)) << 4));
              const int grow = tile_row0 + r, gcol = n0 + unit * ELEMS_PER_UNIT;
              if (grow < p.M && gcol + ELEMS_PER_UNIT <= p.N)
                multimem_st_v4(mc + (int64_t(grow) * p.ldc + gcol) * OUT_BYTES, val);
            }
            ++boxes;
            continue;
          }
          fence_proxy_async_smem();
          UW_BEGIN(w_rd);
          if (store_thread) tma_store_wait_read<0>();  // the other buffer is free for the next box
          UW_END(w_rd);
          UW_BEGIN(w_bar);
          named_barrier_sync(1, kEpiThreads);
          UW_END(w_bar);
          if (store_thread) {
            // Destination 0 (by convention the local copy) goes last; the others (peer GPUs) are
            // walked from a start that rotates with the CTA and the box count, so that every sender
            // spreads its traffic over all receivers at all times instead of all senders hitting
            // the same receiver together.
            if (p.n_dest > 1) {
              const int peers = p.n_dest - 1;
              int g = 1 + int((uint32_t(first_tile) + boxes) % uint32_t(peers));
              for (int i = 0; i < peers; ++i) {
                tma_store_2d_hint(&tmap_c.m[g], buf, n0, tile_row0, pol_c);
                if (++g == p.n_dest) g = 1;
              }
            }
            tma_store_2d_hint(&tmap_c.m[0], buf, n0, tile_row0, pol_c);
            tma_store_commit();
          }
          ++boxes;
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          const int n0 = nb * BN + c * 32;
          if (n0 >= p.N) break;  // uniform across the warp
          uint32_t v[32], w[32];
          tmem_ld_32x32(taddr + uint32_t(c * 32), v);
          tmem_ld_wait();
          pack_chunk<EPI>(p, n0, v, rs, w);
          if (row < p.M) store_chunk<EPI>(p, row, n0, w);
        }
      }
      }  // row blocks
      if (!released) {
        UW_END(w_drain);
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          if constexpr (CG == 2) mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty[ab]), 0));
          else mbar_arrive(&acc_empty[ab]);
        }
      }
    }
    UW_END(w_all);
    if (store_thread) {
      UW_PUT(5, w_accfull);
      UW_PUT(6, w_all);
      UW_PUT(8, w_drain);
      UW_PUT(9, w_rd);
      UW_PUT(10, w_bar);
    }
    if (store_thread && p.store_mode == STORE_TMA) tma_store_wait_all<0>();  // every output tile has left for global memory
    }  // four-warp epilogue
  }

  // Every role gets here: either its loop ended or its wait was abandoned.
  __syncwarp();
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0) atomicOr(&g_umma_status, 1u);
    // Give copies and MMAs still in flight time to land before shared and tensor memory go away.
    uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  tc_fence_before_sync();
  if constexpr (CG == 2) cluster_sync_all(); else __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    if constexpr (CG == 2) tmem_dealloc_pair(tmem_base, T::TMEM_COLS); else tmem_dealloc(tmem_base, T::TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------ host side

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                   CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                   CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  });
  return fn;
}

// 2-D tensor map over a row-major [rows, cols] matrix with leading dimension `ld` (elements):
// box = box_cols x box_rows, 128-byte swizzle, zero fill outside the matrix.
int make_map(CUtensorMap* map, int kind, const void* base, int64_t rows, int64_t cols, int64_t ld,
             int box_cols, int box_rows, bool chunks32 = false) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return fail(B200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  int elem = kind == KIND_I8 ? 1 : (kind == KIND_TF32 ? 4 : 2);
  CUtensorMapDataType dt = kind == KIND_I8     ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                           : kind == KIND_F16  ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                           : kind == KIND_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                               : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  cuuint64_t dims[2] = {cuuint64_t(cols), cuuint64_t(rows)};
  cuuint64_t strides[1] = {cuuint64_t(ld) * cuuint64_t(elem)};
  cuuint32_t box[2] = {cuuint32_t(box_cols), cuuint32_t(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   chunks32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(B200_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", int(r));
  return B200_OK;
}

// Tensor map for storing 128-row x 128-byte tiles of a row-major [rows, cols] C.
int make_c_map(CUtensorMap* map, int epi, void* base, int64_t rows, int64_t cols, int64_t ld, int box_rows) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return fail(B200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  const int elem = (epi == EPI_I32 || epi == EPI_F32) ? 4 : 2;
  CUtensorMapDataType dt = epi == EPI_I32   ? CU_TENSOR_MAP_DATA_TYPE_INT32
                           : epi == EPI_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                           : epi == EPI_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                            : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  cuuint64_t dims[2] = {cuuint64_t(cols), cuuint64_t(rows)};
  cuuint64_t strides[1] = {cuuint64_t(ld) * cuuint64_t(elem)};
  cuuint32_t box[2] = {cuuint32_t(128 / elem), cuuint32_t(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, dt, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(B200_ERR_CUDA, "cuTensorMapEncodeTiled (C) failed with CUresult %d", int(r));
  return B200_OK;
}

#ifdef B200_SKINNY_STAMPS
}  // namespace
}  // namespace b200
// Measurement build only: where the GEMM kernel writes its wait accounting (16 words per CTA), or null.
extern "C" int b200_debug_set_umma_waits(void* device_buffer) {
  unsigned long long* p = static_cast<unsigned long long*>(device_buffer);
  return cudaMemcpyToSymbol(b200::g_umma_waits, &p, sizeof(p)) == cudaSuccess ? 0 : 3;
}
namespace b200 {
namespace {
#endif

int sm_count_of_current_device(int* out) {
  static int cached[64] = {0};
  int dev = 0;
  B200_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 64 && cached[dev]) { *out = cached[dev]; return B200_OK; }
  int n = 0;
  B200_CUDA_TRY(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev));
  if (dev < 64) cached[dev] = n;
  *out = n;
  return B200_OK;
}

template <int KIND, int BN, bool B_NK, int EPI, int CG, int RB = 1>
int launch_one(const void* A, const void* B, const GemmArgs& args, int64_t lda, int64_t ldb,
               cudaStream_t stream) {
  using T = Tile<KIND, BN, CG, RB>;
  auto kernel = gemm_umma_kernel<KIND, BN, B_NK, EPI, CG, RB>;
  // The shared-memory attribute is per device: set it whenever this thread meets a new device.
  static thread_local int last_dev = -1;
  int dev = 0;
  B200_CUDA_TRY(cudaGetDevice(&dev));
  if (dev != last_dev) {
    cudaError_t attr_err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, T::SMEM_BYTES);
    if (attr_err != cudaSuccess)
      return fail(B200_ERR_CUDA, "cudaFuncSetAttribute(%d bytes of shared memory): %s", T::SMEM_BYTES,
                  cudaGetErrorString(attr_err));
    last_dev = dev;
  }
  CUtensorMap ma, mb;
  const int64_t planes = (KIND == KIND_TF32 && !args.single_pass) ? 2 : 1;  // split fp32 operands: low plane, then high plane
  int rc = make_map(&ma, KIND, A, planes * args.M, args.K, lda, T::BK, BM * RB);
  if (rc) return rc;
  if (B_NK)
    rc = make_map(&mb, KIND, B, planes * args.N, args.K, ldb, T::BK, T::BN_CTA);
  else
    rc = make_map(&mb, KIND, B, planes * args.K, args.N, ldb, T::SPAN < T::BN_CTA ? T::SPAN : T::BN_CTA, T::BK,
                  /*chunks32=*/KIND == KIND_TF32);
  if (rc) return rc;
  CMaps mc;
  memset(&mc, 0, sizeof(mc));
  if (args.store_mode == STORE_TMA) {
    for (int g = 0; g < args.n_dest; ++g) {
      rc = make_c_map(&mc.m[g], EPI, args.C[g], args.M, args.N, args.ldc, T::C_BOX_ROWS);
      if (rc) return rc;
    }
  }
  int sms = 0;
  rc = sm_count_of_current_device(&sms);
  if (rc) return rc;
  const int tiles = args.tiles_m * args.tiles_n;
  // Launch with programmatic stream serialisation: this grid's CTAs may be scheduled, and run their
  // set-up (barrier init, TMEM allocation, descriptor prefetch), while the kernel before it in the
  // stream is still draining; they touch no global data before griddepcontrol.wait, which holds them
  // until that kernel has completed.
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(T::THREADS);
  cfg.dynamicSmemBytes = T::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int nattr = 0;
  if (g_use_pdl) {
    attr[nattr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[nattr].val.programmaticStreamSerializationAllowed = 1;
    ++nattr;
  }
  if constexpr (CG == 2) {
    int pairs = tiles < sms / 2 ? tiles : sms / 2;
    cfg.gridDim = dim3(unsigned(2 * pairs));
    attr[nattr].id = cudaLaunchAttributeClusterDimension;
    attr[nattr].val.clusterDim.x = 2;
    attr[nattr].val.clusterDim.y = 1;
    attr[nattr].val.clusterDim.z = 1;
    ++nattr;
  } else {
    cfg.gridDim = dim3(unsigned(tiles < sms ? tiles : sms));
  }
  cfg.attrs = attr;
  cfg.numAttrs = nattr;
  B200_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, ma, mb, mc, args));
  return B200_OK;
}

template <int KIND, int BN, int EPI, int CG, int RB = 1>
int launch_major(bool b_nk, const void* A, const void* B, const GemmArgs& args, int64_t lda, int64_t ldb,
                 cudaStream_t stream) {
  // An N-contiguous B is staged in whole 128-byte spans of N, so a CTA's share of the tile cannot be
  // narrower than one span.
  if constexpr (BN / CG < Tile<KIND, BN, CG>::SPAN) {
    if (!b_nk) return fail(B200_ERR_BAD_ARGUMENT, "tile width %d is narrower than a 128-byte span", BN / CG);
    return launch_one<KIND, BN, true, EPI, CG, RB>(A, B, args, lda, ldb, stream);
  } else {
    return b_nk ? launch_one<KIND, BN, true, EPI, CG, RB>(A, B, args, lda, ldb, stream)
                : launch_one<KIND, BN, false, EPI, CG, RB>(A, B, args, lda, ldb, stream);
  }
}

int g_force_cg = 0, g_force_bn = 0, g_group_rows = 0;  // 0 = automatic; set through b200_set_tile_policy
int g_force_store = 0;                                  // 0 = automatic, STORE_VECTOR = register stores
unsigned long long g_wait_budget_ns = kWaitBudgetNs;    // per-wait limit handed to the kernels
int g_lose_kb = -1;                                     // give-up test: k-block whose arrival is left out
int g_l2_hints = -1;                                    // -1 = automatic, else the bit set of GemmArgs::l2_hints
thread_local bool g_multicast_call = false;              // set by launch_umma_gemm_multicast around its launch
thread_local bool g_tf32_single_pass_call = false;      // set by launch_sgemm_tf32 around its launch

// Stream-ordered memory pool for per-call scratch (the split planes of the 3xTF32 product), one per
// device.  It keeps what it has handed out before (release threshold at the maximum), so that after
// the first call an allocation is a host-side bookkeeping step and never reaches the driver's
// allocator; an allocation and its release are ordered on the caller's stream, so calls on
// different streams never share scratch.
int scratch_pool(cudaMemPool_t* out) {
  static std::mutex mu;
  static cudaMemPool_t pools[64] = {nullptr};
  int dev = 0;
  B200_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(B200_ERR_UNSUPPORTED, "device ordinal %d is beyond the pool table", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (!pools[dev]) {
    cudaMemPoolProps props;
    memset(&props, 0, sizeof(props));
    props.allocType = cudaMemAllocationTypePinned;
    props.handleTypes = cudaMemHandleTypeNone;
    props.location.type = cudaMemLocationTypeDevice;
    props.location.id = dev;
    cudaMemPool_t pool = nullptr;
    B200_CUDA_TRY(cudaMemPoolCreate(&pool, &props));
    uint64_t keep = ~uint64_t(0);
    B200_CUDA_TRY(cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep));
    pools[dev] = pool;
  }
  *out = pools[dev];
  return B200_OK;
}

template <int KIND, int EPI>
int launch_bn(int bn, int cg, int rb, bool b_nk, const void* A, const void* B, GemmArgs args, int64_t lda, int64_t ldb,
              cudaStream_t stream) {
  const int tile_m = BM * cg * rb;
  args.tiles_n = int((args.N + bn - 1) / bn);
  args.tiles_m = int((args.M + tile_m - 1) / tile_m);
  args.group_m = (g_group_rows ? g_group_rows : kDefaultGroupRows) / tile_m;
  if (args.group_m < 1) args.group_m = 1;
  if (cg == 2) {
    if (bn == 256 && rb == 2) return launch_major<KIND, 256, EPI, 2, 2>(b_nk, A, B, args, lda, ldb, stream);
    if (bn == 256) return launch_major<KIND, 256, EPI, 2>(b_nk, A, B, args, lda, ldb, stream);
    return fail(B200_ERR_BAD_ARGUMENT, "CTA pairs are built for 256-wide tiles only");
  }
  switch (bn) {
    case 256: return launch_major<KIND, 256, EPI, 1>(b_nk, A, B, args, lda, ldb, stream);
    case 128: return launch_major<KIND, 128, EPI, 1>(b_nk, A, B, args, lda, ldb, stream);
    case 64: return launch_major<KIND, 64, EPI, 1>(b_nk, A, B, args, lda, ldb, stream);
  }
  return fail(B200_ERR_BAD_ARGUMENT, "tile width %d is not built", bn);
}

}  // namespace

int encode_operand_map(CUtensorMap* map, int kind, const void* base, int64_t rows, int64_t cols, int64_t ld,
                       int box_cols, int box_rows, bool chunks32) {
  return make_map(map, kind, base, rows, cols, ld, box_cols, box_rows, chunks32);
}

bool dependent_launch_enabled() { return g_use_pdl; }

int set_tile_policy(int cg, int bn, int group_rows) {
  if (group_rows < 0 || (group_rows % 256) != 0)
    return fail(B200_ERR_BAD_ARGUMENT, "tile policy: group rows must be a non-negative multiple of 256");
  if (cg == 3) {  // the K-split cluster kernel for skinny products, at a width of its own choice or a given one
    if (bn != 0 && bn != 128 && bn != 192 && bn != 256)
      return fail(B200_ERR_BAD_ARGUMENT, "tile policy: the skinny kernel has widths 128, 192 and 256");
    g_force_cg = cg;
    g_force_bn = bn;
    g_group_rows = group_rows;
    return B200_OK;
  }
  if ((cg != 0 && cg != 1 && cg != 2 && cg != 4) || (bn != 0 && bn != 64 && bn != 128 && bn != 256))
    return fail(B200_ERR_BAD_ARGUMENT, "tile policy: cta group must be 0, 1, 2 or 4 and width 0, 64, 128 or 256");
  if (cg >= 2 && bn != 0 && bn != 256) return fail(B200_ERR_BAD_ARGUMENT, "CTA pairs need 256-wide tiles");
  g_force_cg = cg;
  g_force_bn = bn;
  g_group_rows = group_rows;
  return B200_OK;
}

int set_wait_test(long long lose_kb, unsigned long long budget_ns) {
  if (lose_kb < -1 || lose_kb > (1 << 20)) return fail(B200_ERR_BAD_ARGUMENT, "wait test: k-block out of range");
  g_lose_kb = int(lose_kb);
  g_wait_budget_ns = budget_ns ? budget_ns : kWaitBudgetNs;
  return B200_OK;
}

int set_l2_hints(int hints) {
  if (hints < -1 || hints > 7) return fail(B200_ERR_BAD_ARGUMENT, "L2 hints: -1 (automatic) or a bit set 0..7");
  g_l2_hints = hints;
  return B200_OK;
}

int set_dependent_launch(int enabled) {
  g_use_pdl = enabled != 0;
  return B200_OK;
}

int set_store_policy(int register_stores) {
  g_force_store = register_stores ? STORE_VECTOR : 0;
  return B200_OK;
}

int read_and_clear_umma_status(cudaStream_t stream, uint32_t* out) {
  uint32_t zero = 0;
  B200_CUDA_TRY(cudaStreamSynchronize(stream));
  B200_CUDA_TRY(cudaMemcpyFromSymbol(out, g_umma_status, sizeof(uint32_t)));
  if (*out) B200_CUDA_TRY(cudaMemcpyToSymbol(g_umma_status, &zero, sizeof(uint32_t)));
  return B200_OK;
}

namespace {
int launch_kind(int kind, int epi, int bn, int cg, int rb, bool b_is_nk, const void* A, const void* B, const GemmArgs& args,
                int64_t lda, int64_t ldb, cudaStream_t stream);
}

int launch_umma_gemm(int kind, int epi, const void* A, const void* B, void* C, int64_t M, int64_t N,
                     int64_t K, int64_t lda, int64_t ldb, int64_t ldc, bool b_is_nk,
                     const float* row_scale, const float* col_scale, int force_bn,
                     cudaStream_t stream, const Tail& tail) {
  void* one[1] = {C};
  return launch_umma_gemm_multi(kind, epi, A, B, one, 1, M, N, K, lda, ldb, ldc, b_is_nk, row_scale, col_scale,
                                force_bn, stream, tail);
}

int launch_umma_gemm_multicast(int kind, int epi, const void* A, const void* B, void* C_multicast, int64_t M, int64_t N,
                               int64_t K, int64_t lda, int64_t ldb, int64_t ldc, const float* row_scale,
                               const float* col_scale, cudaStream_t stream) {
  void* one[1] = {C_multicast};
  g_multicast_call = true;
  const int rc = launch_umma_gemm_multi(kind, epi, A, B, one, 1, M, N, K, lda, ldb, ldc, false, row_scale, col_scale, 0,
                                        stream, Tail());
  g_multicast_call = false;
  return rc;
}

int launch_umma_gemm_multi(int kind, int epi, const void* A, const void* B, void* const* C_list, int n_dest,
                           int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc, bool b_is_nk,
                           const float* row_scale, const float* col_scale, int force_bn, cudaStream_t stream,
                           const Tail& tail) {
  if (!A || !B || !C_list) return fail(B200_ERR_BAD_ARGUMENT, "null matrix pointer");
  if ((tail.bias || tail.flags) && (epi == EPI_I32 || epi == EPI_W8A8_BF16))
    return fail(B200_ERR_BAD_ARGUMENT, "bias and activation exist for floating-point products only");
  if (n_dest < 1 || n_dest > kMaxDest)
    return fail(B200_ERR_BAD_ARGUMENT, "number of destinations must be between 1 and %d", kMaxDest);
  for (int g = 0; g < n_dest; ++g)
    if (!C_list[g]) return fail(B200_ERR_BAD_ARGUMENT, "null matrix pointer (destination %d)", g);
  if (M <= 0 || N <= 0 || K <= 0) return fail(B200_ERR_BAD_ARGUMENT, "M, N and K must be positive");
  if (M > (1 << 30) || N > (1 << 30) || K > (1 << 30))
    return fail(B200_ERR_TOO_LARGE, "a dimension exceeds 2^30");
  const int elem = kind == KIND_I8 ? 1 : (kind == KIND_TF32 ? 4 : 2);
  const int out_elem = (epi == EPI_I32 || epi == EPI_F32) ? 4 : 2;
  if (lda < K || ldb < (b_is_nk ? K : N) || ldc < N)
    return fail(B200_ERR_BAD_ARGUMENT, "a leading dimension is smaller than the row it spans");
  // A and B are read by TMA: 16-byte aligned base and row pitch.  C is written with plain
  // stores: 16-byte vectors when its base and pitch allow, element by element otherwise.
  if ((lda * elem) % 16 || (ldb * elem) % 16 || reinterpret_cast<uintptr_t>(A) % 16 ||
      reinterpret_cast<uintptr_t>(B) % 16)
    return fail(B200_ERR_UNSUPPORTED,
                "tensor-core GEMM needs 16-byte aligned A and B pointers and leading dimensions "
                "(lda=%lld ldb=%lld, element %d bytes)",
                (long long)lda, (long long)ldb, elem);
  bool c_aligned16 = (ldc * out_elem) % 16 == 0;
  for (int g = 0; g < n_dest; ++g) {
    if (reinterpret_cast<uintptr_t>(C_list[g]) % out_elem)
      return fail(B200_ERR_UNSUPPORTED, "C is not aligned to its element size");
    if (reinterpret_cast<uintptr_t>(C_list[g]) % 16) c_aligned16 = false;
  }
  if (epi == EPI_W8A8_BF16 && (!row_scale || !col_scale))
    return fail(B200_ERR_BAD_ARGUMENT, "null scale pointer");

  GemmArgs args;
  memset(&args, 0, sizeof(args));
  for (int g = 0; g < n_dest; ++g) args.C[g] = C_list[g];
  args.n_dest = n_dest;
  args.ldc = ldc;
  args.M = int(M);
  args.N = int(N);
  args.K = int(K);
  args.tiles_m = int((M + BM - 1) / BM);
  args.tiles_n = 0;
  // Aligned C: staged TMA stores (or 16-byte register stores when forced); otherwise element by element.
  args.store_mode = !c_aligned16 ? STORE_SCALAR : (g_force_store == STORE_VECTOR ? STORE_VECTOR : STORE_TMA);
  if (g_multicast_call) {
    // the destination is a multicast address: only multimem instructions may touch it
    if (!c_aligned16 || (N * out_elem) % 16)
      return fail(B200_ERR_UNSUPPORTED, "a multicast destination needs 16-byte aligned rows of C (N and ldc)");
    args.store_mode = STORE_MULTIMEM;
  }
  args.row_scale = row_scale;
  args.col_scale = col_scale;
  args.bias = tail.bias;
  args.tail_flags = tail.flags;
  args.single_pass = (kind == KIND_TF32 && g_tf32_single_pass_call) ? 1 : 0;
  args.wait_budget_ns = g_wait_budget_ns;
  args.lose_kb = g_lose_kb;
  args.l2_hints = g_l2_hints >= 0 ? g_l2_hints : 0;

  int sms = 0;
  int rc = sm_count_of_current_device(&sms);
  if (rc) return rc;
  const bool skinny_forced = g_force_cg == 3;  // tile policy 3: the K-split cluster kernel or nothing
  const bool skinny_kind = kind == KIND_F16 || kind == KIND_BF16 || kind == KIND_I8;
  if (skinny_forced && !(skinny_kind && n_dest == 1))
    return fail(B200_ERR_UNSUPPORTED, "the skinny kernel takes fp16, bf16 and int8 products with one destination");
  int bn = force_bn ? force_bn : (skinny_forced ? 0 : g_force_bn);
  int cg = skinny_forced ? 1 : g_force_cg;
  int rb = 1;
  if (cg == 4) { cg = 2; rb = 2; }  // tile policy 4: CTA pairs with two row blocks per CTA (512 x 256 tiles)
  if (g_multicast_call) rb = 1;     // the multicast epilogue is the four-warp one
  if (cg == 0) {
    // CTA pairs (256 x 256 tiles) once they give every pair of SMs a tile; single CTAs below that.
    const int64_t pair_tiles = ((M + 2 * BM - 1) / (2 * BM)) * ((N + 255) / 256);
    cg = (bn == 0 || bn == 256) && M > BM && pair_tiles >= sms / 2 ? 2 : 1;  // a pair needs more than one CTA's rows
    // Two row blocks per CTA (512 x 256 tiles): a quarter fewer bytes from L2 per flop against an
    // epilogue that the next tile's MMAs no longer hide.  Measured back to back from a cool start,
    // 256-row / 512-row tiles: tf32 8192^3 1550 / 1306 us, 4096^3 213 / 180 us; bf16 8192^3 718 / 676 us,
    // 4096^3 99.8 / 95.5 us; int8 -> int32 8192^3 374 / 354 us, 4096^3 56.5 / 55.6 us.  Run for seconds
    // under the power cap, bf16 gains 2.3 / 5.0 / 6.3 % at 4096^3 / 6144^3 / 8192^3, int8 -> int32
    // -1 / 0.4 / 1.7 % (its 4-byte outputs leave the MMA lane waiting 11 % of its loop for the epilogue),
    // and the W8A8 epilogue (two multiplications per value before the accumulators go back) loses 2-7 %.
    // So: tf32 (twice the bytes per flop) takes them whenever they cost at most one extra wave in
    // eight, 16-bit kinds from K = 4096 and int8 -> int32 from K = 8192 where they cost no extra wave,
    // W8A8 never.
    if (cg == 2 && !g_multicast_call && n_dest == 1 && epi != EPI_W8A8_BF16) {  // several destinations: measured with 256-row tiles only
      const int64_t pairs = sms / 2;
      const int64_t tiles_n = (N + 255) / 256;
      const int64_t waves256 = (pair_tiles + pairs - 1) / pairs;
      const int64_t waves512 = 2 * ((((M + 4 * BM - 1) / (4 * BM)) * tiles_n + pairs - 1) / pairs);
      const int64_t k_from = kind == KIND_I8 ? 8192 : 4096;
      if (kind == KIND_TF32 ? waves512 * 7 <= waves256 * 8 : (K >= k_from && waves512 <= waves256)) rb = 2;
    }
  }
  if (cg == 2) bn = 256;
  if (bn == 0) {
    // Tile width with the smallest estimated time: waves of tiles over the SMs, each costing its
    // width plus a fixed part (pipeline fill, A traffic).  A narrow tile that spills into a second,
    // mostly empty wave loses to a wider tile that fits in one.
    int64_t best_cost = 0;
    for (int cand = 256; cand >= 64; cand >>= 1) {
      const int64_t tiles = int64_t(args.tiles_m) * ((N + cand - 1) / cand);
      const int64_t cost = ((tiles + sms - 1) / sms) * (cand + 64);
      if (bn == 0 || cost < best_cost) { bn = cand; best_cost = cost; }
    }
  }
  if (kind == KIND_I8 && !b_is_nk && bn < 128) bn = 128;  // an int8 span of N is 128 elements wide

  // A product of at most 128 rows streams B and little else.  If splitting K inside clusters
  // lets every SM pull clearly less through its TMA unit than the tiles chosen above would (columns
  // of B per k-block, plus the 128 rows of A at the 0.3 they were measured to weigh, coming from L2),
  // that kernel takes it.
  const bool nothing_forced = force_bn == 0 && g_force_bn == 0 && g_force_cg == 0 && g_force_store == 0;
  if (skinny_kind && n_dest == 1 && (skinny_forced || (nothing_forced && M <= BM))) {
    const int64_t k_blocks = (K * elem + 127) / 128;
    const int64_t tiles = int64_t(args.tiles_m) * ((N + bn - 1) / bn);
    const int64_t general_cost = ((tiles + sms - 1) / sms) * (int64_t(bn) * 10 + BM * 3) * k_blocks / 10;
    bool used = false;
    rc = launch_skinny_gemm(kind, epi, A, B, C_list[0], M, N, K, lda, ldb, ldc, b_is_nk, row_scale, col_scale, tail,
                            skinny_forced ? g_force_bn : 0, skinny_forced, general_cost, stream, &used);
    if (rc || used) return rc;
  }

  return launch_kind(kind, epi, bn, cg, rb, b_is_nk, A, B, args, lda, ldb, stream);
}

namespace {
int launch_kind(int kind, int epi, int bn, int cg, int rb, bool b_is_nk, const void* A, const void* B, const GemmArgs& args,
                int64_t lda, int64_t ldb, cudaStream_t stream) {
  switch (kind) {
    case KIND_I8:
      if (epi == EPI_I32) return launch_bn<KIND_I8, EPI_I32>(bn, cg, rb, b_is_nk, A, B, args, lda, ldb, stream);
      if (epi == EPI_W8A8_BF16)
        return launch_bn<KIND_I8, EPI_W8A8_BF16>(bn, cg, rb, b_is_nk, A, B, args, lda, ldb, stream);
      break;
    case KIND_F16:
      if (epi == EPI_F16) return launch_bn<KIND_F16, EPI_F16>(bn, cg, rb, b_is_nk, A, B, args, lda, ldb, stream);
      if (epi == EPI_F32) return launch_bn<KIND_F16, EPI_F32>(bn, cg, rb, b_is_nk, A, B, args, lda, ldb, stream);
      break;
    case KIND_BF16:
      if (epi == EPI_BF16) return launch_bn<KIND_BF16, EPI_BF16>(bn, cg, rb, b_is_nk, A, B, args, lda, ldb, stream);
      if (epi == EPI_F32) return launch_bn<KIND_BF16, EPI_F32>(bn, cg, rb, b_is_nk, A, B, args, lda, ldb, stream);
      break;
    case KIND_TF32:  // A and B are the stacked low/high planes made by launch_sgemm_3xtf32
      if (epi == EPI_F32) return launch_bn<KIND_TF32, EPI_F32>(bn, cg, rb, b_is_nk, A, B, args, lda, ldb, stream);
      break;
    default:
      break;
  }
  return fail(B200_ERR_BAD_ARGUMENT, "unsupported operand kind %d with epilogue %d", kind, epi);
}
}  // namespace

// ------------------------------------------------------------------------------ 3xTF32
namespace {

__device__ __forceinline__ float round_to_tf32(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}

// Splits a row-major [rows, cols] fp32 matrix into two tf32-exact planes stacked in `out`
// ([2 * rows, ld_out]): plane 0 holds the low parts, plane 1 the high parts, x ~= hi + lo with
// hi = tf32(x) and lo = tf32(x - hi).  Padding columns [cols, ld_out) are left untouched; the
// tensor map that reads the planes stops at `cols`.
__global__ void split_tf32_kernel(const float* __restrict__ x, float* __restrict__ out, int64_t rows,
                                  int64_t cols, int64_t ld_in, int64_t ld_out) {
  const int64_t total = rows * cols;
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t r = i / cols, c = i - r * cols;
    const float v = x[r * ld_in + c];
    const float hi = round_to_tf32(v);
    const float lo = round_to_tf32(v - hi);
    out[r * ld_out + c] = lo;
    out[(rows + r) * ld_out + c] = hi;
  }
}

}  // namespace

int split_tf32_into(const float* A, const float* B, float* scratch, int64_t M, int64_t N, int64_t K,
                    int64_t lda, int64_t ldb, bool b_is_nk, int64_t* ld_a_out, int64_t* ld_b_out,
                    float** planes_b, cudaStream_t stream) {
  const int64_t a_cols = K, a_rows = M;
  const int64_t b_cols = b_is_nk ? K : N, b_rows = b_is_nk ? N : K;
  const int64_t lda_p = (a_cols + 3) & ~int64_t(3), ldb_p = (b_cols + 3) & ~int64_t(3);  // 16-byte rows
  float* pa = scratch;
  float* pb = scratch + 2 * a_rows * lda_p;
  const int grid = 148 * 8;
  split_tf32_kernel<<<grid, 256, 0, stream>>>(A, pa, a_rows, a_cols, lda, lda_p);
  split_tf32_kernel<<<grid, 256, 0, stream>>>(B, pb, b_rows, b_cols, ldb, ldb_p);
  B200_CUDA_TRY(cudaGetLastError());
  *ld_a_out = lda_p;
  *ld_b_out = ldb_p;
  *planes_b = pb;
  return B200_OK;
}

size_t split_tf32_scratch_floats(int64_t M, int64_t N, int64_t K, bool b_is_nk) {
  const int64_t b_cols = b_is_nk ? K : N, b_rows = b_is_nk ? N : K;
  return size_t(2 * M * ((K + 3) & ~int64_t(3)) + 2 * b_rows * ((b_cols + 3) & ~int64_t(3)));
}

// fp32 inputs multiplied as tf32 (the tensor cores keep sign, exponent and the top 10 mantissa bits of
// each operand) with fp32 accumulation: one pass, no scratch.  Relative error of a product ~ 2^-10.
int launch_sgemm_tf32(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K, int64_t lda,
                      int64_t ldb, int64_t ldc, bool b_is_nk, cudaStream_t stream, const Tail& tail) {
  g_tf32_single_pass_call = true;
  int rc = launch_umma_gemm(KIND_TF32, EPI_F32, A, B, C, M, N, K, lda, ldb, ldc, b_is_nk, nullptr, nullptr, 0, stream,
                            tail);
  g_tf32_single_pass_call = false;
  return rc;
}

extern int g_x3_path;
bool x3_on_chip_applies(const float* A, const float* B, int64_t lda, int64_t ldb);
int launch_sgemm_3xtf32_on_chip(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K,
                                int64_t lda, int64_t ldb, int64_t ldc, bool b_is_nk, cudaStream_t stream,
                                const Tail& tail);

int launch_sgemm_3xtf32(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K,
                        int64_t lda, int64_t ldb, int64_t ldc, bool b_is_nk, cudaStream_t stream, const Tail& tail) {
  if (!A || !B || !C) return fail(B200_ERR_BAD_ARGUMENT, "null matrix pointer");
  if (M <= 0 || N <= 0 || K <= 0) return fail(B200_ERR_BAD_ARGUMENT, "M, N and K must be positive");
  if (lda < K || ldb < (b_is_nk ? K : N) || ldc < N)
    return fail(B200_ERR_BAD_ARGUMENT, "a leading dimension is smaller than the row it spans");
  // Small and medium products are bound by the per-k-block hand-shake between TMA and the MMA lane,
  // not by the tensor pipe: they take the kernel that splits the operands on chip (one hand-shake
  // per k-block instead of three, no scratch, one launch).  Large ones keep the split planes in
  // global memory and run on CTA pairs (measured on chip / split planes: 1024^3 29.7 / 48.4 us,
  // 2048^3 113 / 147 us, 4096^3 797 / 640 us), except for very long sums: the pair kernel adds a
  // whole K into one accumulator, whose truncation error grows with K (9.6e-6 at K = 4096), while
  // the on-chip kernel sums K in ranges (4.9e-6 there).
  if (g_x3_path != 1 && x3_on_chip_applies(A, B, lda, ldb) &&
      (g_x3_path == 2 || M * N <= int64_t(2048) * 2048 || K > 4096))
    return launch_sgemm_3xtf32_on_chip(A, B, C, M, N, K, lda, ldb, ldc, b_is_nk, stream, tail);
  // The split planes live for this call only: taken from the stream-ordered pool on `stream` and
  // given back on `stream` right behind the GEMM, so calls on different streams (or from different
  // host threads) never share scratch, and nothing is freed while a kernel may still read it.
  const size_t need = split_tf32_scratch_floats(M, N, K, b_is_nk) * sizeof(float);
  cudaMemPool_t pool = nullptr;
  int rc = scratch_pool(&pool);
  if (rc) return rc;
  void* mem = nullptr;
  B200_CUDA_TRY(cudaMallocFromPoolAsync(&mem, need, pool, stream));
  float* scratch = static_cast<float*>(mem);
  int64_t lda_p = 0, ldb_p = 0;
  float* pb = nullptr;
  rc = split_tf32_into(A, B, scratch, M, N, K, lda, ldb, b_is_nk, &lda_p, &ldb_p, &pb, stream);
  if (rc == B200_OK)
    rc = launch_umma_gemm(KIND_TF32, EPI_F32, scratch, pb, C, M, N, K, lda_p, ldb_p, ldc, b_is_nk, nullptr, nullptr, 0,
                          stream, tail);
  const cudaError_t fe = cudaFreeAsync(mem, stream);  // stream-ordered: released after the kernels above
  if (rc == B200_OK && fe != cudaSuccess) rc = fail(B200_ERR_CUDA, "cudaFreeAsync: %s", cudaGetErrorString(fe));
  return rc;
}

}  // namespace b200

// ------------------------------------------------------------------------------ 3xTF32, operands split on chip
//
// The same three-product fp32 GEMM without split planes in global memory.  TMA brings the fp32
// tiles of A and B into a ring of "raw" stages.  Eight converter warps split them: every thread owns
// half a row of the A tile, reads its 16 floats from the stage and writes the tf32 high parts (top 19
// bits) and the remainders, rounded to tf32, into tensor memory, where the MMA takes its A operand
// from; B is cut to its high part in place and its remainder goes to one of two small shared-memory
// buffers.  The MMA lane then issues lo*hi, hi*lo and hi*hi for the k-block.  Against the
// split-plane form a k-block crosses the TMA -> MMA hand-shake once instead of three times, nothing
// but A, B and C touches global memory, and the tensor cores read only B from shared memory (a tf32
// operand is four bytes per element, and shared-memory bandwidth is what bounds a tf32 main loop).
// Tensor memory also holds several accumulators: number 0 takes the two small products of every
// k-block, the others each take hi*hi over one contiguous range of K.  The tensor cores add into
// an fp32 accumulator by truncation, so the error of one long chain grows in proportion to K;
// short chains added with correctly rounded fp32 additions in the epilogue keep it small.
// One tile of 128 x BN per CTA, no persistence; C is written from registers.
//   warp 0 producer, warp 1 MMA + tensor memory, warps 2-5 epilogue, warps 6-13 converters (two warps per
//   32-row quarter of the A tile, each taking half of the k-block's columns).
namespace b200 {
namespace {

constexpr int kX3ConvThreads = 256;               // eight converter warps: two per quarter of tensor memory
constexpr int kX3Threads = 192 + kX3ConvThreads;

template <int BN>
struct X3Tile {
  static constexpr int BK = 32;                       // floats of K per stage: one 128-byte swizzle row
  static constexpr int A_BYTES = BM * 128;
  static constexpr int B_BYTES = BN * 128;
  static constexpr int RAW_BYTES = A_BYTES + B_BYTES;  // one stage of fp32 tiles
  static constexpr int SPAN = 32;                      // floats of N in one 128-byte span of an N-contiguous B
  static constexpr int NSPANS = BN / SPAN;
  static constexpr int SPAN_BYTES = BK * 128;
  static constexpr int LO_BUFS = 2;                    // low parts of B (shared memory) and both parts of A (tensor memory);
                                                       // three changed nothing (1024^3: 29.5 against 29.7 us)
  static constexpr int STAGES_FIT = (kSmemBudget - 2048 - LO_BUFS * B_BYTES) / RAW_BYTES;
  static constexpr int STAGES = STAGES_FIT > 8 ? 8 : STAGES_FIT;
  // Tensor memory, 512 columns: LO_BUFS A buffers of 32 high + 32 low columns each; then NACC accumulators.
  static constexpr int A_COLS = LO_BUFS * 2 * BK;
  static constexpr int NACC = (512 - A_COLS) / BN;
  static constexpr int TMEM_COLS = 512;
  static constexpr int SMEM_BYTES = STAGES * RAW_BYTES + LO_BUFS * B_BYTES + 1024 /*alignment*/ + 256 /*barriers*/;
  static_assert(STAGES >= 3 && NACC >= 2, "ring or accumulator budget too small");
};

template <int BN, bool B_NK>
__global__ void __launch_bounds__(kX3Threads, 1)
gemm_tf32x3_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                   const GemmArgs p) {
  using T = X3Tile<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* lo_base = smem + T::STAGES * T::RAW_BYTES;  // LO_BUFS buffers of B_BYTES: low parts of B
  uint64_t* bars = reinterpret_cast<uint64_t*>(lo_base + T::LO_BUFS * T::B_BYTES);
  uint64_t* full_bar = bars;                        // [STAGES] TMA -> converters
  uint64_t* empty_bar = bars + T::STAGES;           // [STAGES] MMA -> producer
  uint64_t* lo_full = bars + 2 * T::STAGES;         // [LO_BUFS] converters -> MMA: the k-block is split
  uint64_t* lo_empty = lo_full + T::LO_BUFS;        // [LO_BUFS] MMA -> converters: its buffers are free again
  uint64_t* acc_full = lo_empty + T::LO_BUFS;       // [1] MMA -> epilogue
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_kb = (p.K + T::BK - 1) / T::BK;
  int mb, nb;
  tile_coords(int(blockIdx.x), p.tiles_m, p.tiles_n, p.group_m, mb, nb);
  const int m0 = mb * BM, n0 = nb * BN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < T::STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int j = 0; j < T::LO_BUFS; ++j) {
      mbar_init(&lo_full[j], kX3ConvThreads);  // every converter thread arrives
      mbar_init(&lo_empty[j], 1);
    }
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, T::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t acc_base = tmem_base + uint32_t(T::A_COLS);

  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int kb = 0; kb < num_kb; ++kb) {
        if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1u, abort_flag, p.wait_budget_ns)) break;
        uint8_t* sa = smem + stage * T::RAW_BYTES;
        uint8_t* sb = sa + T::A_BYTES;
        mbar_arrive_expect_tx(&full_bar[stage], T::RAW_BYTES);
        tma_load_2d(sa, &tmap_a, &full_bar[stage], kb * T::BK, m0);
        if constexpr (B_NK) {
          tma_load_2d(sb, &tmap_b, &full_bar[stage], kb * T::BK, n0);
        } else {
#pragma unroll
          for (int sp = 0; sp < T::NSPANS; ++sp)
            tma_load_2d(sb + sp * T::SPAN_BYTES, &tmap_b, &full_bar[stage], n0 + sp * T::SPAN, kb * T::BK);
        }
        if (++stage == T::STAGES) { stage = 0; phase ^= 1u; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_instr_desc(KIND_TF32, BM, BN, 0, B_NK ? 0 : 1);
      const uint32_t ring = smem_u32(smem);
      const uint32_t lo_ring = smem_u32(lo_base);
      auto b_desc_at = [](uint32_t base) {
        return B_NK ? make_smem_desc_sw128(base, 16, 1024) : make_smem_desc(base, T::SPAN_BYTES, 512, 1);
      };
      int stage = 0, j = 0;
      uint32_t lo_phase = 0;
      bool ok = true;
      const int big_ranges = min(T::NACC - 1, num_kb);  // accumulators 1 .. big_ranges take hi*hi
      uint32_t started = 0;                             // bit a: accumulator a has been written
      for (int kb = 0; kb < num_kb && ok; ++kb) {
        // the converters waited for the stage themselves; their arrival covers it
        if (!mbar_wait_bounded(&lo_full[j], lo_phase, abort_flag, p.wait_budget_ns)) { ok = false; break; }
        tc_fence_after_sync();
        const uint64_t b_hi = b_desc_at(ring + stage * T::RAW_BYTES + T::A_BYTES);
        const uint64_t b_lo = b_desc_at(lo_ring + j * T::B_BYTES);
        const uint32_t a_hi = tmem_base + uint32_t(j * 2 * T::BK);  // 32 columns of high parts, then 32 of low parts
        const uint32_t a_lo = a_hi + uint32_t(T::BK);
        const int big = 1 + (kb * big_ranges) / num_kb;
#pragma unroll
        for (int prod = 0; prod < 3; ++prod) {  // lo*hi, hi*lo into accumulator 0; hi*hi into its range's
          const uint32_t at = prod == 0 ? a_lo : a_hi;
          const uint64_t bd = prod == 1 ? b_lo : b_hi;
          const int acc = prod == 2 ? big : 0;
          const uint32_t d_tmem = acc_base + uint32_t(acc * BN);
#pragma unroll
          for (int q = 0; q < 4; ++q) {  // 8 floats of K per instruction: 8 columns of A, 32 bytes of B's K
            const uint64_t b_adv = B_NK ? uint64_t((q * 32) >> 4) : uint64_t((q * 8 * 128) >> 4);
            umma_tf32_a_in_tmem(d_tmem, at + uint32_t(q * 8), bd + b_adv, idesc, (started >> acc) & 1u);
            started |= 1u << acc;
          }
        }
        umma_commit(&empty_bar[stage]);
        umma_commit(&lo_empty[j]);
        if (++stage == T::STAGES) stage = 0;
        if (++j == T::LO_BUFS) { j = 0; lo_phase ^= 1u; }
      }
      if (ok) umma_commit(acc_full);
    }
  } else if (warp >= 6) {
    // ------------------------------------------------------------------ converters
    const int ct = int(threadIdx.x) - 6 * 32;  // 0..255
    const int quarter = warp & 3;              // the tensor-memory lanes this warp may touch
    const int half = (warp - 6) >> 2;          // which 16 of the k-block's 32 columns this warp splits
    const int r = quarter * 32 + lane;         // row of the A tile this thread works on
    constexpr int B_CHUNKS = T::B_BYTES / 16;
    int stage = 0, j = 0;
    uint32_t phase = 0, lo_phase = 0;
    for (int kb = 0; kb < num_kb; ++kb) {
      bool ok = mbar_wait_bounded(&full_bar[stage], phase, abort_flag, p.wait_budget_ns) &&
                mbar_wait_bounded(&lo_empty[j], lo_phase ^ 1u, abort_flag, p.wait_budget_ns);
      ok = __all_sync(0xffffffffu, ok) != 0;  // the warp stays together for the aligned tensor-memory stores
      if (!ok) break;
      tc_fence_after_sync();
      // A: half of this thread's row, 4 swizzled 16-byte chunks -> 16 high and 16 low words in tensor memory
      const uint8_t* arow = smem + stage * T::RAW_BYTES + r * 128;
      uint32_t hi[16], lo[16];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const uint4 x = *reinterpret_cast<const uint4*>(arow + (((half * 4 + c) ^ (r & 7)) << 4));
        const uint32_t xs[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const uint32_t h = xs[e] & 0xffffe000u;
          hi[4 * c + e] = h;
          lo[4 * c + e] = __float_as_uint(round_to_tf32(__uint_as_float(xs[e]) - __uint_as_float(h)));
        }
      }
      const uint32_t a_t = tmem_base + (uint32_t(quarter * 32) << 16) + uint32_t(j * 2 * T::BK + half * 16);
      tmem_st_32x16(a_t, hi);
      tmem_st_32x16(a_t + uint32_t(T::BK), lo);
      // B: element-wise on the stage's bytes, whatever their layout: high parts in place, low parts aside
      uint4* braw = reinterpret_cast<uint4*>(smem + stage * T::RAW_BYTES + T::A_BYTES);
      uint4* blo = reinterpret_cast<uint4*>(lo_base + j * T::B_BYTES);
#pragma unroll 4
      for (int c = ct; c < B_CHUNKS; c += kX3ConvThreads) {
        const uint4 x = braw[c];
        uint4 h, l;
        h.x = x.x & 0xffffe000u; h.y = x.y & 0xffffe000u; h.z = x.z & 0xffffe000u; h.w = x.w & 0xffffe000u;
        l.x = __float_as_uint(round_to_tf32(__uint_as_float(x.x) - __uint_as_float(h.x)));
        l.y = __float_as_uint(round_to_tf32(__uint_as_float(x.y) - __uint_as_float(h.y)));
        l.z = __float_as_uint(round_to_tf32(__uint_as_float(x.z) - __uint_as_float(h.z)));
        l.w = __float_as_uint(round_to_tf32(__uint_as_float(x.w) - __uint_as_float(h.w)));
        braw[c] = h;
        blo[c] = l;
      }
      tmem_st_wait();             // the tensor-memory stores have landed
      fence_proxy_async_smem();   // the tensor cores read the shared-memory bytes through the async proxy
      tc_fence_before_sync();
      mbar_arrive(&lo_full[j]);
      if (++stage == T::STAGES) { stage = 0; phase ^= 1u; }
      if (++j == T::LO_BUFS) { j = 0; lo_phase ^= 1u; }
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps
    const int quarter = warp & 3;
    const int r_in_tile = quarter * 32 + lane;
    const int row = m0 + r_in_tile;
    if (mbar_wait_bounded_idle(acc_full, 0u, abort_flag, p.wait_budget_ns)) {
      tc_fence_after_sync();
      const uint32_t taddr = acc_base + (uint32_t(quarter * 32) << 16);
      const int big_ranges = min(T::NACC - 1, num_kb);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int cn0 = n0 + c * 32;
        if (cn0 >= p.N) break;
        // hi*hi ranges in ascending K, then the small products: plain fp32 additions, rounded to nearest
        uint32_t v[32], w[32];
        tmem_ld_32x32(taddr + uint32_t(BN + c * 32), v);
        tmem_ld_wait();
        for (int a = 2; a <= big_ranges + 1; ++a) {
          uint32_t u[32];
          tmem_ld_32x32(taddr + uint32_t((a > big_ranges ? 0 : a) * BN + c * 32), u);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) + __uint_as_float(u[i]));
        }
        pack_chunk<EPI_F32>(p, cn0, v, 0.f, w);
        if (row < p.M) store_chunk<EPI_F32>(p, row, cn0, w);
      }
    }
  }

  __syncwarp();
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0) atomicOr(&g_umma_status, 1u);
    uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, T::TMEM_COLS);
  }
}

template <int BN, bool B_NK>
int launch_x3(const float* A, const float* B, GemmArgs args, int64_t lda, int64_t ldb, cudaStream_t stream) {
  using T = X3Tile<BN>;
  auto kernel = gemm_tf32x3_kernel<BN, B_NK>;
  static thread_local int last_dev = -1;
  int dev = 0;
  B200_CUDA_TRY(cudaGetDevice(&dev));
  if (dev != last_dev) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, T::SMEM_BYTES);
    if (e != cudaSuccess)
      return fail(B200_ERR_CUDA, "cudaFuncSetAttribute(%d bytes of shared memory): %s", T::SMEM_BYTES,
                  cudaGetErrorString(e));
    last_dev = dev;
  }
  args.tiles_m = (args.M + BM - 1) / BM;
  args.tiles_n = (args.N + BN - 1) / BN;
  args.group_m = args.tiles_m;  // m fastest: CTAs that are resident together share columns of B
  CUtensorMap ma, mb;
  int rc = make_map(&ma, KIND_TF32, A, args.M, args.K, lda, T::BK, BM);
  if (rc) return rc;
  if (B_NK)
    rc = make_map(&mb, KIND_TF32, B, args.N, args.K, ldb, T::BK, BN);
  else
    rc = make_map(&mb, KIND_TF32, B, args.K, args.N, ldb, T::SPAN, T::BK, /*chunks32=*/true);
  if (rc) return rc;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(unsigned(args.tiles_m * args.tiles_n));
  cfg.blockDim = dim3(kX3Threads);
  cfg.dynamicSmemBytes = T::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  int nattr = 0;
  if (g_use_pdl) {
    attr[nattr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[nattr].val.programmaticStreamSerializationAllowed = 1;
    ++nattr;
  }
  cfg.attrs = attr;
  cfg.numAttrs = nattr;
  B200_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, ma, mb, args));
  return B200_OK;
}

}  // namespace

int g_x3_path = 0;  // 0 = automatic, 1 = split planes in global memory, 2 = split on chip

int set_x3_path(int path) {
  if (path < 0 || path > 2) return fail(B200_ERR_BAD_ARGUMENT, "3xTF32 path: 0 (automatic), 1 or 2");
  g_x3_path = path;
  return B200_OK;
}

// The on-chip form needs what TMA needs of fp32 operands: 16-byte aligned bases and row pitches.
bool x3_on_chip_applies(const float* A, const float* B, int64_t lda, int64_t ldb) {
  return lda % 4 == 0 && ldb % 4 == 0 && reinterpret_cast<uintptr_t>(A) % 16 == 0 &&
         reinterpret_cast<uintptr_t>(B) % 16 == 0;
}

int launch_sgemm_3xtf32_on_chip(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K,
                                int64_t lda, int64_t ldb, int64_t ldc, bool b_is_nk, cudaStream_t stream,
                                const Tail& tail) {
  GemmArgs args;
  memset(&args, 0, sizeof(args));
  args.C[0] = C;
  args.n_dest = 1;
  args.ldc = ldc;
  args.M = int(M);
  args.N = int(N);
  args.K = int(K);
  const bool c_aligned16 = (ldc * 4) % 16 == 0 && reinterpret_cast<uintptr_t>(C) % 16 == 0;
  args.store_mode = c_aligned16 ? STORE_VECTOR : STORE_SCALAR;
  args.bias = tail.bias;
  args.tail_flags = tail.flags;
  args.wait_budget_ns = g_wait_budget_ns;
  args.lose_kb = -1;
  int sms = 0;
  int rc = sm_count_of_current_device(&sms);
  if (rc) return rc;
  // Narrow tiles until the grid covers the machine: 128 x 128 when that already gives every SM a
  // tile, else 128 x 64.
  const int64_t tiles128 = ((M + BM - 1) / BM) * ((N + 127) / 128);
  const bool wide = tiles128 >= sms;
  if (wide)
    return b_is_nk ? launch_x3<128, true>(A, B, args, lda, ldb, stream) : launch_x3<128, false>(A, B, args, lda, ldb, stream);
  return b_is_nk ? launch_x3<64, true>(A, B, args, lda, ldb, stream) : launch_x3<64, false>(A, B, args, lda, ldb, stream);
}

}  // namespace b200

// ------------------------------------------------------------------------------ 3xTF32 without allocation
//
// Some hosts cannot let a plug-in allocate device memory: an inference server that handed the
// whole GPU to its own memory pool at start-up and treats any later cudaMalloc as a bug, or a
// control loop with a hard latency bound, where the implicit device-wide synchronisation of
// cudaMalloc / cudaFree (and the chance of it failing for lack of memory) is not acceptable.
// For them the split planes of the 3xTF32 GEMM live in a fixed array that is part of the
// library image: every GPU that loads the library carries it until the process ends.
namespace b200 {
namespace {

constexpr size_t kStaticSplitFloats = size_t(8) << 20;  // 8 Mi floats = 32 MiB per device

static __device__ __align__(256) float g_static_split[kStaticSplitFloats];

// Device address of g_static_split on each device, looked up once per device.  In host code the
// array's name is only a handle for the runtime, not an address a kernel could use.
std::mutex g_static_mu;
float* g_static_ptr[64] = {nullptr};

int static_split_address(float** out) {
  int dev = 0;
  B200_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(B200_ERR_UNSUPPORTED, "device ordinal %d is beyond the scratch table", dev);
  std::lock_guard<std::mutex> lock(g_static_mu);
  if (!g_static_ptr[dev]) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_static_split);  // for the device that is current now
    if (e != cudaSuccess)
      return fail(B200_ERR_CUDA, "cudaGetSymbolAddress(static scratch) on device %d: %s", dev, cudaGetErrorString(e));
    g_static_ptr[dev] = static_cast<float*>(p);
  }
  *out = g_static_ptr[dev];
  return B200_OK;
}

}  // namespace
}  // namespace b200

extern "C" int b200_gemm_f32_3xtf32_static(const float* A, const float* B, float* C, int64_t M, int64_t N,
                                           int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int layout,
                                           void* stream_) {
  using namespace b200;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!A || !B || !C) return fail(B200_ERR_BAD_ARGUMENT, "null matrix pointer");
  if (M <= 0 || N <= 0 || K <= 0) return fail(B200_ERR_BAD_ARGUMENT, "M, N and K must be positive");
  if (layout != B200_ROW_MAJOR && layout != B200_COL_MAJOR_NN && layout != B200_ROW_MAJOR_BT)
    return fail(B200_ERR_BAD_ARGUMENT, "unknown layout %d", layout);
  // Same mapping onto the kernels' row-major form as the allocating entry point: a column-major
  // product is the row-major product of the swapped operands.
  const float* a = A;
  const float* b = B;
  int64_t m = M, n = N;
  bool b_is_nk = layout == B200_ROW_MAJOR_BT;
  if (lda == 0) lda = layout == B200_COL_MAJOR_NN ? M : K;
  if (ldb == 0) ldb = layout == B200_ROW_MAJOR ? N : K;
  if (ldc == 0) ldc = layout == B200_COL_MAJOR_NN ? M : N;
  if (layout == B200_COL_MAJOR_NN) {
    a = B; b = A; m = N; n = M;
    int64_t t = lda; lda = ldb; ldb = t;
  }
  if (lda < K || ldb < (b_is_nk ? K : n) || ldc < n)
    return fail(B200_ERR_BAD_ARGUMENT, "a leading dimension is smaller than the row it spans");
  const size_t need = split_tf32_scratch_floats(m, n, K, b_is_nk);
  if (need > kStaticSplitFloats)
    return fail(B200_ERR_TOO_LARGE,
                "the split planes of this %lld x %lld x %lld product need %zu floats; the built-in scratch "
                "holds %zu (2*M*K + 2*K*N, rows padded to 4 floats, must not exceed it)",
                (long long)M, (long long)N, (long long)K, need, kStaticSplitFloats);
  float* scratch = nullptr;
  int rc = static_split_address(&scratch);
  if (rc) return rc;
  // Every word of the scratch that the GEMM reads is rewritten by the split below, so nothing left
  // over from an earlier call has to be cleared.
  int64_t lda_p = 0, ldb_p = 0;
  float* pb = nullptr;
  rc = split_tf32_into(a, b, scratch, m, n, K, lda, ldb, b_is_nk, &lda_p, &ldb_p, &pb, stream);
  if (rc) return rc;
  return launch_umma_gemm(KIND_TF32, EPI_F32, scratch, pb, C, m, n, K, lda_p, ldb_p, ldc, b_is_nk, nullptr, nullptr,
                          0, stream);
}

// ------------------------------------------------------------------------------ cross-GPU completion marker
//
// After a multi-destination GEMM every rank has to learn that all ranks' tiles have landed in its
// copy of C.  Each rank owns a small flag array in peer-mapped memory, one slot per rank; the
// marker kernel (one warp, launched on the same stream right after the GEMM) writes this step's
// number into its slot on every peer and then waits until every slot of its own array has
// reached that number.  The GEMM's stores precede the flag in stream order and the flag is
// written with system-scope release, so a rank that sees the flag also sees the tiles.
// The wait is bounded (two seconds); a rank that gives up records bit 1 of the status word
// that b200_check_device reports.  The ranks must run on different GPUs.
namespace b200 {
namespace {

struct PeerFlagArgs {
  uint32_t* flags[kMaxDest];  // flags[g]: the flag array (kMaxDest words) that lives on rank g
  int world;
  int rank;
  uint32_t value;
};

__global__ void peer_marker_kernel(const PeerFlagArgs a) {
  const int g = threadIdx.x;
  if (g >= a.world) return;
  __threadfence_system();
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(a.flags[g] + a.rank), "r"(a.value) : "memory");
  const uint32_t* mine = a.flags[a.rank] + g;
  const uint64_t t0 = global_timer_ns();
  uint32_t seen;
  for (;;) {
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
    if (int32_t(seen - a.value) >= 0) break;
    if (global_timer_ns() - t0 > 2000000000ull) {
      atomicOr(&g_umma_status, 2u);
      break;
    }
    __nanosleep(200);
  }
}

}  // namespace
}  // namespace b200

extern "C" int b200_peer_marker(void* const* flag_arrays, int world, int rank, uint32_t value, void* stream) {
  using namespace b200;
  if (!flag_arrays || world < 1 || world > kMaxDest || rank < 0 || rank >= world)
    return fail(B200_ERR_BAD_ARGUMENT, "peer marker: bad argument");
  PeerFlagArgs a;
  memset(&a, 0, sizeof(a));
  for (int g = 0; g < world; ++g) {
    if (!flag_arrays[g]) return fail(B200_ERR_BAD_ARGUMENT, "peer marker: null flag array for rank %d", g);
    a.flags[g] = static_cast<uint32_t*>(flag_arrays[g]);
  }
  a.world = world;
  a.rank = rank;
  a.value = value;
  peer_marker_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(a);
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}
