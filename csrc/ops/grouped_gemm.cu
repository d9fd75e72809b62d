// Grouped (per-expert) block-scaled fp8 GEMM on the Blackwell tensor cores.
//
//   for every local expert e with rows [row_start(e), row_start(e) + count(e)):
//     D = dequant(A rows) x dequant(B[e])^T
//   A  e4m3 [rows, K]      one fp32 scale per row and 128 columns (1x128)
//   B  e4m3 [E, N, K]      one fp32 scale per 128x128 block
//
// Two epilogues:
//   kSwiGLUQuant  B = [gate; up] stacked along N (N = 2 I): out = silu(gate) * up, re-quantised
//                 to e4m3 with 1x128 scales -> the input of the down projection
//   kBf16         out = D as bf16 -> the rows handed to combine
//
// Structure: one persistent CTA per SM, twelve warps, launched as clusters of two CTAs. The
// body is a template on the CTAs per tile:
//   pairs (256-row tiles)  the two CTAs of a cluster compute one 256 x 256 tile with
//               tcgen05.mma.cta_group::2 (M 256, N 256, K 32 x 4 per K block). Each CTA loads its
//               own 128 rows of A and its own half of B's rows (TMA with cta_group::2, bytes
//               counted on the leader's mbarrier, 128-byte swizzle) and keeps its 128 rows of the
//               accumulator in its own tensor memory; the leader's commit (two-CTA mask) releases
//               the stage and publishes the accumulator in both CTAs.
//   lone CTA (128-row tiles)  cta_group::1, all four B boxes per stage; chosen when an expert's
//               capacity is 192 rows or less, where the second CTA of a pair would idle.
//   warp 0      TMA producer into a four-stage shared-memory ring (the count must be even, see
//               kStages) and, before the loop, the tile schedule from the experts' row counts
//   warps 1, 2  (leader CTA) one MMA issuer per 256-column TMEM accumulator, even / odd K blocks
//   warp 3      idle; the first warpgroup gives most of its registers away with setmaxnreg
//   warps 4-11  epilogue: tcgen05.ld the K block's partial sums, scale them by
//               a_scale[row, kb] * b_scale[nb, kb] and add into fp32 registers (the per-block
//               scales differ along K, so the running sum cannot stay in TMEM), then SwiGLU +
//               re-quantise or bf16, staged through shared memory into full-line stores
// The two TMEM accumulators let the tensor cores work on K block i+1 while block i is being
// folded. No TMA multicast anywhere: B is shared inside a pair by each CTA loading half of it.
//
// The reference has no GEMM of any kind (its "expert" is x * 2 in tests and benchmarks:
// tests/p2p_all_to_all/test_p2p_all_to_all.py:44-50); this kernel is the expert-side half of
// the fused MoE layer built on top of dispatch / combine.

#include "grouped_gemm.h"

#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include <algorithm>

#include "../core/cu_driver.h"
#include "../core/error.h"
#include "tcgen05.cuh"

// The profiling aids (per-role wait totals, SM-clock stamps, stage removal) exist only in the
// translation unit built with PPLX_GEMM_PROFILE (grouped_gemm_profile.cu, entry point
// grouped_fp8_gemm_profiled); here they compile to nothing.
#ifdef PPLX_GEMM_PROFILE
#define PPLX_GEMM_ENTRY grouped_fp8_gemm_profiled
constexpr bool kProfile = true;
#else
#define PPLX_GEMM_ENTRY grouped_fp8_gemm
constexpr bool kProfile = false;
#endif

namespace pplx::ops {
namespace {

using namespace pplx::tc;

constexpr int kBM = 128, kBN = 256, kBK = 128;   // per CTA; a CTA pair computes 256 x 256
// The kernel body exists for tiles worked on by a pair of CTAs (kCtas 2: 256 rows, each CTA loads
// half of B) and by one CTA (kCtas 1: 128 rows, for experts with so few rows that a pair's second
// CTA would idle). Stage and staging sizes differ; arrays are sized for the larger.
constexpr int kStages = 4;
// The two MMA issuers take alternate K blocks and every issuer waits only for its own blocks'
// operand barriers, by phase parity. That is sound only if a stage always belongs to the same
// issuer, i.e. if the number of stages is even: with an odd count the two issuers share each
// stage's barrier, an issuer skips every other phase of it, and a parity wait can then be
// satisfied by the phase before the one it means when two TMA loads complete out of order
// (seen as a launch failure about once in a hundred launches with three stages).
static_assert(kStages % 2 == 0, "a stage must always be consumed by the same MMA issuer");
constexpr int kThreads = 384;
constexpr int kFirstEpilogueWarp = 4;
constexpr int kEpilogueThreads = 256;
constexpr uint32_t kABytes = kBM * kBK;        // 16 KiB
constexpr uint32_t kBBoxBytes = 64 * kBK;      // 8 KiB; a CTA of a pair holds two boxes (its half of the tile's B rows), a lone CTA four
template <int kCtas> constexpr int kBBoxesOf = kCtas == 2 ? 2 : 4;
template <int kCtas> constexpr uint32_t kStageBytesOf = kABytes + kBBoxesOf<kCtas> * kBBoxBytes;  // 32 / 48 KiB
constexpr uint32_t kBulkRowStride = 144;          // staged rows for bulk copies: 128 B + 16 B against bank conflicts
// per epilogue warp, for coalesced output stores: 128-byte row chunks (padded for bulk copies) in
// the pair kernel; the lone-CTA kernel's four 48 KiB stages leave room for 64-byte chunks only
template <int kCtas> constexpr uint32_t kWarpStageBytesOf = kCtas == 2 ? 32 * kBulkRowStride : 32 * 64;
constexpr uint32_t kTmemCols = 512;
// Register split between the first warpgroup (copies, MMA issue) and the epilogue warps. The
// pool is what the CTA was launched with, 168 registers for each of its 384 threads, not the
// whole register file: setmaxnreg.inc waits until the registers it asks for are free, so a split
// that asks for more than the first warpgroup gave back would wait for ever.
constexpr int kLaunchRegs = 168;
constexpr int kLightRegs = 48;
constexpr int kEpilogueRegs = 224;
static_assert(kFirstEpilogueWarp * 32 * kLightRegs + kEpilogueThreads * kEpilogueRegs <= kThreads * kLaunchRegs,
              "the epilogue's setmaxnreg.inc could never be granted");
static_assert(kLightRegs % 8 == 0 && kEpilogueRegs % 8 == 0, "setmaxnreg takes multiples of 8");
constexpr int kMaxExperts = 128;
constexpr int kTraceTiles = 64;
// Rows 32..61 of the trace hold stamps for CTA 0's first K blocks, one row each: MMA committed,
// epilogue saw the partial sums, epilogue released the accumulator, MMA got the accumulator,
// MMA got the operands, MMA issued.
constexpr int kTraceBlockBase = 32 * 8;
constexpr uint32_t kTraceBlocks = 30;
constexpr uint64_t kWaitNs = 2000000000ull;  // every mbarrier wait gives up after 2 s

struct KernelArgs {
  alignas(64) CUtensorMap map_a;
  alignas(64) CUtensorMap map_b;
  const float* a_scale;
  int64_t a_scale_stride_row;
  int64_t a_scale_stride_k;
  const float* b_scale;            // [E][N/128][K/128]
  const int32_t* expert_num_tokens;
  uint8_t* out;
  int64_t out_stride;              // bytes per output row
  float* out_scale;
  int64_t out_scale_stride_row;    // elements
  uint32_t* error_flag;
  unsigned long long* wait_cycles;  // optional [grid][4]: cycles each role spent waiting
  long long* trace;                 // optional [kTraceTiles][8]: SM clock at the phases of CTA 0's tiles
  int num_experts;
  int N, K;
  int expert_padding;
  int max_rows;
  int mode;
  CombineScatter scatter;
  int debug_skip;   // profiling aid, 0 in production: 1 epilogue reads nothing, 2 no MMAs, 4 no TMA loads, 8 every MMA is issued twice
};

struct Schedule {
  int row_start[kMaxExperts];
  int count[kMaxExperts];
  int tile_prefix[kMaxExperts + 1];
};

// `*e` is a cursor: a CTA's tiles come in increasing order, so the search resumes at the expert of
// the previous call (start it at 0) and costs a step or two instead of a scan.
__device__ __forceinline__ void decode_tile(const Schedule& s, int num_experts, int n_tiles, int t, int* e,
                                            int* m_tile, int* n_tile) {
  int lo = *e;
  while (lo + 1 < num_experts && t >= s.tile_prefix[lo + 1]) ++lo;
  const int local = t - s.tile_prefix[lo];
  *e = lo;
  *m_tile = local / n_tiles;
  *n_tile = local % n_tiles;
}

// One warp writes 64 bytes per row for its 32 rows (lane = row, as tensor memory hands them out)
// with coalesced stores: the rows are transposed through a 2 KiB staging buffer so that one store
// instruction covers 8 rows x 64 contiguous bytes instead of 32 rows x 16 bytes. The 16-byte units
// of a row are XOR-swizzled with the row pair index, which keeps both sides free of bank conflicts.
__device__ __forceinline__ void store_rows_64B(uint8_t* stage, int lane, const uint32_t (&w)[16], uint8_t* dst_row0,
                                               int64_t row_stride, uint32_t valid_mask) {
  #pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int pu = u ^ ((lane >> 1) & 3);
    *reinterpret_cast<uint4*>(stage + lane * 64 + pu * 16) = make_uint4(w[4 * u], w[4 * u + 1], w[4 * u + 2], w[4 * u + 3]);
  }
  __syncwarp();
  #pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = 8 * i + (lane >> 2);
    const int u = lane & 3;
    const uint4 v = *reinterpret_cast<const uint4*>(stage + r * 64 + ((u ^ ((r >> 1) & 3)) * 16));
    if ((valid_mask >> r) & 1u) *reinterpret_cast<uint4*>(dst_row0 + r * row_stride + u * 16) = v;
  }
  __syncwarp();
}

// The 64-byte transposition with a row address functor (null = skip the row), for bf16 rows in the
// lone-CTA kernel.
template <typename RowBase>
__device__ __forceinline__ void store_rows_64B_fn(uint8_t* stage, int lane, const uint32_t (&w)[16], bool streaming,
                                                  RowBase row_base) {
  #pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int pu = u ^ ((lane >> 1) & 3);
    *reinterpret_cast<uint4*>(stage + lane * 64 + pu * 16) = make_uint4(w[4 * u], w[4 * u + 1], w[4 * u + 2], w[4 * u + 3]);
  }
  __syncwarp();
  #pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = 8 * i + (lane >> 2);
    const int u = lane & 3;
    const uint4 v = *reinterpret_cast<const uint4*>(stage + r * 64 + ((u ^ ((r >> 1) & 3)) * 16));
    uint8_t* const base = row_base(r);
    if (base != nullptr) {
      if (streaming) {
        Vec16 out;
        out.x = v.x; out.y = v.y; out.z = v.z; out.w = v.w;
        st_stream_v4(base + u * 16, out);
      } else {
        *reinterpret_cast<uint4*>(base + u * 16) = v;
      }
    }
  }
  __syncwarp();
}

// 128 bytes per row (64 bf16 columns): one store instruction then covers 4 rows x one full
// 128-byte line, which is what both the L2 and NVLink move best. `row_base(r)` gives the address
// of row r's chunk or null. Units of 16 bytes are XOR-swizzled with the row index (conflict-free
// on both sides: a quarter warp writes one unit of 8 rows, and reads the 8 units of one row).
template <typename RowBase>
__device__ __forceinline__ void store_rows_128B(uint8_t* stage, int lane, const uint32_t (&w)[32], bool streaming,
                                                RowBase row_base) {
  #pragma unroll
  for (int u = 0; u < 8; ++u) {
    const int pu = u ^ (lane & 7);
    *reinterpret_cast<uint4*>(stage + lane * 128 + pu * 16) = make_uint4(w[4 * u], w[4 * u + 1], w[4 * u + 2], w[4 * u + 3]);
  }
  __syncwarp();
  #pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = 4 * i + (lane >> 3);
    const int u = lane & 7;
    const uint4 v = *reinterpret_cast<const uint4*>(stage + r * 128 + ((u ^ (r & 7)) * 16));
    uint8_t* const base = row_base(r);
    if (base != nullptr) {
      if (streaming) {
        Vec16 out;
        out.x = v.x; out.y = v.y; out.z = v.z; out.w = v.w;
        st_stream_v4(base + u * 16, out);
      } else {
        *reinterpret_cast<uint4*>(base + u * 16) = v;
      }
    }
  }
  __syncwarp();
}

template <int kCtas>
__device__ __forceinline__ void grouped_fp8_gemm_body(const KernelArgs& a) {
  constexpr uint32_t kStageBytes = kStageBytesOf<kCtas>;
  constexpr int kBBoxes = kBBoxesOf<kCtas>;
  constexpr uint32_t kWarpStageBytes = kWarpStageBytesOf<kCtas>;
  extern __shared__ __align__(1024) uint8_t smem[];
  __shared__ uint64_t full_bar[kStages], empty_bar[kStages], tmem_full_bar[2], tmem_empty_bar[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ Schedule sched;
  __shared__ float s_amax[2][kBM][2];
  __shared__ uint32_t s_failed;

  // broadcast from lane 0 so that the compiler knows the warp index is the same in every lane
  // and keeps the role code (loop counters, descriptors, addresses) in the uniform datapath
  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);
  const int lane = threadIdx.x & 31;
  const bool swiglu = a.mode == kSwiGLUQuant;
  const int I = a.N / 2;
  const int n_tiles = swiglu ? I / 128 : a.N / kBN;
  const int nkb = a.K / kBK;
  // The two CTAs of a cluster form a pair: rank 0 (the leader) issues the MMAs for both. A lone CTA
  // is a "pair" of one: rank 0, its own leader.
  const uint32_t rank = kCtas == 2 ? cluster_ctarank() : 0u;
  const int pair = blockIdx.x / kCtas;
  const int num_pairs = gridDim.x / kCtas;

  if (threadIdx.x == 0) {
    if (kProfile && a.trace != nullptr && blockIdx.x == 0) {   // last row: kernel start / end, SM clock and ns
      a.trace[(kTraceTiles - 1) * 8 + 0] = clock64();
      a.trace[(kTraceTiles - 1) * 8 + 1] = static_cast<long long>(globaltimer_ns());
    }
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full_bar[b], 1);
      mbar_init(&tmem_empty_bar[b], kCtas * kEpilogueThreads / 32);   // the epilogue warps of every CTA of the tile (leader's copy is used)
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    s_failed = 0;
    prefetch_tensormap(&a.map_a);
    prefetch_tensormap(&a.map_b);
  }
  if (warp == 0) {
    // Expert-major row layout (each expert's block starts at a multiple of the padding) and the
    // tile count before each expert. The counts live in global memory: the lanes fetch four
    // experts each at once and combine with a warp scan, instead of one thread walking through
    // up to 128 dependent cache misses in front of every launch.
    constexpr int kPerLane = kMaxExperts / 32;
    int n[kPerLane], rows_of[kPerLane], tiles_of[kPerLane];
    int my_rows = 0, my_tiles = 0;
    #pragma unroll
    for (int j = 0; j < kPerLane; ++j) {
      const int e = lane * kPerLane + j;
      n[j] = e < a.num_experts ? max(a.expert_num_tokens[e], 0) : 0;
    }
    #pragma unroll
    for (int j = 0; j < kPerLane; ++j) {
      rows_of[j] = (n[j] + a.expert_padding - 1) / a.expert_padding * a.expert_padding;
      tiles_of[j] = (n[j] + kCtas * kBM - 1) / (kCtas * kBM) * n_tiles;   // one tile = 128 rows per CTA working on it
      my_rows += rows_of[j];
      my_tiles += tiles_of[j];
    }
    int row = my_rows, tiles = my_tiles;   // inclusive scan over the lanes
    #pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int r_up = __shfl_up_sync(0xffffffffu, row, off);
      const int t_up = __shfl_up_sync(0xffffffffu, tiles, off);
      if (lane >= off) {
        row += r_up;
        tiles += t_up;
      }
    }
    const int total_tiles_all = __shfl_sync(0xffffffffu, tiles, 31);
    row -= my_rows;      // exclusive
    tiles -= my_tiles;
    #pragma unroll
    for (int j = 0; j < kPerLane; ++j) {
      const int e = lane * kPerLane + j;
      if (e < a.num_experts) {
        sched.row_start[e] = row;
        sched.count[e] = n[j];
        sched.tile_prefix[e] = tiles;
      }
      row += rows_of[j];
      tiles += tiles_of[j];
    }
    if (lane == 0) sched.tile_prefix[a.num_experts] = total_tiles_all;
  }
  if (warp == 1) {
    if constexpr (kCtas == 2) {
      tmem_alloc_pair(&tmem_base_slot, kTmemCols);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(&tmem_base_slot, kTmemCols);
      tmem_relinquish();
    }
  }
  // Both CTAs' barriers and tensor memory must exist before either signals the other.
  fence_before_thread_sync();
  if constexpr (kCtas == 2) {
    cluster_sync_all();
  } else {
    __syncthreads();
  }
  fence_after_thread_sync();
  const uint32_t tmem_base = tmem_base_slot;
  const int total_tiles = sched.tile_prefix[a.num_experts];
  // operand tiles need the 1024-byte alignment of the 128-byte swizzle atom
  uint8_t* const tiles = smem + ((1024u - (smem_u32(smem) & 1023u)) & 1023u);

  if (warp < kFirstEpilogueWarp) {
    // The first warpgroup only issues copies and MMAs: it keeps kLightRegs registers per thread and
    // the epilogue warpgroups take the rest of the register file.
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kLightRegs) : "memory");
  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      long long waited = 0;
      int e = 0;
      // the leader's barriers count both CTAs' bytes
      const uint32_t full_leader = kCtas == 2 ? map_to_cta(&full_bar[0], 0) : smem_u32(&full_bar[0]);
      for (int t = pair; t < total_tiles && !s_failed; t += num_pairs) {
        int m_pair, n_tile;
        decode_tile(sched, a.num_experts, n_tiles, t, &e, &m_pair, &n_tile);
        const int row0 = sched.row_start[e] + (kCtas * m_pair + static_cast<int>(rank)) * kBM;
        // This CTA's half of the tile's 256 B rows (accumulator columns [128 rank, 128 rank + 128)).
        // SwiGLU interleaves gate and up in 64-row boxes so that a thread's columns hold both.
        // A lone CTA loads all four boxes: gate, up, gate + 64, up + 64.
        int brow[kBBoxes];
        if constexpr (kCtas == 2) {
          if (swiglu) {
            brow[0] = e * a.N + n_tile * 128 + 64 * static_cast<int>(rank);
            brow[1] = brow[0] + I;
          } else {
            brow[0] = e * a.N + n_tile * kBN + 128 * static_cast<int>(rank);
            brow[1] = brow[0] + 64;
          }
        } else {
          if (swiglu) {
            brow[0] = e * a.N + n_tile * 128;
            brow[1] = brow[0] + I;
            brow[2] = brow[0] + 64;
            brow[3] = brow[1] + 64;
          } else {
            #pragma unroll
            for (int i = 0; i < kBBoxes; ++i) brow[i] = e * a.N + n_tile * kBN + 64 * i;
          }
        }
        const int trace_row = (kProfile && a.trace != nullptr && blockIdx.x == 0 && t / num_pairs < 32) ? t / num_pairs : -1;
        if (trace_row >= 0) a.trace[trace_row * 8 + 6] = clock64();
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t parity = ((it / kStages) & 1u) ^ 1u;
          const long long w0 = clock64();
          const bool got = mbar_wait_timed(&empty_bar[s], parity, kWaitNs);
          waited += clock64() - w0;
          if (!got) {
            s_failed = 1;
            atomicExch(a.error_flag, 1u);
            break;
          }
          uint8_t* stage = tiles + static_cast<size_t>(s) * kStageBytes;
          if (kProfile && (a.debug_skip & 4)) {   // profiling aid: hand over the stage without loading it
            if (rank == 0) mbar_arrive(&full_bar[s]);
            continue;
          }
          if (rank == 0) mbar_expect_tx(&full_bar[s], kCtas * kStageBytes);
          const uint32_t full_s = full_leader + static_cast<uint32_t>(s) * 8u;
          if constexpr (kCtas == 2) {
            tma_load_2d_pair(stage, &a.map_a, kb * kBK, row0, full_s);
          } else {
            tma_load_2d(stage, &a.map_a, kb * kBK, row0, &full_bar[s]);
          }
          #pragma unroll
          for (int i = 0; i < kBBoxes; ++i) {
            if constexpr (kCtas == 2) {
              tma_load_2d_pair(stage + kABytes + i * kBBoxBytes, &a.map_b, kb * kBK, brow[i], full_s);
            } else {
              tma_load_2d(stage + kABytes + i * kBBoxBytes, &a.map_b, kb * kBK, brow[i], &full_bar[s]);
            }
          }
        }
        if (trace_row >= 0) a.trace[trace_row * 8 + 7] = clock64();
      }
      if (kProfile && a.wait_cycles != nullptr) a.wait_cycles[blockIdx.x * 4 + 0] = static_cast<unsigned long long>(waited);
    }
  } else if ((warp == 1 || warp == 2) && rank == 0) {
    // ------------------------------------------------------------------ MMA issuers
    // Two issuing threads, one per accumulator: warp 1 takes the even K blocks, warp 2 the odd
    // ones. One thread's loop (two mbarrier waits, four tcgen05.mma, two commits) takes longer
    // than the tensor cores need for a K block, so a single issuer leaves them idle half the
    // time; the two streams are independent (different accumulators, different stages).
    {
      // The whole warp runs the loop and one elected lane issues: descriptors and addresses then
      // stay in uniform registers, which is what tcgen05.mma takes, instead of being moved there
      // one by one in front of every instruction.
      constexpr uint32_t idesc = idesc_e4m3_f32(kCtas * kBM, kBN);
      const uint32_t w = warp - 1;
      const uint32_t my_tiles = pair < total_tiles ? (total_tiles - pair + num_pairs - 1) / num_pairs : 0;
      const uint32_t total_blocks = my_tiles * static_cast<uint32_t>(nkb);
      const bool timing = kProfile && a.wait_cycles != nullptr;
      const bool stamps = kProfile && a.trace != nullptr && blockIdx.x == 0 && w == 0 && lane == 0;
      const int reps = (kProfile && (a.debug_skip & 2)) ? 0 : ((kProfile && (a.debug_skip & 8)) ? 2 : 1);   // profiling aid
      const uint32_t d_tmem = tmem_base + w * kBN;
      long long waited_tmem = 0, waited_full = 0;
      for (uint32_t it = w; it < total_blocks; it += 2) {
        // one lane's reading for all: lanes that disagreed about leaving would split the warp
        // in front of the warp-wide votes below
        if (__shfl_sync(0xffffffffu, *reinterpret_cast<volatile uint32_t*>(&s_failed), 0) != 0) break;
        const int s = it % kStages;
        // Operands first: they are usually there already (the producer runs ahead), so that
        // nothing but the MMAs stands between getting the accumulator and using it.
        const long long w0 = timing ? clock64() : 0;
        const bool got_full = __all_sync(0xffffffffu, mbar_wait_timed(&full_bar[s], (it / kStages) & 1u, kWaitNs));
        const uint8_t* stage = tiles + static_cast<size_t>(s) * kStageBytes;
        const uint64_t a_desc = smem_desc_k_sw128(stage);
        const uint64_t b_desc = smem_desc_k_sw128(stage + kABytes);
        const long long w1 = (timing || stamps) ? clock64() : 0;
        if (stamps && it < kTraceBlocks) a.trace[kTraceBlockBase + it * 8 + 4] = w1;
        const bool got_tmem =
            got_full && __all_sync(0xffffffffu, mbar_wait_timed(&tmem_empty_bar[w], ((it >> 1) & 1u) ^ 1u, kWaitNs));
        if (timing) {
          waited_full += w1 - w0;
          waited_tmem += clock64() - w1;
        }
        if (!got_tmem || !got_full) {
          if (lane == 0) {
            s_failed = 1;
            atomicExch(a.error_flag, 2u);
          }
          break;
        }
        fence_after_thread_sync();
        if (stamps && it < kTraceBlocks) a.trace[kTraceBlockBase + it * 8 + 3] = clock64();
        if (elect_one()) {
          for (int rep = 0; rep < reps; ++rep) {
            #pragma unroll
            for (int k4 = 0; k4 < kBK / 32; ++k4) {
              // advancing 32 bytes along K inside the 128-byte swizzled row: +2 in 16-byte units
              if constexpr (kCtas == 2) {
                mma_f8f6f4_pair(d_tmem, a_desc + 2 * k4, b_desc + 2 * k4, idesc, k4 > 0 ? 1u : 0u);
              } else {
                mma_f8f6f4(d_tmem, a_desc + 2 * k4, b_desc + 2 * k4, idesc, k4 > 0 ? 1u : 0u);
              }
            }
          }
          // in both CTAs: the partial sums may be read once these MMAs are done, and the stage refilled
          if constexpr (kCtas == 2) {
            mma_commit_pair(&tmem_full_bar[w], 0x3);
            mma_commit_pair(&empty_bar[s], 0x3);
          } else {
            mma_commit(&tmem_full_bar[w]);
            mma_commit(&empty_bar[s]);
          }
        }
        __syncwarp();
        if (stamps && it < kTraceBlocks) a.trace[kTraceBlockBase + it * 8 + 0] = clock64();
      }
      if (timing && lane == 0) {   // the two issuers' waits are summed
        atomicAdd(&a.wait_cycles[blockIdx.x * 4 + 1], static_cast<unsigned long long>(waited_tmem));
        atomicAdd(&a.wait_cycles[blockIdx.x * 4 + 2], static_cast<unsigned long long>(waited_full));
      }
    }
  }
  } else {
    // ------------------------------------------------------------------ epilogue warps
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kEpilogueRegs) : "memory");
    const int q = warp & 3;                      // TMEM lane quarter this warp may read
    const int h = (warp - kFirstEpilogueWarp) >> 2;  // column half: 0 -> cols [0,128), 1 -> [128,256)
    const int row_in_tile = q * 32 + lane;
    uint8_t* const warp_stage = tiles + static_cast<size_t>(kStages) * kStageBytes + (warp - kFirstEpilogueWarp) * kWarpStageBytes;
    const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
    uint32_t acc_it = 0;
    uint32_t tile_parity = 0;
    long long waited_acc = 0;
    const int nkb_scale = a.K / 128;
    const int nb_per_expert = a.N / 128;
    // Where a tile's scales live for this thread: its row's a_scale and the two block rows of
    // b_scale its columns fall into (gate / up under SwiGLU; one block row otherwise).
    struct TileScales {
      const float* a_row;
      const float* b0;
      const float* b1;
    };
    auto tile_scales = [&](int e, int m_tile, int n_tile) {
      const int row = sched.row_start[e] + m_tile * kBM + row_in_tile;
      const bool valid = m_tile * kBM + row_in_tile < sched.count[e] && row < a.max_rows;
      const int nb0 = swiglu ? n_tile : n_tile * 2 + h;
      const int nb1 = swiglu ? I / 128 + n_tile : nb0;
      TileScales ts;
      ts.a_row = a.a_scale + static_cast<int64_t>(valid ? row : 0) * a.a_scale_stride_row;
      ts.b0 = a.b_scale + (static_cast<int64_t>(e) * nb_per_expert + nb0) * nkb_scale;
      ts.b1 = a.b_scale + (static_cast<int64_t>(e) * nb_per_expert + nb1) * nkb_scale;
      return ts;
    };
    // The first K block's scales of a tile are fetched one tile ahead: at a tile boundary they
    // would otherwise be a cold read in front of the first fold.
    float as_first = 0.f, b0_first = 0.f, b1_first = 0.f;
    int e = 0, e_ahead = 0;   // expert cursors of this tile and of the next one
    const uint32_t tmem_empty_leader = kCtas == 2 ? map_to_cta(&tmem_empty_bar[0], 0) : smem_u32(&tmem_empty_bar[0]);
    if (pair < total_tiles) {
      int m_ahead, n_ahead;
      decode_tile(sched, a.num_experts, n_tiles, pair, &e_ahead, &m_ahead, &n_ahead);
      const TileScales ts = tile_scales(e_ahead, kCtas * m_ahead + static_cast<int>(rank), n_ahead);
      as_first = ts.a_row[0];
      b0_first = ts.b0[0];
      b1_first = ts.b1[0];
    }
    for (int t = pair; t < total_tiles; t += num_pairs, tile_parity ^= 1u) {
      int m_pair, n_tile;
      const int trace_row = (kProfile && a.trace != nullptr && blockIdx.x == 0 && warp == kFirstEpilogueWarp && lane == 0 &&
                             t / num_pairs < 32) ? t / num_pairs : -1;
      if (trace_row >= 0) a.trace[trace_row * 8 + 0] = clock64();
      decode_tile(sched, a.num_experts, n_tiles, t, &e, &m_pair, &n_tile);
      const int m_tile = kCtas * m_pair + static_cast<int>(rank);   // this CTA's 128 rows of the tile
      const int row = sched.row_start[e] + m_tile * kBM + row_in_tile;
      const bool valid = m_tile * kBM + row_in_tile < sched.count[e] && row < a.max_rows;
      const TileScales cur = tile_scales(e, m_tile, n_tile);
      const float* a_scale_row = cur.a_row;
      const float* bs0 = cur.b0;
      const float* bs1 = cur.b1;
      float as_next = as_first, b0_next = b0_first, b1_next = b1_first;
      if (t + num_pairs < total_tiles) {
        int m_ahead, n_ahead;
        decode_tile(sched, a.num_experts, n_tiles, t + num_pairs, &e_ahead, &m_ahead, &n_ahead);
        const TileScales nx = tile_scales(e_ahead, kCtas * m_ahead + static_cast<int>(rank), n_ahead);
        as_first = nx.a_row[0];
        b0_first = nx.b0[0];
        b1_first = nx.b1[0];
      }

      float acc[128];
      #pragma unroll
      for (int i = 0; i < 128; ++i) acc[i] = 0.f;
      bool failed = false;
      for (int kb = 0; kb < nkb; ++kb, ++acc_it) {
        const int buf = acc_it & 1;
        const float as = as_next, b0 = b0_next, b1 = b1_next;
        if (kb + 1 < nkb) {
          as_next = a_scale_row[(kb + 1) * a.a_scale_stride_k];
          b0_next = bs0[kb + 1];
          b1_next = bs1[kb + 1];
        }
        // thread columns [0,64) belong to block row nb0 and [64,128) to nb1 (gate / up under
        // SwiGLU; the same block row twice otherwise)
        const float sc0 = as * b0, sc1 = as * b1;
        // the outcome must be the same for the whole warp: tcgen05.ld below is warp-collective
        const long long w0 = clock64();
        const bool got = mbar_wait_timed(&tmem_full_bar[buf], (acc_it >> 1) & 1u, kWaitNs);
        waited_acc += clock64() - w0;
        if (!__all_sync(0xffffffffu, got)) {
          failed = true;
          break;
        }
        fence_after_thread_sync();
        if (kb == 0 && trace_row >= 0) a.trace[trace_row * 8 + 1] = clock64();
        const bool trace_block = trace_row >= 0 && acc_it < kTraceBlocks;
        if (trace_block) a.trace[kTraceBlockBase + acc_it * 8 + 1] = clock64();
        if (kProfile && (a.debug_skip & 1)) {   // profiling aid: leave the partial sums unread
          fence_before_thread_sync();
          __syncwarp();
          if (lane == 0) {
            if constexpr (kCtas == 2) {
              mbar_arrive_cluster(tmem_empty_leader + static_cast<uint32_t>(buf) * 8u);
            } else {
              mbar_arrive(&tmem_empty_bar[buf]);
            }
          }
          if (trace_block) a.trace[kTraceBlockBase + acc_it * 8 + 2] = clock64();
          continue;
        }
        const uint32_t taddr = tmem_base + lane_addr + static_cast<uint32_t>(buf) * kBN + static_cast<uint32_t>(h) * 128;
        // Four chunks of 32 columns, software-pipelined. A warp's tensor-memory loads do not
        // overlap one another (a 32-column load takes about 90 cycles however many are in
        // flight), but they do overlap its FMAs: the load of chunk c+1 runs while chunk c is folded.
        uint32_t ta[32], tb[32];
        tmem_ld32(taddr, ta);
        tmem_ld_wait();
        tmem_ld32(taddr + 32, tb);
        #pragma unroll
        for (int i = 0; i < 32; ++i) acc[i] = fmaf(sc0, __uint_as_float(ta[i]), acc[i]);
        tmem_ld_wait();
        tmem_ld32(taddr + 64, ta);
        #pragma unroll
        for (int i = 0; i < 32; ++i) acc[32 + i] = fmaf(sc0, __uint_as_float(tb[i]), acc[32 + i]);
        tmem_ld_wait();
        tmem_ld32(taddr + 96, tb);
        #pragma unroll
        for (int i = 0; i < 32; ++i) acc[64 + i] = fmaf(sc1, __uint_as_float(ta[i]), acc[64 + i]);
        tmem_ld_wait();
        // everything this warp needs from the buffer is in registers: hand it back
        fence_before_thread_sync();
        __syncwarp();
        if (lane == 0) {
            if constexpr (kCtas == 2) {
              mbar_arrive_cluster(tmem_empty_leader + static_cast<uint32_t>(buf) * 8u);
            } else {
              mbar_arrive(&tmem_empty_bar[buf]);
            }
          }
        if (trace_block) a.trace[kTraceBlockBase + acc_it * 8 + 2] = clock64();
        #pragma unroll
        for (int i = 0; i < 32; ++i) acc[96 + i] = fmaf(sc1, __uint_as_float(tb[i]), acc[96 + i]);
      }
      if (failed) {
        atomicExch(a.error_flag, 3u);
        s_failed = 1;
      }
      if (trace_row >= 0) a.trace[trace_row * 8 + 2] = clock64();

      // Rows of this warp that may be written, and the address of its first row.
      const uint32_t valid_mask = __ballot_sync(0xffffffffu, valid && !failed);
      const int64_t warp_row0 = static_cast<int64_t>(sched.row_start[e] + m_tile * kBM + q * 32);
      if (swiglu) {
        // out[c] = silu(gate[c]) * up[c] for this thread's 64 columns
        float amax = 0.f;
        #pragma unroll
        for (int i = 0; i < 64; ++i) {
          const float g = acc[i];
          const float v = __fdividef(g, 1.f + __expf(-g)) * acc[64 + i];
          acc[i] = v;
          amax = fmaxf(amax, fabsf(v));
        }
        s_amax[tile_parity][row_in_tile][h] = amax;
        // Every epilogue thread gets here, also after a failed wait, and all of them leave with
        // the same outcome: a warp that went on alone would wait at this barrier for ever.
        const bool any_failed = bar_red_or(1, kEpilogueThreads, failed || s_failed != 0);
        amax = fmaxf(s_amax[tile_parity][row_in_tile][0], s_amax[tile_parity][row_in_tile][1]);
        const float scale = fmaxf(amax, 1e-10f) * (1.0f / 448.0f);
        const float inv = 1.0f / scale;
        uint32_t w[16];
        #pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int i = j * 4;
          const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(acc[i] * inv, acc[i + 1] * inv), __NV_SATFINITE, __NV_E4M3);
          const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(acc[i + 2] * inv, acc[i + 3] * inv), __NV_SATFINITE, __NV_E4M3);
          w[j] = lo | (hi << 16);
        }
        store_rows_64B(warp_stage, lane, w, a.out + warp_row0 * a.out_stride + n_tile * 128 + h * 64, a.out_stride,
                       any_failed ? 0u : valid_mask);
        if (h == 0 && valid && !any_failed) a.out_scale[static_cast<int64_t>(row) * a.out_scale_stride_row + n_tile] = scale;
        failed = any_failed;
      } else if (a.mode == kBf16Scatter) {
        // this lane's row: which GPU its token came from and which slot of that GPU's combine
        // receive buffer it fills
        uint8_t* row_ptr = nullptr;
        if (valid && !failed) {
          const uint32_t src = a.scatter.row_src[row];
          if (src < static_cast<uint32_t>(a.scatter.world)) {
            row_ptr = a.scatter.peer_recv[src] + static_cast<uint64_t>(a.scatter.row_tk[row]) * a.scatter.slot_stride;
          }
        }
        const uint32_t col0 = static_cast<uint32_t>(n_tile * kBN + h * 128) * 2u;
        const unsigned long long mine = reinterpret_cast<unsigned long long>(row_ptr);
        if constexpr (kCtas == 1) {
          // the lone-CTA kernel stages 64-byte chunks (its stages leave no room for more)
          #pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t w[16];
            #pragma unroll
            for (int j = 0; j < 16; ++j) {
              const __nv_bfloat162 p2 = __floats2bfloat162_rn(acc[c * 32 + 2 * j], acc[c * 32 + 2 * j + 1]);
              w[j] = *reinterpret_cast<const uint32_t*>(&p2);
            }
            store_rows_64B_fn(warp_stage, lane, w, true, [&](int r) {
              uint8_t* const base = reinterpret_cast<uint8_t*>(__shfl_sync(0xffffffffu, mine, r));
              return base == nullptr ? base : base + col0 + c * 64;
            });
          }
        } else {
        #pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t w[32];
          #pragma unroll
          for (int j = 0; j < 32; ++j) {
            const __nv_bfloat162 p2 = __floats2bfloat162_rn(acc[c * 64 + 2 * j], acc[c * 64 + 2 * j + 1]);
            w[j] = *reinterpret_cast<const uint32_t*>(&p2);
          }
          if (a.scatter.bulk) {
            // Each lane stages its own row's 128 bytes and hands them to the bulk-copy engine; the
            // warp goes on while the bytes cross NVLink. The staging buffer is reused as soon as the
            // engine has read it (wait_group.read), not when the peer has the data.
            bulk_wait_read0();
            __syncwarp();
            #pragma unroll
            for (int u = 0; u < 8; ++u) {
              *reinterpret_cast<uint4*>(warp_stage + lane * kBulkRowStride + u * 16) =
                  make_uint4(w[4 * u], w[4 * u + 1], w[4 * u + 2], w[4 * u + 3]);
            }
            fence_proxy_async_smem();
            if (row_ptr != nullptr) bulk_s2g(row_ptr + col0 + c * 128, warp_stage + lane * kBulkRowStride, 128);
            bulk_commit();
          } else {
            store_rows_128B(warp_stage, lane, w, true, [&](int r) {
              uint8_t* const base = reinterpret_cast<uint8_t*>(__shfl_sync(0xffffffffu, mine, r));
              return base == nullptr ? base : base + col0 + c * 128;
            });
          }
        }
        }
      } else {
        uint8_t* dst = a.out + warp_row0 * a.out_stride + (static_cast<int64_t>(n_tile) * kBN + h * 128) * 2;
        if constexpr (kCtas == 1) {
          #pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t w[16];
            #pragma unroll
            for (int j = 0; j < 16; ++j) {
              const __nv_bfloat162 p2 = __floats2bfloat162_rn(acc[c * 32 + 2 * j], acc[c * 32 + 2 * j + 1]);
              w[j] = *reinterpret_cast<const uint32_t*>(&p2);
            }
            store_rows_64B_fn(warp_stage, lane, w, false, [&](int r) {
              return ((valid_mask >> r) & 1u) ? dst + r * a.out_stride + c * 64 : static_cast<uint8_t*>(nullptr);
            });
          }
        } else {
        #pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t w[32];
          #pragma unroll
          for (int j = 0; j < 32; ++j) {
            const __nv_bfloat162 p2 = __floats2bfloat162_rn(acc[c * 64 + 2 * j], acc[c * 64 + 2 * j + 1]);
            w[j] = *reinterpret_cast<const uint32_t*>(&p2);
          }
          store_rows_128B(warp_stage, lane, w, false, [&](int r) {
            return ((valid_mask >> r) & 1u) ? dst + r * a.out_stride + c * 128 : static_cast<uint8_t*>(nullptr);
          });
        }
        }
      }
      if (trace_row >= 0) a.trace[trace_row * 8 + 3] = clock64();
      if (failed) break;
    }
    if (kProfile && a.wait_cycles != nullptr && warp == kFirstEpilogueWarp && lane == 0) {
      a.wait_cycles[blockIdx.x * 4 + 3] = static_cast<unsigned long long>(waited_acc);
    }
    // bulk copies this thread handed over must have been performed before the arrival signal
    if (kCtas == 2 && a.mode == kBf16Scatter && a.scatter.bulk) bulk_wait0();
  }

  // Neither CTA may leave, or give its tensor memory back, while the other can still signal its
  // barriers or write its accumulators.
  fence_before_thread_sync();
  if constexpr (kCtas == 2) {
    cluster_sync_all();
  } else {
    __syncthreads();
  }
  if (a.mode == kBf16Scatter && threadIdx.x == 0) {
    // The last CTA to get here tells every GPU that this rank's rows have been written. Each CTA's
    // stores are ordered before its increment (system fence after the barrier above), the last
    // CTA's increment reads all the others' (acq_rel), and its release covers what it has seen.
    fence_acq_rel_sys();
    const uint32_t before = atom_acq_rel_gpu_add(a.scatter.done_counter, 1u);
    if (before == gridDim.x - 1) {
      *a.scatter.done_counter = 0;   // ready for the next launch
      const bool healthy = *a.scatter.status == 0 && s_failed == 0 && *a.error_flag == 0;
      if (healthy) {
        fence_acq_rel_sys();
        for (int p = 0; p < a.scatter.world; ++p) red_release_sys_add(a.scatter.peer_flag[p], a.scatter.signal_value);
      }
    }
  }
  if (kProfile && a.trace != nullptr && blockIdx.x == 0 && threadIdx.x == 0) {
    a.trace[(kTraceTiles - 1) * 8 + 2] = clock64();
    a.trace[(kTraceTiles - 1) * 8 + 3] = static_cast<long long>(globaltimer_ns());
  }
  if (warp == 1) {
    fence_after_thread_sync();
    if constexpr (kCtas == 2) {
      tmem_dealloc_pair(tmem_base, kTmemCols);
    } else {
      tmem_dealloc(tmem_base, kTmemCols);
    }
  }
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
    grouped_fp8_gemm_kernel(const __grid_constant__ KernelArgs a) {
  grouped_fp8_gemm_body<2>(a);
}

// One CTA per 128-row tile: for experts with so few rows that the second CTA of a pair would idle.
__global__ void __launch_bounds__(kThreads, 1) grouped_fp8_gemm_kernel_1cta(const __grid_constant__ KernelArgs a) {
  grouped_fp8_gemm_body<1>(a);
}

CUtensorMap make_map(const void* base, uint64_t rows, uint64_t cols_bytes, uint64_t row_stride_bytes,
                     uint32_t box_rows) {
  const CuDriver& cu = CuDriver::get();
  PPLX_REQUIRE(cu.cuTensorMapEncodeTiled != nullptr, "this CUDA driver has no cuTensorMapEncodeTiled");
  CUtensorMap map;
  const cuuint64_t dims[2] = {cols_bytes, rows};
  const cuuint64_t strides[1] = {row_stride_bytes};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(kBK), box_rows};
  const cuuint32_t elem_strides[2] = {1, 1};
  PPLX_CU_CHECK(cu.cuTensorMapEncodeTiled(&map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims,
                                          strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE));
  return map;
}

}  // namespace

void PPLX_GEMM_ENTRY(const GroupedGemmParams& p, cudaStream_t stream) {
  PPLX_REQUIRE(p.K % kBK == 0 && p.K >= kBK, "K must be a multiple of 128");
  PPLX_REQUIRE(p.num_experts >= 1 && p.num_experts <= kMaxExperts, "between 1 and 128 local experts");
  PPLX_REQUIRE(p.expert_padding >= 1, "expert_padding must be positive");
  if (p.mode == kSwiGLUQuant) {
    PPLX_REQUIRE(p.N % 256 == 0, "SwiGLU needs N = 2 * intermediate with intermediate a multiple of 128");
    PPLX_REQUIRE(p.out_scale != nullptr, "the SwiGLU epilogue writes scales");
  } else {
    PPLX_REQUIRE(p.N % kBN == 0, "N must be a multiple of 256");
  }
  if (p.mode == kBf16Scatter) {
    const CombineScatter& sc = p.scatter;
    PPLX_REQUIRE(sc.row_src != nullptr && sc.row_tk != nullptr && sc.done_counter != nullptr && sc.status != nullptr &&
                     sc.world >= 1 && sc.world <= CombineScatter::kMaxPeers,
                 "kBf16Scatter needs the combine scatter description");
    PPLX_REQUIRE(sc.slot_stride % 16 == 0 && sc.slot_stride >= static_cast<uint64_t>(p.N) * 2,
                 "combine slots must hold a bf16 row and be 16-byte aligned");
    for (int i = 0; i < sc.world; ++i) {
      PPLX_REQUIRE(sc.peer_recv[i] != nullptr && reinterpret_cast<uintptr_t>(sc.peer_recv[i]) % 16 == 0 &&
                       sc.peer_flag[i] != nullptr,
                   "kBf16Scatter: missing peer pointer");
    }
    PPLX_REQUIRE(p.error_flag != nullptr, "kBf16Scatter needs an error flag");
  }
  PPLX_REQUIRE(reinterpret_cast<uintptr_t>(p.a) % 16 == 0 && reinterpret_cast<uintptr_t>(p.b) % 16 == 0 &&
                   p.a_stride % 16 == 0 && reinterpret_cast<uintptr_t>(p.out) % 16 == 0 && p.out_stride % 16 == 0,
               "operands must be 16-byte aligned");
  KernelArgs a{};
  a.map_a = make_map(p.a, static_cast<uint64_t>(p.max_rows), static_cast<uint64_t>(p.K),
                     static_cast<uint64_t>(p.a_stride), kBM);
  a.map_b = make_map(p.b, static_cast<uint64_t>(p.num_experts) * p.N, static_cast<uint64_t>(p.K),
                     static_cast<uint64_t>(p.K), 64);
  a.a_scale = p.a_scale;
  a.a_scale_stride_row = p.a_scale_stride_row;
  a.a_scale_stride_k = p.a_scale_stride_k;
  a.b_scale = p.b_scale;
  a.expert_num_tokens = p.expert_num_tokens;
  a.out = static_cast<uint8_t*>(p.out);
  a.out_stride = p.out_stride;
  a.out_scale = p.out_scale;
  a.out_scale_stride_row = p.out_scale_stride_row;
  a.error_flag = p.error_flag;
  a.wait_cycles = p.wait_cycles;
  a.trace = p.trace;
  a.num_experts = p.num_experts;
  a.N = p.N;
  a.K = p.K;
  a.expert_padding = p.expert_padding;
  a.max_rows = p.max_rows;
  a.mode = p.mode;
  a.scatter = p.scatter;
  a.debug_skip = p.debug_skip;

  int device = 0, sms = 0;
  PPLX_CUDA_CHECK(cudaGetDevice(&device));
  PPLX_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
  // Pairs of CTAs on 256-row tiles unless the experts are small: with no more than 192 rows per
  // expert on average (by capacity; the counts themselves stay on the device) the second CTA of a
  // pair would mostly idle, and single CTAs on 128-row tiles do the same work with half the waste.
  const bool wants_pairs = p.mode == kBf16Scatter && p.scatter.bulk;   // the bulk-copy sender stages 128-byte rows
  const int tile_rows =
      p.tile_rows != 0 ? p.tile_rows : ((wants_pairs || p.max_rows / p.num_experts > 192) ? 256 : 128);
  PPLX_REQUIRE(tile_rows == 128 || tile_rows == 256, "tile_rows must be 0 (automatic), 128 or 256");
  const int ctas = p.num_ctas > 0 ? p.num_ctas : sms;
  if (tile_rows == 256) {
    const size_t smem = static_cast<size_t>(kStages) * kStageBytesOf<2> + (kEpilogueThreads / 32) * kWarpStageBytesOf<2> + 1024;
    PPLX_CUDA_CHECK(cudaFuncSetAttribute(grouped_fp8_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem)));
    const int grid = std::max(2, ctas & ~1);   // whole CTA pairs
    grouped_fp8_gemm_kernel<<<grid, kThreads, smem, stream>>>(a);
  } else {
    PPLX_REQUIRE(!(p.mode == kBf16Scatter && p.scatter.bulk), "the bulk-copy sender needs 256-row tiles");
    const size_t smem = static_cast<size_t>(kStages) * kStageBytesOf<1> + (kEpilogueThreads / 32) * kWarpStageBytesOf<1> + 1024;
    PPLX_CUDA_CHECK(cudaFuncSetAttribute(grouped_fp8_gemm_kernel_1cta, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem)));
    grouped_fp8_gemm_kernel_1cta<<<std::max(1, ctas), kThreads, smem, stream>>>(a);
  }
  PPLX_CUDA_CHECK(cudaGetLastError());
}

}  // namespace pplx::ops
