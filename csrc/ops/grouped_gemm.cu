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

#include "grouped_gemm_common.cuh"

namespace pplx::ops {
namespace {

using namespace pplx::ops::gemm_detail;

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
  if (warp == 0) build_schedule<kCtas>(a, sched, n_tiles, lane);
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
      // rows past the count read their own (clamped) row's scales: one shared fallback row would be a hot line in L2
      ts.a_row = a.a_scale + static_cast<int64_t>(min(row, a.max_rows - 1)) * a.a_scale_stride_row;
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

      tile_epilogue<kCtas, false>(a, sched, acc, failed, valid, row, e, m_tile, n_tile, q, h, lane, row_in_tile, tile_parity,
                                  warp_stage, swiglu, s_amax, s_failed);
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
  if (a.mode == kBf16Scatter && threadIdx.x == 0) scatter_signal(a, s_failed);
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

}  // namespace

void PPLX_GEMM_ENTRY(const GroupedGemmParams& p, cudaStream_t stream) {
#ifndef PPLX_GEMM_PROFILE
  if (p.scale_format == kScalesPow2) {
    grouped_fp8_gemm_mx(p, stream);
    return;
  }
#endif
  PPLX_REQUIRE(p.scale_format == kScalesFp32, "the profiled kernel takes fp32 scales only");
  const KernelArgs a = prepare_kernel_args(p);

  int device = 0, sms = 0;
  PPLX_CUDA_CHECK(cudaGetDevice(&device));
  PPLX_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
  // Pairs of CTAs on 256-row tiles unless the experts are small: with no more than 192 rows per
  // expert on average (by capacity; the counts themselves stay on the device) the second CTA of a
  // pair would mostly idle, and single CTAs on 128-row tiles do the same work with half the waste.
  const int tile_rows = choose_tile_rows(p);
  const int ctas = p.num_ctas > 0 ? p.num_ctas : sms;
  if (tile_rows == 256) {
    const size_t smem = static_cast<size_t>(kStages) * kStageBytesOf<2> + (kEpilogueThreads / 32) * kWarpStageBytesOf<2> + 1024;
    PPLX_CUDA_CHECK(cudaFuncSetAttribute(grouped_fp8_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem)));
    const int grid = std::max(2, ctas & ~1);   // whole CTA pairs
    grouped_fp8_gemm_kernel<<<grid, kThreads, smem, stream>>>(a);
  } else {
    const size_t smem = static_cast<size_t>(kStages) * kStageBytesOf<1> + (kEpilogueThreads / 32) * kWarpStageBytesOf<1> + 1024;
    PPLX_CUDA_CHECK(cudaFuncSetAttribute(grouped_fp8_gemm_kernel_1cta, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem)));
    grouped_fp8_gemm_kernel_1cta<<<std::max(1, ctas), kThreads, smem, stream>>>(a);
  }
  PPLX_CUDA_CHECK(cudaGetLastError());
}

}  // namespace pplx::ops
