// Grouped fp8 GEMM with power-of-two block scales applied by the tensor cores.
//
// Same problem, tiles and epilogues as grouped_gemm.cu (per expert D = dequant(A) dequant(B[e])^T,
// A e4m3 with 1x128 scales, B e4m3 with 128x128 block scales; SwiGLU + re-quantise, bf16, or bf16
// scattered into the peers' combine buffers), for callers whose scales are powers of two. The
// MMA is tcgen05.mma kind::mxf8f6f4.block_scale: each K = 32 instruction multiplies A's rows and
// B's rows by a UE8M0 scale read from tensor memory, so the 128-wide scale blocks are applied
// inside the tensor core and the sum over the whole of K stays in one tensor-memory accumulator.
// The epilogue warps no longer read and fold partial sums once per K block (which is what holds
// grouped_gemm.cu at about half of the tensor cores' rate); they read the accumulator once per tile.
//
// Roles, per CTA (one persistent CTA per SM, twelve warps, pairs of CTAs on 256-row tiles or
// lone CTAs on 128-row tiles as in grouped_gemm.cu):
//   warp 0      TMA producer: A rows and B rows of a K block into a ring of stages
//   warp 1      (leader CTA) MMA issuer: every fourth K block it copies a group of scale words
//               from shared to tensor memory (tcgen05.cp 32x128b.warpx4), then four MMAs per
//               K block whose descriptor picks the K block's byte of the scale words
//   warp 3      scale warp: fetches four K blocks' fp32 scales of this CTA's 128 rows of A and of
//               the tile's rows of B (cp.async, six groups in flight), keeps the exponent bytes and
//               writes them to shared memory in the order tcgen05.cp wants (row r of a 128-row
//               block at byte 16 (r % 32) + 4 (r / 32), the four K blocks in the four bytes of the word)
//   warps 4-11  epilogue: when the tile's last MMA has completed they copy the accumulator into
//               registers (128 columns per thread), hand tensor memory back and finish the tile
//               (SwiGLU, quantise, stores) while the tensor cores work on the next one
// Tensor memory: columns [0, 256) the accumulator, [256, 260) A's scale words, [260, 268) B's.
// The scale words in tensor memory are single-buffered: tcgen05.cp and tcgen05.mma of one thread
// execute in issue order, so a copy cannot overtake the MMAs that still read the previous group.
// Optional `trace` (int64 [64][8]): SM clock of CTA 0 per tile: 0 the MMA issuer got the accumulator,
// 5 it has issued the first K block, 1 the last; 6 the first epilogue warp starts waiting, 2 sees
// the sums, 3 has them in registers, 4 has stored the tile; 7 the issuer's waits of the tile, for
// operands in the low word and for scale words in the high word.
// No TMA multicast anywhere. Every wait is bounded and sets error_flag (1 producer, 2 MMA issuer,
// 3 epilogue, 4 scale warp).
//
// The reference has no GEMM (its "expert" is x * 2: tests/p2p_all_to_all/test_p2p_all_to_all.py:44-50).

#include "grouped_gemm.h"

#include "grouped_gemm_common.cuh"

namespace pplx::ops {
namespace {

using namespace pplx::ops::gemm_detail;

// A single issuer consumes the stages in order, so any count works; what fits beside the
// epilogue's staging buffers: five 32 KiB stages for pairs, four 48 KiB stages for lone CTAs.
template <int kCtas> constexpr int kMxStagesOf = kCtas == 2 ? 5 : 4;
template <int kCtas> constexpr int kSfSlotsOf = kCtas == 2 ? 4 : 3;   // groups of four K blocks the scale warp may run ahead
constexpr uint32_t kSfaBytes = 512;         // 128 rows x one word
constexpr uint32_t kSfbBytes = 1024;        // 256 rows of B x one word
constexpr uint32_t kSfSlotBytes = kSfaBytes + kSfbBytes;
constexpr uint32_t kSfaCol = 256, kSfbCol = 260;
constexpr int kScaleWarp = 3;
// The scale warp's landing area for raw fp32 scales: per group of four K blocks 128 rows x 4 of
// A's scales and 2 x 4 of B's; kRawAhead groups are in flight at any time.
// (six for pairs; three for lone CTAs, whose larger stages leave less room).
template <int kCtas> constexpr int kRawSlotsOf = kCtas == 2 ? 8 : 4;
template <int kCtas> constexpr int kRawAheadOf = kCtas == 2 ? 6 : 3;
constexpr uint32_t kRawSlotBytes = 2048 + 64;
static_assert(kRawSlotsOf<1> > kRawAheadOf<1> && kRawSlotsOf<2> > kRawAheadOf<2>,
              "a landing slot is refilled only after it has been packed");
constexpr int kMxLightRegs = 56;
static_assert(kFirstEpilogueWarp * 32 * kMxLightRegs + kEpilogueThreads * kEpilogueRegs <= kThreads * kLaunchRegs,
              "the epilogue's setmaxnreg.inc could never be granted");

template <int kCtas>
constexpr size_t mx_smem_bytes() {
  return static_cast<size_t>(kMxStagesOf<kCtas>) * kStageBytesOf<kCtas> + (kEpilogueThreads / 32) * kWarpStageBytesOf<kCtas> +
         kSfSlotsOf<kCtas> * kSfSlotBytes + kRawSlotsOf<kCtas> * kRawSlotBytes + 1024;
}
// 227 KiB per CTA, of which the kernel's static variables (schedule, row maxima, barriers) take 4 KiB
constexpr size_t kStaticSmemBytes = 4096;
static_assert(mx_smem_bytes<2>() + kStaticSmemBytes <= 227 * 1024 && mx_smem_bytes<1>() + kStaticSmemBytes <= 227 * 1024,
              "shared memory per CTA");

// Asynchronous global -> shared copies of one thread (4 or 16 bytes, both addresses aligned to the size).
__device__ __forceinline__ void cp_async_4(void* smem_dst, const void* gmem_src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" : : "r"(smem_u32(smem_dst)), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gmem_src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" : : "r"(smem_u32(smem_dst)), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int kPending>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" : : "n"(kPending) : "memory");
}

template <int kCtas>
__device__ __forceinline__ void grouped_fp8_gemm_mx_body(const KernelArgs& a) {
  constexpr int kStagesMx = kMxStagesOf<kCtas>;
  constexpr int kSfSlots = kSfSlotsOf<kCtas>;
  constexpr uint32_t kStageBytes = kStageBytesOf<kCtas>;
  constexpr int kBBoxes = kBBoxesOf<kCtas>;
  constexpr uint32_t kWarpStageBytes = kWarpStageBytesOf<kCtas>;
  extern __shared__ __align__(1024) uint8_t smem[];
  __shared__ uint64_t full_bar[kStagesMx], empty_bar[kStagesMx], sf_full_bar[kSfSlots], sf_empty_bar[kSfSlots];
  __shared__ uint64_t tmem_full_bar, tmem_empty_bar;
  __shared__ uint32_t tmem_base_slot;
  __shared__ Schedule sched;
  __shared__ float s_amax[2][kBM][2];
  __shared__ uint32_t s_failed;

  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);
  const int lane = threadIdx.x & 31;
  const bool swiglu = a.mode == kSwiGLUQuant;
  const int I = a.N / 2;
  const int n_tiles = swiglu ? I / 128 : a.N / kBN;
  const int nkb = a.K / kBK;
  const uint32_t rank = kCtas == 2 ? cluster_ctarank() : 0u;
  const int pair = blockIdx.x / kCtas;
  const int num_pairs = gridDim.x / kCtas;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStagesMx; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int s = 0; s < kSfSlots; ++s) {
      mbar_init(&sf_full_bar[s], kCtas);    // one arrival per CTA's scale warp (the leader's copy is used)
      mbar_init(&sf_empty_bar[s], 1);
    }
    mbar_init(&tmem_full_bar, 1);
    mbar_init(&tmem_empty_bar, kCtas * kEpilogueThreads / 32);   // the epilogue warps of every CTA of the tile (the leader's copy is used)
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
  uint8_t* const tiles = smem + ((1024u - (smem_u32(smem) & 1023u)) & 1023u);
  uint8_t* const warp_stages = tiles + static_cast<size_t>(kStagesMx) * kStageBytes;
  uint8_t* const sf_slots = warp_stages + (kEpilogueThreads / 32) * kWarpStageBytes;
  uint8_t* const raw_slots = sf_slots + kSfSlots * kSfSlotBytes;

  if (warp < kFirstEpilogueWarp) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kMxLightRegs) : "memory");
    if (warp == 0) {
      // ------------------------------------------------------------------ TMA producer
      if (lane == 0) {
        uint32_t it = 0;
        int e = 0;
        const uint32_t full_leader = kCtas == 2 ? map_to_cta(&full_bar[0], 0) : smem_u32(&full_bar[0]);
        for (int t = pair; t < total_tiles && !s_failed; t += num_pairs) {
          int m_pair, n_tile;
          decode_tile(sched, a.num_experts, n_tiles, t, &e, &m_pair, &n_tile);
          const int row0 = sched.row_start[e] + (kCtas * m_pair + static_cast<int>(rank)) * kBM;
          // This CTA's rows of B: accumulator columns [128 rank, 128 rank + 128) for a pair, all 256
          // for a lone CTA. SwiGLU interleaves gate and up in 64-row boxes so that a thread's
          // columns hold both.
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
          for (int kb = 0; kb < nkb; ++kb, ++it) {
            const int s = it % kStagesMx;
            const uint32_t parity = ((it / kStagesMx) & 1u) ^ 1u;
            if (!mbar_wait_timed(&empty_bar[s], parity, kWaitNs)) {
              s_failed = 1;
              atomicExch(a.error_flag, 1u);
              break;
            }
            uint8_t* stage = tiles + static_cast<size_t>(s) * kStageBytes;
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
        }
      }
    } else if (warp == 1 && rank == 0) {
      // ------------------------------------------------------------------ MMA issuer
      // The whole warp runs the loop and one elected lane issues, so that descriptors and
      // addresses stay in uniform registers.
      const uint32_t d_tmem = tmem_base;
      const uint32_t sfa_tmem = tmem_base + kSfaCol;
      const uint32_t sfb_tmem = tmem_base + kSfbCol;
      uint32_t it = 0, sf_it = 0, tile_i = 0;
      bool ok = true;
      for (int t = pair; t < total_tiles && ok; t += num_pairs, ++tile_i) {
        const bool stamp = a.trace != nullptr && blockIdx.x == 0 && lane == 0 && tile_i < kTraceTiles;
        long long waited_full = 0, waited_sf = 0;
        for (int kb = 0; kb < nkb && ok; ++kb, ++it) {
          if (__shfl_sync(0xffffffffu, *reinterpret_cast<volatile uint32_t*>(&s_failed), 0) != 0) {
            ok = false;
            break;
          }
          const int s = it % kStagesMx;
          const uint32_t sub = static_cast<uint32_t>(kb) & 3u;   // which byte of the scale words
          const bool last_of_group = sub == 3u || kb == nkb - 1;
          const uint32_t slot = sf_it % kSfSlots;
          const long long w0 = stamp ? clock64() : 0;
          ok = __all_sync(0xffffffffu, mbar_wait_timed(&full_bar[s], (it / kStagesMx) & 1u, kWaitNs));
          const long long w1 = stamp ? clock64() : 0;
          if (ok && sub == 0u) {
            ok = __all_sync(0xffffffffu,
                            mbar_wait_timed_acquire_cluster(&sf_full_bar[slot], (sf_it / kSfSlots) & 1u, kWaitNs));
          }
          if (stamp) {   // low word: cycles spent waiting for operands, high word: for scale words
            waited_full += w1 - w0;
            waited_sf += clock64() - w1;
          }
          if (!ok) break;
          fence_after_thread_sync();
          const uint8_t* stage = tiles + static_cast<size_t>(s) * kStageBytes;
          const uint64_t a_desc = smem_desc_k_sw128(stage);
          const uint64_t b_desc = smem_desc_k_sw128(stage + kABytes);
          const uint8_t* sf = sf_slots + slot * kSfSlotBytes;
          if (sub == 0u && elect_one()) {
            tmem_cp_sf<kCtas>(sfa_tmem, smem_desc_sf(sf));
            tmem_cp_sf<kCtas>(sfb_tmem, smem_desc_sf(sf + kSfaBytes));
            tmem_cp_sf<kCtas>(sfb_tmem + 4, smem_desc_sf(sf + kSfaBytes + 512));
          }
          if (kb == 0) {
            // Only now the accumulator: the previous tile's sums must have been read out before the
            // first MMA overwrites them, but the operands, the scale words and their copy into
            // tensor memory do not have to wait for that.
            ok = __all_sync(0xffffffffu, mbar_wait_timed(&tmem_empty_bar, (tile_i & 1u) ^ 1u, kWaitNs));
            if (!ok) break;
            fence_after_thread_sync();
            if (stamp) a.trace[tile_i * 8 + 0] = clock64();
          }
          if (elect_one()) {
            const uint32_t idesc = idesc_mx_e4m3_ue8m0(kCtas * kBM, kBN, sub);
            // the byte index also rides in the top two bits of the scale addresses
            const uint32_t sfa = sfa_tmem | (sub << 30), sfb = sfb_tmem | (sub << 30);
            #pragma unroll
            for (int k4 = 0; k4 < kBK / 32; ++k4) {
              // advancing 32 bytes along K inside the 128-byte swizzled row: +2 in 16-byte units
              mma_mxf8<kCtas>(d_tmem, a_desc + 2 * k4, b_desc + 2 * k4, idesc, sfa, sfb, (kb > 0 || k4 > 0) ? 1u : 0u);
            }
            // in both CTAs: the stage may be refilled; the scale slot too once its last K block is
            // through (the commit also covers the copies into tensor memory); the sums may be read
            if constexpr (kCtas == 2) {
              mma_commit_pair(&empty_bar[s], 0x3);
              if (last_of_group) mma_commit_pair(&sf_empty_bar[slot], 0x3);
              if (kb == nkb - 1) mma_commit_pair(&tmem_full_bar, 0x3);
            } else {
              mma_commit(&empty_bar[s]);
              if (last_of_group) mma_commit(&sf_empty_bar[slot]);
              if (kb == nkb - 1) mma_commit(&tmem_full_bar);
            }
          }
          __syncwarp();
          if (last_of_group) ++sf_it;
          if (stamp && kb == 0) a.trace[tile_i * 8 + 5] = clock64();
        }
        if (stamp) {
          a.trace[tile_i * 8 + 1] = clock64();
          a.trace[tile_i * 8 + 7] = (waited_sf << 32) | (waited_full & 0xffffffffll);
        }
      }
      if (!ok && lane == 0) {
        s_failed = 1;
        atomicExch(a.error_flag, 2u);
      }
    } else if (warp == kScaleWarp) {
      // ------------------------------------------------------------------ scale warp
      // The fp32 scales come in through cp.async with kRawAhead groups (of four K blocks) in
      // flight: one group at a time would cost a memory round trip per group, which is longer
      // than the tensor cores need for its four K blocks. A lane fetches and later packs the
      // scales of its own four rows of A (lane, lane + 32, lane + 64, lane + 96); lanes 0-7 fetch
      // the two block rows of B.
      constexpr int kRawSlots = kRawSlotsOf<kCtas>, kRawAhead = kRawAheadOf<kCtas>;
      const int ngroups = (nkb + 3) / 4;
      const int nb_per_expert = a.N / 128;
      const uint32_t sf_full_leader = kCtas == 2 ? map_to_cta(&sf_full_bar[0], 0) : smem_u32(&sf_full_bar[0]);
      const int my_tiles = pair < total_tiles ? (total_tiles - pair + num_pairs - 1) / num_pairs : 0;
      const int total = my_tiles * ngroups;
      const bool vec_ok = a.a_scale_stride_k == 1 && (a.a_scale_stride_row & 3) == 0 &&
                          (reinterpret_cast<uintptr_t>(a.a_scale) & 15) == 0;
      // issue cursor
      int t_issue = pair, g_issue = 0, e = 0;
      const float* arow[4] = {a.a_scale, a.a_scale, a.a_scale, a.a_scale};
      const float* b0 = a.b_scale;
      const float* b1 = a.b_scale;
      uint32_t sf_it = 0;
      bool ok = true;
      for (int i = 0; i < total + kRawAhead && ok; ++i) {
        if (i < total) {
          if (g_issue == 0) {
            int m_pair, n_tile;
            decode_tile(sched, a.num_experts, n_tiles, t_issue, &e, &m_pair, &n_tile);
            const int m_tile = kCtas * m_pair + static_cast<int>(rank);
            #pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int in_tile = m_tile * kBM + 32 * j + lane;
              // Rows past the expert's count are not stored, so any finite scale will do for them,
              // but not one shared address: with every such lane of every CTA fetching row 0, the
              // L2 slice holding that line ran at 70 % of its request rate (3.5x the others) and
              // the operand tiles queued behind it (64 experts x 264 rows: 163 us against 58 us
              // for 64 x 256). Their own row, clamped to the buffer, spreads the fetches.
              const int row = min(sched.row_start[e] + in_tile, a.max_rows - 1);
              arow[j] = a.a_scale + static_cast<int64_t>(row) * a.a_scale_stride_row;
            }
            // B's 128-row blocks behind the accumulator columns. SwiGLU: every 128 columns are 64 of
            // gate and 64 of up; otherwise columns [0,128) and [128,256) are two consecutive blocks.
            const int nb0 = swiglu ? n_tile : n_tile * 2;
            const int nb1 = swiglu ? I / 128 + n_tile : n_tile * 2 + 1;
            b0 = a.b_scale + (static_cast<int64_t>(e) * nb_per_expert + nb0) * nkb;
            b1 = a.b_scale + (static_cast<int64_t>(e) * nb_per_expert + nb1) * nkb;
          }
          uint8_t* raw = raw_slots + static_cast<uint32_t>(i % kRawSlots) * kRawSlotBytes;
          const int kb0 = 4 * g_issue;
          if (vec_ok && kb0 + 4 <= nkb) {
            #pragma unroll
            for (int j = 0; j < 4; ++j) cp_async_16(raw + (32 * j + lane) * 16, arow[j] + kb0);
          } else {
            #pragma unroll
            for (int j = 0; j < 4; ++j) {
              #pragma unroll
              for (int k = 0; k < 4; ++k) {
                if (kb0 + k < nkb) cp_async_4(raw + (32 * j + lane) * 16 + 4 * k, arow[j] + (kb0 + k) * a.a_scale_stride_k);
              }
            }
          }
          if (lane < 8 && kb0 + (lane & 3) < nkb) {
            cp_async_4(raw + 2048 + lane * 4, (lane < 4 ? b0 : b1) + kb0 + (lane & 3));
          }
          if (++g_issue == ngroups) {
            g_issue = 0;
            t_issue += num_pairs;
          }
        }
        cp_async_commit();
        if (i < kRawAhead) continue;
        // group i - kRawAhead has landed
        cp_async_wait<kRawAhead>();
        __syncwarp();
        const uint8_t* raw = raw_slots + static_cast<uint32_t>((i - kRawAhead) % kRawSlots) * kRawSlotBytes;
        uint32_t wa[4];
        #pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint4 v = *reinterpret_cast<const uint4*>(raw + (32 * j + lane) * 16);
          wa[j] = ((v.x >> 23) & 0xffu) | (((v.y >> 23) & 0xffu) << 8) | (((v.z >> 23) & 0xffu) << 16) |
                  (((v.w >> 23) & 0xffu) << 24);
        }
        const uint4 vb0 = *reinterpret_cast<const uint4*>(raw + 2048);
        const uint4 vb1 = *reinterpret_cast<const uint4*>(raw + 2048 + 16);
        const uint32_t wb0 = ((vb0.x >> 23) & 0xffu) | (((vb0.y >> 23) & 0xffu) << 8) | (((vb0.z >> 23) & 0xffu) << 16) |
                             (((vb0.w >> 23) & 0xffu) << 24);
        const uint32_t wb1 = ((vb1.x >> 23) & 0xffu) | (((vb1.y >> 23) & 0xffu) << 8) | (((vb1.z >> 23) & 0xffu) << 16) |
                             (((vb1.w >> 23) & 0xffu) << 24);
        const uint32_t slot = sf_it % kSfSlots;
        ok = __all_sync(0xffffffffu, mbar_wait_timed(&sf_empty_bar[slot], ((sf_it / kSfSlots) & 1u) ^ 1u, kWaitNs));
        if (!ok || *reinterpret_cast<volatile uint32_t*>(&s_failed) != 0) {
          ok = false;
          break;
        }
        uint8_t* sf = sf_slots + slot * kSfSlotBytes;
        *reinterpret_cast<uint4*>(sf + lane * 16) = make_uint4(wa[0], wa[1], wa[2], wa[3]);
        const uint4 first = swiglu ? make_uint4(wb0, wb0, wb1, wb1) : make_uint4(wb0, wb0, wb0, wb0);
        const uint4 second = swiglu ? first : make_uint4(wb1, wb1, wb1, wb1);
        *reinterpret_cast<uint4*>(sf + kSfaBytes + lane * 16) = first;
        *reinterpret_cast<uint4*>(sf + kSfaBytes + 512 + lane * 16) = second;
        fence_proxy_async_smem();   // tcgen05.cp reads shared memory through the async proxy
        __syncwarp();
        // Default (CTA-scope) release on purpose: a cluster-scope release would first wait for this
        // thread's cp.async copies in flight, one memory round trip per group. The words are in this
        // CTA's shared memory and fenced for the async proxy above; the copy into tensor memory
        // that the leader triggers reads them on this SM.
        if (lane == 0) mbar_arrive_cluster(sf_full_leader + slot * 8u);
        ++sf_it;
      }
      cp_async_wait<0>();   // nothing of this thread's may still be landing when the CTA leaves
      if (!ok && lane == 0) {
        s_failed = 1;
        atomicExch(a.error_flag, 4u);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kEpilogueRegs) : "memory");
    const int q = warp & 3;                          // TMEM lane quarter this warp may read
    const int h = (warp - kFirstEpilogueWarp) >> 2;  // column half: 0 -> cols [0,128), 1 -> [128,256)
    const int row_in_tile = q * 32 + lane;
    uint8_t* const warp_stage = warp_stages + (warp - kFirstEpilogueWarp) * kWarpStageBytes;
    const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(h) * 128;
    const uint32_t tmem_empty_leader = kCtas == 2 ? map_to_cta(&tmem_empty_bar, 0) : smem_u32(&tmem_empty_bar);
    uint32_t tile_i = 0;
    int e = 0;
    for (int t = pair; t < total_tiles; t += num_pairs, ++tile_i) {
      int m_pair, n_tile;
      decode_tile(sched, a.num_experts, n_tiles, t, &e, &m_pair, &n_tile);
      const int m_tile = kCtas * m_pair + static_cast<int>(rank);   // this CTA's 128 rows of the tile
      const int row = sched.row_start[e] + m_tile * kBM + row_in_tile;
      const bool valid = m_tile * kBM + row_in_tile < sched.count[e] && row < a.max_rows;
      float acc[128];
      // the outcome must be the same for the whole warp: tcgen05.ld below is warp-collective
      const bool stamp = a.trace != nullptr && blockIdx.x == 0 && warp == kFirstEpilogueWarp && lane == 0 && tile_i < kTraceTiles;
      if (stamp) a.trace[tile_i * 8 + 6] = clock64();
      bool failed = !__all_sync(0xffffffffu, mbar_wait_timed(&tmem_full_bar, tile_i & 1u, kWaitNs));
      if (stamp) a.trace[tile_i * 8 + 2] = clock64();
      if (!failed) {
        fence_after_thread_sync();
        uint32_t c0[32], c1[32], c2[32], c3[32];
        tmem_ld32(taddr, c0);
        tmem_ld32(taddr + 32, c1);
        tmem_ld32(taddr + 64, c2);
        tmem_ld32(taddr + 96, c3);
        tmem_ld_wait();
        #pragma unroll
        for (int i = 0; i < 32; ++i) {
          acc[i] = __uint_as_float(c0[i]);
          acc[32 + i] = __uint_as_float(c1[i]);
          acc[64 + i] = __uint_as_float(c2[i]);
          acc[96 + i] = __uint_as_float(c3[i]);
        }
        // everything this warp needs is in registers: the tensor cores may start the next tile
        fence_before_thread_sync();
        __syncwarp();
        if (stamp) a.trace[tile_i * 8 + 3] = clock64();
        if (lane == 0) {
          if constexpr (kCtas == 2) {
            mbar_arrive_cluster(tmem_empty_leader);
          } else {
            mbar_arrive(&tmem_empty_bar);
          }
        }
      } else {
        #pragma unroll
        for (int i = 0; i < 128; ++i) acc[i] = 0.f;
        atomicExch(a.error_flag, 3u);
        s_failed = 1;
      }
      tile_epilogue<kCtas, true>(a, sched, acc, failed, valid, row, e, m_tile, n_tile, q, h, lane, row_in_tile, tile_i & 1u,
                                 warp_stage, swiglu, s_amax, s_failed);
      if (stamp) a.trace[tile_i * 8 + 4] = clock64();
      if (failed) break;
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
    grouped_fp8_gemm_mx_kernel(const __grid_constant__ KernelArgs a) {
  grouped_fp8_gemm_mx_body<2>(a);
}

__global__ void __launch_bounds__(kThreads, 1) grouped_fp8_gemm_mx_kernel_1cta(const __grid_constant__ KernelArgs a) {
  grouped_fp8_gemm_mx_body<1>(a);
}

}  // namespace

void grouped_fp8_gemm_mx(const GroupedGemmParams& p, cudaStream_t stream) {
  PPLX_REQUIRE(p.scale_format == kScalesPow2, "grouped_fp8_gemm_mx takes power-of-two scales");
  const KernelArgs a = prepare_kernel_args(p);
  int device = 0, sms = 0;
  PPLX_CUDA_CHECK(cudaGetDevice(&device));
  PPLX_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
  const int tile_rows = choose_tile_rows(p);
  const int ctas = p.num_ctas > 0 ? p.num_ctas : sms;
  if (tile_rows == 256) {
    constexpr size_t smem = mx_smem_bytes<2>();
    PPLX_CUDA_CHECK(cudaFuncSetAttribute(grouped_fp8_gemm_mx_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem)));
    const int grid = std::max(2, ctas & ~1);   // whole CTA pairs
    grouped_fp8_gemm_mx_kernel<<<grid, kThreads, smem, stream>>>(a);
  } else {
    constexpr size_t smem = mx_smem_bytes<1>();
    PPLX_CUDA_CHECK(cudaFuncSetAttribute(grouped_fp8_gemm_mx_kernel_1cta, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem)));
    grouped_fp8_gemm_mx_kernel_1cta<<<std::max(1, ctas), kThreads, smem, stream>>>(a);
  }
  PPLX_CUDA_CHECK(cudaGetLastError());
}

}  // namespace pplx::ops
