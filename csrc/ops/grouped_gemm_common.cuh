// Pieces shared by the two grouped fp8 GEMM kernels (grouped_gemm.cu: fp32 scales folded in per
// K block by the epilogue; grouped_gemm_mx.cu: power-of-two scales applied inside the MMA): tile
// sizes, kernel arguments, the tile schedule, the staged row stores and the tile-end epilogue.
// Everything here is inline.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include <algorithm>

#include "../core/cu_driver.h"
#include "../core/error.h"
#include "grouped_gemm.h"
#include "tcgen05.cuh"

namespace pplx::ops::gemm_detail {

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

// Expert-major row layout (each expert's block starts at a multiple of the padding) and the tile
// count before each expert, computed by one warp. The counts live in global memory: the lanes
// fetch four experts each at once and combine with a warp scan, instead of one thread walking
// through up to 128 dependent cache misses in front of every launch.
template <int kCtas>
__device__ __forceinline__ void build_schedule(const KernelArgs& a, Schedule& sched, int n_tiles, int lane) {
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

// End of a tile for one epilogue thread: `acc` holds its row's 128 columns of D (columns
// [128 h, 128 h + 128) of the CTA's accumulator; under SwiGLU the first 64 are gate, the last 64 up).
// SwiGLU + re-quantise, bf16, or bf16 scattered into the peers' combine buffers. With kPow2 the
// scales written by the SwiGLU epilogue are powers of two. Every epilogue thread of the CTA must
// call this for every tile (a named barrier exchanges the row maxima under SwiGLU); `failed`
// comes back true for all of them if any saw a failure.
template <int kCtas, bool kPow2>
__device__ __forceinline__ void tile_epilogue(const KernelArgs& a, const Schedule& sched, float (&acc)[128], bool& failed,
                                              bool valid, int row, int e, int m_tile, int n_tile, int q, int h, int lane,
                                              int row_in_tile, uint32_t tile_parity, uint8_t* warp_stage, bool swiglu,
                                              float (&s_amax)[2][kBM][2], const uint32_t& s_failed) {
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
    float scale = fmaxf(amax, 1e-10f) * (1.0f / 448.0f);
    if constexpr (kPow2) {   // next power of two at or above: the consumer takes the exponent only
      scale = __uint_as_float((__float_as_uint(scale) + 0x007fffffu) & 0x7f800000u);
    }
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
}

// After the CTA's (or cluster's) final barrier, one thread per CTA: the last CTA of the grid to
// get here tells every GPU that this rank's rows have been written.
__device__ __forceinline__ void scatter_signal(const KernelArgs& a, const uint32_t& s_failed) {
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

inline CUtensorMap make_map(const void* base, uint64_t rows, uint64_t cols_bytes, uint64_t row_stride_bytes,
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

// Argument checks common to both kernels, and the kernel's argument block.
inline KernelArgs prepare_kernel_args(const GroupedGemmParams& p) {
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
  return a;
}

// Pairs of CTAs on 256-row tiles unless the experts are small: with no more than 192 rows per
// expert on average (by capacity; the counts themselves stay on the device) the second CTA of a
// pair would mostly idle, and single CTAs on 128-row tiles do the same work with half the waste.
inline int choose_tile_rows(const GroupedGemmParams& p) {
  const bool wants_pairs = p.mode == kBf16Scatter && p.scatter.bulk;   // the bulk-copy sender stages 128-byte rows
  const int tile_rows =
      p.tile_rows != 0 ? p.tile_rows : ((wants_pairs || p.max_rows / p.num_experts > 192) ? 256 : 128);
  PPLX_REQUIRE(tile_rows == 128 || tile_rows == 256, "tile_rows must be 0 (automatic), 128 or 256");
  PPLX_REQUIRE(tile_rows == 256 || !(p.mode == kBf16Scatter && p.scatter.bulk), "the bulk-copy sender needs 256-row tiles");
  return tile_rows;
}

}  // namespace pplx::ops::gemm_detail
