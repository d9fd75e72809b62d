// Host interface of the grouped block-scaled fp8 GEMM (see grouped_gemm.cu).
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

namespace pplx::ops {

enum GroupedGemmMode : int {
  kSwiGLUQuant = 0,  // B = [gate; up]; out = e4m3(silu(gate) * up) with 1x128 fp32 scales
  kBf16 = 1,         // out = bf16(A B^T)
  // out = bf16(A B^T), every row written straight into the combine receive buffer of the GPU
  // its token came from (peer stores over NVLink), followed by the arrival signal that the
  // receivers' combine_recv waits for: the down projection and the combine's send phase in one
  // kernel, so that the transfer of a tile overlaps the math of the next ones.
  kBf16Scatter = 2,
};

// How the scales of A and B are applied.
enum GroupedGemmScales : int {
  // any fp32 value; the epilogue reads every K block's partial sums out of tensor memory and
  // folds them with a_scale * b_scale (the tensor cores wait for it)
  kScalesFp32 = 0,
  // every scale is a power of two (mantissa bits zero; what a UE8M0 scale can express). The kernel
  // takes the exponents and the tensor cores apply them (tcgen05.mma kind::mxf8f6f4.block_scale),
  // so the sum over K stays in tensor memory; the SwiGLU epilogue then writes power-of-two scales
  // too. A scale with mantissa bits set is truncated to the power of two below it.
  kScalesPow2 = 1,
};

// Where the rows of a kBf16Scatter GEMM go. Filled by A2AContext::combine_scatter_begin().
struct CombineScatter {
  static constexpr int kMaxPeers = 8;
  const uint32_t* row_src = nullptr;   // [max_rows] rank the row's token came from, 0xffffffff = padding row
  const uint32_t* row_tk = nullptr;    // [max_rows] token * topk + k at that rank: the slot to write
  uint8_t* peer_recv[kMaxPeers] = {};  // combine receive area of every rank, as mapped on this GPU
  uint64_t slot_stride = 0;            // bytes per slot
  uint32_t* peer_flag[kMaxPeers] = {}; // this rank's combine arrival counter at every rank
  int world = 0;
  uint32_t signal_value = 0;           // arrivals a receiver expects from one sender per combine
  uint32_t* done_counter = nullptr;    // device word, zero between launches (counts finished CTAs)
  const uint32_t* status = nullptr;    // the all-to-all's status word: non-zero = do not signal
  // 0: the epilogue warps store the rows themselves; 1: they hand each row chunk to the bulk-copy
  // engine (cp.async.bulk shared -> peer global), so that NVLink back-pressure does not hold them up
  int bulk = 0;
};

struct GroupedGemmParams {
  const void* a = nullptr;          // e4m3 [max_rows, K], expert-major rows
  int64_t a_stride = 0;             // bytes per row
  const float* a_scale = nullptr;   // [max_rows, K / 128]
  int64_t a_scale_stride_row = 0;   // elements
  int64_t a_scale_stride_k = 1;
  const void* b = nullptr;          // e4m3 [num_experts, N, K] contiguous
  const float* b_scale = nullptr;   // [num_experts, N / 128, K / 128] contiguous
  const int32_t* expert_num_tokens = nullptr;  // device, [num_experts]
  void* out = nullptr;
  int64_t out_stride = 0;           // bytes per row
  float* out_scale = nullptr;       // kSwiGLUQuant: [max_rows, N / 256]
  int64_t out_scale_stride_row = 0;
  uint32_t* error_flag = nullptr;   // device word, set non-zero when a bounded wait ran out
  // Optional device array [num CTAs][4]: cycles spent waiting by the TMA producer (for a free
  // stage), the MMA issuer (for a free accumulator, for operands) and the first epilogue warp
  // (for partial sums). Shows which stage of the pipeline is the bottleneck.
  unsigned long long* wait_cycles = nullptr;
  // Optional device array [64][8] of SM clock readings for the first 64 tiles of CTA 0: epilogue
  // tile start, first partial sums ready, K loop done, tile stored; MMA first issue, last commit;
  // producer first load, last load.
  long long* trace = nullptr;
  int num_experts = 0;
  int N = 0, K = 0;
  int expert_padding = 1;           // every expert's rows start at a multiple of this
  int max_rows = 0;
  int mode = kBf16;
  int num_ctas = 0;                 // 0: one per SM
  // Rows per tile: 256 = pairs of CTAs (each loads half of B), 128 = one CTA per tile (for experts
  // with few rows), 0 = choose from max_rows / num_experts.
  int tile_rows = 0;
  // Profiling aid, 0 in production (results are wrong otherwise). Bit 0: the epilogue leaves the
  // partial sums unread; bit 1: no MMAs are issued; bit 2: no TMA loads;
  // bit 3: every MMA is issued twice. Timing the kernel with
  // one stage removed shows what the other stages can sustain.
  int debug_skip = 0;
  int scale_format = kScalesFp32;  // GroupedGemmScales
  CombineScatter scatter;          // kBf16Scatter only
};

void grouped_fp8_gemm(const GroupedGemmParams& params, cudaStream_t stream);

// The kScalesPow2 kernel (grouped_gemm_mx.cu); grouped_fp8_gemm() forwards to it.
void grouped_fp8_gemm_mx(const GroupedGemmParams& params, cudaStream_t stream);

// The same kernel built with its profiling aids (wait_cycles, trace, debug_skip); the regular
// entry point ignores those three fields.
void grouped_fp8_gemm_profiled(const GroupedGemmParams& params, cudaStream_t stream);

}  // namespace pplx::ops
