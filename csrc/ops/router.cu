// One warp per token. Each lane keeps num_experts / 32 logits in registers (expert = j * 32 +
// lane, so the loads of a warp are coalesced); k rounds of a warp-wide arg-max (ties go to the
// lower expert index) pick the experts, and the chosen logits stay in a register of lane r for
// round r, so the softmax over them is one more pair of warp reductions.
#include "router.h"

#include <cuda_bf16.h>

#include <cfloat>

#include "../core/error.h"

namespace pplx::ops {
namespace {

constexpr int kWarpsPerBlock = 8;

template <int PER_LANE>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) topk_route_kernel(const TopkRouteParams p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int token = blockIdx.x * kWarpsPerBlock + warp;
  if (token >= p.tokens) return;

  float key[PER_LANE];   // logit + bias: what the choice is made on
  float val[PER_LANE];   // logit: what the weight is made of
  #pragma unroll
  for (int j = 0; j < PER_LANE; ++j) {
    const int e = j * 32 + lane;
    float v = -FLT_MAX;
    if (e < p.num_experts) {
      v = p.logits_bf16
              ? __bfloat162float(static_cast<const __nv_bfloat16*>(p.logits)[token * p.logits_stride + e])
              : static_cast<const float*>(p.logits)[token * p.logits_stride + e];
    }
    val[j] = v;
    key[j] = (e < p.num_experts && p.bias != nullptr) ? v + p.bias[e] : v;
  }

  float my_val = -FLT_MAX;   // lane r keeps the logit chosen in round r
  uint32_t my_idx = 0;
  for (int r = 0; r < p.k; ++r) {
    // this lane's best remaining candidate
    float best = -FLT_MAX;
    int best_j = 0;
    #pragma unroll
    for (int j = 0; j < PER_LANE; ++j) {
      if (key[j] > best) {   // strict: the lower j (lower expert index) wins a tie
        best = key[j];
        best_j = j;
      }
    }
    int best_e = best_j * 32 + lane;
    float w_best = best;
    int w_e = best_e;
    #pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, w_best, off);
      const int oe = __shfl_xor_sync(0xffffffffu, w_e, off);
      if (ob > w_best || (ob == w_best && oe < w_e)) {
        w_best = ob;
        w_e = oe;
      }
    }
    // the owner retires the winner and hands its plain logit to lane r
    float chosen = 0.f;
    if ((w_e & 31) == lane) {
      #pragma unroll
      for (int j = 0; j < PER_LANE; ++j) {
        if (j == (w_e >> 5)) {
          chosen = val[j];
          key[j] = -FLT_MAX;
        }
      }
    }
    chosen = __shfl_sync(0xffffffffu, chosen, w_e & 31);
    if (lane == r) {
      my_val = chosen;
      my_idx = static_cast<uint32_t>(w_e);
    }
  }

  // softmax over the k chosen logits (lanes >= k hold -FLT_MAX and contribute exp() = 0)
  float m = my_val;
  #pragma unroll
  for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
  const float ex = lane < p.k ? __expf(my_val - m) : 0.f;
  float sum = ex;
  #pragma unroll
  for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
  if (lane < p.k) {
    p.indices[token * p.indices_stride + lane] = my_idx;
    p.weights[token * p.weights_stride + lane] = ex / sum;
  }
}

}  // namespace

void topk_route(const TopkRouteParams& p, cudaStream_t stream) {
  PPLX_REQUIRE(p.num_experts >= 1 && p.num_experts <= 1024, "between 1 and 1024 experts");
  PPLX_REQUIRE(p.k >= 1 && p.k <= 32 && p.k <= p.num_experts, "k must be in [1, min(32, num_experts)]");
  if (p.tokens == 0) return;
  const int blocks = (p.tokens + kWarpsPerBlock - 1) / kWarpsPerBlock;
  const int per_lane = (p.num_experts + 31) / 32;
  if (per_lane <= 4) {
    topk_route_kernel<4><<<blocks, kWarpsPerBlock * 32, 0, stream>>>(p);
  } else if (per_lane <= 8) {
    topk_route_kernel<8><<<blocks, kWarpsPerBlock * 32, 0, stream>>>(p);
  } else if (per_lane <= 16) {
    topk_route_kernel<16><<<blocks, kWarpsPerBlock * 32, 0, stream>>>(p);
  } else {
    topk_route_kernel<32><<<blocks, kWarpsPerBlock * 32, 0, stream>>>(p);
  }
  PPLX_CUDA_CHECK(cudaGetLastError());
}

}  // namespace pplx::ops
