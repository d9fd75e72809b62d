// Top-k routing of one token by one warp, shared by the stand-alone routing kernel (router.cu)
// and by the all-to-all's dispatch, which can route a token in the team that is about to send it.
//
// Each lane keeps PER_LANE logits in registers (expert = j * 32 + lane, so the loads of a warp
// are coalesced). The choice is made on logit + bias, mapped to an unsigned key of the same
// order, so that a round of the arg-max is two warp reductions in hardware (redux.sync): the
// maximum key, then the lowest expert index among the lanes that hold it (ties go to the lower
// expert index, as torch.topk does). The chosen logits stay in a register of lane r for round r,
// so the softmax over them is one more pair of warp reductions; the weight is made of the plain
// logit.
#pragma once

#include <cuda_bf16.h>

#include <cfloat>
#include <cstdint>

namespace pplx::ops {

// All 32 lanes call. On return lane r < k holds the r-th chosen expert in *idx and its softmax
// weight in *weight; the other lanes hold (0, 0).
template <int PER_LANE>
__device__ __forceinline__ void route_token_warp(const void* logits_row, bool logits_bf16, const float* bias,
                                                 int num_experts, int k, uint32_t* idx, float* weight) {
  const int lane = threadIdx.x & 31;
  uint32_t key[PER_LANE];   // logit + bias as an order-preserving unsigned; 0 = no candidate
  float val[PER_LANE];      // logit: what the weight is made of
  #pragma unroll
  for (int j = 0; j < PER_LANE; ++j) {
    const int e = j * 32 + lane;
    float v = -FLT_MAX;
    uint32_t u = 0;
    if (e < num_experts) {
      v = logits_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(logits_row)[e])
                      : static_cast<const float*>(logits_row)[e];
      const float choice = (bias != nullptr ? v + bias[e] : v) + 0.0f;   // + 0: -0 and +0 compare equal
      const uint32_t bits = __float_as_uint(choice);
      u = bits ^ ((bits >> 31) != 0 ? 0xffffffffu : 0x80000000u);       // monotone in the float order
      u = max(u, 1u);
    }
    val[j] = v;
    key[j] = u;
  }

  float my_val = -FLT_MAX;   // lane r keeps the logit chosen in round r
  uint32_t my_idx = 0;
  #pragma unroll 1
  for (int r = 0; r < k; ++r) {
    uint32_t best = 0;
    #pragma unroll
    for (int j = 0; j < PER_LANE; ++j) best = max(best, key[j]);
    const uint32_t top = __reduce_max_sync(0xffffffffu, best);
    // the lowest expert index that holds the maximum: in this lane the lowest j, then over the warp
    uint32_t cand = 0xffffffffu;
    #pragma unroll
    for (int j = PER_LANE - 1; j >= 0; --j) {
      if (key[j] == top) cand = static_cast<uint32_t>(j * 32 + lane);
    }
    const uint32_t w_e = __reduce_min_sync(0xffffffffu, cand);
    // the owner retires the winner and hands its plain logit to lane r
    float chosen = 0.f;
    if ((w_e & 31u) == static_cast<uint32_t>(lane)) {
      #pragma unroll
      for (int j = 0; j < PER_LANE; ++j) {
        if (j == static_cast<int>(w_e >> 5)) {
          chosen = val[j];
          key[j] = 0u;
        }
      }
    }
    chosen = __shfl_sync(0xffffffffu, chosen, w_e & 31u);
    if (lane == r) {
      my_val = chosen;
      my_idx = w_e;
    }
  }

  // softmax over the k chosen logits (lanes >= k hold -FLT_MAX and contribute exp() = 0)
  float m = my_val;
  #pragma unroll
  for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
  const float ex = lane < k ? __expf(my_val - m) : 0.f;
  float sum = ex;
  #pragma unroll
  for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
  *idx = lane < k ? my_idx : 0u;
  *weight = lane < k ? ex / sum : 0.f;
}

}  // namespace pplx::ops
