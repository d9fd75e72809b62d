// Top-k routing of one token by one warp, shared by the stand-alone routing kernel (router.cu)
// and by the all-to-all's dispatch, which can route a token in the team that is about to send it.
//
// Each lane keeps PER_LANE logits in registers (expert = j * 32 + lane, so the loads of a warp
// are coalesced); k rounds of a warp-wide arg-max (ties go to the lower expert index) pick the
// experts, and the chosen logits stay in a register of lane r for round r, so the softmax over
// them is one more pair of warp reductions. The choice is made on logit + bias, the weight on
// the plain logit.
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
  float key[PER_LANE];   // logit + bias: what the choice is made on
  float val[PER_LANE];   // logit: what the weight is made of
  #pragma unroll
  for (int j = 0; j < PER_LANE; ++j) {
    const int e = j * 32 + lane;
    float v = -FLT_MAX;
    if (e < num_experts) {
      v = logits_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(logits_row)[e])
                      : static_cast<const float*>(logits_row)[e];
    }
    val[j] = v;
    key[j] = (e < num_experts && bias != nullptr) ? v + bias[e] : v;
  }

  float my_val = -FLT_MAX;   // lane r keeps the logit chosen in round r
  uint32_t my_idx = 0;
  #pragma unroll 1
  for (int r = 0; r < k; ++r) {
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
  const float ex = lane < k ? __expf(my_val - m) : 0.f;
  float sum = ex;
  #pragma unroll
  for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
  *idx = lane < k ? my_idx : 0u;
  *weight = lane < k ? ex / sum : 0.f;
}

}  // namespace pplx::ops
