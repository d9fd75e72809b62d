// Top-k routing: for every token, the k experts with the largest router logit (plus an optional
// per-expert bias used for the choice only) and the softmax of the chosen logits, i.e. softmax
// weights renormalised over the chosen k. Output in the layout dispatch / combine take:
// indices uint32 [tokens, k], weights float32 [tokens, k], both sorted by decreasing logit.
//
// The reference leaves routing to the caller (its tests draw indices directly:
// tests/p2p_all_to_all/data.py:9-108); this kernel is the first stage of the fused MoE layer.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

namespace pplx::ops {

struct TopkRouteParams {
  const void* logits = nullptr;    // [tokens, num_experts], fp32 or bf16, row stride in elements
  int64_t logits_stride = 0;
  bool logits_bf16 = false;
  const float* bias = nullptr;     // optional [num_experts], added for the choice, not for the weights
  uint32_t* indices = nullptr;     // [tokens, k]
  int64_t indices_stride = 0;
  float* weights = nullptr;        // [tokens, k]
  int64_t weights_stride = 0;
  int tokens = 0;
  int num_experts = 0;             // at most 1024
  int k = 0;                       // at most 32
};

void topk_route(const TopkRouteParams& p, cudaStream_t stream);

}  // namespace pplx::ops
