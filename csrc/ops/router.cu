// Stand-alone top-k routing: one warp per token (the per-token work is in router.cuh).
#include "router.h"

#include <cuda_bf16.h>

#include <cfloat>

#include "../core/error.h"
#include "router.cuh"

namespace pplx::ops {
namespace {

constexpr int kWarpsPerBlock = 8;

template <int PER_LANE>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) topk_route_kernel(const TopkRouteParams p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int token = blockIdx.x * kWarpsPerBlock + warp;
  if (token >= p.tokens) return;
  const size_t elem = p.logits_bf16 ? 2 : 4;
  const void* row = static_cast<const char*>(p.logits) + static_cast<size_t>(token) * p.logits_stride * elem;
  uint32_t idx;
  float weight;
  route_token_warp<PER_LANE>(row, p.logits_bf16, p.bias, p.num_experts, p.k, &idx, &weight);
  if (lane < p.k) {
    p.indices[token * p.indices_stride + lane] = idx;
    p.weights[token * p.weights_stride + lane] = weight;
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
