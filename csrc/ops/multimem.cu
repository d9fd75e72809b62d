#include "multimem.h"

#include "../core/error.h"

namespace pplx::ops {

namespace {
__global__ void multimem_red_add_kernel(uint32_t* mc_ptr, uint32_t value) {
  asm volatile("multimem.red.relaxed.sys.global.add.u32 [%0], %1;" : : "l"(mc_ptr), "r"(value) : "memory");
}
}  // namespace

void multimem_red_add_u32(uint32_t* mc_ptr, uint32_t value, cudaStream_t stream) {
  PPLX_REQUIRE(mc_ptr != nullptr && reinterpret_cast<uintptr_t>(mc_ptr) % 4 == 0,
               "multimem_red_add_u32: the address must be a 4-byte aligned multicast address");
  multimem_red_add_kernel<<<1, 1, 0, stream>>>(mc_ptr, value);
  PPLX_CUDA_CHECK(cudaGetLastError());
}

}  // namespace pplx::ops
