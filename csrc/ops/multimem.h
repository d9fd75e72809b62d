// Reductions through an NVSwitch multicast mapping (NVLS): one instruction updates the word at
// the same offset in the memory of every GPU bound to the multicast object.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

namespace pplx::ops {

// `mc_ptr`: address inside a mapping of a CUDA multicast object. Adds `value` to the 32-bit word
// there on every bound GPU (multimem.red.relaxed.sys.global.add.u32), stream ordered, one thread.
void multimem_red_add_u32(uint32_t* mc_ptr, uint32_t value, cudaStream_t stream);

}  // namespace pplx::ops
