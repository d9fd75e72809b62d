// Device-side copy engine of the intra-box transport: moves pages (KV-cache blocks) or one
// large range (weight shards) from local memory into a peer GPU's memory over NVLink.
// There is no counterpart in the reference, whose transfers are executed by RDMA NICs
// (fabric-lib/src/verbs/verbs_rdma_op.rs:122-224 builds the per-page work requests that
// this kernel replaces on a single NVSwitch box).
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

namespace pplx::fabric {

struct PagedCopyArgs {
  const uint8_t* src_base;
  uint8_t* dst_base;            // local or peer mapping
  const uint32_t* src_pages;    // device pointer, or nullptr: page i is at index i
  const uint32_t* dst_pages;
  uint64_t src_stride, dst_stride;
  uint64_t src_offset, dst_offset;
  uint64_t length;              // bytes per page
  uint32_t num_pages;
  uint32_t* error_flag;         // device word set to non-zero if a bounded wait ran out
};

// Launches the copy on `stream`. With addresses, strides and length all multiples of 16 bytes:
// pages of up to 16 KiB (64 or more of them) are copied one warp per page on every SM, larger
// ones through the bulk-copy (TMA) engine with a few CTAs; otherwise a byte-wise SIMT loop.
// `max_ctas` <= 0 picks a default that saturates NVLink with a fraction of the SMs.
cudaError_t launch_paged_copy(const PagedCopyArgs& args, int max_ctas, cudaStream_t stream);

// Loads the copy kernels on the current device (empty launches) and waits for them. Call once
// per device at set-up time, never while a kernel that depends on a later copy is running.
cudaError_t warm_up_paged_copy(cudaStream_t stream);

}  // namespace pplx::fabric
