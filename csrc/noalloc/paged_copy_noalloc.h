// Paged device-to-device copy for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference: the reference moves pages with RDMA
// work requests built on the host (fabric-lib/src/verbs/verbs_rdma_op.rs:122-224) and never
// stages page tables on the GPU.
//
// Who needs it: code that runs where cudaMalloc is off limits. A serving process that
// handed every free byte to its KV-cache arena cannot get more memory from the driver; a
// component embedded in someone else's runtime (a plugin, a callback on a worker thread that
// owns no allocator) has no allocator to ask; and cudaMalloc / cudaFree synchronise the whole
// device, which a latency-critical decode loop cannot afford in the middle of a step. The
// regular path of this library (LocalDomain in csrc/fabric/local_domain.cpp) grows a
// cudaMalloc'd scratch buffer for the page tables of a paged write; this variant keeps that
// scratch in a fixed array that is part of the loaded library image instead.
//
// Contract
//   * The caller passes the source and destination base pointers (device memory reachable
//     from the current device, e.g. local memory or a mapped peer region) and two page tables
//     in HOST memory. Page i of the source, at src_base + src_pages[i] * src_stride +
//     src_offset, is copied to dst_base + dst_pages[i] * dst_stride + dst_offset; `length`
//     bytes per page.
//   * At most pplx_paged_copy_noalloc_max_pages() pages per call (65,536). More is refused
//     with an error, nothing is copied.
//   * The page tables are staged in a file-scope device array of 2 x 65,536 x 4 bytes
//     (512 KiB). Every GPU on which the library is used holds that array until the process
//     exits.
//   * The first call on a device resolves the device address of that array (one
//     cudaGetSymbolAddress with that device current). Make that first call outside of any
//     stream capture. Later calls on the same device skip the set-up.
//   * All calls on one device share the array, and it keeps the tables of the last call.
//     Nothing in it has to start out zeroed: a call overwrites the entries it reads before
//     the kernel runs. Two calls that may overlap on the GPU (different streams without an
//     ordering between them) race on the array; order them, e.g. by using one stream.
//   * The work is enqueued on `stream` and is asynchronous like any kernel launch. The two
//     host page tables are read by two cudaMemcpyAsync calls on `stream`. Tables in pageable
//     memory (malloc, a Python list turned into a ctypes array) are staged by the runtime
//     before the call returns and may be reused at once. Tables in pinned or registered host
//     memory are read when the stream reaches the copies: keep them unchanged until then
//     (an event or a stream synchronisation after the call tells you).
//   * No cudaMalloc, cudaFree or other allocating routine is called.
//
// Returns 0 on success, a cudaError_t value when a CUDA call failed, -1 for invalid
// arguments. pplx_noalloc_last_error() gives the message of the last failure on the calling
// thread.
#pragma once

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

__attribute__((visibility("default")))
int pplx_paged_copy_noalloc(const void* src_base, void* dst_base, const uint32_t* src_pages_host,
                            const uint32_t* dst_pages_host, uint32_t num_pages, uint64_t src_stride,
                            uint64_t dst_stride, uint64_t src_offset, uint64_t dst_offset,
                            uint64_t length, void* stream);

__attribute__((visibility("default")))
uint32_t pplx_paged_copy_noalloc_max_pages(void);

__attribute__((visibility("default")))
const char* pplx_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
