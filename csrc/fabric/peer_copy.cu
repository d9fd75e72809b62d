#include "peer_copy.h"

#include <algorithm>

#include "../a2a/ptx.cuh"

namespace pplx::fabric {
namespace {

constexpr uint32_t kChunkBytes = 32 * 1024;  // one bulk copy
constexpr int kStages = 4;                   // chunks in flight per CTA (128 KiB of smem)
constexpr int kBulkThreads = 32;
constexpr uint64_t kSmallPageBytes = 16 * 1024;  // at or below: one warp per page (paged_copy_rows_kernel)

__device__ __forceinline__ uint64_t page_offset(const uint32_t* pages, uint32_t i, uint64_t stride,
                                                uint64_t offset) {
  const uint64_t idx = pages != nullptr ? pages[i] : i;
  return idx * stride + offset;
}

// One elected thread per CTA drives a ring of shared-memory stages:
//   global --cp.async.bulk--> smem stage --cp.async.bulk--> (peer) global
// Loads complete on an mbarrier per stage, stores in bulk groups; a stage is reused once
// the store that read it has finished reading. SMs only issue descriptors.
__global__ void __launch_bounds__(kBulkThreads)
paged_copy_bulk_kernel(const __grid_constant__ PagedCopyArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ uint64_t bars[kStages];
  if (threadIdx.x != 0) return;

  for (int s = 0; s < kStages; ++s) mbar_init(&bars[s], 1);
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");

  const uint32_t chunks_per_page = static_cast<uint32_t>((a.length + kChunkBytes - 1) / kChunkBytes);
  const uint64_t total = static_cast<uint64_t>(a.num_pages) * chunks_per_page;
  uint32_t phase[kStages] = {0, 0, 0, 0};
  uint64_t issued = 0;
  bool failed = false;

  // Software pipeline: keep up to kStages loads in flight, store each as it lands.
  auto item_of = [&](uint64_t n) { return blockIdx.x + n * gridDim.x; };
  auto load = [&](uint64_t n) {
    const uint64_t item = item_of(n);
    const uint32_t page = static_cast<uint32_t>(item / chunks_per_page);
    const uint64_t within = (item % chunks_per_page) * kChunkBytes;
    const uint32_t bytes = static_cast<uint32_t>(min(static_cast<uint64_t>(kChunkBytes), a.length - within));
    const int s = static_cast<int>(n % kStages);
    mbar_expect_tx(&bars[s], bytes);
    bulk_g2s(smem + s * kChunkBytes, a.src_base + page_offset(a.src_pages, page, a.src_stride, a.src_offset) + within,
             bytes, &bars[s]);
  };
  uint64_t mine = 0;
  if (total > blockIdx.x) mine = (total - blockIdx.x + gridDim.x - 1) / gridDim.x;

  for (; issued < mine && issued < kStages; ++issued) load(issued);
  for (uint64_t n = 0; n < mine; ++n) {
    const int s = static_cast<int>(n % kStages);
    if (!mbar_wait_timed(&bars[s], phase[s], 2000000000ull)) {
      failed = true;
      break;
    }
    phase[s] ^= 1u;
    const uint64_t item = item_of(n);
    const uint32_t page = static_cast<uint32_t>(item / chunks_per_page);
    const uint64_t within = (item % chunks_per_page) * kChunkBytes;
    const uint32_t bytes = static_cast<uint32_t>(min(static_cast<uint64_t>(kChunkBytes), a.length - within));
    fence_proxy_async_smem();
    bulk_s2g(a.dst_base + page_offset(a.dst_pages, page, a.dst_stride, a.dst_offset) + within,
             smem + s * kChunkBytes, bytes);
    bulk_commit();
    // All but the newest store have finished reading their stage: the stage of store
    // n - 1 is free for the next load, while store n still overlaps with it.
    asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
    if (n >= 1 && issued < mine) {
      load(issued);  // issued == n - 1 + kStages: lands in stage (n - 1) % kStages
      ++issued;
    }
  }
  // Stores must be complete (not merely read) before the kernel, and with it the stream
  // event the host polls, finishes.
  bulk_wait0();
  if (failed) {
    atomicExch(a.error_flag, 1u);
    // loads that are still in flight land in this CTA's shared memory: wait for them
    // (bounded) before the CTA may exit
    for (uint64_t n = 0; n < issued; ++n) {
      const int s = static_cast<int>(n % kStages);
      (void)mbar_wait_timed(&bars[s], phase[s], 100000000ull);
    }
  }
}

// Fallback for arbitrary alignment: 16-byte vectors where both sides allow it, bytes else.
__global__ void __launch_bounds__(256) paged_copy_simt_kernel(const __grid_constant__ PagedCopyArgs a) {
  const uint32_t chunks_per_page = static_cast<uint32_t>((a.length + kChunkBytes - 1) / kChunkBytes);
  const uint64_t total = static_cast<uint64_t>(a.num_pages) * chunks_per_page;
  for (uint64_t item = blockIdx.x; item < total; item += gridDim.x) {
    const uint32_t page = static_cast<uint32_t>(item / chunks_per_page);
    const uint64_t within = (item % chunks_per_page) * kChunkBytes;
    const uint64_t bytes = min(static_cast<uint64_t>(kChunkBytes), a.length - within);
    const uint8_t* src = a.src_base + page_offset(a.src_pages, page, a.src_stride, a.src_offset) + within;
    uint8_t* dst = a.dst_base + page_offset(a.dst_pages, page, a.dst_stride, a.dst_offset) + within;
    const bool aligned = ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15u) == 0;
    if (aligned) {
      const uint64_t nvec = bytes / 16;
      for (uint64_t i = threadIdx.x; i < nvec; i += blockDim.x) {
        st_stream_v4(dst + 16 * i, ld_input_v4(src + 16 * i));
      }
      for (uint64_t i = nvec * 16 + threadIdx.x; i < bytes; i += blockDim.x) dst[i] = src[i];
    } else {
      for (uint64_t i = threadIdx.x; i < bytes; i += blockDim.x) dst[i] = src[i];
    }
  }
}

// Many small pages (rows of a weight shard, short KV pages): one warp per page, 16-byte vectors,
// four loads in flight per lane, as many CTAs as it takes to have every SM storing. A page this
// small is not worth a bulk-copy descriptor and a shared-memory round trip per page; what counts
// is how many independent pages are in flight.
constexpr int kRowsWarps = 8;

__global__ void __launch_bounds__(kRowsWarps * 32) paged_copy_rows_kernel(const __grid_constant__ PagedCopyArgs a) {
  const uint32_t lane = threadIdx.x & 31u;
  const uint64_t warp = static_cast<uint64_t>(blockIdx.x) * kRowsWarps + (threadIdx.x >> 5);
  const uint64_t warps = static_cast<uint64_t>(gridDim.x) * kRowsWarps;
  const uint32_t nvec = static_cast<uint32_t>(a.length / 16);
  for (uint64_t page = warp; page < a.num_pages; page += warps) {
    const uint8_t* src = a.src_base + page_offset(a.src_pages, static_cast<uint32_t>(page), a.src_stride, a.src_offset);
    uint8_t* dst = a.dst_base + page_offset(a.dst_pages, static_cast<uint32_t>(page), a.dst_stride, a.dst_offset);
    for (uint32_t i0 = lane; i0 < nvec; i0 += 128) {
      Vec16 v[4];
      #pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (i0 + 32 * u < nvec) v[u] = ld_input_v4(src + 16ull * (i0 + 32 * u));
      }
      #pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (i0 + 32 * u < nvec) st_stream_v4(dst + 16ull * (i0 + 32 * u), v[u]);
      }
    }
  }
}

}  // namespace

cudaError_t launch_paged_copy(const PagedCopyArgs& args, int max_ctas, cudaStream_t stream) {
  if (args.num_pages == 0 || args.length == 0) return cudaSuccess;
  const uint64_t chunks_per_page = (args.length + kChunkBytes - 1) / kChunkBytes;
  const uint64_t total = args.num_pages * chunks_per_page;
  if (max_ctas <= 0) max_ctas = 64;
  const int grid = static_cast<int>(std::min<uint64_t>(total, static_cast<uint64_t>(max_ctas)));
  const uint64_t all = reinterpret_cast<uintptr_t>(args.src_base) | reinterpret_cast<uintptr_t>(args.dst_base) |
                       args.src_stride | args.dst_stride | args.src_offset | args.dst_offset | args.length;
  if ((all & 15u) == 0 && args.length <= kSmallPageBytes && args.num_pages >= 64) {
    int sms = 0, device = 0;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    const uint64_t wanted = (args.num_pages + kRowsWarps - 1) / kRowsWarps;
    const int rows_grid = static_cast<int>(std::min<uint64_t>(wanted, static_cast<uint64_t>(std::max(sms, 1)) * 4));
    paged_copy_rows_kernel<<<rows_grid, kRowsWarps * 32, 0, stream>>>(args);
  } else if ((all & 15u) == 0) {
    const size_t smem = static_cast<size_t>(kStages) * kChunkBytes;
    // per device and cheap: set it on every launch rather than tracking devices
    cudaError_t e = cudaFuncSetAttribute(paged_copy_bulk_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem));
    if (e != cudaSuccess) return e;
    paged_copy_bulk_kernel<<<grid, kBulkThreads, smem, stream>>>(args);
  } else {
    paged_copy_simt_kernel<<<grid, 256, 0, stream>>>(args);
  }
  return cudaGetLastError();
}

cudaError_t warm_up_paged_copy(cudaStream_t stream) {
  // Empty launches: the kernels return at once, but their code is loaded and their attributes
  // are set. With lazy module loading the first launch of a kernel may otherwise have to wait
  // for kernels that are running, and one of those may be waiting for this copy.
  PagedCopyArgs args{};
  const size_t smem = static_cast<size_t>(kStages) * kChunkBytes;
  cudaError_t e = cudaFuncSetAttribute(paged_copy_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(smem));
  if (e != cudaSuccess) return e;
  paged_copy_bulk_kernel<<<1, kBulkThreads, smem, stream>>>(args);
  paged_copy_simt_kernel<<<1, 256, 0, stream>>>(args);
  paged_copy_rows_kernel<<<1, kRowsWarps * 32, 0, stream>>>(args);
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  return cudaStreamSynchronize(stream);
}

}  // namespace pplx::fabric
