#include "paged_copy_noalloc.h"

#include <cuda_runtime.h>

#include <mutex>
#include <string>

namespace {

constexpr uint32_t kMaxPages = 65536;
constexpr int kMaxDevices = 64;
constexpr uint32_t kChunkBytes = 32 * 1024;

// Page tables of the call in flight: [0, kMaxPages) source pages, [kMaxPages, 2 kMaxPages)
// destination pages. In host code this name is only a handle for cudaGetSymbolAddress; the
// device address is looked up once per device below.
static __device__ __align__(256) uint32_t g_page_tables[2 * kMaxPages];

uint32_t* g_tables_on_device[kMaxDevices] = {};
std::mutex g_setup_mutex;
thread_local std::string t_last_error;

int fail(int code, const std::string& what) {
  t_last_error = what;
  return code;
}

// Same copy loop as the library's SIMT paged copy, reading its page tables from the
// static array: one CTA per 32 KiB chunk of a page, 16-byte vectors when both sides are
// aligned, bytes otherwise.
__global__ void __launch_bounds__(256)
paged_copy_static_tables_kernel(const uint8_t* __restrict__ src_base, uint8_t* __restrict__ dst_base,
                                const uint32_t* __restrict__ tables, uint32_t num_pages,
                                uint64_t src_stride, uint64_t dst_stride, uint64_t src_offset,
                                uint64_t dst_offset, uint64_t length) {
  const uint32_t chunks_per_page = static_cast<uint32_t>((length + kChunkBytes - 1) / kChunkBytes);
  const uint64_t total = static_cast<uint64_t>(num_pages) * chunks_per_page;
  for (uint64_t item = blockIdx.x; item < total; item += gridDim.x) {
    const uint32_t page = static_cast<uint32_t>(item / chunks_per_page);
    const uint64_t within = (item % chunks_per_page) * kChunkBytes;
    const uint64_t bytes = min(static_cast<uint64_t>(kChunkBytes), length - within);
    const uint8_t* src = src_base + static_cast<uint64_t>(tables[page]) * src_stride + src_offset + within;
    uint8_t* dst = dst_base + static_cast<uint64_t>(tables[kMaxPages + page]) * dst_stride + dst_offset + within;
    const bool aligned = ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15u) == 0;
    if (aligned) {
      const uint64_t nvec = bytes / 16;
      const uint4* s4 = reinterpret_cast<const uint4*>(src);
      uint4* d4 = reinterpret_cast<uint4*>(dst);
      for (uint64_t i = threadIdx.x; i < nvec; i += blockDim.x) d4[i] = s4[i];
      for (uint64_t i = nvec * 16 + threadIdx.x; i < bytes; i += blockDim.x) dst[i] = src[i];
    } else {
      for (uint64_t i = threadIdx.x; i < bytes; i += blockDim.x) dst[i] = src[i];
    }
  }
}

}  // namespace

extern "C" uint32_t pplx_paged_copy_noalloc_max_pages(void) { return kMaxPages; }

extern "C" const char* pplx_noalloc_last_error(void) { return t_last_error.c_str(); }

extern "C" int pplx_paged_copy_noalloc(const void* src_base, void* dst_base,
                                       const uint32_t* src_pages_host, const uint32_t* dst_pages_host,
                                       uint32_t num_pages, uint64_t src_stride, uint64_t dst_stride,
                                       uint64_t src_offset, uint64_t dst_offset, uint64_t length,
                                       void* stream) {
  if (num_pages > kMaxPages) {
    return fail(-1, "pplx_paged_copy_noalloc: " + std::to_string(num_pages) + " pages exceed the limit of " +
                        std::to_string(kMaxPages) + " per call; split the transfer");
  }
  if (num_pages == 0 || length == 0) return 0;
  if (src_base == nullptr || dst_base == nullptr || src_pages_host == nullptr || dst_pages_host == nullptr) {
    return fail(-1, "pplx_paged_copy_noalloc: null pointer argument");
  }
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return fail(static_cast<int>(e), std::string("cudaGetDevice: ") + cudaGetErrorString(e));
  if (device < 0 || device >= kMaxDevices) return fail(-1, "pplx_paged_copy_noalloc: device ordinal out of range");

  uint32_t* tables = nullptr;
  {
    // Set-up, once per device and with that device current: turn the host-side handle of the
    // static array into the address kernels on this device can use.
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (g_tables_on_device[device] == nullptr) {
      uint32_t* ptr = nullptr;
      e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_page_tables);
      if (e != cudaSuccess) {
        return fail(static_cast<int>(e), std::string("cudaGetSymbolAddress(page tables): ") + cudaGetErrorString(e));
      }
      g_tables_on_device[device] = ptr;
    }
    tables = g_tables_on_device[device];
  }

  cudaStream_t s = static_cast<cudaStream_t>(stream);
  e = cudaMemcpyAsync(tables, src_pages_host, sizeof(uint32_t) * num_pages, cudaMemcpyHostToDevice, s);
  if (e == cudaSuccess) {
    e = cudaMemcpyAsync(tables + kMaxPages, dst_pages_host, sizeof(uint32_t) * num_pages,
                        cudaMemcpyHostToDevice, s);
  }
  if (e != cudaSuccess) return fail(static_cast<int>(e), std::string("staging the page tables: ") + cudaGetErrorString(e));

  const uint64_t chunks = static_cast<uint64_t>(num_pages) * ((length + kChunkBytes - 1) / kChunkBytes);
  const unsigned grid = static_cast<unsigned>(chunks < 1184 ? chunks : 1184);  // 8 CTAs per SM of a B200
  paged_copy_static_tables_kernel<<<grid, 256, 0, s>>>(static_cast<const uint8_t*>(src_base),
                                                       static_cast<uint8_t*>(dst_base), tables, num_pages,
                                                       src_stride, dst_stride, src_offset, dst_offset, length);
  e = cudaGetLastError();
  if (e != cudaSuccess) return fail(static_cast<int>(e), std::string("kernel launch: ") + cudaGetErrorString(e));
  return 0;
}
