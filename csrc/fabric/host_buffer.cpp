#include "host_buffer.h"

#include <cstdlib>

#include "../core/error.h"

namespace pplx::fabric {

HostBuffer::~HostBuffer() { owner_->recycle(data_, capacity_); }

HostBufferAllocator::HostBufferAllocator(RegisterFn on_new, RegisterFn on_free)
    : on_new_(std::move(on_new)), on_free_(std::move(on_free)) {}

HostBufferAllocator::~HostBufferAllocator() {
  for (auto& [ptr, len] : all_) {
    if (on_free_) on_free_(ptr, len);
    std::free(ptr);
  }
}

std::unique_ptr<HostBuffer> HostBufferAllocator::allocate(size_t len) {
  size_t cap = 4096;
  while (cap < len) cap <<= 1;
  {
    std::lock_guard<std::mutex> lock(mu_);
    auto it = free_.find(cap);
    if (it != free_.end() && !it->second.empty()) {
      uint8_t* p = it->second.back();
      it->second.pop_back();
      return std::unique_ptr<HostBuffer>(new HostBuffer(this, p, cap));
    }
  }
  void* mem = nullptr;
  if (posix_memalign(&mem, 4096, cap) != 0) throw Error::from_errno("posix_memalign(bounce buffer)");
  uint8_t* p = static_cast<uint8_t*>(mem);
  if (on_new_) on_new_(p, cap);
  {
    std::lock_guard<std::mutex> lock(mu_);
    all_.emplace_back(p, cap);
    allocated_ += cap;
  }
  return std::unique_ptr<HostBuffer>(new HostBuffer(this, p, cap));
}

void HostBufferAllocator::recycle(uint8_t* data, size_t capacity) {
  std::lock_guard<std::mutex> lock(mu_);
  free_[capacity].push_back(data);
}

size_t HostBufferAllocator::cached_buffers() const {
  std::lock_guard<std::mutex> lock(mu_);
  size_t n = 0;
  for (const auto& kv : free_) n += kv.second.size();
  return n;
}

}  // namespace pplx::fabric
