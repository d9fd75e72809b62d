// Registered host bounce buffers, handed out in power-of-two sizes and recycled through
// per-size free lists (reference: fabric-lib/src/host_buffer.rs:9-129).
#pragma once

#include <cstdint>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <vector>

namespace pplx::fabric {

class HostBufferAllocator;

class HostBuffer {
 public:
  ~HostBuffer();
  HostBuffer(const HostBuffer&) = delete;
  HostBuffer& operator=(const HostBuffer&) = delete;
  uint8_t* data() const { return data_; }
  size_t capacity() const { return capacity_; }

 private:
  friend class HostBufferAllocator;
  HostBuffer(HostBufferAllocator* owner, uint8_t* data, size_t capacity)
      : owner_(owner), data_(data), capacity_(capacity) {}
  HostBufferAllocator* owner_;
  uint8_t* data_;
  size_t capacity_;
};

class HostBufferAllocator {
 public:
  using RegisterFn = std::function<void(uint8_t* ptr, size_t len)>;
  // `on_new` is called once for every fresh allocation (to register it with the domains),
  // `on_free` when the allocator is destroyed.
  explicit HostBufferAllocator(RegisterFn on_new = nullptr, RegisterFn on_free = nullptr);
  ~HostBufferAllocator();
  // Buffer of at least `len` bytes (capacity is the next power of two, at least 4 KiB).
  std::unique_ptr<HostBuffer> allocate(size_t len);
  size_t allocated_bytes() const { return allocated_; }
  size_t cached_buffers() const;

 private:
  friend class HostBuffer;
  void recycle(uint8_t* data, size_t capacity);
  RegisterFn on_new_, on_free_;
  mutable std::mutex mu_;
  std::map<size_t, std::vector<uint8_t*>> free_;
  std::vector<std::pair<uint8_t*, size_t>> all_;
  size_t allocated_ = 0;
};

}  // namespace pplx::fabric
