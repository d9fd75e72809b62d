// Small utilities of the transfer engine (reference: fabric-lib/src/utils/{defer,obj_pool,
// memory}.rs): a scope guard, a pool of stable-address objects and a fixed-chunk memory pool.
#pragma once

#include <cstddef>
#include <cstdint>
#include <memory>
#include <utility>
#include <vector>

namespace pplx::fabric {

template <typename F>
class Defer {
 public:
  explicit Defer(F f) : f_(std::move(f)) {}
  ~Defer() {
    if (armed_) f_();
  }
  void cancel() { armed_ = false; }
  Defer(const Defer&) = delete;
  Defer& operator=(const Defer&) = delete;

 private:
  F f_;
  bool armed_ = true;
};

// Objects live in chunks that never move, so pointers stay valid while the pool grows;
// released objects are reused before a new chunk is added.
template <typename T, size_t kChunk = 64>
class ObjectPool {
 public:
  template <typename... Args>
  T* acquire(Args&&... args) {
    if (free_.empty()) grow();
    T* slot = free_.back();
    free_.pop_back();
    return new (slot) T(std::forward<Args>(args)...);
  }
  void release(T* obj) {
    obj->~T();
    free_.push_back(obj);
  }
  size_t capacity() const { return chunks_.size() * kChunk; }
  size_t in_use() const { return capacity() - free_.size(); }

 private:
  struct alignas(alignof(T)) Slot { unsigned char bytes[sizeof(T)]; };
  void grow() {
    chunks_.emplace_back(new Slot[kChunk]);
    Slot* base = chunks_.back().get();
    for (size_t i = kChunk; i-- > 0;) free_.push_back(reinterpret_cast<T*>(&base[i]));
  }
  std::vector<std::unique_ptr<Slot[]>> chunks_;
  std::vector<T*> free_;
};

// Fixed-size chunks carved out of one caller-provided region (e.g. a registered buffer).
class MemoryPool {
 public:
  MemoryPool(uint8_t* base, size_t total, size_t chunk) : base_(base), chunk_(chunk) {
    for (size_t off = 0; off + chunk <= total; off += chunk) free_.push_back(base + off);
  }
  uint8_t* acquire() {
    if (free_.empty()) return nullptr;
    uint8_t* p = free_.back();
    free_.pop_back();
    return p;
  }
  void release(uint8_t* p) { free_.push_back(p); }
  size_t chunk_size() const { return chunk_; }
  size_t available() const { return free_.size(); }

 private:
  uint8_t* base_;
  size_t chunk_;
  std::vector<uint8_t*> free_;
};

}  // namespace pplx::fabric
