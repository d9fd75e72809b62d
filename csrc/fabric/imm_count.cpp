#include "imm_count.h"

#include <mutex>

namespace pplx::fabric {

std::optional<std::pair<uint32_t, uint32_t>> ImmCountMap::set_expected(uint32_t imm, uint32_t expected) {
  std::unique_lock lock(mu_);
  std::optional<std::pair<uint32_t, uint32_t>> prev;
  auto it = map_.find(imm);
  if (it != map_.end()) {
    prev = std::make_pair(static_cast<uint32_t>(it->second.counter->load()), it->second.expected);
  }
  Entry e{Entry::Kind::kExpected, std::make_shared<std::atomic<int64_t>>(0), expected, nullptr};
  map_[imm] = std::move(e);
  return prev;
}

std::shared_ptr<std::atomic<int64_t>> ImmCountMap::set_free(uint32_t imm) {
  std::unique_lock lock(mu_);
  Entry e{Entry::Kind::kFree, std::make_shared<std::atomic<int64_t>>(0), 0, nullptr};
  auto cell = e.counter;
  map_[imm] = std::move(e);
  return cell;
}

std::shared_ptr<std::atomic<int64_t>> ImmCountMap::set_flag(uint32_t imm, volatile uint32_t* flag) {
  std::unique_lock lock(mu_);
  Entry e{Entry::Kind::kFlag, std::make_shared<std::atomic<int64_t>>(0), 0, flag};
  auto cell = e.counter;
  map_[imm] = std::move(e);
  return cell;
}

std::optional<std::pair<uint32_t, uint32_t>> ImmCountMap::remove(uint32_t imm) {
  std::unique_lock lock(mu_);
  auto it = map_.find(imm);
  if (it == map_.end()) return std::nullopt;
  auto out = std::make_pair(static_cast<uint32_t>(it->second.counter->load()), it->second.expected);
  map_.erase(it);
  return out;
}

ImmIncResult ImmCountMap::inc(uint32_t imm, uint32_t n) {
  std::shared_lock lock(mu_);
  auto it = map_.find(imm);
  if (it == map_.end()) return ImmIncResult::kVacant;
  Entry& e = it->second;
  switch (e.kind) {
    case Entry::Kind::kExpected: {
      // Consumes exactly `expected` arrivals: the one that completes the count reports
      // kReached, every later one is surplus and is treated as if no counter existed.
      const int64_t prev = e.counter->fetch_add(n, std::memory_order_acq_rel);
      if (prev >= e.expected) {
        e.counter->fetch_sub(n, std::memory_order_acq_rel);
        return ImmIncResult::kVacant;
      }
      return prev + n >= e.expected ? ImmIncResult::kReached : ImmIncResult::kNotReached;
    }
    case Entry::Kind::kFree:
      e.counter->fetch_add(n, std::memory_order_acq_rel);
      return ImmIncResult::kNotReached;
    case Entry::Kind::kFlag: {
      const int64_t now = e.counter->fetch_add(n, std::memory_order_acq_rel) + n;
      if (now == 0 && e.flag != nullptr) {
        *e.flag = 1u;
        std::atomic_thread_fence(std::memory_order_seq_cst);
      }
      return ImmIncResult::kNotReached;
    }
  }
  return ImmIncResult::kVacant;
}

size_t ImmCountMap::size() const {
  std::shared_lock lock(mu_);
  return map_.size();
}

}  // namespace pplx::fabric
