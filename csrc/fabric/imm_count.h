// Arrival counters keyed by the 32-bit immediate value of one-sided writes.
//
// Three flavours, as in the reference's fabric-lib/src/imm_count.rs:15-144:
//   Expected  fire once when the count reaches an expected value; later arrivals are surplus
//             and are reported as if no counter were installed, until it is set again;
//   Free      count forever, the user waits on the counter (ImmCounter::wait);
//   Flag      count upwards from a negative "debt"; when the debt is paid (value 0) raise a
//             flag in mapped memory that a GPU kernel polls (the reference raises a GDRCopy
//             flag; here it is a word in device-mapped pinned host memory).
#pragma once

#include <atomic>
#include <cstdint>
#include <memory>
#include <optional>
#include <shared_mutex>
#include <unordered_map>

namespace pplx::fabric {

enum class ImmIncResult { kVacant, kNotReached, kReached };

class ImmCountMap {
 public:
  // Registers (or replaces) an Expected counter. Returns the previous (count, expected)
  // if `imm` already was a counter.
  std::optional<std::pair<uint32_t, uint32_t>> set_expected(uint32_t imm, uint32_t expected);
  // Registers a free-running counter and returns the shared cell.
  std::shared_ptr<std::atomic<int64_t>> set_free(uint32_t imm);
  // Registers a flag counter: `flag` is set to 1 when the counter comes back to zero.
  std::shared_ptr<std::atomic<int64_t>> set_flag(uint32_t imm, volatile uint32_t* flag);
  // Removes the counter; returns (count, expected or 0).
  std::optional<std::pair<uint32_t, uint32_t>> remove(uint32_t imm);
  // One arrival (or `n` coalesced arrivals) of `imm`.
  ImmIncResult inc(uint32_t imm, uint32_t n = 1);
  size_t size() const;

 private:
  struct Entry {
    enum class Kind { kExpected, kFree, kFlag } kind;
    std::shared_ptr<std::atomic<int64_t>> counter;
    uint32_t expected = 0;
    volatile uint32_t* flag = nullptr;
  };
  mutable std::shared_mutex mu_;
  std::unordered_map<uint32_t, Entry> map_;
};

}  // namespace pplx::fabric
