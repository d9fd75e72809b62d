// A provider decorator that misbehaves on request: fails, swallows, delays or reorders the
// completions of writes. It is the engine's fault-injection seam for tests that must not touch a
// GPU to make something go wrong: the failure is made here, on the host, and the layers above
// (callbacks, error counters, the all-to-all's proxy, bounded waits) have to cope.
//
// The reference exports mockall mocks of its engine traits for the same purpose
// (fabric-lib/src/interface.rs:72,99,119-188) and no test of its own uses them.
#pragma once

#include <atomic>
#include <chrono>
#include <deque>
#include <memory>
#include <mutex>

#include "provider.h"

namespace pplx::fabric {

enum class FaultKind : int {
  kNone = 0,
  kFailWrite = 1,     // the n-th write from now completes with an error, nothing is copied
  kDropWrite = 2,     // the n-th write from now vanishes: no copy, no completion, ever
  kDelayWrites = 3,   // completions of writes are held back for `value` milliseconds
  kReorderWrites = 4, // completions are released in batches of `value`, newest first
};

class FaultyDomain : public Domain {
 public:
  explicit FaultyDomain(std::unique_ptr<Domain> inner) : inner_(std::move(inner)) {}

  Domain& inner() { return *inner_; }
  // Arms one fault. `value`: see FaultKind. kNone clears delay and reorder.
  void inject(FaultKind kind, uint64_t value);
  // Completions currently held back (delayed or waiting for their batch).
  size_t held() const;

  const DomainInfo& info() const override { return inner_->info(); }
  DomainAddress address() const override { return inner_->address(); }
  MemoryRegionRemoteKey register_mr(uint64_t ptr, uint64_t len, int device) override {
    return inner_->register_mr(ptr, len, device);
  }
  void unregister_mr(uint64_t ptr) override { inner_->unregister_mr(ptr); }
  void submit_write(TransferId transfer_id, const DomainAddress& dst, WriteOp op) override;
  void submit_send(TransferId transfer_id, const DomainAddress& dst, std::string data) override {
    inner_->submit_send(transfer_id, dst, std::move(data));
  }
  void post_recvs(TransferId transfer_id, size_t count, size_t len) override {
    inner_->post_recvs(transfer_id, count, len);
  }
  void poll_progress(std::vector<DomainCompletion>* out) override;
  bool busy() const override;

 private:
  using Clock = std::chrono::steady_clock;
  struct Held {
    DomainCompletion completion;
    Clock::time_point release_at;
  };
  std::unique_ptr<Domain> inner_;
  mutable std::mutex mu_;       // inject() comes from other threads than the worker
  uint64_t writes_ = 0;         // writes seen so far
  uint64_t fail_at_ = 0, drop_at_ = 0;
  uint64_t delay_ms_ = 0, reorder_batch_ = 0;
  std::deque<DomainCompletion> injected_;  // error completions made here
  std::deque<Held> held_;
};

}  // namespace pplx::fabric
