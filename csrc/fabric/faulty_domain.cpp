#include "faulty_domain.h"

#include <algorithm>

namespace pplx::fabric {

void FaultyDomain::inject(FaultKind kind, uint64_t value) {
  std::lock_guard<std::mutex> lock(mu_);
  switch (kind) {
    case FaultKind::kNone:
      fail_at_ = drop_at_ = delay_ms_ = reorder_batch_ = 0;
      break;
    case FaultKind::kFailWrite:
      fail_at_ = value == 0 ? 0 : writes_ + value;
      break;
    case FaultKind::kDropWrite:
      drop_at_ = value == 0 ? 0 : writes_ + value;
      break;
    case FaultKind::kDelayWrites:
      delay_ms_ = value;
      break;
    case FaultKind::kReorderWrites:
      reorder_batch_ = value;
      break;
  }
}

size_t FaultyDomain::held() const {
  std::lock_guard<std::mutex> lock(mu_);
  return held_.size();
}

void FaultyDomain::submit_write(TransferId transfer_id, const DomainAddress& dst, WriteOp op) {
  {
    std::lock_guard<std::mutex> lock(mu_);
    ++writes_;
    if (fail_at_ != 0 && writes_ == fail_at_) {
      fail_at_ = 0;
      DomainCompletion c;
      c.kind = DomainCompletion::Kind::kError;
      c.transfer_id = transfer_id;
      c.error = "injected write failure";
      injected_.push_back(std::move(c));
      return;
    }
    if (drop_at_ != 0 && writes_ == drop_at_) {
      drop_at_ = 0;
      return;  // as if the message had been lost for good
    }
  }
  inner_->submit_write(transfer_id, dst, std::move(op));
}

void FaultyDomain::poll_progress(std::vector<DomainCompletion>* out) {
  std::vector<DomainCompletion> fresh;
  inner_->poll_progress(&fresh);
  std::lock_guard<std::mutex> lock(mu_);
  while (!injected_.empty()) {
    out->push_back(std::move(injected_.front()));
    injected_.pop_front();
  }
  const Clock::time_point now = Clock::now();
  for (DomainCompletion& c : fresh) {
    const bool is_write = c.kind == DomainCompletion::Kind::kWriteDone;
    if (is_write && (delay_ms_ != 0 || reorder_batch_ > 1)) {
      held_.push_back(Held{std::move(c), now + std::chrono::milliseconds(delay_ms_)});
    } else {
      out->push_back(std::move(c));
    }
  }
  if (held_.empty()) return;
  if (reorder_batch_ > 1) {
    // whole batches whose members are all due, newest member first
    while (held_.size() >= reorder_batch_) {
      bool due = true;
      for (size_t i = 0; i < reorder_batch_; ++i) due &= held_[i].release_at <= now;
      if (!due) break;
      for (size_t i = reorder_batch_; i-- > 0;) out->push_back(std::move(held_[i].completion));
      held_.erase(held_.begin(), held_.begin() + static_cast<long>(reorder_batch_));
    }
  } else {
    while (!held_.empty() && held_.front().release_at <= now) {
      out->push_back(std::move(held_.front().completion));
      held_.pop_front();
    }
  }
  if (delay_ms_ == 0 && reorder_batch_ <= 1) {
    // faults were cleared: let everything go
    while (!held_.empty()) {
      out->push_back(std::move(held_.front().completion));
      held_.pop_front();
    }
  }
}

bool FaultyDomain::busy() const {
  if (inner_->busy()) return true;
  std::lock_guard<std::mutex> lock(mu_);
  // a partial reorder batch waits for more writes, not for time: it must not keep the worker spinning
  const bool timed = delay_ms_ != 0 && !held_.empty();
  return !injected_.empty() || timed;
}

}  // namespace pplx::fabric
