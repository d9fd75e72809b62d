#include "domain_group.h"

#include <algorithm>

#include "../core/error.h"
#include "shard.h"

namespace pplx::fabric {

DomainGroup::DomainGroup(std::vector<std::unique_ptr<Domain>> domains) : domains_(std::move(domains)) {
  PPLX_REQUIRE(!domains_.empty(), "a domain group needs at least one domain");
}

uint64_t DomainGroup::aggregated_link_speed() const {
  uint64_t total = 0;
  for (const auto& d : domains_) total += d->info().link_speed;
  return total;
}

MemoryRegionDescriptor DomainGroup::register_mr(uint64_t ptr, uint64_t len, int device) {
  MemoryRegionDescriptor desc;
  desc.ptr = ptr;
  for (auto& d : domains_) desc.addr_rkey_list.emplace_back(d->address(), d->register_mr(ptr, len, device));
  return desc;
}

void DomainGroup::unregister_mr(uint64_t ptr) {
  for (auto& d : domains_) d->unregister_mr(ptr);
}

PeerGroupHandle DomainGroup::add_peer_group(std::vector<DomainAddress> main_addresses) {
  peer_groups_.push_back(std::move(main_addresses));
  return PeerGroupHandle{static_cast<uint32_t>(peer_groups_.size() - 1)};
}

void DomainGroup::check_descriptor(const MemoryRegionDescriptor& d) const {
  if (d.addr_rkey_list.size() != domains_.size()) {
    throw Error(ErrorKind::kInvalidArgument,
                "Number of target addresses must match the number of domains");
  }
}

void DomainGroup::track(TransferId id, size_t parts, std::optional<TransferCounter> counter) {
  Pending p;
  p.expected = parts;
  p.counter = std::move(counter);
  pending_[id] = std::move(p);
}

size_t DomainGroup::next_round_robin() {
  const size_t i = rr_next_;
  rr_next_ = (rr_next_ + 1) % domains_.size();
  return i;
}

void DomainGroup::submit(TransferId id, const TransferRequest& request,
                         std::optional<TransferCounter> counter) {
  std::visit(
      [&](const auto& r) {
        using T = std::decay_t<decltype(r)>;
        if constexpr (std::is_same_v<T, SingleTransferRequest>) submit_single(id, r, std::move(counter));
        else if constexpr (std::is_same_v<T, PagedTransferRequest>) submit_paged(id, r, std::move(counter));
        else if constexpr (std::is_same_v<T, ScatterTransferRequest>) submit_scatter(id, r, std::move(counter));
        else if constexpr (std::is_same_v<T, ImmTransferRequest>) submit_imm(id, r, std::move(counter));
        else submit_barrier(id, r, std::move(counter));
      },
      request);
}

void DomainGroup::submit_imm(TransferId id, const ImmTransferRequest& r, std::optional<TransferCounter> c) {
  check_descriptor(r.dst_mr);
  size_t i = 0;
  if (r.domain.kind == DomainGroupRouting::Kind::kPinned) {
    PPLX_REQUIRE(r.domain.domain_idx < domains_.size(), "DomainGroupRouting::Pinned.domain_idx is out of bounds");
    i = r.domain.domain_idx;
  } else {
    i = next_round_robin();
  }
  track(id, 1, std::move(c));
  WriteOp op;
  op.kind = WriteOp::Kind::kImm;
  op.imm = ImmWriteOp{r.imm_data, r.dst_mr.ptr, r.dst_mr.addr_rkey_list[i].second};
  domains_[i]->submit_write(id, r.dst_mr.addr_rkey_list[i].first, std::move(op));
}

void DomainGroup::submit_barrier(TransferId id, const BarrierTransferRequest& r,
                                 std::optional<TransferCounter> c) {
  for (const auto& d : r.dst_mrs) check_descriptor(d);
  size_t i = 0;
  if (r.domain.kind == DomainGroupRouting::Kind::kPinned) {
    PPLX_REQUIRE(r.domain.domain_idx < domains_.size(), "DomainGroupRouting::Pinned.domain_idx is out of bounds");
    i = r.domain.domain_idx;
  }
  if (r.dst_mrs.empty()) {
    track(id, 1, std::move(c));
    scratch_.push_back(DomainCompletion{DomainCompletion::Kind::kWriteDone, id, {}, 0, 1, {}});
    return;
  }
  track(id, r.dst_mrs.size(), std::move(c));
  for (const auto& d : r.dst_mrs) {
    WriteOp op;
    op.kind = WriteOp::Kind::kImm;
    op.imm = ImmWriteOp{r.imm_data, d.ptr, d.addr_rkey_list[i].second};
    domains_[i]->submit_write(id, d.addr_rkey_list[i].first, std::move(op));
  }
}

void DomainGroup::submit_single(TransferId id, const SingleTransferRequest& r,
                                std::optional<TransferCounter> c) {
  check_descriptor(r.dst_mr);
  size_t num_shards = 1;
  if (r.domain.kind == DomainGroupRouting::Kind::kRoundRobinSharded) {
    num_shards = r.domain.num_shards;
    PPLX_REQUIRE(num_shards >= 1, "num_shards must be positive");
    if (num_shards > domains_.size()) {
      throw Error(ErrorKind::kInvalidArgument,
                  "DomainGroupRouting::RoundRobinSharded.num_shards is greater than the number of domains");
    }
  } else {
    PPLX_REQUIRE(r.domain.domain_idx < domains_.size(), "DomainGroupRouting::Pinned.domain_idx is out of bounds");
  }
  const auto ranges = shard_single_transfer(r.length, num_shards);
  track(id, ranges.size(), std::move(c));
  for (const auto& [offset, len] : ranges) {
    const size_t i = r.domain.kind == DomainGroupRouting::Kind::kPinned ? r.domain.domain_idx
                                                                       : next_round_robin();
    WriteOp op;
    op.kind = WriteOp::Kind::kSingle;
    op.single.src_ptr = r.src_mr.ptr;
    op.single.src_offset = r.src_offset + offset;
    op.single.length = len;
    op.single.imm_data = r.imm_data;   // every shard carries the immediate: the receiver counts
    op.single.dst_ptr = r.dst_mr.ptr;
    op.single.dst_rkey = r.dst_mr.addr_rkey_list[i].second;
    op.single.dst_offset = len > 0 ? r.dst_offset + offset : 0;
    if (len == 0) op.single.src_offset = 0;
    domains_[i]->submit_write(id, r.dst_mr.addr_rkey_list[i].first, std::move(op));
  }
}

void DomainGroup::submit_paged(TransferId id, const PagedTransferRequest& r,
                               std::optional<TransferCounter> c) {
  check_descriptor(r.dst_mr);
  PPLX_REQUIRE(r.src_page_indices && r.dst_page_indices, "paged write needs both page lists");
  PPLX_REQUIRE(r.src_page_indices->size() == r.dst_page_indices->size(),
               "source and destination page lists differ in length");
  const size_t pages = r.src_page_indices->size();
  const auto runs = shard_pages(pages, domains_.size());
  if (runs.empty()) {
    track(id, 1, std::move(c));
    scratch_.push_back(DomainCompletion{DomainCompletion::Kind::kWriteDone, id, {}, 0, 1, {}});
    return;
  }
  track(id, runs.size(), std::move(c));
  for (const auto& [begin, end] : runs) {
    const size_t i = next_round_robin();
    WriteOp op;
    op.kind = WriteOp::Kind::kPaged;
    PagedWriteOp& p = op.paged;
    p.src_ptr = r.src_mr.ptr;
    p.length = r.length;
    p.src_page_indices = r.src_page_indices;
    p.dst_page_indices = r.dst_page_indices;
    p.page_begin = begin;
    p.page_end = end;
    p.src_stride = r.src_stride;
    p.src_offset = r.src_offset;
    p.dst_ptr = r.dst_mr.ptr;
    p.dst_rkey = r.dst_mr.addr_rkey_list[i].second;
    p.dst_stride = r.dst_stride;
    p.dst_offset = r.dst_offset;
    p.imm_data = r.imm_data;
    domains_[i]->submit_write(id, r.dst_mr.addr_rkey_list[i].first, std::move(op));
  }
}

void DomainGroup::submit_scatter(TransferId id, const ScatterTransferRequest& r,
                                 std::optional<TransferCounter> c) {
  PPLX_REQUIRE(r.dsts != nullptr, "scatter needs a target list");
  for (const auto& t : *r.dsts) check_descriptor(t.dst_mr);
  if (r.dst_handle.has_value()) {
    PPLX_REQUIRE(r.dst_handle->id < peer_groups_.size(), "unknown peer group handle");
    PPLX_REQUIRE(peer_groups_[r.dst_handle->id].size() == r.dsts->size(),
                 "scatter targets must match the peer group one to one");
  }
  const size_t n = domains_.size();
  struct Part {
    size_t domain;
    const ScatterTarget* target;
    uint64_t offset, length;
  };
  std::vector<Part> parts;
  switch (r.domain.kind) {
    case GroupTransferRouting::Kind::kSingle:
      PPLX_REQUIRE(r.domain.domain_idx < n, "GroupTransferRouting::Single.domain_idx is out of bounds");
      for (const auto& t : *r.dsts) parts.push_back({r.domain.domain_idx, &t, 0, t.length});
      break;
    case GroupTransferRouting::Kind::kAllDomainsShardPeers: {
      size_t peer = 0;
      for (const auto& t : *r.dsts) parts.push_back({(peer++) % n, &t, 0, t.length});
      break;
    }
    case GroupTransferRouting::Kind::kAllDomainsShardBytes:
      for (const auto& t : *r.dsts) {
        const auto ranges = shard_single_transfer(t.length, n);
        for (size_t i = 0; i < ranges.size(); ++i) {
          parts.push_back({i, &t, ranges[i].second ? ranges[i].first : 0, ranges[i].second});
        }
      }
      break;
  }
  if (parts.empty()) {
    track(id, 1, std::move(c));
    scratch_.push_back(DomainCompletion{DomainCompletion::Kind::kWriteDone, id, {}, 0, 1, {}});
    return;
  }
  track(id, parts.size(), std::move(c));
  for (const Part& p : parts) {
    WriteOp op;
    op.kind = WriteOp::Kind::kSingle;
    op.single.src_ptr = r.src_mr.ptr;
    op.single.src_offset = p.length ? p.target->src_offset + p.offset : 0;
    op.single.length = p.length;
    op.single.imm_data = r.imm_data;
    op.single.dst_ptr = p.target->dst_mr.ptr;
    op.single.dst_rkey = p.target->dst_mr.addr_rkey_list[p.domain].second;
    op.single.dst_offset = p.length ? p.target->dst_offset + p.offset : 0;
    domains_[p.domain]->submit_write(id, p.target->dst_mr.addr_rkey_list[p.domain].first, std::move(op));
  }
}

void DomainGroup::submit_send(TransferId id, const DomainAddress& dst, std::string data) {
  // two-sided traffic always uses the first domain
  domains_[0]->submit_send(id, dst, std::move(data));
}

void DomainGroup::post_recvs(TransferId id, size_t count, size_t len) { domains_[0]->post_recvs(id, count, len); }

void DomainGroup::poll(std::vector<GroupCompletion>* out) {
  for (auto& d : domains_) d->poll_progress(&scratch_);
  for (DomainCompletion& c : scratch_) {
    switch (c.kind) {
      case DomainCompletion::Kind::kSendDone:
        out->push_back(GroupCompletion{GroupCompletion::Kind::kSendDone, c.transfer_id, {}, 0, 1, {}});
        break;
      case DomainCompletion::Kind::kRecv:
        out->push_back(GroupCompletion{GroupCompletion::Kind::kRecv, c.transfer_id, std::move(c.data), 0, 1, {}});
        break;
      case DomainCompletion::Kind::kImm:
        out->push_back(GroupCompletion{GroupCompletion::Kind::kImm, 0, {}, c.imm, c.imm_count, {}});
        break;
      case DomainCompletion::Kind::kWriteDone:
      case DomainCompletion::Kind::kError: {
        auto it = pending_.find(c.transfer_id);
        if (it == pending_.end()) {
          // sends and receives are not tracked: pass their errors through
          if (c.kind == DomainCompletion::Kind::kError) {
            out->push_back(GroupCompletion{GroupCompletion::Kind::kError, c.transfer_id, {}, 0, 1, std::move(c.error)});
          }
          break;
        }
        Pending& p = it->second;
        ++p.seen;
        if (c.kind == DomainCompletion::Kind::kError && !p.failed) {
          p.failed = true;
          p.error = std::move(c.error);
        }
        if (p.seen == p.expected) {
          if (p.counter.has_value()) {
            if (p.failed) p.counter->mark_error(); else p.counter->mark_done();
          }
          if (p.failed) {
            out->push_back(GroupCompletion{GroupCompletion::Kind::kError, c.transfer_id, {}, 0, 1, std::move(p.error)});
          } else if (!p.counter.has_value()) {
            out->push_back(GroupCompletion{GroupCompletion::Kind::kTransferDone, c.transfer_id, {}, 0, 1, {}});
          }
          pending_.erase(it);
        }
        break;
      }
    }
  }
  scratch_.clear();
}

bool DomainGroup::busy() const {
  if (!pending_.empty()) return true;
  for (const auto& d : domains_) {
    if (d->busy()) return true;
  }
  return false;
}

}  // namespace pplx::fabric
