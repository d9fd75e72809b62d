// Several domains (NIC ports / copy queues) of one GPU driven as one unit: registers
// memory on all of them, spreads single writes by bytes and paged writes by pages, fans
// scatters out by peer or by bytes, and merges the per-domain completions of one transfer.
// Reference: DomainGroup<D, N> in fabric-lib/src/domain_group.rs:52-550.
#pragma once

#include <map>
#include <memory>
#include <unordered_map>
#include <vector>

#include "api.h"
#include "provider.h"

namespace pplx::fabric {

struct GroupCompletion {
  enum class Kind { kTransferDone, kSendDone, kRecv, kImm, kError } kind;
  TransferId transfer_id = 0;
  std::string data;
  uint32_t imm = 0;
  uint32_t imm_count = 1;
  std::string error;
};

class DomainGroup {
 public:
  explicit DomainGroup(std::vector<std::unique_ptr<Domain>> domains);

  size_t num_domains() const { return domains_.size(); }
  Domain& domain(size_t i) { return *domains_[i]; }
  DomainAddress main_address() const { return domains_[0]->address(); }
  uint64_t aggregated_link_speed() const;

  // Registers on every domain; the descriptor lists one (address, key) per domain.
  MemoryRegionDescriptor register_mr(uint64_t ptr, uint64_t len, int device);
  void unregister_mr(uint64_t ptr);

  // Pre-resolved list of peers for scatters (one descriptor list index per peer).
  PeerGroupHandle add_peer_group(std::vector<DomainAddress> main_addresses);

  // Throws pplx::Error(kInvalidArgument) when the request does not fit the group
  // (wrong number of remote addresses, shard count above the domain count, ...).
  void submit(TransferId id, const TransferRequest& request,
              std::optional<TransferCounter> counter = std::nullopt);
  void submit_send(TransferId id, const DomainAddress& dst, std::string data);
  void post_recvs(TransferId id, size_t count, size_t len);

  void poll(std::vector<GroupCompletion>* out);
  bool busy() const;

 private:
  struct Pending {
    size_t expected = 0;   // per-domain completions still to come
    size_t seen = 0;
    bool failed = false;
    std::string error;
    std::optional<TransferCounter> counter;
  };
  void track(TransferId id, size_t parts, std::optional<TransferCounter> counter);
  size_t next_round_robin();
  void submit_single(TransferId id, const SingleTransferRequest& r, std::optional<TransferCounter> c);
  void submit_paged(TransferId id, const PagedTransferRequest& r, std::optional<TransferCounter> c);
  void submit_scatter(TransferId id, const ScatterTransferRequest& r, std::optional<TransferCounter> c);
  void submit_imm(TransferId id, const ImmTransferRequest& r, std::optional<TransferCounter> c);
  void submit_barrier(TransferId id, const BarrierTransferRequest& r, std::optional<TransferCounter> c);
  void check_descriptor(const MemoryRegionDescriptor& d) const;

  std::vector<std::unique_ptr<Domain>> domains_;
  std::unordered_map<TransferId, Pending> pending_;
  std::vector<std::vector<DomainAddress>> peer_groups_;
  size_t rr_next_ = 0;
  std::vector<DomainCompletion> scratch_;
};

}  // namespace pplx::fabric
