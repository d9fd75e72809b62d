// Public value types of the transfer engine: addresses, memory-region handles and
// descriptors, transfer requests, routing policies, completion entries and counters.
// They mirror the reference's fabric-lib/src/api.rs:26-258 one to one, so that code (and
// pickles of descriptors exchanged between ranks) keeps its shape; the wire encoding is
// this library's own.
#pragma once

#include <atomic>
#include <cstdint>
#include <memory>
#include <optional>
#include <string>
#include <utility>
#include <variant>
#include <vector>

namespace pplx::fabric {

using TransferId = uint64_t;

// Opaque bytes that identify one domain (one transport endpoint) of one process.
class DomainAddress {
 public:
  DomainAddress() = default;
  explicit DomainAddress(std::string bytes) : bytes_(std::move(bytes)) {}
  const std::string& bytes() const { return bytes_; }
  std::string to_hex() const;                       // lower-case hex, as printed
  static DomainAddress from_hex(const std::string& hex);
  bool operator==(const DomainAddress& o) const { return bytes_ == o.bytes_; }
  bool operator!=(const DomainAddress& o) const { return bytes_ != o.bytes_; }
  bool operator<(const DomainAddress& o) const { return bytes_ < o.bytes_; }
  size_t hash() const { return std::hash<std::string>()(bytes_); }

 private:
  std::string bytes_;
};

// Local handle of a registered region: its base pointer.
struct MemoryRegionHandle {
  uint64_t ptr = 0;
};

using MemoryRegionRemoteKey = uint64_t;

// What a peer needs to write into a region: the base pointer in the owner's address
// space and one (address, key) pair per domain the owner registered it with.
struct MemoryRegionDescriptor {
  uint64_t ptr = 0;
  std::vector<std::pair<DomainAddress, MemoryRegionRemoteKey>> addr_rkey_list;

  std::string serialize() const;
  static MemoryRegionDescriptor deserialize(const std::string& bytes);
  std::string debug_str() const;
};

struct UvmWatcherId {
  uint32_t slot = 0;
  uint32_t generation = 0;
};

// ---- routing ----
struct DomainGroupRouting {
  enum class Kind { kRoundRobinSharded, kPinned } kind = Kind::kRoundRobinSharded;
  uint8_t num_shards = 1;  // kRoundRobinSharded
  uint8_t domain_idx = 0;  // kPinned
  static DomainGroupRouting sharded(uint8_t n) { return {Kind::kRoundRobinSharded, n, 0}; }
  static DomainGroupRouting pinned(uint8_t i) { return {Kind::kPinned, 1, i}; }
};

struct GroupTransferRouting {
  enum class Kind { kAllDomainsShardPeers, kAllDomainsShardBytes, kSingle } kind =
      Kind::kAllDomainsShardPeers;
  uint8_t domain_idx = 0;  // kSingle
};

// ---- requests ----
struct ImmTransferRequest {
  uint32_t imm_data = 0;
  MemoryRegionDescriptor dst_mr;
  DomainGroupRouting domain;
};

struct BarrierTransferRequest {
  uint32_t imm_data = 0;
  std::vector<MemoryRegionDescriptor> dst_mrs;
  DomainGroupRouting domain;
};

struct SingleTransferRequest {
  MemoryRegionHandle src_mr;
  uint64_t src_offset = 0;
  uint64_t length = 0;
  std::optional<uint32_t> imm_data;
  MemoryRegionDescriptor dst_mr;
  uint64_t dst_offset = 0;
  DomainGroupRouting domain;
};

struct PagedTransferRequest {
  uint64_t length = 0;  // bytes per page
  MemoryRegionHandle src_mr;
  std::shared_ptr<const std::vector<uint32_t>> src_page_indices;
  uint64_t src_stride = 0;
  uint64_t src_offset = 0;
  MemoryRegionDescriptor dst_mr;
  std::shared_ptr<const std::vector<uint32_t>> dst_page_indices;
  uint64_t dst_stride = 0;
  uint64_t dst_offset = 0;
  std::optional<uint32_t> imm_data;
};

struct PeerGroupHandle {
  uint32_t id = 0;
};

struct ScatterTarget {
  MemoryRegionDescriptor dst_mr;
  uint64_t length = 0;
  uint64_t src_offset = 0;
  uint64_t dst_offset = 0;
};

struct ScatterTransferRequest {
  MemoryRegionHandle src_mr;
  std::optional<PeerGroupHandle> dst_handle;
  std::shared_ptr<const std::vector<ScatterTarget>> dsts;
  std::optional<uint32_t> imm_data;
  GroupTransferRouting domain;
};

using TransferRequest = std::variant<ImmTransferRequest, SingleTransferRequest, PagedTransferRequest,
                                     ScatterTransferRequest, BarrierTransferRequest>;

// ---- completions ----
struct TransferCompletionEntry {
  enum class Kind { kRecv, kSend, kTransfer, kImmData, kImmCountReached, kUvmWatch, kError } kind;
  TransferId transfer_id = 0;
  size_t data_len = 0;        // kRecv
  std::string data;           // kRecv payload
  uint32_t imm = 0;           // kImmData / kImmCountReached
  UvmWatcherId watcher;       // kUvmWatch
  uint64_t old_value = 0, new_value = 0;
  std::string error;          // kError
};

// A free-running arrival counter the user can block on: wait(n) consumes n arrivals.
class ImmCounter {
 public:
  explicit ImmCounter(std::shared_ptr<std::atomic<int64_t>> c) : counter_(std::move(c)) {}
  // Returns false if `deadline_ms` (>= 0) elapsed first; a negative deadline waits forever.
  bool wait(uint32_t target, int64_t deadline_ms = -1) const;
  int64_t value() const { return counter_->load(std::memory_order_relaxed); }

 private:
  std::shared_ptr<std::atomic<int64_t>> counter_;
};

// Completion counters for submit_transfer_atomic: `done` counts finished transfers
// (successful or not), `errors` the failed ones.
class TransferCounter {
 public:
  TransferCounter(std::shared_ptr<std::atomic<int64_t>> done,
                  std::shared_ptr<std::atomic<int64_t>> errors)
      : done_(std::move(done)), errors_(std::move(errors)) {}
  void mark_done() const { done_->fetch_add(1, std::memory_order_release); }
  void mark_error() const {
    errors_->fetch_add(1, std::memory_order_release);
    done_->fetch_add(1, std::memory_order_release);
  }
  int64_t done() const { return done_->load(std::memory_order_acquire); }
  int64_t errors() const { return errors_->load(std::memory_order_acquire); }

 private:
  std::shared_ptr<std::atomic<int64_t>> done_;
  std::shared_ptr<std::atomic<int64_t>> errors_;
};

// ---- helpers shared by tests and providers ----
std::string hex_encode(const std::string& bytes);
std::string hex_decode(const std::string& hex);  // throws pplx::Error on bad input

}  // namespace pplx::fabric

namespace std {
template <>
struct hash<pplx::fabric::DomainAddress> {
  size_t operator()(const pplx::fabric::DomainAddress& a) const { return a.hash(); }
};
}  // namespace std
