// Transport provider interface: one Domain is one endpoint (a NIC port in the RDMA
// providers, a copy queue of one GPU in the intra-box provider). A DomainGroup drives
// several domains of one GPU from a single worker thread, so a Domain is NOT thread safe:
// every method is called from its owning worker thread only.
//
// Reference: trait RdmaDomain (fabric-lib/src/provider.rs:16-72) and the provider-neutral
// operations in fabric-lib/src/rdma_op.rs:8-90.
#pragma once

#include <cstdint>
#include <memory>
#include <optional>
#include <string>
#include <vector>

#include "api.h"

namespace pplx::fabric {

struct DomainInfo {
  std::string name;          // e.g. "nvl0:cuda3", "mlx5_0"
  uint64_t link_speed = 0;   // bits per second
  std::string provider;      // "local", "verbs", "efa"
};

struct SingleWriteOp {
  uint64_t src_ptr = 0;      // base of the source region
  uint64_t src_offset = 0;
  uint64_t length = 0;
  std::optional<uint32_t> imm_data;
  uint64_t dst_ptr = 0;      // base of the destination region in the owner's address space
  MemoryRegionRemoteKey dst_rkey = 0;
  uint64_t dst_offset = 0;
};

struct ImmWriteOp {
  uint32_t imm_data = 0;
  uint64_t dst_ptr = 0;
  MemoryRegionRemoteKey dst_rkey = 0;
};

struct PagedWriteOp {
  uint64_t src_ptr = 0;
  uint64_t length = 0;       // bytes per page
  std::shared_ptr<const std::vector<uint32_t>> src_page_indices;
  std::shared_ptr<const std::vector<uint32_t>> dst_page_indices;
  size_t page_begin = 0, page_end = 0;  // the run of page slots this domain handles
  uint64_t src_stride = 0, src_offset = 0;
  uint64_t dst_ptr = 0;
  MemoryRegionRemoteKey dst_rkey = 0;
  uint64_t dst_stride = 0, dst_offset = 0;
  std::optional<uint32_t> imm_data;
};

struct WriteOp {
  enum class Kind { kSingle, kImm, kPaged } kind = Kind::kSingle;
  SingleWriteOp single;
  ImmWriteOp imm;
  PagedWriteOp paged;
};

struct DomainCompletion {
  enum class Kind { kWriteDone, kSendDone, kRecv, kImm, kError } kind;
  TransferId transfer_id = 0;
  std::string data;       // kRecv
  uint32_t imm = 0;       // kImm
  uint32_t imm_count = 1; // kImm: arrivals coalesced into this entry
  std::string error;      // kError
};

class Domain {
 public:
  virtual ~Domain() = default;
  virtual const DomainInfo& info() const = 0;
  virtual DomainAddress address() const = 0;

  // `device` is a CUDA ordinal, or -1 for host memory. Returns the key peers must quote.
  virtual MemoryRegionRemoteKey register_mr(uint64_t ptr, uint64_t len, int device) = 0;
  virtual void unregister_mr(uint64_t ptr) = 0;

  // One-sided write (or bare immediate) towards `dst`. Completion (kWriteDone or kError)
  // is reported by poll_progress under `transfer_id`.
  virtual void submit_write(TransferId transfer_id, const DomainAddress& dst, WriteOp op) = 0;
  // Two-sided message; completion kSendDone.
  virtual void submit_send(TransferId transfer_id, const DomainAddress& dst, std::string data) = 0;
  // Allows `count` more incoming messages of up to `len` bytes to be delivered as kRecv
  // under `transfer_id`.
  virtual void post_recvs(TransferId transfer_id, size_t count, size_t len) = 0;

  // Makes progress and appends whatever completed.
  virtual void poll_progress(std::vector<DomainCompletion>* out) = 0;
  // True while operations are in flight (the worker then polls without sleeping).
  virtual bool busy() const = 0;
};

}  // namespace pplx::fabric
