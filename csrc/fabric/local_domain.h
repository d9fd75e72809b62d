// Intra-box transport provider: one-sided writes between the GPUs (and host memory) of one
// machine without a NIC.
//
//   * device -> device   the peer-copy kernel (peer_copy.h) writes straight into the
//                        destination over NVLink; a region owned by another process is
//                        mapped through its CUDA IPC handle on first use;
//   * host memory        memcpy inside one process, chunks over the control socket between
//                        processes;
//   * immediates, two-sided messages, region look-ups travel over an abstract unix
//     datagram socket per domain (or a direct queue when both ends share a process);
//     a write's immediate is sent after the copy's CUDA event has completed, so its
//     arrival implies the data is visible.
//
// It implements the same Domain interface the RDMA providers of the reference implement
// (VerbsDomain: fabric-lib/src/verbs/verbs_domain.rs, EfaDomain: fabric-lib/src/efa/
// efa_domain.rs) and keeps their semantics: reliable, unordered, every page of a paged
// write counts as one immediate at the receiver.
#pragma once

#include <cuda_runtime.h>

#include <deque>
#include <map>
#include <mutex>
#include <unordered_map>

#include "provider.h"

namespace pplx::fabric {

class LocalDomain : public Domain {
 public:
  // `device`: CUDA ordinal whose copy queue this domain drives, or -1 for a host-only
  // domain (CPU tests, machines without a GPU).
  LocalDomain(int device, int index);
  ~LocalDomain() override;

  const DomainInfo& info() const override { return info_; }
  DomainAddress address() const override { return address_; }
  MemoryRegionRemoteKey register_mr(uint64_t ptr, uint64_t len, int device) override;
  void unregister_mr(uint64_t ptr) override;
  void submit_write(TransferId transfer_id, const DomainAddress& dst, WriteOp op) override;
  void submit_send(TransferId transfer_id, const DomainAddress& dst, std::string data) override;
  void post_recvs(TransferId transfer_id, size_t count, size_t len) override;
  void poll_progress(std::vector<DomainCompletion>* out) override;
  bool busy() const override;

  // Test hook: fail (kError) the n-th write submitted from now on (1-based; 0 disables).
  void inject_write_failure(uint64_t nth) { fail_write_at_ = writes_submitted_ + nth; }

 private:
  struct Region {
    uint64_t ptr = 0, len = 0;
    int device = -1;
    MemoryRegionRemoteKey rkey = 0;
    bool has_ipc = false;
    cudaIpcMemHandle_t ipc{};
    uint64_t ipc_offset = 0;  // ptr - allocation base
    // CUDA virtual-memory allocations (cuMemCreate) have no IPC handle: they travel as a POSIX
    // file descriptor that the importer fetches from this process's descriptor server
    int vmm_fd = -1;
    uint64_t vmm_size = 0;    // bytes of the whole allocation; ipc_offset is the offset into it
  };
  struct RemoteRegion {
    bool resolved = false;
    bool same_process = false;
    int device = -1;
    uint64_t owner_ptr = 0, len = 0;
    uint8_t* mapped = nullptr;  // usable base pointer here (device regions), else nullptr
    void* ipc_base = nullptr;   // to close
    uint64_t vmm_va = 0, vmm_size = 0;   // to unmap (imported virtual-memory allocation)
  };
  struct Message {
    uint32_t type = 0;
    uint64_t a = 0, b = 0;
    uint32_t c = 0;
    std::string payload;
    DomainAddress from;
  };
  struct PendingWrite {
    TransferId id = 0;
    DomainAddress dst;
    WriteOp op;
  };
  struct InFlight {
    TransferId id = 0;
    cudaEvent_t event = nullptr;
    DomainAddress dst;
    bool has_imm = false;
    uint32_t imm = 0, imm_count = 0;
    uint32_t* error_flag = nullptr;  // pinned host word the kernel may raise
  };

  static LocalDomain* find_local(const DomainAddress& addr);
  void deliver(const DomainAddress& dst, Message msg);  // direct queue or socket
  void handle(Message& msg, std::vector<DomainCompletion>* out);
  void drain_socket(std::vector<DomainCompletion>* out);
  RemoteRegion& remote(const DomainAddress& dst, MemoryRegionRemoteKey rkey);
  void start_write(PendingWrite w, std::vector<DomainCompletion>* out);
  void run_write(const PendingWrite& w, RemoteRegion& rr, std::vector<DomainCompletion>* out);
  std::string region_info(const Region& r) const;
  void ensure_stream();
  uint32_t* device_scratch(size_t words);

  DomainInfo info_;
  DomainAddress address_;
  int device_;
  int sock_ = -1;
  cudaStream_t stream_ = nullptr;
  uint32_t* scratch_ = nullptr;
  size_t scratch_words_ = 0;
  uint32_t* error_flag_host_ = nullptr;  // pinned + mapped
  uint32_t* error_flag_dev_ = nullptr;

  std::mutex regions_mu_;                         // other domains of the process look regions up
  std::map<uint64_t, Region> regions_;            // by ptr
  std::map<MemoryRegionRemoteKey, uint64_t> by_rkey_;
  MemoryRegionRemoteKey next_rkey_ = 1;

  std::map<std::pair<DomainAddress, MemoryRegionRemoteKey>, RemoteRegion> remotes_;
  std::map<std::pair<DomainAddress, MemoryRegionRemoteKey>, std::vector<PendingWrite>> waiting_mr_;
  std::deque<InFlight> in_flight_;
  std::deque<DomainCompletion> ready_;

  struct RecvCredit {
    TransferId id;
    size_t remaining;
    size_t len;
  };
  std::deque<RecvCredit> recv_credits_;
  std::deque<Message> unclaimed_;  // messages that arrived before a receive was posted

  std::mutex inbox_mu_;
  std::deque<Message> inbox_;  // deliveries from other domains of this process

  std::unordered_map<TransferId, size_t> host_write_acks_;  // outstanding cross-process host writes
  uint64_t writes_submitted_ = 0;
  uint64_t fail_write_at_ = 0;
  uint64_t stuck_polls_ = 0;   // polls since the oldest copy in flight last made progress
};

}  // namespace pplx::fabric
