// Host proxy of the all-to-all for ranks outside this rank's NVLink domain.
//
// Inside the domain the kernels write into their peers' memory themselves. A rank outside it
// is not mapped here, so the kernels write what is bound for it into local buffers that mirror
// the remote layout (dispatch: counts and records; combine: rows packed densely plus the slot
// each row belongs in) and tell this thread through a word of pinned host memory. The thread
// then moves the bytes with the transfer engine and, once they have all landed, writes the
// arrival flag the remote kernels wait on, again through the engine:
//
//   dispatch  kernel: "send phase n done"  ->  per remote rank: counts slice, record slice
//             -> wait for the completions -> flag "dispatch n started" at every remote rank
//   combine   kernel: "send phase n done"  ->  per remote origin rank: paged write of its rows
//             (dense source pages, destination page = the row's combine slot)
//             -> wait -> flag "combine n delivered" at every remote rank
//
// The flag always travels after the data it announces, so a receiver that sees it may read.
// A failed transfer marks the proxy failed; the context then reports it on the next call, as
// the reference does (p2p-all-to-all/src/a2a_context.rs:332-334).
//
// This is the counterpart of the reference's worker (p2p-all-to-all/src/a2a_worker.rs:340-455,
// scatter of counts :348-354, token scatter :457-523, barrier :778-802). It is much thinner:
// the expert-major layout, the offsets and the combine positions are computed by the kernels
// from the counts, so there is no routing table to build on the host
// (process_routing_info, :526-776) and no table to push to the GPU.
#pragma once

#include <atomic>
#include <memory>
#include <string>
#include <thread>
#include <vector>

#include "../fabric/transfer_engine.h"
#include "a2a_types.h"

namespace pplx {

struct A2AProxyPeer {
  int rank = -1;
  fabric::MemoryRegionDescriptor sync_desc;  // the peer's sync region
  fabric::MemoryRegionDescriptor recv_desc;  // the peer's receive region
};

// Local buffers, all registered with the engine by the caller (the handle is the base pointer).
struct A2AProxyBuffers {
  uint64_t shadow_sync[kMaxRanks] = {};  // stand-in for rank d's sync region, 0 for ranks in the domain
  uint64_t shadow_recv[kMaxRanks] = {};  // stand-in for this rank's group slice of rank d's dispatch records
  uint64_t stage = 0;                    // combine rows for ranks outside the domain, dense
  uint64_t flag_source = 0;              // pinned host words the flags are written from
  volatile uint32_t* flag_source_host = nullptr;  // the same words as the host sees them
  volatile uint32_t* proxy_words = nullptr;       // A2AProxyWord block (host pointer)
  const volatile uint32_t* stage_slot = nullptr;  // combine slot of every staged row (host pointer)
};

class A2AProxy {
 public:
  A2AProxy(const A2AConfig& cfg, int rank, fabric::TransferEngine* engine, std::vector<A2AProxyPeer> peers,
           const A2AProxyBuffers& buffers, int pin_cpu);
  ~A2AProxy();
  A2AProxy(const A2AProxy&) = delete;
  A2AProxy& operator=(const A2AProxy&) = delete;

  bool failed() const { return failed_.load(std::memory_order_acquire); }
  std::string error() const;
  // Dispatches and combines served so far.
  uint32_t dispatches() const { return dispatches_.load(); }
  uint32_t combines() const { return combines_.load(); }

 private:
  void loop();
  void serve_dispatch(uint32_t tag);
  void serve_combine(uint32_t tag);
  // Submits and waits (bounded by the context's wait limit); false on error or timeout.
  bool run(std::vector<fabric::TransferRequest> requests, const char* what);
  bool send_flags(int row, uint32_t tag, const char* what);
  void fail(const std::string& why);

  A2AConfig cfg_;
  int rank_;
  fabric::TransferEngine* engine_;
  std::vector<A2AProxyPeer> peers_;
  A2AProxyBuffers buf_;
  int pin_cpu_;
  std::atomic<bool> stop_{false};
  std::atomic<bool> failed_{false};
  std::atomic<uint32_t> dispatches_{0}, combines_{0};
  mutable std::mutex error_mu_;
  std::string error_;
  std::thread thread_;
};

}  // namespace pplx
