// Host side of one all-to-all context: wire-format/layout arithmetic, the device-local
// workspace, launch wrappers and the status word.
//
// Counterpart of the reference's AllToAllContext (p2p-all-to-all/src/a2a_context.rs:15-488).
// There is no worker thread to spawn or join: the reference's host proxy
// (p2p-all-to-all/src/a2a_worker.rs:340-455) has no equivalent because counts, tokens and
// arrival signals all move as NVLink peer stores issued by the kernels.
#pragma once

#include <cuda_runtime.h>

#include <array>
#include <cstdint>
#include <string>
#include <vector>

#include "a2a_proxy.h"
#include "a2a_types.h"

namespace pplx {

struct A2AParams {
  int world = 1;
  int dp_size = 1;
  int num_experts = 0;
  int topk = 0;
  int max_num_tokens = 0;
  int hidden_dim = 0;
  int hidden_dim_scale = 0;
  int in_elemsize = 2;
  int out_elemsize = 2;
  int scale_elemsize = 4;
  int expert_padding = 1;
  int combine_mode = kCombinePerRoute;
  int wire = kWireAuto;        // auto: flagged lines up to 512 tokens per call, plain above;
                               // PPLX_A2A_WIRE=ll|plain overrides an automatic choice
  // Ranks whose memory is mapped into this process (bit r = rank r, own rank included); 0 means
  // all of them. The others are reached through a transfer engine by a host proxy
  // (A2AContext::enable_proxy), which needs the plain wire format.
  uint32_t node_mask = 0;
  int num_blocks = 0;          // 0: one block per SM (divided among virtual ranks)
  int64_t wait_limit_ms = 0;   // 0: PPLX_A2A_TIMEOUT_MS or 10 s
};

// Pure arithmetic (no CUDA): validated config with wire format and symmetric layout.
A2AConfig a2a_make_config(const A2AParams& p, int num_sms, int virtual_ranks);

struct A2AStatusInfo {
  uint32_t code = 0, phase = 0, who = 0, detail = 0;
  std::string message() const;
};

// What a kernel other than combine_send needs in order to play the combine's send phase
// itself: where each received row goes and how to tell the receivers that it got there.
struct A2AScatterInfo {
  const uint32_t* row_src;         // [max_recv_rows] rank a row's token came from, kNoSlot = padding
  const uint32_t* row_tk;          // [max_recv_rows] token * topk + k at that rank
  uint8_t* peer_recv[kMaxRanks];   // combine receive area of every rank as mapped here
  uint64_t slot_stride;            // bytes per (token, k) slot
  uint32_t* peer_flag[kMaxRanks];  // this rank's combine arrival counter at every rank
  int world;
  uint32_t signal_value;           // what the sender adds to each flag once all its rows are written
  uint32_t* done_counter;          // scratch word, zero between launches
  const uint32_t* status;          // this rank's status word
};

class A2AContext {
 public:
  // `ranks` lists the ranks this process plays (one entry in a real multi-GPU run).
  // sync_ptrs[i][p] / recv_ptrs[i][p]: rank p's symmetric regions as mapped for ranks[i].
  A2AContext(const A2AParams& params, int device, const std::vector<int>& ranks,
             const std::vector<std::vector<uint64_t>>& sync_ptrs,
             const std::vector<std::vector<uint64_t>>& recv_ptrs);
  ~A2AContext();
  A2AContext(const A2AContext&) = delete;
  A2AContext& operator=(const A2AContext&) = delete;

  const A2AConfig& config() const { return cfg_; }
  int num_local_ranks() const { return static_cast<int>(ranks_.size()); }
  int device() const { return device_; }

  void dispatch(const DispatchSendArgs* send, const DispatchRecvArgs* recv, bool do_send,
                bool do_recv, cudaStream_t stream);
  void combine(const CombineSendArgs* send, const CombineRecvArgs* recv, bool do_send,
               bool do_recv, int y_dtype, int out_dtype, cudaStream_t stream);

  // Serves the ranks outside the NVLink domain of local rank `i` (those missing from
  // A2AParams::node_mask): allocates the stand-in buffers the kernels write into instead of the
  // unreachable peers, registers them with `engine` and starts the proxy thread that forwards
  // them. `peers` names every such rank with the descriptors of its sync and receive regions.
  // Call once per local rank, before the first dispatch. The engine must outlive the context.
  void enable_proxy(int i, fabric::TransferEngine* engine, std::vector<A2AProxyPeer> peers, int pin_cpu);

  // (dispatches, combines) the proxy of local rank `i` has forwarded; zeros without a proxy.
  std::array<uint32_t, 2> proxy_counters(int i = 0) const {
    if (i < 0 || static_cast<size_t>(i) >= proxies_.size() || !proxies_[i].proxy) return {0, 0};
    return {proxies_[i].proxy->dispatches(), proxies_[i].proxy->combines()};
  }

  // All ranks of the context meet on the device: returns (in stream order) once every rank has
  // entered. Bounded like every other wait. Collective; may be called between any two phases.
  void barrier(cudaStream_t stream);

  // The send phase of a combine done by somebody else's kernel (the down projection's epilogue
  // writes the rows into the peers' buffers and signals): advances the phase order as
  // combine(do_send only) would and returns, for every local rank, what that kernel needs.
  // Only for per-route combines without replication (dp_size 1) and 2-byte outputs.
  std::vector<A2AScatterInfo> combine_send_external();

  // Synchronous read of the status word of local rank `i` (does not wait for the stream).
  A2AStatusInfo status(int i = 0) const;
  // True once any kernel of this context reported a failure. Reads a pinned host word:
  // no stream synchronisation, safe to call after every launch.
  bool failed() const;
  // Throws pplx::Error when any local rank recorded a failure.
  void check() const;
  // [tokens sent, reserved, max dispatch wait ns, max combine wait ns, ...]
  std::array<uint64_t, 8> stats(int i = 0) const;
  // [completed dispatches, completed combines]
  std::array<uint32_t, 2> iterations(int i = 0) const;
  // Timeline of the last launches (globaltimer ns; see A2ATrace), filled when the context
  // was created with PPLX_A2A_TRACE=1.
  std::array<uint64_t, kTraceSlots> trace(int i = 0) const;
  void set_team_override(int team) { team_override_ = team; }
  // Test hook: pretend the phases before `phase` were already issued.
  void debug_set_next_phase(int phase) { next_phase_ = phase; }

 private:
  int pick(int64_t items, int64_t vectors_per_item) const;
  void require_phase(int first) const;
  void commit_phase(int last);
  void require_proxies() const;

  A2AConfig cfg_{};
  int device_;
  std::vector<int> ranks_;
  A2ARankStates states_{};
  std::vector<void*> allocations_;
  std::vector<uint32_t*> status_ptrs_;
  std::vector<uint32_t*> host_flags_;
  std::vector<unsigned long long*> stats_ptrs_;
  std::vector<uint32_t*> iters_ptrs_;
  std::vector<unsigned long long*> trace_ptrs_;
  std::vector<uint32_t*> scatter_done_ptrs_;
  int next_phase_ = kPhaseDispatchSend;
  int64_t last_tokens_ = 0;
  int team_override_ = 0;
  bool external_send_ = false;  // the pending combine's send phase was played by another kernel
  struct ProxyState {
    std::unique_ptr<A2AProxy> proxy;
    fabric::TransferEngine* engine = nullptr;
    std::vector<uint64_t> registered;   // regions registered with the engine
    std::vector<void*> device_buffers;  // cudaMalloc
    std::vector<void*> host_buffers;    // cudaHostAlloc
  };
  std::vector<ProxyState> proxies_;
};

}  // namespace pplx
