// The transfer engine: worker threads that drive the domain groups (one per GPU), a UVM
// watcher thread, and a callback thread that turns completions into user callbacks.
//
// Layering follows the reference: Worker (fabric-lib/src/worker.rs:137-599) ->
// FabricEngine (fabric_engine.rs:27-343) -> TransferEngine (transfer_engine.rs:68-550),
// built through TransferEngineBuilder (transfer_engine_builder.rs:18-103). Blocking calls
// (register, add_peer_group) are executed on the owning worker thread and waited for;
// submissions are queued and return at once; callbacks run on the callback thread.
#pragma once

#include <atomic>
#include <condition_variable>
#include <deque>
#include <functional>
#include <future>
#include <map>
#include <memory>
#include <mutex>
#include <thread>
#include <unordered_map>

#include "api.h"
#include "domain_group.h"
#include "host_buffer.h"
#include "imm_count.h"
#include "topo.h"

namespace pplx::fabric {

using DomainFactory = std::function<std::unique_ptr<Domain>(int device, int index, const DomainInfo&)>;

struct GpuDomainSpec {
  int cuda_device = -1;
  std::vector<DomainInfo> domains;
  int pin_worker_cpu = -1;
  int pin_uvm_cpu = -1;
};

class UvmWatcher {
 public:
  uint64_t ptr() const { return ptr_; }   // address of the watched 64-bit word (host mapped)
  UvmWatcherId id() const { return id_; }

 private:
  friend class TransferEngine;
  uint64_t ptr_ = 0;
  UvmWatcherId id_;
};

class TransferEngine {
 public:
  using DoneFn = std::function<void()>;
  using ErrorFn = std::function<void(const std::string&)>;
  using RecvFn = std::function<void(const std::string&)>;
  using ImmFn = std::function<void(uint32_t)>;
  using WatchFn = std::function<bool(uint64_t old_value, uint64_t new_value)>;

  // `factory` creates the domains (default: the intra-box provider).
  explicit TransferEngine(std::vector<GpuDomainSpec> gpus, DomainFactory factory = nullptr);
  ~TransferEngine();
  TransferEngine(const TransferEngine&) = delete;
  TransferEngine& operator=(const TransferEngine&) = delete;

  DomainAddress main_address() const { return main_address_; }
  size_t num_domains() const { return num_domains_; }
  size_t nets_per_gpu() const { return nets_per_gpu_; }
  uint64_t aggregated_link_speed() const { return link_speed_; }
  void stop();
  bool stopped() const { return stopped_.load(); }

  // ---- memory ----
  std::pair<MemoryRegionHandle, MemoryRegionDescriptor> register_memory(uint64_t ptr, uint64_t len, int device);
  void unregister_memory(uint64_t ptr);
  PeerGroupHandle add_peer_group(const std::vector<DomainAddress>& addresses, int device = INT32_MIN);

  // ---- one-sided ----
  TransferId submit_transfer(TransferRequest request, DoneFn on_done, ErrorFn on_error);
  // No callback: completion is counted in `counter` (polled by the caller).
  TransferId submit_transfer_atomic(TransferRequest request, TransferCounter counter);

  // ---- two-sided ----
  void submit_send(const DomainAddress& dst, std::string data, DoneFn on_done, ErrorFn on_error);
  void submit_bouncing_recvs(size_t count, size_t len, RecvFn on_recv, ErrorFn on_error);

  // ---- immediates ----
  void set_imm_callback(ImmFn cb);
  // Counts arrivals of `imm`; after `expected` of them `on_reached` runs once, the counter
  // disappears and later arrivals go to the imm callback again.
  std::optional<std::pair<uint32_t, uint32_t>> set_imm_count_expected(uint32_t imm, uint32_t expected, DoneFn on_reached);
  std::optional<std::pair<uint32_t, uint32_t>> remove_imm_count(uint32_t imm);
  ImmCounter get_imm_counter(uint32_t imm);
  // Raises `flag` (a word in device-mapped host memory) every time the counter of `imm`
  // returns to zero; the returned cell is decremented by the user to arm it.
  std::shared_ptr<std::atomic<int64_t>> get_flag_counter(uint32_t imm, volatile uint32_t* flag);

  // ---- UVM watcher ----
  UvmWatcher alloc_scalar_watcher(WatchFn cb);

  // Test hook: the first domain of the worker of `device`.
  Domain* debug_domain(int device, size_t index = 0);

 private:
  struct Worker;
  Worker& worker_for_device(int device);
  Worker& worker_for_mr(uint64_t ptr);
  void worker_loop(Worker* w);
  void callback_loop();
  void uvm_loop();
  void push_completion(TransferCompletionEntry e);
  template <typename F>
  auto call_on(Worker& w, F&& f) -> decltype(f(std::declval<DomainGroup&>()));

  std::vector<std::unique_ptr<Worker>> workers_;
  std::map<int, size_t> worker_of_device_;
  std::mutex mr_mu_;
  std::map<uint64_t, std::pair<uint64_t, size_t>> mr_owner_;  // ptr -> (len, worker index)

  DomainAddress main_address_;
  size_t num_domains_ = 0, nets_per_gpu_ = 0;
  uint64_t link_speed_ = 0;
  std::atomic<bool> stopped_{false};
  std::atomic<TransferId> next_id_{1};

  // completions -> callback thread
  std::mutex cq_mu_;
  std::condition_variable cq_cv_;
  std::deque<TransferCompletionEntry> cq_;
  std::thread callback_thread_;

  std::mutex cb_mu_;
  // Callbacks may wrap Python callables whose copy takes the GIL: they are held through
  // shared_ptr so that no copy ever happens under one of the engine's locks.
  struct TransferCallbacks { std::shared_ptr<DoneFn> done; std::shared_ptr<ErrorFn> error; };
  std::unordered_map<TransferId, TransferCallbacks> transfer_cbs_;
  struct RecvCallbacks { std::shared_ptr<RecvFn> recv; std::shared_ptr<ErrorFn> error; size_t len; size_t worker; };
  std::unordered_map<TransferId, RecvCallbacks> recv_cbs_;
  std::shared_ptr<ImmFn> imm_cb_;
  std::unordered_map<uint32_t, std::shared_ptr<DoneFn>> imm_reached_cbs_;
  ImmCountMap imm_counts_;

  // UVM watcher
  static constexpr size_t kWatchSlots = 512;
  uint64_t* watch_page_ = nullptr;
  bool watch_page_cuda_ = false;
  std::mutex watch_mu_;
  struct WatchSlot { bool used = false; uint32_t generation = 0; uint64_t last = 0; std::shared_ptr<WatchFn> cb; };
  std::vector<WatchSlot> watch_slots_;
  std::thread uvm_thread_;
  int uvm_cpu_ = -1;
};

class TransferEngineBuilder {
 public:
  TransferEngineBuilder& add_gpu_domains(int cuda_device, std::vector<DomainInfo> domains,
                                         int pin_worker_cpu, int pin_uvm_cpu);
  // Validates against the detected topology (device exists, domains belong to it, equal
  // domain counts per GPU) and builds.
  std::unique_ptr<TransferEngine> build(DomainFactory factory = nullptr);

 private:
  std::vector<GpuDomainSpec> gpus_;
};

}  // namespace pplx::fabric
