#include "transfer_engine.h"

#include <cuda_runtime.h>

#include <algorithm>
#include <chrono>
#include <climits>
#include <cstdlib>
#include <cstring>

#include "../core/error.h"
#define PPLX_LOG_TARGET "pplx_garden::fabric"
#include "../core/log.h"
#include "../core/thread_util.h"
#include "faulty_domain.h"
#include "local_domain.h"

namespace pplx::fabric {

struct TransferEngine::Worker {
  int device = -1;
  int pin_cpu = -1;
  std::unique_ptr<DomainGroup> group;
  std::thread thread;
  std::mutex mu;
  std::condition_variable cv;
  std::deque<std::function<void(DomainGroup&)>> commands;
  std::atomic<bool> stop{false};
  std::atomic<bool> failed{false};
};

namespace {
std::unique_ptr<Domain> default_factory(int device, int index, const DomainInfo& info) {
  if (info.provider != "local" && !info.provider.empty()) {
    throw Error(ErrorKind::kDomain, "no provider named '" + info.provider +
                                        "' in this build (RDMA providers need libibverbs / libfabric headers)");
  }
  return std::make_unique<LocalDomain>(device, index);
}
}  // namespace

TransferEngine::TransferEngine(std::vector<GpuDomainSpec> gpus, DomainFactory factory) {
  PPLX_REQUIRE(!gpus.empty(), "a transfer engine needs at least one device");
  if (!factory) factory = default_factory;
  nets_per_gpu_ = gpus[0].domains.size();
  for (const GpuDomainSpec& spec : gpus) {
    PPLX_REQUIRE(!spec.domains.empty(), "every device needs at least one domain");
    PPLX_REQUIRE(spec.domains.size() == nets_per_gpu_, "all devices must use the same number of domains");
    PPLX_REQUIRE(worker_of_device_.count(spec.cuda_device) == 0, "device listed twice");
    auto w = std::make_unique<Worker>();
    w->device = spec.cuda_device;
    w->pin_cpu = spec.pin_worker_cpu;
    std::vector<std::unique_ptr<Domain>> domains;
    for (size_t i = 0; i < spec.domains.size(); ++i) {
      // every provider sits behind the fault-injection decorator (inert until armed)
      domains.push_back(std::make_unique<FaultyDomain>(factory(spec.cuda_device, static_cast<int>(i), spec.domains[i])));
    }
    w->group = std::make_unique<DomainGroup>(std::move(domains));
    num_domains_ += spec.domains.size();
    link_speed_ += w->group->aggregated_link_speed();
    if (workers_.empty()) {
      main_address_ = w->group->main_address();
      uvm_cpu_ = spec.pin_uvm_cpu;
    }
    worker_of_device_[spec.cuda_device] = workers_.size();
    workers_.push_back(std::move(w));
  }
  watch_slots_.resize(kWatchSlots);
  for (auto& w : workers_) {
    Worker* raw = w.get();
    w->thread = std::thread([this, raw] { worker_loop(raw); });
  }
  callback_thread_ = std::thread([this] { callback_loop(); });
  PPLX_INFO("transfer engine up: %zu device(s), %zu domain(s), main address %s", workers_.size(),
            num_domains_, main_address_.to_hex().c_str());
}

TransferEngine::~TransferEngine() { stop(); }

void TransferEngine::stop() {
  if (stopped_.exchange(true)) return;
  for (auto& w : workers_) {
    w->stop = true;
    w->cv.notify_all();
  }
  for (auto& w : workers_) {
    if (w->thread.joinable()) w->thread.join();
  }
  if (uvm_thread_.joinable()) uvm_thread_.join();
  {
    std::lock_guard<std::mutex> lock(cq_mu_);
    cq_cv_.notify_all();
  }
  if (callback_thread_.joinable()) callback_thread_.join();
  // domains (sockets, streams, IPC mappings) go away with their groups
  for (auto& w : workers_) w->group.reset();
  if (watch_page_ != nullptr) {
    if (watch_page_cuda_) cudaFreeHost(watch_page_); else std::free(watch_page_);
    watch_page_ = nullptr;
  }
}

TransferEngine::Worker& TransferEngine::worker_for_device(int device) {
  auto it = worker_of_device_.find(device);
  if (it != worker_of_device_.end()) return *workers_[it->second];
  if (device < 0) return *workers_[0];  // host memory goes through the first worker
  throw Error(ErrorKind::kInvalidArgument, "no domains were added for cuda:" + std::to_string(device));
}

TransferEngine::Worker& TransferEngine::worker_for_mr(uint64_t ptr) {
  std::lock_guard<std::mutex> lock(mr_mu_);
  auto it = mr_owner_.upper_bound(ptr);
  if (it != mr_owner_.begin()) {
    --it;
    if (ptr < it->first + it->second.first) return *workers_[it->second.second];
  }
  throw Error(ErrorKind::kInvalidArgument, "the source memory region is not registered with this engine");
}

template <typename F>
auto TransferEngine::call_on(Worker& w, F&& f) -> decltype(f(std::declval<DomainGroup&>())) {
  using R = decltype(f(std::declval<DomainGroup&>()));
  if (stopped_.load() || w.failed.load()) throw Error(ErrorKind::kWorkerDown, "Worker is down");
  auto task = std::make_shared<std::packaged_task<R(DomainGroup&)>>(std::forward<F>(f));
  std::future<R> fut = task->get_future();
  {
    std::lock_guard<std::mutex> lock(w.mu);
    w.commands.emplace_back([task](DomainGroup& g) { (*task)(g); });
  }
  w.cv.notify_one();
  return fut.get();
}

void TransferEngine::push_completion(TransferCompletionEntry e) {
  {
    std::lock_guard<std::mutex> lock(cq_mu_);
    cq_.push_back(std::move(e));
  }
  cq_cv_.notify_one();
}

// ---------------------------------------------------------------------------
// worker thread
// ---------------------------------------------------------------------------

void TransferEngine::worker_loop(Worker* w) {
  set_thread_name("tx_engine_worker");
  if (w->pin_cpu >= 0) {
    try {
      pin_cpu(w->pin_cpu);
    } catch (const std::exception& e) {
      PPLX_WARN("cannot pin the worker of device %d to cpu %d: %s", w->device, w->pin_cpu, e.what());
    }
  }
  if (w->device >= 0) cudaSetDevice(w->device);
  std::vector<GroupCompletion> done;
  std::deque<std::function<void(DomainGroup&)>> batch;
  auto idle_since = std::chrono::steady_clock::now();
  while (!w->stop.load(std::memory_order_relaxed)) {
    {
      std::unique_lock<std::mutex> lock(w->mu);
      if (w->commands.empty() && !w->group->busy()) {
        // Nothing in flight: immediates and messages from peers still have to be picked
        // up, so sleep only briefly once the engine has been quiet for a while.
        const auto quiet = std::chrono::steady_clock::now() - idle_since;
        if (quiet > std::chrono::milliseconds(2)) {
          w->cv.wait_for(lock, std::chrono::microseconds(200));
        }
      }
      batch.swap(w->commands);
    }
    if (!batch.empty()) idle_since = std::chrono::steady_clock::now();
    for (auto& cmd : batch) {
      try {
        cmd(*w->group);
      } catch (const std::exception& e) {
        PPLX_ERROR("worker command failed: %s", e.what());
      }
    }
    batch.clear();
    try {
      w->group->poll(&done);
    } catch (const std::exception& e) {
      PPLX_ERROR("worker of device %d stops after a provider failure: %s", w->device, e.what());
      w->failed = true;
      return;
    }
    if (!done.empty()) idle_since = std::chrono::steady_clock::now();
    for (GroupCompletion& c : done) {
      TransferCompletionEntry e{};
      e.transfer_id = c.transfer_id;
      switch (c.kind) {
        case GroupCompletion::Kind::kTransferDone:
          e.kind = TransferCompletionEntry::Kind::kTransfer;
          push_completion(std::move(e));
          break;
        case GroupCompletion::Kind::kSendDone:
          e.kind = TransferCompletionEntry::Kind::kSend;
          push_completion(std::move(e));
          break;
        case GroupCompletion::Kind::kRecv:
          e.kind = TransferCompletionEntry::Kind::kRecv;
          e.data_len = c.data.size();
          e.data = std::move(c.data);
          push_completion(std::move(e));
          break;
        case GroupCompletion::Kind::kError:
          e.kind = TransferCompletionEntry::Kind::kError;
          e.error = std::move(c.error);
          push_completion(std::move(e));
          break;
        case GroupCompletion::Kind::kImm:
          // count on the worker thread so that counters move with minimal delay
          for (uint32_t i = 0; i < c.imm_count; ++i) {
            const ImmIncResult r = imm_counts_.inc(c.imm, 1);
            if (r == ImmIncResult::kVacant) {
              TransferCompletionEntry im{};
              im.kind = TransferCompletionEntry::Kind::kImmData;
              im.imm = c.imm;
              push_completion(std::move(im));
            } else if (r == ImmIncResult::kReached) {
              TransferCompletionEntry im{};
              im.kind = TransferCompletionEntry::Kind::kImmCountReached;
              im.imm = c.imm;
              push_completion(std::move(im));
            }
          }
          break;
      }
    }
    done.clear();
  }
}

// ---------------------------------------------------------------------------
// callback thread
// ---------------------------------------------------------------------------

void TransferEngine::callback_loop() {
  set_thread_name("tx_engine_callback");
  for (;;) {
    TransferCompletionEntry e;
    {
      std::unique_lock<std::mutex> lock(cq_mu_);
      cq_cv_.wait_for(lock, std::chrono::milliseconds(50), [this] { return !cq_.empty() || stopped_.load(); });
      if (cq_.empty()) {
        if (stopped_.load()) return;
        continue;
      }
      e = std::move(cq_.front());
      cq_.pop_front();
    }
    try {
      switch (e.kind) {
        case TransferCompletionEntry::Kind::kTransfer:
        case TransferCompletionEntry::Kind::kSend: {
          TransferCallbacks cbs;
          {
            std::lock_guard<std::mutex> lock(cb_mu_);
            auto it = transfer_cbs_.find(e.transfer_id);
            if (it == transfer_cbs_.end()) break;
            cbs = std::move(it->second);
            transfer_cbs_.erase(it);
          }
          if (cbs.done && *cbs.done) (*cbs.done)();
          break;
        }
        case TransferCompletionEntry::Kind::kRecv: {
          std::shared_ptr<RecvFn> fn;
          size_t worker = 0, len = 0;
          {
            std::lock_guard<std::mutex> lock(cb_mu_);
            auto it = recv_cbs_.find(e.transfer_id);
            if (it == recv_cbs_.end()) break;
            fn = it->second.recv;
            worker = it->second.worker;
            len = it->second.len;
          }
          if (fn && *fn) (*fn)(e.data);
          // a bouncing receive is posted again as soon as its buffer has been handed over
          Worker& w = *workers_[worker];
          const TransferId id = e.transfer_id;
          {
            std::lock_guard<std::mutex> lock(w.mu);
            w.commands.emplace_back([id, len](DomainGroup& g) { g.post_recvs(id, 1, len); });
          }
          w.cv.notify_one();
          break;
        }
        case TransferCompletionEntry::Kind::kImmData: {
          std::shared_ptr<ImmFn> fn;
          {
            std::lock_guard<std::mutex> lock(cb_mu_);
            fn = imm_cb_;
          }
          if (fn && *fn) (*fn)(e.imm);
          else PPLX_DEBUG("immediate 0x%x arrived with no callback or counter installed", e.imm);
          break;
        }
        case TransferCompletionEntry::Kind::kImmCountReached: {
          std::shared_ptr<DoneFn> fn;
          {
            std::lock_guard<std::mutex> lock(cb_mu_);
            auto it = imm_reached_cbs_.find(e.imm);
            if (it != imm_reached_cbs_.end()) {
              fn = std::move(it->second);
              imm_reached_cbs_.erase(it);
            }
          }
          if (fn && *fn) (*fn)();
          break;
        }
        case TransferCompletionEntry::Kind::kUvmWatch: {
          std::shared_ptr<WatchFn> fn;
          {
            std::lock_guard<std::mutex> lock(watch_mu_);
            WatchSlot& s = watch_slots_[e.watcher.slot];
            if (!s.used || s.generation != e.watcher.generation) break;
            fn = s.cb;
          }
          const bool keep = (fn && *fn) ? (*fn)(e.old_value, e.new_value) : false;
          if (!keep) {
            std::shared_ptr<WatchFn> dropped;
            std::lock_guard<std::mutex> lock(watch_mu_);
            WatchSlot& s = watch_slots_[e.watcher.slot];
            if (s.used && s.generation == e.watcher.generation) {
              s.used = false;
              dropped = std::move(s.cb);
            }
          }
          break;
        }
        case TransferCompletionEntry::Kind::kError: {
          std::shared_ptr<ErrorFn> fn;
          TransferCallbacks taken;  // destroyed after the lock is released
          {
            std::lock_guard<std::mutex> lock(cb_mu_);
            auto it = transfer_cbs_.find(e.transfer_id);
            if (it != transfer_cbs_.end()) {
              taken = std::move(it->second);
              transfer_cbs_.erase(it);
              fn = taken.error;
            } else {
              auto rit = recv_cbs_.find(e.transfer_id);
              if (rit != recv_cbs_.end()) fn = rit->second.error;
            }
          }
          if (fn && *fn) (*fn)(e.error);
          else PPLX_ERROR("transfer %llu failed: %s", static_cast<unsigned long long>(e.transfer_id), e.error.c_str());
          break;
        }
      }
    } catch (const std::exception& ex) {
      PPLX_ERROR("a completion callback raised: %s", ex.what());
    }
  }
}

// ---------------------------------------------------------------------------
// memory
// ---------------------------------------------------------------------------

std::pair<MemoryRegionHandle, MemoryRegionDescriptor> TransferEngine::register_memory(uint64_t ptr, uint64_t len,
                                                                                        int device) {
  PPLX_REQUIRE(ptr != 0 && len > 0, "cannot register an empty region");
  Worker& w = worker_for_device(device);
  MemoryRegionDescriptor desc = call_on(w, [=](DomainGroup& g) { return g.register_mr(ptr, len, device); });
  {
    std::lock_guard<std::mutex> lock(mr_mu_);
    mr_owner_[ptr] = {len, worker_of_device_.count(device) ? worker_of_device_[device] : 0};
  }
  return {MemoryRegionHandle{ptr}, std::move(desc)};
}

void TransferEngine::unregister_memory(uint64_t ptr) {
  size_t index;
  {
    std::lock_guard<std::mutex> lock(mr_mu_);
    auto it = mr_owner_.find(ptr);
    if (it == mr_owner_.end()) return;
    index = it->second.second;
    mr_owner_.erase(it);
  }
  call_on(*workers_[index], [=](DomainGroup& g) {
    g.unregister_mr(ptr);
    return 0;
  });
}

PeerGroupHandle TransferEngine::add_peer_group(const std::vector<DomainAddress>& addresses, int device) {
  Worker& w = device == INT32_MIN ? *workers_[0] : worker_for_device(device);
  return call_on(w, [=](DomainGroup& g) { return g.add_peer_group(addresses); });
}

// ---------------------------------------------------------------------------
// submissions
// ---------------------------------------------------------------------------

namespace {
uint64_t source_ptr(const TransferRequest& r) {
  return std::visit(
      [](const auto& x) -> uint64_t {
        using T = std::decay_t<decltype(x)>;
        if constexpr (std::is_same_v<T, SingleTransferRequest> || std::is_same_v<T, PagedTransferRequest> ||
                      std::is_same_v<T, ScatterTransferRequest>) {
          return x.src_mr.ptr;
        } else {
          return 0;
        }
      },
      r);
}
}  // namespace

TransferId TransferEngine::submit_transfer(TransferRequest request, DoneFn on_done, ErrorFn on_error) {
  if (stopped_.load()) throw Error(ErrorKind::kWorkerDown, "Worker is down");
  const uint64_t src = source_ptr(request);
  Worker& w = src != 0 ? worker_for_mr(src) : *workers_[0];
  if (w.failed.load()) throw Error(ErrorKind::kWorkerDown, "Worker is down");
  const TransferId id = next_id_.fetch_add(1);
  auto done_ptr = std::make_shared<DoneFn>(std::move(on_done));
  auto error_ptr = std::make_shared<ErrorFn>(std::move(on_error));
  {
    std::lock_guard<std::mutex> lock(cb_mu_);
    transfer_cbs_[id] = TransferCallbacks{std::move(done_ptr), std::move(error_ptr)};
  }
  auto req = std::make_shared<TransferRequest>(std::move(request));
  {
    std::lock_guard<std::mutex> lock(w.mu);
    w.commands.emplace_back([this, id, req](DomainGroup& g) {
      try {
        g.submit(id, *req);
      } catch (const std::exception& e) {
        TransferCompletionEntry err{};
        err.kind = TransferCompletionEntry::Kind::kError;
        err.transfer_id = id;
        err.error = e.what();
        push_completion(std::move(err));
      }
    });
  }
  w.cv.notify_one();
  return id;
}

TransferId TransferEngine::submit_transfer_atomic(TransferRequest request, TransferCounter counter) {
  if (stopped_.load()) throw Error(ErrorKind::kWorkerDown, "Worker is down");
  const uint64_t src = source_ptr(request);
  Worker& w = src != 0 ? worker_for_mr(src) : *workers_[0];
  if (w.failed.load()) throw Error(ErrorKind::kWorkerDown, "Worker is down");
  const TransferId id = next_id_.fetch_add(1);
  auto req = std::make_shared<TransferRequest>(std::move(request));
  {
    std::lock_guard<std::mutex> lock(w.mu);
    w.commands.emplace_back([id, req, counter](DomainGroup& g) {
      try {
        g.submit(id, *req, counter);
      } catch (const std::exception& e) {
        PPLX_ERROR("transfer %llu rejected: %s", static_cast<unsigned long long>(id), e.what());
        counter.mark_error();
      }
    });
  }
  w.cv.notify_one();
  return id;
}

void TransferEngine::submit_send(const DomainAddress& dst, std::string data, DoneFn on_done, ErrorFn on_error) {
  if (stopped_.load()) throw Error(ErrorKind::kWorkerDown, "Worker is down");
  Worker& w = *workers_[0];
  const TransferId id = next_id_.fetch_add(1);
  auto done_ptr = std::make_shared<DoneFn>(std::move(on_done));
  auto error_ptr = std::make_shared<ErrorFn>(std::move(on_error));
  {
    std::lock_guard<std::mutex> lock(cb_mu_);
    transfer_cbs_[id] = TransferCallbacks{std::move(done_ptr), std::move(error_ptr)};
  }
  auto payload = std::make_shared<std::string>(std::move(data));
  {
    std::lock_guard<std::mutex> lock(w.mu);
    w.commands.emplace_back([id, dst, payload](DomainGroup& g) { g.submit_send(id, dst, std::move(*payload)); });
  }
  w.cv.notify_one();
}

void TransferEngine::submit_bouncing_recvs(size_t count, size_t len, RecvFn on_recv, ErrorFn on_error) {
  if (stopped_.load()) throw Error(ErrorKind::kWorkerDown, "Worker is down");
  PPLX_REQUIRE(count > 0 && len > 0, "submit_bouncing_recvs needs a positive count and length");
  Worker& w = *workers_[0];
  const TransferId id = next_id_.fetch_add(1);
  auto recv_ptr = std::make_shared<RecvFn>(std::move(on_recv));
  auto error_ptr = std::make_shared<ErrorFn>(std::move(on_error));
  {
    std::lock_guard<std::mutex> lock(cb_mu_);
    recv_cbs_[id] = RecvCallbacks{std::move(recv_ptr), std::move(error_ptr), len, 0};
  }
  {
    std::lock_guard<std::mutex> lock(w.mu);
    w.commands.emplace_back([id, count, len](DomainGroup& g) { g.post_recvs(id, count, len); });
  }
  w.cv.notify_one();
}

// ---------------------------------------------------------------------------
// immediates
// ---------------------------------------------------------------------------

void TransferEngine::set_imm_callback(ImmFn cb) {
  auto ptr = std::make_shared<ImmFn>(std::move(cb));
  std::shared_ptr<ImmFn> old;
  {
    std::lock_guard<std::mutex> lock(cb_mu_);
    old = std::move(imm_cb_);
    imm_cb_ = std::move(ptr);
  }
}

std::optional<std::pair<uint32_t, uint32_t>> TransferEngine::set_imm_count_expected(uint32_t imm, uint32_t expected,
                                                                                     DoneFn on_reached) {
  PPLX_REQUIRE(expected > 0, "expected_count must be positive");
  auto ptr = std::make_shared<DoneFn>(std::move(on_reached));
  std::shared_ptr<DoneFn> old;
  {
    std::lock_guard<std::mutex> lock(cb_mu_);
    auto& slot = imm_reached_cbs_[imm];
    old = std::move(slot);
    slot = std::move(ptr);
  }
  return imm_counts_.set_expected(imm, expected);
}

std::optional<std::pair<uint32_t, uint32_t>> TransferEngine::remove_imm_count(uint32_t imm) {
  std::shared_ptr<DoneFn> old;
  {
    std::lock_guard<std::mutex> lock(cb_mu_);
    auto it = imm_reached_cbs_.find(imm);
    if (it != imm_reached_cbs_.end()) {
      old = std::move(it->second);
      imm_reached_cbs_.erase(it);
    }
  }
  return imm_counts_.remove(imm);
}

ImmCounter TransferEngine::get_imm_counter(uint32_t imm) { return ImmCounter(imm_counts_.set_free(imm)); }

std::shared_ptr<std::atomic<int64_t>> TransferEngine::get_flag_counter(uint32_t imm, volatile uint32_t* flag) {
  return imm_counts_.set_flag(imm, flag);
}

// ---------------------------------------------------------------------------
// UVM watcher
// ---------------------------------------------------------------------------

UvmWatcher TransferEngine::alloc_scalar_watcher(WatchFn cb) {
  auto cb_ptr = std::make_shared<WatchFn>(std::move(cb));
  std::lock_guard<std::mutex> lock(watch_mu_);
  if (watch_page_ == nullptr) {
    // One 4 KiB page of 64-bit words that both the host thread and kernels can address.
    void* page = nullptr;
    if (cudaHostAlloc(&page, kWatchSlots * sizeof(uint64_t), cudaHostAllocMapped | cudaHostAllocPortable) ==
        cudaSuccess) {
      watch_page_cuda_ = true;
    } else {
      cudaGetLastError();
      if (posix_memalign(&page, 4096, kWatchSlots * sizeof(uint64_t)) != 0) {
        throw Error::from_errno("posix_memalign(watch page)");
      }
    }
    std::memset(page, 0, kWatchSlots * sizeof(uint64_t));
    watch_page_ = static_cast<uint64_t*>(page);
    uvm_thread_ = std::thread([this] { uvm_loop(); });
  }
  for (size_t i = 0; i < kWatchSlots; ++i) {
    WatchSlot& s = watch_slots_[i];
    if (s.used) continue;
    s.used = true;
    s.generation += 1;
    s.last = 0;
    s.cb = std::move(cb_ptr);
    reinterpret_cast<volatile uint64_t*>(watch_page_)[i] = 0;
    UvmWatcher w;
    w.ptr_ = reinterpret_cast<uint64_t>(&watch_page_[i]);
    w.id_ = UvmWatcherId{static_cast<uint32_t>(i), s.generation};
    return w;
  }
  throw Error(ErrorKind::kCustom, "all 512 scalar watcher slots are in use");
}

void TransferEngine::uvm_loop() {
  set_thread_name("tx_engine_uvm");
  if (uvm_cpu_ >= 0) {
    try {
      pin_cpu(uvm_cpu_);
    } catch (const std::exception& e) {
      PPLX_WARN("cannot pin the UVM watcher to cpu %d: %s", uvm_cpu_, e.what());
    }
  }
  uint32_t idle = 0;
  while (!stopped_.load(std::memory_order_relaxed)) {
    bool any = false;
    {
      std::lock_guard<std::mutex> lock(watch_mu_);
      for (size_t i = 0; i < kWatchSlots; ++i) {
        WatchSlot& s = watch_slots_[i];
        if (!s.used) continue;
        // written by a kernel (or, in host-only use, by another thread): an acquire load, so that a
        // callback sees what the writer published before the word
        const uint64_t now = __atomic_load_n(&watch_page_[i], __ATOMIC_ACQUIRE);
        if (now != s.last) {
          TransferCompletionEntry e{};
          e.kind = TransferCompletionEntry::Kind::kUvmWatch;
          e.watcher = UvmWatcherId{static_cast<uint32_t>(i), s.generation};
          e.old_value = s.last;
          e.new_value = now;
          s.last = now;
          push_completion(std::move(e));
          any = true;
        }
      }
    }
    if (any) {
      idle = 0;
    } else if (++idle > 2000) {
      std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
  }
}

Domain* TransferEngine::debug_domain(int device, size_t index) {
  Worker& w = worker_for_device(device);
  return index < w.group->num_domains() ? &w.group->domain(index) : nullptr;
}

// ---------------------------------------------------------------------------
// builder
// ---------------------------------------------------------------------------

TransferEngineBuilder& TransferEngineBuilder::add_gpu_domains(int cuda_device, std::vector<DomainInfo> domains,
                                                              int pin_worker_cpu, int pin_uvm_cpu) {
  gpus_.push_back(GpuDomainSpec{cuda_device, std::move(domains), pin_worker_cpu, pin_uvm_cpu});
  return *this;
}

std::unique_ptr<TransferEngine> TransferEngineBuilder::build(DomainFactory factory) {
  PPLX_REQUIRE(!gpus_.empty(), "add_gpu_domains was never called");
  const std::vector<TopologyGroup>& topo = detect_topology();
  for (const GpuDomainSpec& spec : gpus_) {
    const TopologyGroup* group = nullptr;
    for (const TopologyGroup& g : topo) {
      if (g.cuda_device == spec.cuda_device) group = &g;
    }
    if (group == nullptr) {
      throw Error(ErrorKind::kInvalidArgument, "cuda:" + std::to_string(spec.cuda_device) + " is not in the detected topology");
    }
    PPLX_REQUIRE(!spec.domains.empty(), "every device needs at least one domain");
    for (const DomainInfo& d : spec.domains) {
      const bool known = std::any_of(group->domains.begin(), group->domains.end(),
                                     [&](const DomainInfo& k) { return k.name == d.name; });
      if (!known && !factory) {
        throw Error(ErrorKind::kInvalidArgument, "domain '" + d.name + "' does not belong to cuda:" + std::to_string(spec.cuda_device));
      }
    }
  }
  return std::make_unique<TransferEngine>(gpus_, std::move(factory));
}

}  // namespace pplx::fabric
