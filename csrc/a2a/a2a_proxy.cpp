#include "a2a_proxy.h"

#include <chrono>

#include "../core/error.h"
#define PPLX_LOG_TARGET "pplx_garden::a2a"
#include "../core/log.h"
#include "../core/thread_util.h"

namespace pplx {

using fabric::DomainGroupRouting;
using fabric::MemoryRegionHandle;
using fabric::PagedTransferRequest;
using fabric::SingleTransferRequest;
using fabric::TransferCounter;
using fabric::TransferRequest;

namespace {
// The words come from the kernels (system-scope release stores into pinned host memory) or, in
// host-only tests, from another thread: the phase words are read with acquire, what they publish
// after that with plain atomic loads.
uint32_t load_acquire(const volatile uint32_t* p) {
  return __atomic_load_n(const_cast<const uint32_t*>(p), __ATOMIC_ACQUIRE);
}
uint32_t load_relaxed(const volatile uint32_t* p) {
  return __atomic_load_n(const_cast<const uint32_t*>(p), __ATOMIC_RELAXED);
}

uint64_t flag_offset(int row, int src_rank) {
  return static_cast<uint64_t>(row * kMaxRanks + src_rank) * kFlagStrideWords * sizeof(uint32_t);
}
}  // namespace

A2AProxy::A2AProxy(const A2AConfig& cfg, int rank, fabric::TransferEngine* engine,
                   std::vector<A2AProxyPeer> peers, const A2AProxyBuffers& buffers, int pin_cpu)
    : cfg_(cfg), rank_(rank), engine_(engine), peers_(std::move(peers)), buf_(buffers), pin_cpu_(pin_cpu) {
  PPLX_REQUIRE(engine_ != nullptr, "the all-to-all proxy needs a transfer engine");
  PPLX_REQUIRE(buf_.proxy_words != nullptr && buf_.stage_slot != nullptr && buf_.flag_source_host != nullptr,
               "the all-to-all proxy needs its host-visible words");
  for (const A2AProxyPeer& p : peers_) {
    PPLX_REQUIRE(p.rank >= 0 && p.rank < cfg_.world && ((cfg_.node_mask >> p.rank) & 1u) == 0,
                 "proxy peers are the ranks outside the NVLink domain");
    PPLX_REQUIRE(buf_.shadow_sync[p.rank] != 0 && buf_.shadow_recv[p.rank] != 0,
                 "every proxy peer needs its stand-in buffers");
  }
  // Touch every remote region once now, with empty writes: the engine resolves and maps a
  // region on its first use, and that (address-space changes on this device) must not happen
  // later, while a kernel that waits for the very transfer fills the GPU.
  std::vector<TransferRequest> warm;
  for (const A2AProxyPeer& p : peers_) {
    for (const fabric::MemoryRegionDescriptor* desc : {&p.sync_desc, &p.recv_desc}) {
      SingleTransferRequest r;
      r.src_mr = MemoryRegionHandle{buf_.shadow_sync[p.rank]};
      r.src_offset = 0;
      r.length = 0;
      r.dst_mr = *desc;
      r.dst_offset = 0;
      r.domain = DomainGroupRouting::pinned(0);
      warm.emplace_back(std::move(r));
      for (size_t d = 1; d < engine_->nets_per_gpu(); ++d) {
        SingleTransferRequest more;
        more.src_mr = MemoryRegionHandle{buf_.shadow_sync[p.rank]};
        more.length = 0;
        more.dst_mr = *desc;
        more.domain = DomainGroupRouting::pinned(static_cast<uint8_t>(d));
        warm.emplace_back(std::move(more));
      }
    }
  }
  if (!run(std::move(warm), "connecting to the ranks outside the NVLink domain")) {
    throw Error(ErrorKind::kDomain, "all-to-all proxy: " + error());
  }
  thread_ = std::thread([this] { loop(); });
}

A2AProxy::~A2AProxy() {
  stop_.store(true);
  if (thread_.joinable()) thread_.join();
}

std::string A2AProxy::error() const {
  std::lock_guard<std::mutex> lock(error_mu_);
  return error_;
}

void A2AProxy::fail(const std::string& why) {
  {
    std::lock_guard<std::mutex> lock(error_mu_);
    if (error_.empty()) error_ = why;
  }
  failed_.store(true, std::memory_order_release);
  PPLX_ERROR("all-to-all proxy of rank %d: %s", rank_, why.c_str());
}

void A2AProxy::loop() {
  if (pin_cpu_ >= 0) pin_cpu(pin_cpu_);
  set_thread_name("a2a_proxy");
  uint32_t next_dispatch = 1, next_combine = 1;
  int idle = 0;
  while (!stop_.load(std::memory_order_acquire)) {
    bool worked = false;
    // the kernels write the tag of the phase that has just finished (tags count up from 1)
    const uint32_t d = load_acquire(&buf_.proxy_words[kProxyDispatchSent]);
    if (static_cast<int32_t>(d - next_dispatch) >= 0) {
      serve_dispatch(next_dispatch);
      ++next_dispatch;
      dispatches_.fetch_add(1);
      worked = true;
    }
    const uint32_t c = load_acquire(&buf_.proxy_words[kProxyCombineSent]);
    if (static_cast<int32_t>(c - next_combine) >= 0) {
      serve_combine(next_combine);
      ++next_combine;
      combines_.fetch_add(1);
      worked = true;
    }
    if (worked) {
      idle = 0;
    } else if (++idle > 20000) {
      // nothing for a while: stop burning a core, a new phase still gets picked up within ~50 us
      std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
  }
}

bool A2AProxy::run(std::vector<TransferRequest> requests, const char* what) {
  if (requests.empty()) return true;
  if (failed()) return false;
  auto done = std::make_shared<std::atomic<int64_t>>(0);
  auto errors = std::make_shared<std::atomic<int64_t>>(0);
  const TransferCounter counter(done, errors);
  const int64_t n = static_cast<int64_t>(requests.size());
  try {
    for (TransferRequest& r : requests) engine_->submit_transfer_atomic(std::move(r), counter);
  } catch (const std::exception& e) {
    fail(std::string(what) + ": " + e.what());
    return false;
  }
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::nanoseconds(cfg_.wait_limit_ns);
  while (counter.done() < n) {
    if (stop_.load(std::memory_order_acquire)) return false;
    if (std::chrono::steady_clock::now() > deadline) {
      fail(std::string(what) + ": transfers did not complete within the wait limit");
      return false;
    }
    std::this_thread::yield();
  }
  if (counter.errors() != 0) {
    fail(std::string(what) + ": fabric-lib transfer error");
    return false;
  }
  return true;
}

bool A2AProxy::send_flags(int row, uint32_t tag, const char* what) {
  // one word per (row, tag parity) so that a flag in flight is never overwritten by the next
  const int word = row * 2 + static_cast<int>(tag & 1u);
  __atomic_store_n(const_cast<uint32_t*>(&buf_.flag_source_host[word]), tag, __ATOMIC_RELEASE);
  std::vector<TransferRequest> requests;
  for (const A2AProxyPeer& p : peers_) {
    SingleTransferRequest r;
    r.src_mr = MemoryRegionHandle{buf_.flag_source};
    r.src_offset = static_cast<uint64_t>(word) * sizeof(uint32_t);
    r.length = sizeof(uint32_t);
    r.dst_mr = p.sync_desc;
    r.dst_offset = flag_offset(row, rank_);
    r.domain = DomainGroupRouting::pinned(0);
    requests.emplace_back(std::move(r));
  }
  return run(std::move(requests), what);
}

void A2AProxy::serve_dispatch(uint32_t tag) {
  PPLX_DEBUG("proxy of rank %d: dispatch %u has been sent by the kernels", rank_, tag);
  const uint32_t par = (tag - 1) & 1u;
  const int my_group = rank_ / cfg_.dp_size;
  const int my_tp = rank_ % cfg_.dp_size;
  std::vector<TransferRequest> requests;
  for (const A2AProxyPeer& p : peers_) {
    if (p.rank % cfg_.dp_size != my_tp) continue;   // another rank of my dp group serves this one
    // the counts this rank's kernel wrote for the peer, at the same place in the peer's region
    const uint64_t counts_off =
        cfg_.off_counts + 4ull * (par * cfg_.counts_bank_words + static_cast<uint64_t>(my_group) * cfg_.counts_stride);
    SingleTransferRequest c;
    c.src_mr = MemoryRegionHandle{buf_.shadow_sync[p.rank]};
    c.src_offset = counts_off;
    c.length = 4ull * cfg_.counts_stride;
    c.dst_mr = p.sync_desc;
    c.dst_offset = counts_off;
    c.domain = DomainGroupRouting::pinned(0);
    requests.emplace_back(std::move(c));
    const uint64_t records = load_relaxed(&buf_.proxy_words[kProxyRecords + p.rank]);
    if (records == 0) continue;
    if (records > static_cast<uint64_t>(cfg_.max_num_tokens)) {
      fail("dispatch: the kernel reported more records than a region holds");
      return;
    }
    SingleTransferRequest r;
    r.src_mr = MemoryRegionHandle{buf_.shadow_recv[p.rank]};
    r.src_offset = 0;
    r.length = records * cfg_.d_stride;
    r.dst_mr = p.recv_desc;
    r.dst_offset = cfg_.off_drecv + static_cast<uint64_t>(my_group) * cfg_.drecv_group_stride;
    r.domain = DomainGroupRouting::sharded(static_cast<uint8_t>(engine_->nets_per_gpu()));
    requests.emplace_back(std::move(r));
  }
  if (!run(std::move(requests), "dispatch")) return;
  PPLX_DEBUG("proxy of rank %d: dispatch %u delivered, sending the flags", rank_, tag);
  send_flags(kFlagDispatchStarted, tag, "dispatch flags");
  PPLX_DEBUG("proxy of rank %d: dispatch %u done", rank_, tag);
}

void A2AProxy::serve_combine(uint32_t tag) {
  PPLX_DEBUG("proxy of rank %d: combine %u has been sent by the kernels", rank_, tag);
  std::vector<TransferRequest> requests;
  for (const A2AProxyPeer& p : peers_) {
    const int g = p.rank / cfg_.dp_size;   // rows go to every member of the origin's dp group
    const uint32_t rows = load_relaxed(&buf_.proxy_words[kProxyRows + g]);
    if (rows == 0) continue;
    const uint32_t first = load_relaxed(&buf_.proxy_words[kProxyRowBase + g]);
    if (static_cast<uint64_t>(first) + rows > cfg_.max_recv_rows) {
      fail("combine: the kernel reported more staged rows than the staging buffer holds");
      return;
    }
    auto src_pages = std::make_shared<std::vector<uint32_t>>(rows);
    auto dst_pages = std::make_shared<std::vector<uint32_t>>(rows);
    const uint64_t slots = static_cast<uint64_t>(cfg_.max_num_tokens) * cfg_.c_records_per_token;
    for (uint32_t i = 0; i < rows; ++i) {
      (*src_pages)[i] = first + i;
      const uint32_t slot = load_relaxed(&buf_.stage_slot[first + i]);
      if (slot >= slots) {
        fail("combine: a staged row names a slot outside the receive buffer");
        return;
      }
      (*dst_pages)[i] = slot;
    }
    PagedTransferRequest r;
    r.length = cfg_.c_stride;
    r.src_mr = MemoryRegionHandle{buf_.stage};
    r.src_page_indices = std::move(src_pages);
    r.src_stride = cfg_.c_stride;
    r.src_offset = 0;
    r.dst_mr = p.recv_desc;
    r.dst_page_indices = std::move(dst_pages);
    r.dst_stride = cfg_.c_stride;
    r.dst_offset = cfg_.off_crecv;
    requests.emplace_back(std::move(r));
  }
  if (!run(std::move(requests), "combine")) return;
  PPLX_DEBUG("proxy of rank %d: combine %u delivered, sending the flags", rank_, tag);
  send_flags(kFlagRemoteCombine, tag, "combine flags");
  PPLX_DEBUG("proxy of rank %d: combine %u done", rank_, tag);
}

}  // namespace pplx
