// Native unit tests of the host-side building blocks (the counterpart of the reference's Rust
// unit tests: cuda-lib/src/test_driver.rs, fabric-lib's imm_count / utils modules). No GPU is
// needed. Exit code 0 when every check passes; each failure prints its expression and line.
#include <sys/mman.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "../a2a/a2a_context.h"
#include "../a2a/a2a_proxy.h"
#include "../core/error.h"
#include "../cumem/cumem.h"
#include "../fabric/api.h"
#include "../fabric/host_buffer.h"
#include "../fabric/imm_count.h"
#include "../fabric/shard.h"
#include "../fabric/faulty_domain.h"
#include "../fabric/topo.h"
#include "../fabric/transfer_engine.h"
#include "../fabric/util.h"
#include "../unigram/engine.h"
#include "../unigram/json.h"

namespace {

int g_failures = 0;
int g_checks = 0;

#define CHECK(expr)                                                        \
  do {                                                                     \
    ++g_checks;                                                            \
    if (!(expr)) {                                                         \
      ++g_failures;                                                        \
      std::fprintf(stderr, "FAILED %s:%d: %s\n", __FILE__, __LINE__, #expr); \
    }                                                                      \
  } while (0)

using namespace pplx;
using namespace pplx::fabric;

void test_error() {
  try {
    throw Error(ErrorKind::kTimeout, "waited too long");
  } catch (const Error& e) {
    CHECK(e.kind() == ErrorKind::kTimeout);
    CHECK(std::string(e.what()).find("waited too long") != std::string::npos);
  }
  bool threw = false;
  try {
    PPLX_REQUIRE(1 + 1 == 3, "arithmetic");
  } catch (const Error& e) {
    threw = true;
    CHECK(std::string(e.what()).find("arithmetic") != std::string::npos);
  }
  CHECK(threw);
}

void test_defer_and_pools() {
  int fired = 0;
  {
    Defer d([&] { ++fired; });
  }
  CHECK(fired == 1);
  {
    Defer d([&] { ++fired; });
    d.cancel();
  }
  CHECK(fired == 1);

  ObjectPool<std::string, 4> pool;
  std::vector<std::string*> held;
  for (int i = 0; i < 9; ++i) held.push_back(pool.acquire("item " + std::to_string(i)));
  CHECK(pool.capacity() == 12 && pool.in_use() == 9);
  const std::string* first = held[0];
  CHECK(*first == "item 0");   // growth did not move it
  pool.release(held[3]);
  std::string* again = pool.acquire("reused");
  CHECK(again == held[3] && *again == "reused");
  held[3] = again;
  for (std::string* s : held) pool.release(s);
  CHECK(pool.in_use() == 0);

  std::vector<uint8_t> region(1000);
  MemoryPool mem(region.data(), region.size(), 256);
  CHECK(mem.available() == 3 && mem.chunk_size() == 256);
  uint8_t* a = mem.acquire();
  uint8_t* b = mem.acquire();
  uint8_t* c = mem.acquire();
  CHECK(a && b && c && a != b && b != c && mem.acquire() == nullptr);
  mem.release(b);
  CHECK(mem.acquire() == b);
}

void test_imm_counts() {
  ImmCountMap map;
  CHECK(map.inc(7) == ImmIncResult::kVacant);
  CHECK(!map.set_expected(7, 3).has_value());
  CHECK(map.inc(7) == ImmIncResult::kNotReached);
  CHECK(map.inc(7) == ImmIncResult::kNotReached);
  CHECK(map.inc(7) == ImmIncResult::kReached);
  CHECK(map.inc(7) == ImmIncResult::kVacant);   // fired once; surplus arrivals see no counter
  [[maybe_unused]] auto prev = map.set_expected(7, 2);
  CHECK(map.inc(7, 2) == ImmIncResult::kReached);
  auto free_cell = map.set_free(9);
  map.inc(9);
  map.inc(9, 4);
  CHECK(free_cell->load() == 5);
  volatile uint32_t flag = 0;
  auto debt = map.set_flag(11, &flag);
  debt->store(-2);
  map.inc(11);
  CHECK(flag == 0);
  map.inc(11);
  CHECK(flag == 1);
  CHECK(map.remove(9).has_value() && !map.remove(9).has_value());
}

void test_sharding() {
  const auto one = shard_single_transfer(100, 4);   // a small write stays whole; idle shards are (0, 0)
  CHECK(one.size() == 4 && one[0].first == 0 && one[0].second == 100);
  for (size_t i = 1; i < one.size(); ++i) CHECK(one[i].first == 0 && one[i].second == 0);
  const uint64_t total = (1u << 20) + 12345;
  const auto parts = shard_single_transfer(total, 4);
  uint64_t covered = 0;
  size_t non_empty = 0;
  for (size_t i = 0; i < parts.size(); ++i) {
    if (parts[i].second == 0) continue;
    ++non_empty;
    CHECK(parts[i].first == covered);
    covered += parts[i].second;
    if (covered != total) CHECK(parts[i].second % 8192 == 0);   // all but the last non-empty shard
  }
  CHECK(covered == total && parts.size() == 4 && non_empty >= 2);
  const auto pages = shard_pages(10, 4);   // [begin, end) runs
  size_t sum = 0, next = 0;
  for (const auto& p : pages) {
    CHECK(p.first == next && p.second > p.first);
    sum += p.second - p.first;
    next = p.second;
  }
  CHECK(sum == 10 && pages.size() == 4);
  CHECK(shard_pages(2, 4).size() == 2);    // empty runs are dropped
}

void test_host_buffers() {
  size_t registered = 0, freed = 0;
  {
    HostBufferAllocator alloc([&](uint8_t*, size_t n) { registered += n; }, [&](uint8_t*, size_t n) { freed += n; });
    auto a = alloc.allocate(5000);
    CHECK(a->capacity() == 8192);
    uint8_t* where = a->data();
    std::memset(where, 0xAB, 5000);
    a.reset();                       // back to the free list, not to the system
    CHECK(alloc.cached_buffers() == 1);
    auto b = alloc.allocate(8000);   // same size class: the same memory again
    CHECK(b->data() == where);
    auto c = alloc.allocate(100);
    CHECK(c->capacity() == 4096);
    CHECK(registered == 8192 + 4096);
  }
  CHECK(freed == registered);
}

void test_addresses_and_topology_helpers() {
  const DomainAddress addr(std::string("\x01\x02\xfe", 3));
  CHECK(addr.to_hex() == "0102fe");
  CHECK(DomainAddress::from_hex("0102fe") == addr);
  const std::vector<int> cpus = parse_cpu_list("0-3,8,10-11");
  CHECK((cpus == std::vector<int>{0, 1, 2, 3, 8, 10, 11}));
  const std::vector<int> all{0, 1, 2, 3, 4, 5, 6};
  size_t n = 0;
  for (size_t i = 0; i < 3; ++i) n += split_evenly(all, 3, i).size();
  CHECK(n == all.size());
}

void test_json_numbers() {
  const json::Value v = json::parse(R"({"a": -12.143931267304547, "b": 3, "c": 2.5e-3, "s": "xé"})");
  CHECK(v.find("a")->as_number() == -(static_cast<double>(12143931267304547ull) / 1e15));
  CHECK(v.find("b")->as_number() == 3.0);
  CHECK(v.find("c")->as_number() == 0.0025);
  CHECK(v.find("s")->as_string() == "x\xc3\xa9");
  bool threw = false;
  try {
    json::parse("{\"a\": 01}");
  } catch (const std::exception&) {
    threw = true;
  }
  CHECK(threw);
}

// Two engines on host memory (no GPU), four submitting threads each way, callbacks and counters
// coming back on the engines' own threads, immediates counted at the receiver, a delayed and
// reordered domain under one of them, then shutdown while the last completions arrive. Its job is
// to give the thread and address sanitizer builds (python build.py --sanitize thread|address)
// something that exercises the engine's locking and object lifetimes; the assertions are the
// same a plain build checks.
void test_engine_threads() {
  GpuDomainSpec spec;
  spec.cuda_device = -1;
  spec.domains = {DomainInfo{"host0", 1, "local"}, DomainInfo{"host1", 1, "local"}};
  std::vector<uint8_t> src(1 << 16), dst_a(1 << 16), dst_b(1 << 16);
  for (size_t i = 0; i < src.size(); ++i) src[i] = static_cast<uint8_t>(i * 7);
  {
    TransferEngine a({spec}), b({spec});
    const auto a_src = a.register_memory(reinterpret_cast<uint64_t>(src.data()), src.size(), -1);
    const auto b_dst = b.register_memory(reinterpret_cast<uint64_t>(dst_b.data()), dst_b.size(), -1);
    const auto b_src = b.register_memory(reinterpret_cast<uint64_t>(src.data()), src.size(), -1);
    const auto a_dst = a.register_memory(reinterpret_cast<uint64_t>(dst_a.data()), dst_a.size(), -1);
    if (auto* d = dynamic_cast<FaultyDomain*>(a.debug_domain(-1, 1))) {
      d->inject(FaultKind::kDelayWrites, 1);
      d->inject(FaultKind::kReorderWrites, 2);
    }
    std::atomic<int> imm_seen{0}, reached{0}, done_cb{0}, err_cb{0};
    b.set_imm_callback([&](uint32_t) { imm_seen.fetch_add(1); });
    a.set_imm_count_expected(7, 64, [&] { reached.fetch_add(1); });
    auto done = std::make_shared<std::atomic<int64_t>>(0);
    auto errors = std::make_shared<std::atomic<int64_t>>(0);
    const TransferCounter counter(done, errors);
    constexpr int kThreads = 4, kPerThread = 32;
    std::vector<std::thread> threads;
    for (int t = 0; t < kThreads; ++t) {
      threads.emplace_back([&, t] {
        for (int i = 0; i < kPerThread; ++i) {
          const uint64_t off = static_cast<uint64_t>(t * kPerThread + i) * 256;
          SingleTransferRequest r;
          r.src_mr = a_src.first;
          r.src_offset = off;
          r.length = 256;
          r.dst_mr = b_dst.second;
          r.dst_offset = off;
          r.imm_data = (i % 2 == 0) ? std::optional<uint32_t>(1000 + i) : std::nullopt;
          r.domain = DomainGroupRouting::sharded(2);
          if (i % 4 == 0) {
            a.submit_transfer_atomic(TransferRequest(std::move(r)), counter);
          } else {
            a.submit_transfer(TransferRequest(std::move(r)), [&] { done_cb.fetch_add(1); },
                              [&](const std::string&) { err_cb.fetch_add(1); });
          }
          // and the other way, with an immediate that the first engine counts
          if (i % 2 == 0) {
            SingleTransferRequest back;
            back.src_mr = b_src.first;
            back.src_offset = off;
            back.length = 128;
            back.dst_mr = a_dst.second;
            back.dst_offset = off;
            back.imm_data = 7;
            back.domain = DomainGroupRouting::pinned(static_cast<uint8_t>(i % 2));
            b.submit_transfer(TransferRequest(std::move(back)), [&] { done_cb.fetch_add(1); },
                              [&](const std::string&) { err_cb.fetch_add(1); });
          }
        }
      });
    }
    for (auto& th : threads) th.join();
    const int want_cb = kThreads * kPerThread * 3 / 4 + kThreads * kPerThread / 2;
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::seconds(20);
    while ((done_cb.load() < want_cb || done->load() < kThreads * kPerThread / 4 || reached.load() < 1 ||
            imm_seen.load() < kThreads * kPerThread) &&
           std::chrono::steady_clock::now() < deadline) {
      std::this_thread::sleep_for(std::chrono::milliseconds(1));
    }
    CHECK(done_cb.load() == want_cb);
    CHECK(err_cb.load() == 0 && errors->load() == 0);
    CHECK(done->load() == kThreads * kPerThread / 4);
    CHECK(imm_seen.load() == kThreads * kPerThread);   // two shards per write, each carries the immediate
    CHECK(reached.load() == 1);
    CHECK(std::memcmp(src.data(), dst_b.data(), kThreads * kPerThread * 256) == 0);
    // two-sided messages into bouncing receives, and a watched word changed from another thread
    std::atomic<int> received{0}, sent{0}, watched{0};
    std::atomic<uint64_t> last_seen{0};
    b.submit_bouncing_recvs(2, 256, [&](const std::string& data) { if (data.rfind("message ", 0) == 0) received.fetch_add(1); },
                            [&](const std::string&) { err_cb.fetch_add(1); });
    for (int i = 0; i < 8; ++i) {
      a.submit_send(b.main_address(), "message " + std::to_string(i), [&] { sent.fetch_add(1); },
                    [&](const std::string&) { err_cb.fetch_add(1); });
    }
    const UvmWatcher watcher = a.alloc_scalar_watcher([&](uint64_t, uint64_t now) {
      last_seen.store(now);
      watched.fetch_add(1);
      return true;
    });
    std::thread poker([&] {
      for (uint64_t v = 1; v <= 5; ++v) {
        __atomic_store_n(reinterpret_cast<uint64_t*>(watcher.ptr()), v, __ATOMIC_RELEASE);
        std::this_thread::sleep_for(std::chrono::milliseconds(2));
      }
    });
    poker.join();
    const auto deadline2 = std::chrono::steady_clock::now() + std::chrono::seconds(20);
    while ((received.load() < 8 || sent.load() < 8 || last_seen.load() != 5) && std::chrono::steady_clock::now() < deadline2) {
      std::this_thread::sleep_for(std::chrono::milliseconds(1));
    }
    CHECK(received.load() == 8 && sent.load() == 8);
    CHECK(last_seen.load() == 5 && watched.load() >= 1 && err_cb.load() == 0);
    // a last burst that is still in flight when the engines are stopped and destroyed
    for (int i = 0; i < 16; ++i) {
      SingleTransferRequest r;
      r.src_mr = a_src.first;
      r.length = 4096;
      r.dst_mr = b_dst.second;
      r.domain = DomainGroupRouting::sharded(2);
      a.submit_transfer(TransferRequest(std::move(r)), [] {}, [](const std::string&) {});
    }
    a.stop();
    b.stop();
  }
}

// The all-to-all's host proxy between two one-rank "nodes" over host memory: this test plays the
// kernels (it fills the stand-in buffers and raises the words they would raise) and checks that
// counts, records and combine rows land where the remote kernels expect them, and that a flag
// never arrives before its data. Mainly here so that the proxy thread, the engine's threads and
// the words they share run under the sanitizers.
void test_proxy_between_two_nodes() {
  A2AParams p;
  p.world = 2;
  p.num_experts = 4;
  p.topk = 2;
  p.max_num_tokens = 8;
  p.hidden_dim = 64;
  p.in_elemsize = 2;
  p.out_elemsize = 2;
  p.wire = kWirePlain;
  p.wait_limit_ms = 3000;
  struct Side {
    A2AConfig cfg;
    std::vector<uint8_t> sync, recv, shadow_sync, shadow_recv, stage, flag_source;
    std::vector<uint32_t> words, slots;
    std::unique_ptr<TransferEngine> engine;
    MemoryRegionDescriptor sync_desc, recv_desc;
    std::unique_ptr<A2AProxy> proxy;
  };
  GpuDomainSpec spec;
  spec.cuda_device = -1;
  spec.domains = {DomainInfo{"host0", 1, "local"}};
  Side side[2];
  for (int r = 0; r < 2; ++r) {
    Side& s = side[r];
    p.node_mask = 1u << r;
    s.cfg = a2a_make_config(p, 148, 1);
    s.sync.assign(s.cfg.sync_bytes, 0);
    s.recv.assign(s.cfg.recv_bytes, 0);
    s.shadow_sync.assign(s.cfg.sync_bytes, 0);
    s.shadow_recv.assign(s.cfg.drecv_group_stride, 0);
    s.stage.assign(static_cast<size_t>(s.cfg.max_recv_rows) * s.cfg.c_stride, 0);
    s.flag_source.assign(4096, 0);
    s.words.assign(kProxyWords, 0);
    s.slots.assign(s.cfg.max_recv_rows, 0);
    s.engine = std::make_unique<TransferEngine>(std::vector<GpuDomainSpec>{spec});
    auto reg = [&](std::vector<uint8_t>& v) {
      return s.engine->register_memory(reinterpret_cast<uint64_t>(v.data()), v.size(), -1).second;
    };
    s.sync_desc = reg(s.sync);
    s.recv_desc = reg(s.recv);
    reg(s.shadow_sync);
    reg(s.shadow_recv);
    reg(s.stage);
    reg(s.flag_source);
  }
  for (int r = 0; r < 2; ++r) {
    Side& s = side[r];
    Side& o = side[1 - r];
    A2AProxyPeer peer;
    peer.rank = 1 - r;
    peer.sync_desc = o.sync_desc;
    peer.recv_desc = o.recv_desc;
    A2AProxyBuffers buf;
    buf.shadow_sync[1 - r] = reinterpret_cast<uint64_t>(s.shadow_sync.data());
    buf.shadow_recv[1 - r] = reinterpret_cast<uint64_t>(s.shadow_recv.data());
    buf.stage = reinterpret_cast<uint64_t>(s.stage.data());
    buf.flag_source = reinterpret_cast<uint64_t>(s.flag_source.data());
    buf.flag_source_host = reinterpret_cast<volatile uint32_t*>(s.flag_source.data());
    buf.proxy_words = reinterpret_cast<volatile uint32_t*>(s.words.data());
    buf.stage_slot = reinterpret_cast<const volatile uint32_t*>(s.slots.data());
    s.proxy = std::make_unique<A2AProxy>(s.cfg, r, s.engine.get(), std::vector<A2AProxyPeer>{peer}, buf, -1);
  }
  Side& a = side[0];
  Side& b = side[1];
  const A2AConfig& c = a.cfg;
  auto flag_at = [&](Side& s, int row, int src) {
    const size_t off = static_cast<size_t>(row * kMaxRanks + src) * kFlagStrideWords * sizeof(uint32_t);
    return __atomic_load_n(reinterpret_cast<uint32_t*>(s.sync.data() + off), __ATOMIC_ACQUIRE);
  };
  auto raise = [&](Side& s, int word, uint32_t value) {
    __atomic_store_n(&s.words[word], value, __ATOMIC_RELEASE);
  };
  auto wait_for = [&](auto cond) {
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::seconds(10);
    while (!cond() && std::chrono::steady_clock::now() < deadline) std::this_thread::sleep_for(std::chrono::milliseconds(1));
    return cond();
  };
  // dispatch 1 from rank 0: three records and the counts message
  for (size_t i = 0; i < 3u * c.d_stride; ++i) a.shadow_recv[i] = static_cast<uint8_t>(1 + i % 251);
  const size_t counts_off = c.off_counts;   // bank 0, source group 0
  for (uint32_t i = 0; i < c.counts_stride; ++i) {
    const uint32_t v = i + 1;
    std::memcpy(a.shadow_sync.data() + counts_off + 4 * i, &v, 4);
  }
  a.words[kProxyRecords + 1] = 3;
  raise(a, kProxyDispatchSent, 1);
  CHECK(wait_for([&] { return flag_at(b, kFlagDispatchStarted, 0) == 1u; }));
  CHECK(std::memcmp(b.recv.data() + c.off_drecv, a.shadow_recv.data(), 3u * c.d_stride) == 0);
  CHECK(std::memcmp(b.sync.data() + counts_off, a.shadow_sync.data() + counts_off, 4u * c.counts_stride) == 0);
  // the proxy counts a phase when its own write of the flag has completed, which is after the flag is visible
  CHECK(wait_for([&] { return a.proxy->dispatches() == 1u; }) && !a.proxy->failed());
  // combine 1: four rows for rank 1, staged behind five rows that stay here
  const uint32_t slots[4] = {7, 0, 12, 3};
  for (int i = 0; i < 4; ++i) {
    a.slots[5 + i] = slots[i];
    std::memset(a.stage.data() + static_cast<size_t>(5 + i) * c.c_stride, 0x40 + i, c.c_stride);
  }
  a.words[kProxyRowBase + 1] = 5;
  a.words[kProxyRows + 1] = 4;
  raise(a, kProxyCombineSent, 1);
  CHECK(wait_for([&] { return flag_at(b, kFlagRemoteCombine, 0) == 1u; }));
  for (int i = 0; i < 4; ++i) {
    const uint8_t* row = b.recv.data() + c.off_crecv + static_cast<size_t>(slots[i]) * c.c_stride;
    CHECK(row[0] == 0x40 + i && row[c.c_stride - 1] == 0x40 + i);
  }
  CHECK(wait_for([&] { return a.proxy->combines() == 1u; }));
  // the other direction at the same time as a second dispatch from rank 0
  b.words[kProxyRecords + 0] = 0;
  raise(b, kProxyDispatchSent, 1);
  a.words[kProxyRecords + 1] = 0;
  raise(a, kProxyDispatchSent, 2);
  CHECK(wait_for([&] { return flag_at(a, kFlagDispatchStarted, 1) == 1u && flag_at(b, kFlagDispatchStarted, 0) == 2u; }));
  for (Side& s : side) {
    s.proxy.reset();
    s.engine->stop();
  }
}

// The descriptor server (the SCM_RIGHTS route by which CUDA virtual-memory allocations travel
// between processes): four threads fetch a registered descriptor over the socket while another
// is registered and unregistered; a wrong token and an unregistered number are refused.
void test_fd_server_threads() {
  const int fd = memfd_create("pplx-core-test", MFD_CLOEXEC);
  CHECK(fd >= 0);
  const char text[] = "descriptor contents";
  CHECK(write(fd, text, sizeof(text)) == static_cast<ssize_t>(sizeof(text)));
  const int other = memfd_create("pplx-core-test-2", MFD_CLOEXEC);
  const std::string name = fd_server_name();
  fd_server_register(fd);
  fd_fetch_set_mode("socket");
  std::atomic<int> good{0}, refused{0};
  std::vector<std::thread> threads;
  for (int t = 0; t < 4; ++t) {
    threads.emplace_back([&] {
      for (int i = 0; i < 8; ++i) {
        try {
          const int got = fd_fetch(getpid(), fd, name);
          char buf[sizeof(text)] = {};
          if (pread(got, buf, sizeof(buf), 0) == static_cast<ssize_t>(sizeof(buf)) && std::memcmp(buf, text, sizeof(buf)) == 0) {
            good.fetch_add(1);
          }
          close(got);
        } catch (const std::exception&) {
        }
        try {
          close(fd_fetch(getpid(), fd + 1000, name));   // never registered
        } catch (const std::exception&) {
          refused.fetch_add(1);
        }
      }
    });
  }
  for (int i = 0; i < 16; ++i) {
    fd_server_register(other);
    fd_server_unregister(other);
  }
  for (auto& th : threads) th.join();
  CHECK(good.load() == 32);
  CHECK(refused.load() == 32);
  bool threw = false;
  try {
    const size_t colon = name.find(':');
    close(fd_fetch(getpid(), fd, name.substr(0, colon) + ":0000000000000000"));   // right socket, wrong token
  } catch (const std::exception&) {
    threw = true;
  }
  CHECK(threw);
  fd_fetch_set_mode("auto");
  fd_server_unregister(fd);
  close(fd);
  close(other);
}

// The tokenizer's batch encoder: a small model (empty charsmap, nine pieces), 400 documents, one
// thread against six; the threads share the engine and keep their own states and word caches.
void test_unigram_batch_threads() {
  const std::string spec =
      "{\"version\": \"1.0\", \"added_tokens\": [], \"normalizer\": {\"type\": \"Precompiled\", "
      "\"precompiled_charsmap\": \"AAAAAA==\"}, \"pre_tokenizer\": {\"type\": \"Metaspace\", \"replacement\": \"\u2581\", "
      "\"prepend_scheme\": \"always\", \"split\": true}, \"post_processor\": null, \"decoder\": {\"type\": \"Metaspace\", "
      "\"replacement\": \"\u2581\", \"prepend_scheme\": \"always\", \"split\": true}, \"model\": {\"type\": \"Unigram\", "
      "\"unk_id\": 0, \"vocab\": [[\"<unk>\", 0.0], [\"\u2581\", -2.0], [\"\u2581a\", -1.0], [\"a\", -3.0], [\"b\", -3.0], "
      "[\"ab\", -2.5], [\"\u2581ab\", -1.5], [\"c\", -4.0], [\"\u2581abc\", -1.2]], \"byte_fallback\": false}}";
  const auto engine = pplx::unigram::Engine::from_hf_json_bytes(spec);
  CHECK(engine->vocab_size() == 9);
  std::vector<std::string> docs;
  uint32_t x = 12345;
  for (int d = 0; d < 400; ++d) {
    std::string text;
    for (int w = 0; w < 200; ++w) {
      x = x * 1664525u + 1013904223u;
      static const char* words[] = {"ab", "abc", "a", "cab", "zz", "abcabc", "b", "ca"};
      text += words[(x >> 24) & 7];
      text += ' ';
    }
    docs.push_back(std::move(text));
  }
  std::vector<std::string_view> views(docs.begin(), docs.end());
  const auto one = engine->encode_batch(views, 1);
  const auto six = engine->encode_batch(views, 6);
  CHECK(one.size() == 400 && one == six);
  const std::vector<pplx::unigram::TokenId> want = {6, 8, 2, 1, 7, 5};
  CHECK(engine->encode_batch({std::string_view("ab abc a cab")}, 2)[0] == want);
}

// The symmetric layout of the all-to-all for a grid of shapes: strides are multiples of 16 bytes
// (128 for the flagged-line format), the regions inside the sync and receive areas do not
// overlap and fit, and the receive area holds a worst-case dispatch and combine.
void test_a2a_layout_invariants() {
  int configs = 0;
  for (int world : {1, 2, 4, 8}) {
    for (int dp : {1, 2}) {
      if (world % dp != 0) continue;
      for (int tokens : {1, 8, 128, 4096}) {
        for (int hidden : {16, 64, 7168}) {
          for (int with_scale : {0, 1}) {
            if (with_scale && hidden % 128 != 0) continue;
            for (int wire : {static_cast<int>(kWirePlain), static_cast<int>(kWireLL)}) {
              for (int mode : {static_cast<int>(kCombinePerRoute), static_cast<int>(kCombinePreReduce)}) {
                A2AParams p;
                p.world = world;
                p.dp_size = dp;
                p.num_experts = 8 * world;
                p.topk = 4;
                p.max_num_tokens = tokens;
                p.hidden_dim = hidden;
                p.hidden_dim_scale = with_scale ? hidden / 128 : 0;
                p.in_elemsize = with_scale ? 1 : 2;
                p.out_elemsize = 2;
                p.wire = wire;
                p.combine_mode = mode;
                const A2AConfig c = a2a_make_config(p, 148, 1);
                ++configs;
                const uint32_t unit = c.wire == kWireLL ? 128u : 16u;
                bool ok = c.d_stride % unit == 0 && c.c_stride % unit == 0 && c.d_stride > 0 && c.c_stride > 0;
                ok = ok && c.num_groups == world / dp && c.experts_per_rank == 8;
                ok = ok && c.d_header_bytes % 16 == 0 && c.d_header_bytes >= 4u * (2 + 2 * 4);
                ok = ok && c.d_payload_bytes >= static_cast<uint32_t>(hidden * p.in_elemsize);
                // sync area: two banks of counts, then the per-token arrival words
                // one counts message per source group, or per source rank in the flagged-line format
                ok = ok && c.counts_bank_words == static_cast<uint32_t>(c.wire == kWireLL ? world : c.num_groups) * c.counts_stride;
                ok = ok && c.off_counts % 16 == 0 && c.off_counts + 8ull * c.counts_bank_words <= c.sync_bytes;
                ok = ok && c.off_tok_arrive % 16 == 0 && c.off_tok_arrive + 4ull * tokens <= c.sync_bytes;
                ok = ok && (c.off_tok_arrive >= c.off_counts + 8ull * c.counts_bank_words ||
                            c.off_counts >= c.off_tok_arrive + 4ull * tokens);
                // receive area: every source group's worst case of records, then the combine slots
                ok = ok && c.drecv_group_stride >= static_cast<uint64_t>(tokens) * c.d_stride;
                ok = ok && c.off_drecv % unit == 0 && c.off_crecv % unit == 0;
                ok = ok && c.off_drecv + c.num_groups * c.drecv_group_stride <= c.off_crecv;
                ok = ok && c.c_records_per_token == static_cast<uint32_t>(mode == kCombinePerRoute ? 4 : world);
                ok = ok && c.off_crecv + static_cast<uint64_t>(tokens) * c.c_records_per_token * c.c_stride <= c.recv_bytes;
                ok = ok && c.max_recv_rows >= static_cast<uint32_t>(tokens) * 4u * static_cast<uint32_t>(c.num_groups);
                if (!ok) {
                  std::fprintf(stderr, "layout: world %d dp %d tokens %d hidden %d scale %d wire %d mode %d\n", world, dp, tokens,
                               hidden, with_scale, wire, mode);
                }
                CHECK(ok);
              }
            }
          }
        }
      }
    }
  }
  CHECK(configs > 300);
}

}  // namespace

int main() {
  test_error();
  test_defer_and_pools();
  test_imm_counts();
  test_sharding();
  test_host_buffers();
  test_addresses_and_topology_helpers();
  test_json_numbers();
  test_engine_threads();
  test_proxy_between_two_nodes();
  test_fd_server_threads();
  test_unigram_batch_threads();
  test_a2a_layout_invariants();
  std::printf("%d checks, %d failed\n", g_checks, g_failures);
  return g_failures == 0 ? 0 : 1;
}
