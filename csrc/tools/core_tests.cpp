// Native unit tests of the host-side building blocks (the counterpart of the reference's Rust
// unit tests: cuda-lib/src/test_driver.rs, fabric-lib's imm_count / utils modules). No GPU is
// needed. Exit code 0 when every check passes; each failure prints its expression and line.
#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "../core/error.h"
#include "../fabric/api.h"
#include "../fabric/host_buffer.h"
#include "../fabric/imm_count.h"
#include "../fabric/shard.h"
#include "../fabric/faulty_domain.h"
#include "../fabric/topo.h"
#include "../fabric/transfer_engine.h"
#include "../fabric/util.h"
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
  auto prev = map.set_expected(7, 2);
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
  std::printf("%d checks, %d failed\n", g_checks, g_failures);
  return g_failures == 0 ? 0 : 1;
}
