// pplx-fabric-debug: benchmark and self-check of the transfer engine.
//
//   pplx-fabric-debug                     both ends in this process (GPU 0 -> GPU 1 when two
//                                         GPUs exist, else GPU 0 -> GPU 0, else host memory)
//   pplx-fabric-debug local <src> <dst>   same, explicit CUDA ordinals (-1 = host memory)
//   pplx-fabric-debug server <gpu>        prints "<descriptor-hex>" and serves writes
//   pplx-fabric-debug client <gpu> <descriptor-hex>
//
// For every shape it fills the source with an xorshift stream, writes, verifies the
// destination (local modes), then times 50 warm-up + 100 measured transfers and reports
// latency, Gbit/s, percent of the link speed and million pages per second. Shapes and
// methodology follow the reference's fabric-debug (fabric-lib/fabric-debug/src/main.rs:
// 330-483,706-837): paged writes of 13 (page size, page count) shapes, single writes from
// 1 KiB to 64 MiB, and the latency of a bare immediate.
#include <cuda_runtime.h>

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <iostream>
#include <mutex>
#include <numeric>
#include <random>
#include <string>
#include <thread>
#include <vector>

#include "../core/error.h"
#include "../core/log.h"
#include "../fabric/transfer_engine.h"

using namespace pplx;
using namespace pplx::fabric;
using Clock = std::chrono::steady_clock;

namespace {

struct Buffer {
  int device = -1;
  size_t bytes = 0;
  void* ptr = nullptr;
  Buffer(int dev, size_t n) : device(dev), bytes(n) {
    if (dev >= 0) {
      PPLX_CUDA_CHECK(cudaSetDevice(dev));
      PPLX_CUDA_CHECK(cudaMalloc(&ptr, n));
      PPLX_CUDA_CHECK(cudaMemset(ptr, 0, n));
    } else {
      if (posix_memalign(&ptr, 4096, n) != 0) throw Error::from_errno("posix_memalign");
      std::memset(ptr, 0, n);
    }
  }
  ~Buffer() {
    if (device >= 0) cudaFree(ptr); else std::free(ptr);
  }
  void upload(const std::vector<uint8_t>& host) {
    if (device >= 0) {
      PPLX_CUDA_CHECK(cudaSetDevice(device));
      PPLX_CUDA_CHECK(cudaMemcpy(ptr, host.data(), host.size(), cudaMemcpyHostToDevice));
    } else {
      std::memcpy(ptr, host.data(), host.size());
    }
  }
  std::vector<uint8_t> download() const {
    std::vector<uint8_t> host(bytes);
    if (device >= 0) {
      PPLX_CUDA_CHECK(cudaSetDevice(device));
      PPLX_CUDA_CHECK(cudaMemcpy(host.data(), ptr, bytes, cudaMemcpyDeviceToHost));
    } else {
      std::memcpy(host.data(), ptr, bytes);
    }
    return host;
  }
  void clear() {
    if (device >= 0) {
      PPLX_CUDA_CHECK(cudaSetDevice(device));
      PPLX_CUDA_CHECK(cudaMemset(ptr, 0, bytes));
    } else {
      std::memset(ptr, 0, bytes);
    }
  }
};

std::vector<uint8_t> xorshift_bytes(size_t n, uint64_t seed) {
  std::vector<uint8_t> out(n);
  uint64_t x = seed ? seed : 88172645463325252ull;
  for (size_t i = 0; i < n; i += 8) {
    x ^= x << 13;
    x ^= x >> 7;
    x ^= x << 17;
    std::memcpy(out.data() + i, &x, std::min<size_t>(8, n - i));
  }
  return out;
}

struct Latch {
  std::mutex mu;
  std::condition_variable cv;
  int pending = 0;
  std::string error;
  void add(int n) {
    std::lock_guard<std::mutex> l(mu);
    pending += n;
  }
  void done() {
    std::lock_guard<std::mutex> l(mu);
    --pending;
    cv.notify_all();
  }
  void fail(const std::string& e) {
    std::lock_guard<std::mutex> l(mu);
    error = e;
    --pending;
    cv.notify_all();
  }
  void wait() {
    std::unique_lock<std::mutex> l(mu);
    if (!cv.wait_for(l, std::chrono::seconds(60), [&] { return pending <= 0; })) {
      throw Error(ErrorKind::kTimeout, "transfer did not complete within 60 s");
    }
    if (!error.empty()) throw Error(ErrorKind::kCompletion, error);
  }
};

struct Stats {
  double mean_us, p50_us, min_us;
};

template <typename F>
Stats time_it(F&& one, int warmup = 50, int repeats = 100) {
  for (int i = 0; i < warmup; ++i) one();
  std::vector<double> us;
  for (int i = 0; i < repeats; ++i) {
    const auto t0 = Clock::now();
    one();
    us.push_back(std::chrono::duration<double, std::micro>(Clock::now() - t0).count());
  }
  std::sort(us.begin(), us.end());
  return Stats{std::accumulate(us.begin(), us.end(), 0.0) / us.size(), us[us.size() / 2], us.front()};
}

std::vector<GpuDomainSpec> spec_for(int device, size_t nets) {
  GpuDomainSpec s;
  s.cuda_device = device;
  for (size_t i = 0; i < nets; ++i) {
    s.domains.push_back(DomainInfo{(device >= 0 ? "nvl" : "host") + std::to_string(i), 0, "local"});
  }
  return {s};
}

void bench_pair(TransferEngine& tx, TransferEngine* rx, int src_dev, const MemoryRegionDescriptor& dst_desc,
                Buffer* dst_buf, size_t region) {
  Buffer src(src_dev, region);
  const std::vector<uint8_t> pattern = xorshift_bytes(region, 42);
  src.upload(pattern);
  const auto [src_handle, src_desc] = tx.register_memory(reinterpret_cast<uint64_t>(src.ptr), region, src_dev);
  (void)src_desc;
  const double link_gbps = static_cast<double>(tx.aggregated_link_speed()) / 1e9;

  std::printf("%-34s %12s %12s %10s %8s %10s\n", "shape", "p50 us", "mean us", "Gbit/s", "% link", "Mpages/s");
  // ---- paged writes ----
  const std::pair<size_t, size_t> shapes[] = {{4096, 1},   {4096, 16},  {4096, 256}, {4096, 4096}, {16384, 64},
                                              {16384, 1024}, {65536, 16}, {65536, 256}, {131072, 64}, {131072, 512},
                                              {262144, 128}, {1048576, 32}, {1048576, 64}};
  for (const auto& [page, count] : shapes) {
    if (page * count * 2 > region) continue;
    auto src_pages = std::make_shared<std::vector<uint32_t>>(count);
    auto dst_pages = std::make_shared<std::vector<uint32_t>>(count);
    std::mt19937 rng(7);
    std::vector<uint32_t> perm(region / page / 2);
    std::iota(perm.begin(), perm.end(), 0u);
    std::shuffle(perm.begin(), perm.end(), rng);
    for (size_t i = 0; i < count; ++i) (*src_pages)[i] = perm[i];
    std::shuffle(perm.begin(), perm.end(), rng);
    for (size_t i = 0; i < count; ++i) (*dst_pages)[i] = perm[i];
    auto one = [&] {
      Latch latch;
      latch.add(1);
      PagedTransferRequest r;
      r.length = page;
      r.src_mr = src_handle;
      r.src_page_indices = src_pages;
      r.src_stride = page;
      r.dst_mr = dst_desc;
      r.dst_page_indices = dst_pages;
      r.dst_stride = page;
      tx.submit_transfer(r, [&] { latch.done(); }, [&](const std::string& e) { latch.fail(e); });
      latch.wait();
    };
    bool verified = false;
    if (dst_buf != nullptr) {
      dst_buf->clear();
      one();
      const std::vector<uint8_t> got = dst_buf->download();
      verified = true;
      for (size_t i = 0; i < count && verified; ++i) {
        verified = std::memcmp(got.data() + (*dst_pages)[i] * page, pattern.data() + (*src_pages)[i] * page, page) == 0;
      }
      if (!verified) throw Error(ErrorKind::kCustom, "paged write verification FAILED");
    }
    const Stats st = time_it(one);
    const double gbps = page * count * 8.0 / (st.p50_us * 1e3);
    char name[64];
    std::snprintf(name, sizeof(name), "paged %zu B x %zu%s", page, count, verified ? " VERIFIED" : "");
    std::printf("%-34s %12.1f %12.1f %10.1f %8.1f %10.3f\n", name, st.p50_us, st.mean_us, gbps,
                100.0 * gbps / link_gbps, count / st.p50_us);
  }
  // ---- single writes ----
  for (size_t bytes = 1024; bytes <= (64u << 20) && bytes <= region; bytes *= 4) {
    auto one = [&] {
      Latch latch;
      latch.add(1);
      SingleTransferRequest r;
      r.src_mr = src_handle;
      r.length = bytes;
      r.dst_mr = dst_desc;
      r.domain = DomainGroupRouting::sharded(static_cast<uint8_t>(tx.nets_per_gpu()));
      tx.submit_transfer(r, [&] { latch.done(); }, [&](const std::string& e) { latch.fail(e); });
      latch.wait();
    };
    bool verified = false;
    if (dst_buf != nullptr) {
      dst_buf->clear();
      one();
      const std::vector<uint8_t> got = dst_buf->download();
      verified = std::memcmp(got.data(), pattern.data(), bytes) == 0;
      if (!verified) throw Error(ErrorKind::kCustom, "single write verification FAILED");
    }
    const Stats st = time_it(one);
    const double gbps = bytes * 8.0 / (st.p50_us * 1e3);
    char name[64];
    std::snprintf(name, sizeof(name), "single %zu B%s", bytes, verified ? " VERIFIED" : "");
    std::printf("%-34s %12.1f %12.1f %10.1f %8.1f %10s\n", name, st.p50_us, st.mean_us, gbps,
                100.0 * gbps / link_gbps, "-");
  }
  // ---- immediate latency (needs the receiving engine in this process) ----
  if (rx != nullptr) {
    ImmCounter counter = rx->get_imm_counter(0x1234);
    auto one = [&] {
      ImmTransferRequest r{0x1234, dst_desc, DomainGroupRouting::pinned(0)};
      tx.submit_transfer(r, [] {}, [](const std::string&) {});
      if (!counter.wait(1, 10000)) throw Error(ErrorKind::kTimeout, "immediate did not arrive");
    };
    const Stats st = time_it(one);
    std::printf("%-34s %12.1f %12.1f %10s %8s %10s\n", "imm one-way (submit -> counted)", st.p50_us, st.mean_us,
                "-", "-", "-");
  }
  tx.unregister_memory(reinterpret_cast<uint64_t>(src.ptr));
}

int run_local(int src_dev, int dst_dev) {
  const size_t region = 256u << 20;
  TransferEngine tx(spec_for(src_dev, 1));
  TransferEngine rx(spec_for(dst_dev, 1));
  Buffer dst(dst_dev, region);
  const auto [h, desc] = rx.register_memory(reinterpret_cast<uint64_t>(dst.ptr), region, dst_dev);
  (void)h;
  std::printf("# source %s, destination %s, link %.0f Gbit/s\n",
              src_dev >= 0 ? ("cuda:" + std::to_string(src_dev)).c_str() : "host",
              dst_dev >= 0 ? ("cuda:" + std::to_string(dst_dev)).c_str() : "host",
              static_cast<double>(tx.aggregated_link_speed()) / 1e9);
  bench_pair(tx, &rx, src_dev, desc, &dst, region);
  tx.stop();
  rx.stop();
  return 0;
}

}  // namespace

int main(int argc, char** argv) {
  log_init_from_env();
  try {
    const std::string mode = argc > 1 ? argv[1] : "auto";
    if (mode == "auto") {
      int count = 0;
      if (cudaGetDeviceCount(&count) != cudaSuccess) count = 0;
      return count >= 2 ? run_local(0, 1) : count == 1 ? run_local(0, 0) : run_local(-1, -1);
    }
    if (mode == "local" && argc >= 4) return run_local(std::atoi(argv[2]), std::atoi(argv[3]));
    if (mode == "server" && argc >= 3) {
      const int dev = std::atoi(argv[2]);
      const size_t region = 256u << 20;
      TransferEngine rx(spec_for(dev, 1));
      Buffer dst(dev, region);
      const auto [h, desc] = rx.register_memory(reinterpret_cast<uint64_t>(dst.ptr), region, dev);
      (void)h;
      std::printf("%s\n", hex_encode(desc.serialize()).c_str());
      std::fflush(stdout);
      std::fprintf(stderr, "serving; press enter (or close stdin) to stop\n");
      std::string line;
      std::getline(std::cin, line);
      rx.stop();
      return 0;
    }
    if (mode == "client" && argc >= 4) {
      const int dev = std::atoi(argv[2]);
      const MemoryRegionDescriptor desc = MemoryRegionDescriptor::deserialize(hex_decode(argv[3]));
      TransferEngine tx(spec_for(dev, 1));
      bench_pair(tx, nullptr, dev, desc, nullptr, 256u << 20);
      tx.stop();
      return 0;
    }
    std::fprintf(stderr, "usage: %s [local <src> <dst> | server <gpu> | client <gpu> <descriptor-hex>]\n", argv[0]);
    return 2;
  } catch (const std::exception& e) {
    std::fprintf(stderr, "error: %s\n", e.what());
    return 1;
  }
}
