#include "a2a_context.h"

#include <nvtx3/nvToolsExt.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>

#include "../core/error.h"
#define PPLX_LOG_TARGET "pplx_garden::a2a"
#include "../core/log.h"
#include "a2a_kernels.h"

namespace pplx {

namespace {
uint32_t round_up_u32(uint32_t a, uint32_t b) { return (a + b - 1) / b * b; }

struct NvtxRange {
  explicit NvtxRange(const char* name) { nvtxRangePushA(name); }
  ~NvtxRange() { nvtxRangePop(); }
};
}  // namespace

A2AConfig a2a_make_config(const A2AParams& p, int num_sms, int virtual_ranks) {
  PPLX_REQUIRE(p.world >= 1 && p.world <= kMaxRanks, "world size must be in [1, 8]");
  PPLX_REQUIRE(p.dp_size >= 1 && p.world % p.dp_size == 0, "dp_size must divide the world size");
  PPLX_REQUIRE(p.num_experts >= 1, "num_experts must be positive");
  PPLX_REQUIRE(p.topk >= 1 && p.topk <= kMaxTopK, "num_experts_per_token must be in [1, 16]");
  PPLX_REQUIRE(p.topk <= p.num_experts, "num_experts_per_token exceeds num_experts");
  PPLX_REQUIRE(p.max_num_tokens >= 1, "max_num_tokens must be positive");
  PPLX_REQUIRE(p.hidden_dim >= 8 && p.hidden_dim % 8 == 0, "hidden_dim must be a multiple of 8");
  PPLX_REQUIRE((static_cast<int64_t>(p.hidden_dim) * p.in_elemsize) % 16 == 0,
               "hidden_dim * in_elemsize must be a multiple of 16 bytes");
  PPLX_REQUIRE(p.in_elemsize == 1 || p.in_elemsize == 2 || p.in_elemsize == 4, "bad in_elemsize");
  PPLX_REQUIRE(p.out_elemsize == 2 || p.out_elemsize == 4, "out dtype must be f16, bf16 or f32");
  PPLX_REQUIRE(p.hidden_dim_scale == 0 || p.scale_elemsize == 4, "scales must be float32");
  PPLX_REQUIRE(p.expert_padding >= 1, "expert_padding must be positive");
  PPLX_REQUIRE(virtual_ranks >= 1 && virtual_ranks <= kMaxVirtualRanks, "bad virtual rank count");

  A2AConfig c{};
  c.world = p.world;
  c.dp_size = p.dp_size;
  c.num_groups = p.world / p.dp_size;
  c.num_experts = p.num_experts;
  c.experts_per_rank = (p.num_experts + p.world - 1) / p.world;
  c.topk = p.topk;
  c.max_num_tokens = p.max_num_tokens;
  c.hidden_dim = p.hidden_dim;
  c.hidden_dim_scale = p.hidden_dim_scale;
  c.in_elemsize = p.in_elemsize;
  c.out_elemsize = p.out_elemsize;
  c.expert_padding = p.expert_padding;
  c.combine_mode = p.combine_mode;

  int blocks = p.num_blocks;
  if (blocks <= 0) {
    const char* env = std::getenv("PPLX_A2A_BLOCKS");
    blocks = env ? std::atoi(env) : 0;
  }
  if (blocks <= 0) blocks = std::max(1, num_sms / virtual_ranks);
  c.num_blocks = blocks;

  int wire = p.wire;
  if (wire == kWireAuto) {
    const char* env = std::getenv("PPLX_A2A_WIRE");
    if (env != nullptr && std::strcmp(env, "ll") == 0) wire = kWireLL;
    else if (env != nullptr && std::strcmp(env, "plain") == 0) wire = kWirePlain;
    else wire = p.max_num_tokens <= 512 ? kWireLL : kWirePlain;
  }
  PPLX_REQUIRE(wire == kWirePlain || wire == kWireLL, "wire must be 'plain' or 'll'");
  c.wire = wire;
  const uint32_t all_ranks = p.world >= 32 ? 0xffffffffu : ((1u << p.world) - 1u);
  c.node_mask = p.node_mask == 0 ? all_ranks : (p.node_mask & all_ranks);
  PPLX_REQUIRE(c.node_mask == all_ranks || wire == kWirePlain,
               "ranks outside the NVLink domain need the plain wire format (wire='plain')");

  c.d_header_bytes = round_up_u32(4u * (2 + 2 * p.topk), 16);
  c.d_payload_bytes = static_cast<uint32_t>(p.hidden_dim) * p.in_elemsize;
  c.d_scale_bytes = round_up_u32(static_cast<uint32_t>(p.hidden_dim_scale) * 4u, 16);
  const uint32_t c_row_bytes = round_up_u32(static_cast<uint32_t>(p.hidden_dim) * p.out_elemsize, 16);
  if (wire == kWireLL) {
    // seven data vectors per 128-byte line
    const uint32_t d_vecs = (c.d_header_bytes + c.d_payload_bytes + c.d_scale_bytes) / 16;
    c.d_stride = (d_vecs + 6) / 7 * 128;
    c.c_stride = (c_row_bytes / 16 + 6) / 7 * 128;
  } else {
    c.d_stride = round_up_u32(c.d_header_bytes + c.d_payload_bytes + c.d_scale_bytes, 128);
    c.c_stride = c_row_bytes;
  }
  c.c_records_per_token = p.combine_mode == kCombinePreReduce ? p.world : p.topk;
  c.counts_stride = round_up_u32(1 + c.experts_per_rank, 4);
  int count_sources = c.num_groups;
  if (wire == kWireLL) {
    // flagged lines, one set per source *rank*: seven data vectors per 128-byte line
    c.counts_stride = (c.counts_stride / 4 + 6) / 7 * 32;
    count_sources = p.world;
  }

  const uint64_t rows_per_token = std::min(p.topk, c.experts_per_rank);
  uint64_t rows = static_cast<uint64_t>(c.num_groups) * p.max_num_tokens * rows_per_token +
                  static_cast<uint64_t>(c.experts_per_rank) * (p.expert_padding - 1);
  rows = round_up_u64(rows, p.expert_padding);
  PPLX_REQUIRE(rows < (1ull << 31), "receive row count overflows 31 bits");
  c.max_recv_rows = static_cast<uint32_t>(rows);

  const uint64_t flag_bytes =
      static_cast<uint64_t>(kNumFlagRows) * kMaxRanks * kFlagStrideWords * sizeof(uint32_t);
  c.off_counts = flag_bytes;
  c.counts_bank_words = static_cast<uint32_t>(count_sources) * c.counts_stride;
  c.off_tok_arrive = round_up_u64(c.off_counts + 2ull * 4ull * c.counts_bank_words, 128);
  c.sync_bytes = round_up_u64(c.off_tok_arrive + 4ull * p.max_num_tokens, 4096);

  c.off_drecv = 0;
  c.drecv_group_stride = static_cast<uint64_t>(p.max_num_tokens) * c.d_stride;
  c.off_crecv = round_up_u64(c.drecv_group_stride * c.num_groups, 4096);
  const uint64_t crecv_bytes =
      static_cast<uint64_t>(p.max_num_tokens) * c.c_records_per_token * c.c_stride;
  c.recv_bytes = round_up_u64(c.off_crecv + crecv_bytes, 4096);

  int64_t limit_ms = p.wait_limit_ms;
  if (limit_ms <= 0) {
    const char* env = std::getenv("PPLX_A2A_TIMEOUT_MS");
    limit_ms = env ? std::atoll(env) : 0;
  }
  if (limit_ms <= 0) limit_ms = 10000;
  c.wait_limit_ns = static_cast<uint64_t>(limit_ms) * 1000000ull;
  return c;
}

std::string A2AStatusInfo::message() const {
  static const char* phases[] = {"dispatch_send", "dispatch_recv", "combine_send", "combine_recv"};
  const char* ph = phase < 4 ? phases[phase] : "?";
  switch (code) {
    case kStatusOk: return "ok";
    case kStatusWaitTimeout:
      return std::string("all-to-all ") + ph + ": timed out waiting for source " +
             std::to_string(who) + " (expected arrival count " + std::to_string(detail) + ")";
    case kStatusRowOverflow:
      return std::string("all-to-all ") + ph + ": " + std::to_string(who) +
             " expert rows do not fit the output tensor (" + std::to_string(detail) + " rows)";
    case kStatusBadExpertIndex:
      return std::string("all-to-all ") + ph + ": token " + std::to_string(who) +
             " routes to expert " + std::to_string(detail) + " which does not exist";
    case kStatusRecordOverflow:
      return std::string("all-to-all ") + ph + ": more records for rank " + std::to_string(who) +
             " than its region holds";
    default: return "all-to-all: unknown failure code " + std::to_string(code);
  }
}

A2AContext::A2AContext(const A2AParams& params, int device, const std::vector<int>& ranks,
                       const std::vector<std::vector<uint64_t>>& sync_ptrs,
                       const std::vector<std::vector<uint64_t>>& recv_ptrs)
    : device_(device), ranks_(ranks) {
  PPLX_REQUIRE(!ranks.empty() && ranks.size() <= static_cast<size_t>(kMaxVirtualRanks),
               "a context plays between 1 and 8 ranks");
  PPLX_REQUIRE(sync_ptrs.size() == ranks.size() && recv_ptrs.size() == ranks.size(),
               "one pointer table per local rank is required");
  PPLX_CUDA_CHECK(cudaSetDevice(device));
  int num_sms = 0;
  PPLX_CUDA_CHECK(cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, device));
  cfg_ = a2a_make_config(params, num_sms, static_cast<int>(ranks.size()));
  if (ranks.size() > 1) {
    PPLX_REQUIRE(static_cast<int>(ranks.size()) * cfg_.num_blocks <= num_sms,
                 "virtual ranks x blocks must fit the GPU at one block per SM");
  }

  PPLX_CUDA_CHECK(a2a_preload_kernels(cfg_));
  const char* trace_env = std::getenv("PPLX_A2A_TRACE");
  cfg_.trace = (trace_env != nullptr && std::atoi(trace_env) != 0) ? 1 : 0;
  const char* team_env = std::getenv("PPLX_A2A_TEAM");
  if (team_env != nullptr) team_override_ = std::atoi(team_env);

  const size_t GL = static_cast<size_t>(cfg_.num_groups) * cfg_.experts_per_rank;
  const size_t L = cfg_.experts_per_rank;
  const size_t rows = cfg_.max_recv_rows;
  const size_t recs = static_cast<size_t>(cfg_.num_groups) * cfg_.max_num_tokens;
  const bool pre = cfg_.combine_mode == kCombinePreReduce;

  for (size_t i = 0; i < ranks.size(); ++i) {
    PPLX_REQUIRE(ranks[i] >= 0 && ranks[i] < cfg_.world, "rank out of range");
    PPLX_REQUIRE(sync_ptrs[i].size() == static_cast<size_t>(cfg_.world) &&
                     recv_ptrs[i].size() == static_cast<size_t>(cfg_.world),
                 "pointer tables must have one entry per rank of the world");
    A2ARankState& st = states_.r[i];
    st.rank = ranks[i];
    for (int p = 0; p < cfg_.world; ++p) {
      PPLX_REQUIRE(sync_ptrs[i][p] % 128 == 0 && recv_ptrs[i][p] % 128 == 0,
                   "symmetric regions must be 128-byte aligned");
      st.sync[p] = reinterpret_cast<uint8_t*>(sync_ptrs[i][p]);
      st.recv[p] = reinterpret_cast<uint8_t*>(recv_ptrs[i][p]);
    }
    // One zero-filled allocation for the whole device-local workspace.
    size_t off = 0;
    auto take = [&](size_t bytes) {
      const size_t at = off;
      off += (bytes + 255) / 256 * 256;
      return at;
    };
    const size_t o_epochs = take(sizeof(uint32_t) * 4);
    const size_t o_done = take(sizeof(uint32_t) * 2);
    const size_t o_send_cursor = take(sizeof(uint32_t) * 2 * kMaxRanks);
    const size_t o_place_cursor = take(sizeof(uint32_t) * 2 * GL);
    const size_t o_row_src = take(sizeof(uint32_t) * rows);
    const size_t o_row_tk = take(sizeof(uint32_t) * rows);
    const size_t o_meta = take(sizeof(uint32_t) * (2 + 2 * L));
    const size_t o_rec_rows = take(pre ? sizeof(uint32_t) * recs * cfg_.topk : 4);
    const size_t o_rec_w = take(pre ? sizeof(float) * recs * cfg_.topk : 4);
    const size_t o_rec_tok = take(pre ? sizeof(uint32_t) * 2 * recs : 4);
    const size_t o_status = take(sizeof(uint32_t) * 4);
    const size_t o_stats = take(sizeof(unsigned long long) * 8);
    const size_t o_trace = take(sizeof(unsigned long long) * kTraceSlots);
    const size_t o_scatter_done = take(sizeof(uint32_t));
    const size_t o_route_hist = take(sizeof(uint32_t) * 2 * cfg_.num_experts);
    const size_t o_route_nrec = take(sizeof(uint32_t) * 2 * kMaxRanks);
    const size_t o_route_done = take(sizeof(uint32_t) * 2);
    void* base = nullptr;
    PPLX_CUDA_CHECK(cudaMalloc(&base, off));
    allocations_.push_back(base);
    PPLX_CUDA_CHECK(cudaMemset(base, 0, off));
    uint8_t* b = static_cast<uint8_t*>(base);
    st.local.epochs = reinterpret_cast<uint32_t*>(b + o_epochs);
    st.local.done = reinterpret_cast<uint32_t*>(b + o_done);
    st.local.send_cursor = reinterpret_cast<uint32_t*>(b + o_send_cursor);
    st.local.place_cursor = reinterpret_cast<uint32_t*>(b + o_place_cursor);
    st.local.row_src = reinterpret_cast<uint32_t*>(b + o_row_src);
    st.local.row_tk = reinterpret_cast<uint32_t*>(b + o_row_tk);
    st.local.expert_meta = reinterpret_cast<uint32_t*>(b + o_meta);
    st.local.rec_rows = reinterpret_cast<uint32_t*>(b + o_rec_rows);
    st.local.rec_weights = reinterpret_cast<float*>(b + o_rec_w);
    st.local.rec_token = reinterpret_cast<uint32_t*>(b + o_rec_tok);
    st.local.status = reinterpret_cast<uint32_t*>(b + o_status);
    st.local.stats = reinterpret_cast<unsigned long long*>(b + o_stats);
    st.local.trace = reinterpret_cast<unsigned long long*>(b + o_trace);
    st.local.route_hist = reinterpret_cast<uint32_t*>(b + o_route_hist);
    st.local.route_nrec = reinterpret_cast<uint32_t*>(b + o_route_nrec);
    st.local.route_done = reinterpret_cast<uint32_t*>(b + o_route_done);
    trace_ptrs_.push_back(st.local.trace);
    scatter_done_ptrs_.push_back(reinterpret_cast<uint32_t*>(b + o_scatter_done));
    uint32_t* host_flag = nullptr;
    PPLX_CUDA_CHECK(cudaHostAlloc(reinterpret_cast<void**>(&host_flag), 64, cudaHostAllocMapped));
    std::memset(host_flag, 0, 64);
    uint32_t* host_flag_dev = nullptr;
    PPLX_CUDA_CHECK(cudaHostGetDevicePointer(reinterpret_cast<void**>(&host_flag_dev), host_flag, 0));
    st.local.host_flag = host_flag_dev;
    host_flags_.push_back(host_flag);
    status_ptrs_.push_back(st.local.status);
    stats_ptrs_.push_back(st.local.stats);
    iters_ptrs_.push_back(st.local.epochs);
  }
  PPLX_CUDA_CHECK(cudaDeviceSynchronize());
  PPLX_INFO("a2a context: world=%d dp=%d experts=%d topk=%d hidden=%d record=%uB/%uB blocks=%d "
            "local_ranks=%zu recv=%.1f MiB wire=%s",
            cfg_.world, cfg_.dp_size, cfg_.num_experts, cfg_.topk, cfg_.hidden_dim, cfg_.d_stride,
            cfg_.c_stride, cfg_.num_blocks, ranks.size(), cfg_.recv_bytes / 1048576.0,
            cfg_.wire == kWireLL ? "ll" : "plain");
}

void A2AContext::enable_proxy(int i, fabric::TransferEngine* engine, std::vector<A2AProxyPeer> peers,
                              int pin_cpu) {
  PPLX_REQUIRE(i >= 0 && i < num_local_ranks(), "enable_proxy: no such local rank");
  PPLX_REQUIRE(engine != nullptr, "enable_proxy: a transfer engine is required");
  PPLX_REQUIRE(cfg_.wire == kWirePlain, "enable_proxy: the plain wire format is required");
  if (proxies_.size() < ranks_.size()) proxies_.resize(ranks_.size());
  PPLX_REQUIRE(!proxies_[i].proxy, "enable_proxy: this local rank already has a proxy");
  PPLX_CUDA_CHECK(cudaSetDevice(device_));
  A2ARankState& st = states_.r[i];
  ProxyState& ps = proxies_[i];
  ps.engine = engine;
  const int my_group = st.rank / cfg_.dp_size;

  auto device_alloc = [&](size_t bytes) {
    void* p = nullptr;
    PPLX_CUDA_CHECK(cudaMalloc(&p, bytes));
    PPLX_CUDA_CHECK(cudaMemset(p, 0, bytes));
    ps.device_buffers.push_back(p);
    return reinterpret_cast<uint64_t>(p);
  };
  auto host_alloc = [&](size_t bytes, uint32_t** device_view) {
    uint32_t* p = nullptr;
    PPLX_CUDA_CHECK(cudaHostAlloc(reinterpret_cast<void**>(&p), bytes, cudaHostAllocMapped));
    std::memset(p, 0, bytes);
    ps.host_buffers.push_back(p);
    if (device_view != nullptr) {
      PPLX_CUDA_CHECK(cudaHostGetDevicePointer(reinterpret_cast<void**>(device_view), p, 0));
    }
    return p;
  };
  auto reg = [&](uint64_t ptr, uint64_t len, int device) {
    engine->register_memory(ptr, len, device);
    ps.registered.push_back(ptr);
  };

  A2AProxyBuffers buf;
  // device-local words of this rank that only exist with a proxy
  const uint64_t extra = device_alloc(256 + 256);
  st.local.send_done = reinterpret_cast<uint32_t*>(extra);
  st.local.stage_cursor = reinterpret_cast<uint32_t*>(extra + 256);
  uint32_t* proxy_dev = nullptr;
  uint32_t* proxy_host = host_alloc(sizeof(uint32_t) * kProxyWords, &proxy_dev);
  st.local.proxy = proxy_dev;
  buf.proxy_words = proxy_host;
  uint32_t* slot_dev = nullptr;
  uint32_t* slot_host = host_alloc(sizeof(uint32_t) * std::max<size_t>(cfg_.max_recv_rows, 1), &slot_dev);
  st.local.stage_slot = slot_dev;
  buf.stage_slot = slot_host;
  const size_t stage_bytes = round_up_u64(static_cast<uint64_t>(cfg_.max_recv_rows) * cfg_.c_stride, 4096);
  buf.stage = device_alloc(stage_bytes);
  st.local.stage = reinterpret_cast<uint8_t*>(buf.stage);
  reg(buf.stage, stage_bytes, device_);
  uint32_t* flag_host = host_alloc(4096, nullptr);
  buf.flag_source = reinterpret_cast<uint64_t>(flag_host);
  buf.flag_source_host = flag_host;
  reg(buf.flag_source, 4096, -1);

  const uint64_t slice_bytes = round_up_u64(cfg_.drecv_group_stride, 4096);
  for (const A2AProxyPeer& p : peers) {
    PPLX_REQUIRE(p.rank >= 0 && p.rank < cfg_.world && ((cfg_.node_mask >> p.rank) & 1u) == 0,
                 "enable_proxy: a peer is inside the NVLink domain");
    buf.shadow_sync[p.rank] = device_alloc(cfg_.sync_bytes);
    reg(buf.shadow_sync[p.rank], cfg_.sync_bytes, device_);
    buf.shadow_recv[p.rank] = device_alloc(slice_bytes);
    reg(buf.shadow_recv[p.rank], slice_bytes, device_);
    // The kernels address "rank p's regions" exactly as they would a mapped peer; only this
    // rank's group slice of the dispatch records is ever touched there, so only that is backed.
    st.sync[p.rank] = reinterpret_cast<uint8_t*>(buf.shadow_sync[p.rank]);
    st.recv[p.rank] = reinterpret_cast<uint8_t*>(buf.shadow_recv[p.rank]) -
                      (cfg_.off_drecv + static_cast<uint64_t>(my_group) * cfg_.drecv_group_stride);
  }
  for (int r = 0; r < cfg_.world; ++r) {
    if (((cfg_.node_mask >> r) & 1u) == 0) {
      PPLX_REQUIRE(buf.shadow_sync[r] != 0, "enable_proxy: a rank outside the NVLink domain has no peer entry");
    }
  }
  PPLX_CUDA_CHECK(cudaDeviceSynchronize());
  ps.proxy = std::make_unique<A2AProxy>(cfg_, st.rank, engine, std::move(peers), buf, pin_cpu);
  PPLX_INFO("a2a proxy for rank %d: %zu remote rank(s), staging %.1f MiB", st.rank,
            static_cast<size_t>(__builtin_popcount(~cfg_.node_mask & ((1u << cfg_.world) - 1u))),
            stage_bytes / 1048576.0);
}

A2AContext::~A2AContext() {
  for (ProxyState& ps : proxies_) {
    ps.proxy.reset();   // joins the thread before its buffers go away
    for (uint64_t ptr : ps.registered) {
      try {
        ps.engine->unregister_memory(ptr);
      } catch (const std::exception&) {
        // the engine may already have been stopped
      }
    }
    for (void* p : ps.device_buffers) cudaFree(p);
    for (void* p : ps.host_buffers) cudaFreeHost(p);
  }
  for (void* p : allocations_) cudaFree(p);
  for (uint32_t* p : host_flags_) cudaFreeHost(p);
}

bool A2AContext::failed() const {
  for (const uint32_t* p : host_flags_) {
    if (*reinterpret_cast<const volatile uint32_t*>(p) != 0) return true;
  }
  for (const ProxyState& p : proxies_) {
    if (p.proxy && p.proxy->failed()) return true;
  }
  return false;
}

void A2AContext::require_phase(int first) const {
  // The device protocol tags records with the dispatch number and counts arrivals, so the
  // four phases must be issued in order, each exactly once per layer.
  static const char* names[] = {"dispatch_send", "dispatch_recv", "combine_send", "combine_recv"};
  if (first != next_phase_) {
    throw Error(ErrorKind::kInvalidArgument,
                std::string("all-to-all phases out of order: got ") + names[first] +
                    " but the next phase of this context is " + names[next_phase_] +
                    " (sequence: dispatch_send, dispatch_recv, combine_send, combine_recv)");
  }
}

void A2AContext::require_proxies() const {
  const uint32_t all_ranks = cfg_.world >= 32 ? 0xffffffffu : ((1u << cfg_.world) - 1u);
  if (cfg_.node_mask == all_ranks) return;
  for (size_t i = 0; i < ranks_.size(); ++i) {
    PPLX_REQUIRE(i < proxies_.size() && proxies_[i].proxy != nullptr,
                 "ranks outside the NVLink domain need enable_proxy() before the first dispatch");
  }
}

void A2AContext::commit_phase(int last) { next_phase_ = (last + 1) % kNumPhases; }

int A2AContext::pick(int64_t items, int64_t vectors_per_item) const {
  if (team_override_ == 32 || team_override_ == 128 || team_override_ == 512) return team_override_;
  return a2a_pick_team(cfg_, std::max<int64_t>(items, 1), std::max<int64_t>(vectors_per_item, 1));
}

void A2AContext::dispatch(const DispatchSendArgs* send, const DispatchRecvArgs* recv, bool do_send,
                          bool do_recv, cudaStream_t stream) {
  PPLX_REQUIRE(do_send || do_recv, "dispatch: nothing to do");
  require_proxies();
  // Nothing is committed before the launch went through: a rejected call leaves the context
  // where it was, so a corrected call may follow.
  require_phase(do_send ? kPhaseDispatchSend : kPhaseDispatchRecv);
  NvtxRange range(do_send && do_recv ? "a2a_dispatch" : do_send ? "a2a_dispatch_send" : "a2a_dispatch_recv");
  PerRank<DispatchSendArgs> s{};
  PerRank<DispatchRecvArgs> r{};
  const int n = num_local_ranks();
  for (int i = 0; i < n; ++i) {
    if (do_send) {
      s.r[i] = send[i];
      PPLX_REQUIRE(send[i].num_tokens >= 0 && send[i].num_tokens <= cfg_.max_num_tokens,
                   "dispatch: num_tokens exceeds max_num_tokens");
      PPLX_REQUIRE(reinterpret_cast<uintptr_t>(send[i].x) % 16 == 0 && send[i].x_stride % 16 == 0,
                   "dispatch: dp_x rows must be 16-byte aligned");
      if (send[i].quantize) {
        PPLX_REQUIRE(cfg_.in_elemsize == 1 && cfg_.hidden_dim % 128 == 0 &&
                         cfg_.hidden_dim_scale == cfg_.hidden_dim / 128,
                     "fused quantisation needs a 1-byte wire type and one scale per 128 elements");
      } else if (cfg_.hidden_dim_scale > 0) {
        PPLX_REQUIRE(send[i].x_scale != nullptr, "dispatch: dp_x_scale is required");
      }
      if (send[i].logits != nullptr) {
        PPLX_REQUIRE(cfg_.num_experts <= 512, "routing fused into dispatch handles at most 512 experts");
        PPLX_REQUIRE(send[i].logits_stride >= cfg_.num_experts, "dispatch: logits rows are shorter than num_experts");
      }
      last_tokens_ = std::max<int64_t>(send[i].num_tokens, 1);
    }
    if (do_recv) {
      r.r[i] = recv[i];
      PPLX_REQUIRE(reinterpret_cast<uintptr_t>(recv[i].out_x) % 16 == 0 &&
                       recv[i].out_x_stride % 16 == 0,
                   "dispatch: out_expert_x rows must be 16-byte aligned");
    }
  }
  PPLX_CUDA_CHECK(cudaSetDevice(device_));
  // send: one item per token; recv: one item per (source group, token) slot
  const int64_t vectors = cfg_.d_payload_bytes / 16;
  const int send_team = do_send ? pick(last_tokens_, vectors) : 0;
  const int recv_team = do_recv ? pick(last_tokens_ * cfg_.num_groups, vectors) : 0;
  PPLX_CUDA_CHECK(a2a_launch_dispatch(cfg_, states_, n, s, r, send_team, recv_team, stream));
  commit_phase(do_recv ? kPhaseDispatchRecv : kPhaseDispatchSend);
}

void A2AContext::combine(const CombineSendArgs* send, const CombineRecvArgs* recv, bool do_send,
                         bool do_recv, int y_dtype, int out_dtype, cudaStream_t stream) {
  PPLX_REQUIRE(do_send || do_recv, "combine: nothing to do");
  require_phase(do_send ? kPhaseCombineSend : kPhaseCombineRecv);
  NvtxRange range(do_send && do_recv ? "a2a_combine" : do_send ? "a2a_combine_send" : "a2a_combine_recv");
  PerRank<CombineSendArgs> s{};
  PerRank<CombineRecvArgs> r{};
  const int n = num_local_ranks();
  int64_t tokens = last_tokens_;
  for (int i = 0; i < n; ++i) {
    if (do_send) {
      s.r[i] = send[i];
      PPLX_REQUIRE(reinterpret_cast<uintptr_t>(send[i].expert_y) % 16 == 0 &&
                       send[i].expert_y_stride % 16 == 0,
                   "combine: expert_y rows must be 16-byte aligned");
    }
    if (do_recv) {
      r.r[i] = recv[i];
      r.r[i].external = (!do_send && external_send_) ? 1 : 0;
      PPLX_REQUIRE(recv[i].num_tokens >= 0 && recv[i].num_tokens <= cfg_.max_num_tokens,
                   "combine: num_tokens exceeds max_num_tokens");
      tokens = std::max<int64_t>(recv[i].num_tokens, 1);
    }
  }
  const int y_size = y_dtype == kDtypeF32 ? 4 : 2;
  PPLX_REQUIRE(y_size == cfg_.out_elemsize,
               "combine: expert_y element size differs from the context's out dtype");
  PPLX_CUDA_CHECK(cudaSetDevice(device_));
  // send: one item per expert row (per-route) or per received record (pre-reduce);
  // recv: one item per token, whose reduction reads up to eight records per output vector.
  int send_team = 0, recv_team = 0;
  if (do_send) {
    const int64_t per_token = cfg_.combine_mode == kCombinePreReduce
                                  ? std::min<int64_t>(cfg_.topk, cfg_.world)
                                  : cfg_.topk;
    send_team = pick(tokens * cfg_.num_groups * per_token / cfg_.world + 1, cfg_.c_stride / 16);
  }
  if (do_recv) recv_team = pick(tokens, static_cast<int64_t>(cfg_.hidden_dim / 8) * 8);
  PPLX_CUDA_CHECK(a2a_launch_combine(cfg_, states_, n, s, r, send_team, recv_team, y_dtype,
                                     out_dtype, stream));
  if (do_send) external_send_ = false;
  if (do_recv) external_send_ = false;
  commit_phase(do_recv ? kPhaseCombineRecv : kPhaseCombineSend);
}

void A2AContext::barrier(cudaStream_t stream) {
  NvtxRange range("a2a_barrier");
  PPLX_CUDA_CHECK(cudaSetDevice(device_));
  PPLX_CUDA_CHECK(a2a_launch_barrier(cfg_, states_, num_local_ranks(), stream));
}

std::vector<A2AScatterInfo> A2AContext::combine_send_external() {
  PPLX_REQUIRE(cfg_.combine_mode == kCombinePerRoute, "an external combine send needs the per_route mode");
  PPLX_REQUIRE(cfg_.dp_size == 1, "an external combine send does not replicate to dp peers");
  PPLX_REQUIRE(cfg_.out_elemsize == 2, "an external combine send writes 2-byte elements");
  PPLX_REQUIRE(cfg_.wire == kWirePlain, "an external combine send needs the plain wire format (wire='plain')");
  require_phase(kPhaseCombineSend);
  commit_phase(kPhaseCombineSend);
  external_send_ = true;
  std::vector<A2AScatterInfo> out(ranks_.size());
  for (size_t i = 0; i < ranks_.size(); ++i) {
    const A2ARankState& st = states_.r[i];
    A2AScatterInfo& s = out[i];
    s = A2AScatterInfo{};
    s.row_src = st.local.row_src;
    s.row_tk = st.local.row_tk;
    for (int p = 0; p < cfg_.world; ++p) {
      s.peer_recv[p] = st.recv[p] + cfg_.off_crecv;
      // one counter per sending rank: externally sent combines that have fully landed
      s.peer_flag[p] = reinterpret_cast<uint32_t*>(st.sync[p]) +
                       (kFlagExternalCombine * kMaxRanks + st.rank) * kFlagStrideWords;
    }
    s.slot_stride = cfg_.c_stride;
    s.world = cfg_.world;
    s.signal_value = 1;
    s.done_counter = scatter_done_ptrs_[i];
    s.status = st.local.status;
  }
  return out;
}

A2AStatusInfo A2AContext::status(int i) const {
  uint32_t w[4] = {0, 0, 0, 0};
  PPLX_CUDA_CHECK(cudaMemcpy(w, status_ptrs_.at(i), sizeof(w), cudaMemcpyDeviceToHost));
  A2AStatusInfo s;
  s.code = w[0];
  s.phase = w[1];
  s.who = w[2];
  s.detail = w[3];
  return s;
}

void A2AContext::check() const {
  for (size_t i = 0; i < proxies_.size(); ++i) {
    if (proxies_[i].proxy && proxies_[i].proxy->failed()) {
      // the reference's wording for a failed RDMA completion (p2p-all-to-all/src/a2a_context.rs:332-334)
      throw Error(ErrorKind::kCustom, "rank " + std::to_string(ranks_[i]) + ": fabric-lib transfer error (" +
                                          proxies_[i].proxy->error() + ")");
    }
  }
  for (int i = 0; i < num_local_ranks(); ++i) {
    const A2AStatusInfo s = status(i);
    if (s.code != kStatusOk) {
      throw Error(s.code == kStatusWaitTimeout ? ErrorKind::kTimeout : ErrorKind::kCustom,
                  "rank " + std::to_string(ranks_[i]) + ": " + s.message());
    }
  }
}

std::array<uint64_t, 8> A2AContext::stats(int i) const {
  std::array<uint64_t, 8> out{};
  PPLX_CUDA_CHECK(cudaMemcpy(out.data(), stats_ptrs_.at(i), sizeof(uint64_t) * 8, cudaMemcpyDeviceToHost));
  return out;
}

std::array<uint32_t, 2> A2AContext::iterations(int i) const {
  std::array<uint32_t, 2> out{};
  PPLX_CUDA_CHECK(cudaMemcpy(out.data(), iters_ptrs_.at(i), sizeof(uint32_t) * 2, cudaMemcpyDeviceToHost));
  return out;
}

std::array<uint64_t, kTraceSlots> A2AContext::trace(int i) const {
  std::array<uint64_t, kTraceSlots> out{};
  PPLX_CUDA_CHECK(cudaMemcpy(out.data(), trace_ptrs_.at(i), sizeof(uint64_t) * kTraceSlots, cudaMemcpyDeviceToHost));
  return out;
}

}  // namespace pplx
