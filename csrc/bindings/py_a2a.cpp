// Bindings of the all-to-all context. Method names and keyword arguments follow the
// reference's python-ext/src/py_p2p_all_to_all.rs:17-210 (typed in
// pplx_garden/native/p2p_all_to_all.pyi); arguments that only its RDMA proxy needs are
// accepted and ignored. Extra entry points: fused send+recv launches, a layout query,
// virtual-rank (single GPU, several ranks) launches and status/statistics readers.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "../a2a/a2a_context.h"
#include "../core/error.h"
#include "py_fabric.h"
#include "py_util.h"

namespace py = pybind11;
using namespace pplx;

namespace {

uint64_t opt_u64(const py::handle& o) { return o.is_none() ? 0ull : o.cast<uint64_t>(); }
int64_t opt_i64(const py::handle& o) { return o.is_none() ? 0ll : o.cast<int64_t>(); }

int combine_mode_from(const py::object& mode) {
  if (mode.is_none()) return kCombinePerRoute;
  if (py::isinstance<py::int_>(mode)) return mode.cast<int>();
  const std::string s = mode.cast<std::string>();
  if (s == "per_route") return kCombinePerRoute;
  if (s == "pre_reduce") return kCombinePreReduce;
  throw Error(ErrorKind::kInvalidArgument, "combine_mode must be 'per_route' or 'pre_reduce'");
}

int wire_from(const py::object& wire) {
  if (wire.is_none()) return kWireAuto;
  if (py::isinstance<py::int_>(wire)) return wire.cast<int>();
  const std::string s = wire.cast<std::string>();
  if (s == "auto") return kWireAuto;
  if (s == "plain") return kWirePlain;
  if (s == "ll") return kWireLL;
  throw Error(ErrorKind::kInvalidArgument, "wire must be 'auto', 'plain' or 'll'");
}

A2AParams make_params(int hidden_dim, const py::object& hidden_dim_scale, int in_elemsize,
                      int out_elemsize, const py::object& scale_elemsize, int max_num_tokens,
                      int num_experts, int expert_padding, int num_experts_per_token, int dp_size,
                      int world_size, const py::object& combine_mode, int num_blocks,
                      int64_t wait_limit_ms, const py::object& wire = py::none(), uint32_t node_mask = 0) {
  A2AParams p;
  p.world = world_size;
  p.dp_size = dp_size;
  p.num_experts = num_experts;
  p.topk = num_experts_per_token;
  p.max_num_tokens = max_num_tokens;
  p.hidden_dim = hidden_dim;
  p.hidden_dim_scale = hidden_dim_scale.is_none() ? 0 : hidden_dim_scale.cast<int>();
  p.in_elemsize = in_elemsize;
  p.out_elemsize = out_elemsize;
  p.scale_elemsize = scale_elemsize.is_none() ? 4 : scale_elemsize.cast<int>();
  p.expert_padding = expert_padding;
  p.combine_mode = combine_mode_from(combine_mode);
  p.num_blocks = num_blocks;
  p.wait_limit_ms = wait_limit_ms;
  p.wire = wire_from(wire);
  p.node_mask = node_mask;
  return p;
}

py::dict config_dict(const A2AConfig& c) {
  py::dict d;
  d["world"] = c.world;
  d["dp_size"] = c.dp_size;
  d["num_groups"] = c.num_groups;
  d["num_experts"] = c.num_experts;
  d["experts_per_rank"] = c.experts_per_rank;
  d["topk"] = c.topk;
  d["max_num_tokens"] = c.max_num_tokens;
  d["num_blocks"] = c.num_blocks;
  d["combine_mode"] = c.combine_mode;
  d["wire"] = c.wire == kWireLL ? "ll" : "plain";
  d["node_mask"] = c.node_mask;
  d["dispatch_header_bytes"] = c.d_header_bytes;
  d["dispatch_payload_bytes"] = c.d_payload_bytes;
  d["dispatch_scale_bytes"] = c.d_scale_bytes;
  d["dispatch_record_bytes"] = c.d_stride;
  d["combine_record_bytes"] = c.c_stride;
  d["combine_records_per_token"] = c.c_records_per_token;
  d["counts_stride"] = c.counts_stride;
  d["max_recv_rows"] = c.max_recv_rows;
  d["sync_bytes"] = c.sync_bytes;
  d["off_counts"] = c.off_counts;
  d["off_tok_arrive"] = c.off_tok_arrive;
  d["counts_bank_words"] = c.counts_bank_words;
  d["recv_bytes"] = c.recv_bytes;
  d["off_drecv"] = c.off_drecv;
  d["drecv_group_stride"] = c.drecv_group_stride;
  d["off_crecv"] = c.off_crecv;
  d["wait_limit_ns"] = c.wait_limit_ns;
  return d;
}

DispatchSendArgs send_args(int num_tokens, uint64_t x_ptr, uint64_t x_stride,
                           const py::handle& x_scale_ptr, const py::handle& sse,
                           const py::handle& sst, uint64_t indices_ptr, uint64_t indices_stride,
                           uint64_t weights_ptr, uint64_t weights_stride,
                           const py::handle& bound_m_ptr, int quantize,
                           const py::handle& logits_ptr = py::none(), int64_t logits_stride = 0,
                           bool logits_bf16 = false, const py::handle& logits_bias_ptr = py::none()) {
  DispatchSendArgs a{};
  a.num_tokens = num_tokens;
  a.x = reinterpret_cast<const uint8_t*>(x_ptr);
  a.x_stride = x_stride;
  a.x_scale = reinterpret_cast<const uint8_t*>(opt_u64(x_scale_ptr));
  a.x_scale_stride_elem = opt_i64(sse);
  a.x_scale_stride_token = opt_i64(sst);
  a.indices = reinterpret_cast<const uint32_t*>(indices_ptr);
  a.indices_stride = indices_stride;
  a.weights = reinterpret_cast<const float*>(weights_ptr);
  a.weights_stride = weights_stride;
  a.bound_m = reinterpret_cast<const int32_t*>(opt_u64(bound_m_ptr));
  PPLX_REQUIRE(quantize >= 0 && quantize <= 2, "quantize is 0 (no), 1 (fp32 scales) or 2 (power-of-two scales)");
  a.quantize = quantize;
  a.logits = reinterpret_cast<const void*>(opt_u64(logits_ptr));
  a.logits_stride = logits_stride;
  a.logits_bf16 = logits_bf16 ? 1 : 0;
  a.logits_bias = reinterpret_cast<const float*>(opt_u64(logits_bias_ptr));
  return a;
}

DispatchRecvArgs recv_args(uint64_t out_num_tokens_ptr, uint64_t out_x_ptr, uint64_t out_x_stride,
                           const py::handle& out_x_scale_ptr, const py::handle& sse,
                           const py::handle& sst, uint32_t out_rows) {
  DispatchRecvArgs a{};
  a.out_num_tokens = reinterpret_cast<int32_t*>(out_num_tokens_ptr);
  a.out_x = reinterpret_cast<uint8_t*>(out_x_ptr);
  a.out_x_stride = out_x_stride;
  a.out_x_scale = reinterpret_cast<uint8_t*>(opt_u64(out_x_scale_ptr));
  a.out_x_scale_stride_elem = opt_i64(sse);
  a.out_x_scale_stride_token = opt_i64(sst);
  a.out_rows = out_rows;
  return a;
}

CombineSendArgs csend_args(uint64_t expert_x_ptr, uint64_t expert_x_stride) {
  CombineSendArgs a{};
  a.expert_y = reinterpret_cast<const uint8_t*>(expert_x_ptr);
  a.expert_y_stride = expert_x_stride;
  return a;
}

CombineRecvArgs crecv_args(int num_tokens, uint64_t out_tokens_ptr, uint64_t out_tokens_stride,
                           uint64_t indices_ptr, uint64_t indices_stride, uint64_t weights_ptr,
                           uint64_t weights_stride, const py::handle& bound_m_ptr,
                           bool accumulate) {
  CombineRecvArgs a{};
  a.num_tokens = num_tokens;
  a.out_tokens = reinterpret_cast<uint8_t*>(out_tokens_ptr);
  a.out_tokens_stride = out_tokens_stride;
  a.indices = reinterpret_cast<const uint32_t*>(indices_ptr);
  a.indices_stride = indices_stride;
  a.weights = reinterpret_cast<const float*>(weights_ptr);
  a.weights_stride = weights_stride;
  a.bound_m = reinterpret_cast<const int32_t*>(opt_u64(bound_m_ptr));
  a.accumulate = accumulate ? 1 : 0;
  return a;
}

int dtype_code(const py::object& dtype) {
  if (py::isinstance<py::int_>(dtype)) return dtype.cast<int>();
  const pplx_py::DtypeInfo info = pplx_py::dtype_info(dtype);
  PPLX_REQUIRE(info.code == kDtypeF16 || info.code == kDtypeBF16 || info.code == kDtypeF32,
               "combine supports float16, bfloat16 and float32");
  return info.code;
}

cudaStream_t as_stream(uint64_t s) { return reinterpret_cast<cudaStream_t>(s); }

struct PyA2A {
  std::unique_ptr<A2AContext> ctx;
  int out_dtype = kDtypeBF16;

  void after_launch() const {
    if (ctx->failed()) ctx->check();
  }
};

std::vector<std::vector<uint64_t>> ptr_tables(const py::object& ptrs, size_t nlocal) {
  std::vector<std::vector<uint64_t>> out;
  py::list l = ptrs.cast<py::list>();
  if (l.size() > 0 && py::isinstance<py::int_>(l[0])) {
    PPLX_REQUIRE(nlocal == 1, "a flat pointer list describes exactly one local rank");
    out.push_back(l.cast<std::vector<uint64_t>>());
  } else {
    for (const auto& row : l) out.push_back(row.cast<std::vector<uint64_t>>());
  }
  return out;
}

}  // namespace

// The host proxy on its own, over buffers the caller owns and has registered with the engine
// (host memory in CPU tests, where Python plays the kernels' part).
struct PyProxyProbe {
  std::unique_ptr<A2AProxy> proxy;
};

void bind_a2a(py::module_& m) {
  py::class_<PyProxyProbe>(m, "_A2AProxyProbe")
      .def(py::init([](const py::dict& layout_args, int rank, PyEngine& engine, const py::list& peers,
                       const py::dict& shadow_sync, const py::dict& shadow_recv, uint64_t stage,
                       uint64_t flag_source, uint64_t proxy_words, uint64_t stage_slot) {
             auto get = [&](const char* key, py::object fallback) -> py::object {
               return layout_args.contains(key) ? py::reinterpret_borrow<py::object>(layout_args[key]) : fallback;
             };
             const A2AParams p = make_params(
                 get("hidden_dim", py::int_(0)).cast<int>(), get("hidden_dim_scale", py::none()),
                 get("in_elemsize", py::int_(2)).cast<int>(), get("out_elemsize", py::int_(2)).cast<int>(),
                 get("scale_elemsize", py::none()), get("max_num_tokens", py::int_(0)).cast<int>(),
                 get("num_experts", py::int_(0)).cast<int>(), get("expert_padding", py::int_(1)).cast<int>(),
                 get("num_experts_per_token", py::int_(0)).cast<int>(), get("dp_size", py::int_(1)).cast<int>(),
                 get("world_size", py::int_(1)).cast<int>(), get("combine_mode", py::none()), 0,
                 get("wait_limit_ms", py::int_(0)).cast<int64_t>(), py::str("plain"),
                 get("node_mask", py::int_(0)).cast<uint32_t>());
             const A2AConfig cfg = a2a_make_config(p, 148, 1);
             std::vector<A2AProxyPeer> list;
             for (const auto& item : peers) {
               const py::tuple t = item.cast<py::tuple>();
               A2AProxyPeer peer;
               peer.rank = t[0].cast<int>();
               peer.sync_desc = t[1].cast<fabric::MemoryRegionDescriptor>();
               peer.recv_desc = t[2].cast<fabric::MemoryRegionDescriptor>();
               list.push_back(std::move(peer));
             }
             A2AProxyBuffers buf;
             for (const auto& kv : shadow_sync) buf.shadow_sync[kv.first.cast<int>()] = kv.second.cast<uint64_t>();
             for (const auto& kv : shadow_recv) buf.shadow_recv[kv.first.cast<int>()] = kv.second.cast<uint64_t>();
             buf.stage = stage;
             buf.flag_source = flag_source;
             buf.flag_source_host = reinterpret_cast<volatile uint32_t*>(flag_source);
             buf.proxy_words = reinterpret_cast<volatile uint32_t*>(proxy_words);
             buf.stage_slot = reinterpret_cast<const volatile uint32_t*>(stage_slot);
             auto self = std::make_unique<PyProxyProbe>();
             fabric::TransferEngine* eng = &engine.get();
             py::gil_scoped_release release;
             self->proxy = std::make_unique<A2AProxy>(cfg, rank, eng, std::move(list), buf, -1);
             return self;
           }),
           py::arg("layout_args"), py::arg("rank"), py::arg("transfer_engine"), py::arg("peers"),
           py::arg("shadow_sync"), py::arg("shadow_recv"), py::arg("stage"), py::arg("flag_source"),
           py::arg("proxy_words"), py::arg("stage_slot"))
      .def("failed", [](const PyProxyProbe& s) { return s.proxy && s.proxy->failed(); })
      .def("error", [](const PyProxyProbe& s) { return s.proxy ? s.proxy->error() : std::string(); })
      .def("counters",
           [](const PyProxyProbe& s) { return py::make_tuple(s.proxy->dispatches(), s.proxy->combines()); })
      .def("close", [](PyProxyProbe& s) {
        py::gil_scoped_release release;
        s.proxy.reset();
      });

  py::class_<PyA2A>(m, "AllToAllContext")
      .def_static(
          "layout",
          [](int hidden_dim, const py::object& hidden_dim_scale, int in_elemsize, int out_elemsize,
             const py::object& scale_elemsize, int max_num_tokens, int num_experts,
             int expert_padding, int num_experts_per_token, int dp_size, int world_size,
             const py::object& combine_mode, int num_blocks, int num_sms, int virtual_ranks,
             const py::object& wire, uint32_t node_mask) {
            const A2AParams p = make_params(hidden_dim, hidden_dim_scale, in_elemsize, out_elemsize,
                                            scale_elemsize, max_num_tokens, num_experts,
                                            expert_padding, num_experts_per_token, dp_size,
                                            world_size, combine_mode, num_blocks, 0, wire, node_mask);
            return config_dict(a2a_make_config(p, num_sms, virtual_ranks));
          },
          py::kw_only(), py::arg("hidden_dim"), py::arg("hidden_dim_scale") = py::none(),
          py::arg("in_elemsize"), py::arg("out_elemsize"), py::arg("scale_elemsize") = py::none(),
          py::arg("max_num_tokens"), py::arg("num_experts"), py::arg("expert_padding") = 1,
          py::arg("num_experts_per_token"), py::arg("dp_size") = 1, py::arg("world_size"),
          py::arg("combine_mode") = py::none(), py::arg("num_blocks") = 0,
          py::arg("num_sms") = 148, py::arg("virtual_ranks") = 1, py::arg("wire") = py::none(), py::arg("node_mask") = 0,
          "Wire format and symmetric-buffer layout for a configuration (no GPU needed).")
      .def_static(
          "create",
          [](int hidden_dim, const py::object& hidden_dim_scale, int in_elemsize, int out_elemsize,
             const py::object& out_dtype, const py::object& scale_elemsize, int max_num_tokens,
             const py::object& /*max_recv_tokens*/, const py::object& /*max_private_tokens*/,
             int num_experts, int expert_padding, int num_experts_per_token, const py::object& rank,
             int dp_size, const py::object& /*node_size*/, int world_size,
             const py::object& /*num_routed_ptr*/, const py::object& /*num_routed_mr*/,
             const py::object& /*send_buffer_ptr*/, const py::object& /*send_buffer_mr*/,
             const py::object& /*recv_buffer_ptr*/, const py::object& /*recv_buffer_mr*/,
             const py::object& sync_ptrs, const py::object& /*send_ptrs*/,
             const py::object& recv_ptrs, int device, const py::object& /*imm_base*/,
             const py::object& /*ranks*/, const py::object& /*transfer_engine*/,
             const py::object& /*worker_cpu*/, const py::object& combine_mode, int num_blocks,
             int64_t wait_limit_ms, const py::object& wire, uint32_t node_mask) {
            std::vector<int> local_ranks;
            if (py::isinstance<py::int_>(rank)) {
              local_ranks.push_back(rank.cast<int>());
            } else {
              local_ranks = rank.cast<std::vector<int>>();
            }
            const A2AParams p = make_params(hidden_dim, hidden_dim_scale, in_elemsize, out_elemsize,
                                            scale_elemsize, max_num_tokens, num_experts,
                                            expert_padding, num_experts_per_token, dp_size,
                                            world_size, combine_mode, num_blocks, wait_limit_ms, wire, node_mask);
            auto self = std::make_unique<PyA2A>();
            self->out_dtype = dtype_code(out_dtype);
            self->ctx = std::make_unique<A2AContext>(p, device, local_ranks,
                                                     ptr_tables(sync_ptrs, local_ranks.size()),
                                                     ptr_tables(recv_ptrs, local_ranks.size()));
            return self;
          },
          py::kw_only(), py::arg("hidden_dim"), py::arg("hidden_dim_scale") = py::none(),
          py::arg("in_elemsize"), py::arg("out_elemsize"), py::arg("out_dtype"),
          py::arg("scale_elemsize") = py::none(), py::arg("max_num_tokens"),
          py::arg("max_recv_tokens") = py::none(), py::arg("max_private_tokens") = py::none(),
          py::arg("num_experts"), py::arg("expert_padding") = 1, py::arg("num_experts_per_token"),
          py::arg("rank"), py::arg("dp_size") = 1, py::arg("node_size") = py::none(),
          py::arg("world_size"), py::arg("num_routed_ptr") = py::none(),
          py::arg("num_routed_mr") = py::none(), py::arg("send_buffer_ptr") = py::none(),
          py::arg("send_buffer_mr") = py::none(), py::arg("recv_buffer_ptr") = py::none(),
          py::arg("recv_buffer_mr") = py::none(), py::arg("sync_ptrs"),
          py::arg("send_ptrs") = py::none(), py::arg("recv_ptrs"), py::arg("device"),
          py::arg("imm_base") = py::none(), py::arg("ranks") = py::none(),
          py::arg("transfer_engine") = py::none(), py::arg("worker_cpu") = py::none(),
          py::arg("combine_mode") = py::none(), py::arg("num_blocks") = 0,
          py::arg("wait_limit_ms") = 0, py::arg("wire") = py::none(), py::arg("node_mask") = 0,
          "Create a context. `rank` may be a list: the context then plays several ranks on one "
          "GPU and sync_ptrs / recv_ptrs hold one pointer table per local rank.")
      .def("config", [](const PyA2A& s) { return config_dict(s.ctx->config()); })
      .def("dispatch_send",
           [](PyA2A& s, int num_tokens, uint64_t x_ptr, uint64_t x_stride,
              const py::object& x_scale_ptr, const py::object& sse, const py::object& sst,
              uint64_t indices_ptr, uint64_t indices_stride, uint64_t weights_ptr,
              uint64_t weights_stride, const py::object& bound_m_ptr, uint64_t stream,
              int quantize, const py::object& logits_ptr, int64_t logits_stride, bool logits_bf16,
              const py::object& logits_bias_ptr) {
             pplx_py::TorchProfilerGuard profiler_range("a2a_dispatch_send");
             const DispatchSendArgs a =
                 send_args(num_tokens, x_ptr, x_stride, x_scale_ptr, sse, sst, indices_ptr,
                           indices_stride, weights_ptr, weights_stride, bound_m_ptr, quantize, logits_ptr,
                           logits_stride, logits_bf16, logits_bias_ptr);
             s.ctx->dispatch(&a, nullptr, true, false, as_stream(stream));
             s.after_launch();
           },
           py::arg("num_tokens"), py::arg("x_ptr"), py::arg("x_stride"), py::arg("x_scale_ptr"),
           py::arg("x_scale_stride_elem"), py::arg("x_scale_stride_token"), py::arg("indices_ptr"),
           py::arg("indices_stride"), py::arg("weights_ptr"), py::arg("weights_stride"),
           py::arg("bound_m_ptr"), py::arg("stream"), py::arg("quantize") = 0,
           py::arg("logits_ptr") = py::none(), py::arg("logits_stride") = 0, py::arg("logits_bf16") = false,
           py::arg("logits_bias_ptr") = py::none())
      .def("dispatch_recv",
           [](PyA2A& s, uint64_t out_num_tokens_ptr, uint64_t out_x_ptr, uint64_t out_x_stride,
              const py::object& out_x_scale_ptr, const py::object& sse, const py::object& sst,
              uint64_t stream, uint32_t out_rows) {
             pplx_py::TorchProfilerGuard profiler_range("a2a_dispatch_recv");
             const DispatchRecvArgs a = recv_args(out_num_tokens_ptr, out_x_ptr, out_x_stride,
                                                  out_x_scale_ptr, sse, sst, out_rows);
             s.ctx->dispatch(nullptr, &a, false, true, as_stream(stream));
             s.after_launch();
           },
           py::arg("out_num_tokens_ptr"), py::arg("out_x_ptr"), py::arg("out_x_stride"),
           py::arg("out_x_scale_ptr"), py::arg("out_x_scale_stride_elem"),
           py::arg("out_x_scale_stride_token"), py::arg("stream"), py::arg("out_rows") = 0)
      .def("dispatch",
           [](PyA2A& s, int num_tokens, uint64_t x_ptr, uint64_t x_stride,
              const py::object& x_scale_ptr, const py::object& sse, const py::object& sst,
              uint64_t indices_ptr, uint64_t indices_stride, uint64_t weights_ptr,
              uint64_t weights_stride, const py::object& bound_m_ptr, uint64_t out_num_tokens_ptr,
              uint64_t out_x_ptr, uint64_t out_x_stride, const py::object& out_x_scale_ptr,
              const py::object& osse, const py::object& osst, uint64_t stream, uint32_t out_rows,
              int quantize, const py::object& logits_ptr, int64_t logits_stride, bool logits_bf16,
              const py::object& logits_bias_ptr) {
             pplx_py::TorchProfilerGuard profiler_range("a2a_dispatch");
             const DispatchSendArgs a =
                 send_args(num_tokens, x_ptr, x_stride, x_scale_ptr, sse, sst, indices_ptr,
                           indices_stride, weights_ptr, weights_stride, bound_m_ptr, quantize, logits_ptr,
                           logits_stride, logits_bf16, logits_bias_ptr);
             const DispatchRecvArgs r = recv_args(out_num_tokens_ptr, out_x_ptr, out_x_stride,
                                                  out_x_scale_ptr, osse, osst, out_rows);
             s.ctx->dispatch(&a, &r, true, true, as_stream(stream));
             s.after_launch();
           },
           py::arg("num_tokens"), py::arg("x_ptr"), py::arg("x_stride"), py::arg("x_scale_ptr"),
           py::arg("x_scale_stride_elem"), py::arg("x_scale_stride_token"), py::arg("indices_ptr"),
           py::arg("indices_stride"), py::arg("weights_ptr"), py::arg("weights_stride"),
           py::arg("bound_m_ptr"), py::arg("out_num_tokens_ptr"), py::arg("out_x_ptr"),
           py::arg("out_x_stride"), py::arg("out_x_scale_ptr"), py::arg("out_x_scale_stride_elem"),
           py::arg("out_x_scale_stride_token"), py::arg("stream"), py::arg("out_rows") = 0,
           py::arg("quantize") = 0, py::arg("logits_ptr") = py::none(), py::arg("logits_stride") = 0,
           py::arg("logits_bf16") = false, py::arg("logits_bias_ptr") = py::none(),
           "dispatch_send and dispatch_recv fused into one launch.")
      .def("combine_send",
           [](PyA2A& s, uint64_t expert_x_ptr, uint64_t expert_x_stride, uint64_t stream,
              const py::object& expert_y_dtype) {
             pplx_py::TorchProfilerGuard profiler_range("a2a_combine_send");
             const CombineSendArgs a = csend_args(expert_x_ptr, expert_x_stride);
             const int y = expert_y_dtype.is_none() ? s.out_dtype : dtype_code(expert_y_dtype);
             s.ctx->combine(&a, nullptr, true, false, y, s.out_dtype, as_stream(stream));
             s.after_launch();
           },
           py::arg("expert_x_ptr"), py::arg("expert_x_stride"), py::arg("stream"),
           py::arg("expert_y_dtype") = py::none())
      .def("combine_send_external",
           [](PyA2A& s) {
             py::list out;
             for (const A2AScatterInfo& i : s.ctx->combine_send_external()) {
               py::list recv, flags;
               for (int p = 0; p < i.world; ++p) {
                 recv.append(reinterpret_cast<uint64_t>(i.peer_recv[p]));
                 flags.append(reinterpret_cast<uint64_t>(i.peer_flag[p]));
               }
               out.append(py::make_tuple(reinterpret_cast<uint64_t>(i.row_src), reinterpret_cast<uint64_t>(i.row_tk),
                                         recv, i.slot_stride, flags, i.world, i.signal_value,
                                         reinterpret_cast<uint64_t>(i.done_counter),
                                         reinterpret_cast<uint64_t>(i.status)));
             }
             return out;
           },
           "The combine's send phase is done by another kernel (grouped_fp8_gemm in its scatter mode): "
           "counts as combine_send in the phase order and returns one descriptor per local rank.")
      .def("combine_recv",
           [](PyA2A& s, int num_tokens, const py::object& /*num_recv_tokens*/,
              const py::object& expert_y_dtype, uint64_t out_tokens_ptr,
              uint64_t out_tokens_stride, uint64_t indices_ptr, uint64_t indices_stride,
              uint64_t weights_ptr, uint64_t weights_stride, const py::object& bound_m_ptr,
              bool accumulate, uint64_t stream) {
             pplx_py::TorchProfilerGuard profiler_range("a2a_combine_recv");
             const CombineRecvArgs a =
                 crecv_args(num_tokens, out_tokens_ptr, out_tokens_stride, indices_ptr,
                            indices_stride, weights_ptr, weights_stride, bound_m_ptr, accumulate);
             s.ctx->combine(nullptr, &a, false, true, dtype_code(expert_y_dtype), s.out_dtype,
                            as_stream(stream));
             s.after_launch();
           },
           py::arg("num_tokens"), py::arg("num_recv_tokens"), py::arg("expert_y_dtype"),
           py::arg("out_tokens_ptr"), py::arg("out_tokens_stride"), py::arg("indices_ptr"),
           py::arg("indices_stride"), py::arg("weights_ptr"), py::arg("weights_stride"),
           py::arg("bound_m_ptr"), py::arg("accumulate"), py::arg("stream"))
      .def("combine",
           [](PyA2A& s, uint64_t expert_x_ptr, uint64_t expert_x_stride, int num_tokens,
              const py::object& expert_y_dtype, uint64_t out_tokens_ptr,
              uint64_t out_tokens_stride, uint64_t indices_ptr, uint64_t indices_stride,
              uint64_t weights_ptr, uint64_t weights_stride, const py::object& bound_m_ptr,
              bool accumulate, uint64_t stream) {
             pplx_py::TorchProfilerGuard profiler_range("a2a_combine");
             const CombineSendArgs a = csend_args(expert_x_ptr, expert_x_stride);
             const CombineRecvArgs r =
                 crecv_args(num_tokens, out_tokens_ptr, out_tokens_stride, indices_ptr,
                            indices_stride, weights_ptr, weights_stride, bound_m_ptr, accumulate);
             s.ctx->combine(&a, &r, true, true, dtype_code(expert_y_dtype), s.out_dtype,
                            as_stream(stream));
             s.after_launch();
           },
           py::arg("expert_x_ptr"), py::arg("expert_x_stride"), py::arg("num_tokens"),
           py::arg("expert_y_dtype"), py::arg("out_tokens_ptr"), py::arg("out_tokens_stride"),
           py::arg("indices_ptr"), py::arg("indices_stride"), py::arg("weights_ptr"),
           py::arg("weights_stride"), py::arg("bound_m_ptr"), py::arg("accumulate"),
           py::arg("stream"), "combine_send and combine_recv fused into one launch.")
      // ---- several ranks in one launch (one tuple per local rank, same order as above) ----
      .def("dispatch_multi",
           [](PyA2A& s, const py::object& send, const py::object& recv, uint64_t stream) {
             pplx_py::TorchProfilerGuard profiler_range("a2a_dispatch");
             std::vector<DispatchSendArgs> sa;
             std::vector<DispatchRecvArgs> ra;
             if (!send.is_none()) {
               for (const auto& item : send.cast<py::list>()) {
                 const py::tuple t = item.cast<py::tuple>();
                 PPLX_REQUIRE(t.size() == 12 || t.size() == 16,
                              "send tuple needs 12 entries (16 with logits, their stride, bf16 flag and bias)");
                 if (t.size() == 16) {
                   sa.push_back(send_args(t[0].cast<int>(), t[1].cast<uint64_t>(), t[2].cast<uint64_t>(), t[3],
                                          t[4], t[5], t[6].cast<uint64_t>(), t[7].cast<uint64_t>(),
                                          t[8].cast<uint64_t>(), t[9].cast<uint64_t>(), t[10],
                                          t[11].cast<int>(), t[12], t[13].cast<int64_t>(), t[14].cast<bool>(),
                                          t[15]));
                   continue;
                 }
                 sa.push_back(send_args(t[0].cast<int>(), t[1].cast<uint64_t>(),
                                        t[2].cast<uint64_t>(), t[3], t[4], t[5],
                                        t[6].cast<uint64_t>(), t[7].cast<uint64_t>(),
                                        t[8].cast<uint64_t>(), t[9].cast<uint64_t>(), t[10],
                                        t[11].cast<int>()));
               }
               PPLX_REQUIRE(static_cast<int>(sa.size()) == s.ctx->num_local_ranks(),
                            "one send tuple per local rank is required");
             }
             if (!recv.is_none()) {
               for (const auto& item : recv.cast<py::list>()) {
                 const py::tuple t = item.cast<py::tuple>();
                 PPLX_REQUIRE(t.size() == 7, "recv tuple needs 7 entries");
                 ra.push_back(recv_args(t[0].cast<uint64_t>(), t[1].cast<uint64_t>(),
                                        t[2].cast<uint64_t>(), t[3], t[4], t[5],
                                        t[6].cast<uint32_t>()));
               }
               PPLX_REQUIRE(static_cast<int>(ra.size()) == s.ctx->num_local_ranks(),
                            "one recv tuple per local rank is required");
             }
             s.ctx->dispatch(sa.empty() ? nullptr : sa.data(), ra.empty() ? nullptr : ra.data(),
                             !sa.empty(), !ra.empty(), as_stream(stream));
             s.after_launch();
           },
           py::arg("send"), py::arg("recv"), py::arg("stream"))
      .def("combine_multi",
           [](PyA2A& s, const py::object& send, const py::object& recv,
              const py::object& expert_y_dtype, uint64_t stream) {
             pplx_py::TorchProfilerGuard profiler_range("a2a_combine");
             std::vector<CombineSendArgs> sa;
             std::vector<CombineRecvArgs> ra;
             if (!send.is_none()) {
               for (const auto& item : send.cast<py::list>()) {
                 const py::tuple t = item.cast<py::tuple>();
                 PPLX_REQUIRE(t.size() == 2, "combine send tuple needs 2 entries");
                 sa.push_back(csend_args(t[0].cast<uint64_t>(), t[1].cast<uint64_t>()));
               }
               PPLX_REQUIRE(static_cast<int>(sa.size()) == s.ctx->num_local_ranks(),
                            "one send tuple per local rank is required");
             }
             if (!recv.is_none()) {
               for (const auto& item : recv.cast<py::list>()) {
                 const py::tuple t = item.cast<py::tuple>();
                 PPLX_REQUIRE(t.size() == 9, "combine recv tuple needs 9 entries");
                 ra.push_back(crecv_args(t[0].cast<int>(), t[1].cast<uint64_t>(),
                                         t[2].cast<uint64_t>(), t[3].cast<uint64_t>(),
                                         t[4].cast<uint64_t>(), t[5].cast<uint64_t>(),
                                         t[6].cast<uint64_t>(), t[7], t[8].cast<bool>()));
               }
               PPLX_REQUIRE(static_cast<int>(ra.size()) == s.ctx->num_local_ranks(),
                            "one recv tuple per local rank is required");
             }
             s.ctx->combine(sa.empty() ? nullptr : sa.data(), ra.empty() ? nullptr : ra.data(),
                            !sa.empty(), !ra.empty(), dtype_code(expert_y_dtype), s.out_dtype,
                            as_stream(stream));
             s.after_launch();
           },
           py::arg("send"), py::arg("recv"), py::arg("expert_y_dtype"), py::arg("stream"))
      .def("enable_proxy",
           [](PyA2A& s, PyEngine& engine, const py::list& peers, int local_rank, int worker_cpu) {
             std::vector<A2AProxyPeer> list;
             for (const auto& item : peers) {
               const py::tuple t = item.cast<py::tuple>();
               PPLX_REQUIRE(t.size() == 3, "a proxy peer is (rank, sync descriptor, receive descriptor)");
               A2AProxyPeer p;
               p.rank = t[0].cast<int>();
               p.sync_desc = t[1].cast<fabric::MemoryRegionDescriptor>();
               p.recv_desc = t[2].cast<fabric::MemoryRegionDescriptor>();
               list.push_back(std::move(p));
             }
             fabric::TransferEngine* eng = &engine.get();
             py::gil_scoped_release release;
             s.ctx->enable_proxy(local_rank, eng, std::move(list), worker_cpu);
           },
           py::arg("transfer_engine"), py::arg("peers"), py::arg("local_rank") = 0, py::arg("worker_cpu") = -1,
           "Serve the ranks outside this rank's NVLink domain through a transfer engine: peers is a list of "
           "(rank, MemoryRegionDescriptor of its sync region, MemoryRegionDescriptor of its receive region).")
      .def("proxy_counters",
           [](const PyA2A& s, int local_rank) { return s.ctx->proxy_counters(local_rank); },
           py::arg("local_rank") = 0, "(dispatches, combines) the host proxy has served.")
      .def("barrier",
           [](PyA2A& s, uint64_t stream) {
             s.ctx->barrier(as_stream(stream));
             s.after_launch();
           },
           py::arg("stream"),
           "Device-side barrier over all ranks of the context (collective, stream ordered).")
      .def("failed", [](const PyA2A& s) { return s.ctx->failed(); })
      .def("check", [](const PyA2A& s) { s.ctx->check(); })
      .def("status",
           [](const PyA2A& s, int i) {
             const A2AStatusInfo st = s.ctx->status(i);
             return py::make_tuple(st.code, st.phase, st.who, st.detail, st.message());
           },
           py::arg("local_rank") = 0)
      .def("stats", [](const PyA2A& s, int i) { return s.ctx->stats(i); }, py::arg("local_rank") = 0)
      .def("iterations", [](const PyA2A& s, int i) { return s.ctx->iterations(i); },
           py::arg("local_rank") = 0)
      .def("trace", [](const PyA2A& s, int i) { return s.ctx->trace(i); }, py::arg("local_rank") = 0)
      .def("_set_next_phase", [](PyA2A& s, int phase) { s.ctx->debug_set_next_phase(phase); })
      .def("set_team", [](PyA2A& s, int team) { s.ctx->set_team_override(team); })
      .def("destroy", [](PyA2A& s) { s.ctx.reset(); });
}
