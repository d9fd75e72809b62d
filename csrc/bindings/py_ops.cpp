// Bindings of the expert-side compute ops (no counterpart in the reference, which ships no
// expert computation at all).
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "../core/error.h"
#include "../ops/grouped_gemm.h"
#include "../ops/multimem.h"
#include "../ops/router.h"

namespace py = pybind11;
using namespace pplx;
using namespace pplx::ops;

void bind_ops(py::module_& m) {
  m.def(
      "multimem_red_add_u32",
      [](uint64_t mc_ptr, uint32_t value, uint64_t stream) {
        multimem_red_add_u32(reinterpret_cast<uint32_t*>(mc_ptr), value, reinterpret_cast<cudaStream_t>(stream));
      },
      py::arg("mc_ptr"), py::arg("value"), py::arg("stream"),
      "Adds value to the 32-bit word at a multicast-mapped address on every bound GPU (one multimem.red).");
  m.def(
      "topk_route",
      [](uint64_t logits, int64_t logits_stride, bool logits_bf16, uint64_t bias, uint64_t indices,
         int64_t indices_stride, uint64_t weights, int64_t weights_stride, int tokens, int num_experts, int k,
         uint64_t stream) {
        TopkRouteParams p;
        p.logits = reinterpret_cast<const void*>(logits);
        p.logits_stride = logits_stride;
        p.logits_bf16 = logits_bf16;
        p.bias = reinterpret_cast<const float*>(bias);
        p.indices = reinterpret_cast<uint32_t*>(indices);
        p.indices_stride = indices_stride;
        p.weights = reinterpret_cast<float*>(weights);
        p.weights_stride = weights_stride;
        p.tokens = tokens;
        p.num_experts = num_experts;
        p.k = k;
        topk_route(p, reinterpret_cast<cudaStream_t>(stream));
      },
      py::arg("logits"), py::arg("logits_stride"), py::arg("logits_bf16"), py::arg("bias"), py::arg("indices"),
      py::arg("indices_stride"), py::arg("weights"), py::arg("weights_stride"), py::arg("tokens"),
      py::arg("num_experts"), py::arg("k"), py::arg("stream"));
  m.def(
      "grouped_fp8_gemm",
      [](uint64_t a, int64_t a_stride, uint64_t a_scale, int64_t a_scale_stride_row, int64_t a_scale_stride_k,
         uint64_t b, uint64_t b_scale, uint64_t expert_num_tokens, uint64_t out, int64_t out_stride,
         uint64_t out_scale, int64_t out_scale_stride_row, uint64_t error_flag, int num_experts, int N, int K,
         int expert_padding, int max_rows, int mode, int num_ctas, uint64_t stream, uint64_t wait_cycles,
         int debug_skip, uint64_t trace, const py::object& scatter, int tile_rows, int scale_format) {
        GroupedGemmParams p;
        p.a = reinterpret_cast<const void*>(a);
        p.a_stride = a_stride;
        p.a_scale = reinterpret_cast<const float*>(a_scale);
        p.a_scale_stride_row = a_scale_stride_row;
        p.a_scale_stride_k = a_scale_stride_k;
        p.b = reinterpret_cast<const void*>(b);
        p.b_scale = reinterpret_cast<const float*>(b_scale);
        p.expert_num_tokens = reinterpret_cast<const int32_t*>(expert_num_tokens);
        p.out = reinterpret_cast<void*>(out);
        p.out_stride = out_stride;
        p.out_scale = reinterpret_cast<float*>(out_scale);
        p.out_scale_stride_row = out_scale_stride_row;
        p.error_flag = reinterpret_cast<uint32_t*>(error_flag);
        p.num_experts = num_experts;
        p.N = N;
        p.K = K;
        p.expert_padding = expert_padding;
        p.max_rows = max_rows;
        p.mode = mode;
        p.num_ctas = num_ctas;
        p.wait_cycles = reinterpret_cast<unsigned long long*>(wait_cycles);
        p.debug_skip = debug_skip;
        p.tile_rows = tile_rows;
        p.scale_format = scale_format;
        p.trace = reinterpret_cast<long long*>(trace);
        if (!scatter.is_none()) {
          // the tuple AllToAllContext.combine_send_external() returns for this rank
          const py::tuple t = scatter.cast<py::tuple>();
          PPLX_REQUIRE(t.size() == 9 || t.size() == 10, "scatter descriptor needs 9 entries (+ optional bulk flag)");
          if (t.size() == 10) p.scatter.bulk = t[9].cast<int>();
          CombineScatter& sc = p.scatter;
          sc.row_src = reinterpret_cast<const uint32_t*>(t[0].cast<uint64_t>());
          sc.row_tk = reinterpret_cast<const uint32_t*>(t[1].cast<uint64_t>());
          const py::list recv = t[2].cast<py::list>();
          const py::list flags = t[4].cast<py::list>();
          sc.world = t[5].cast<int>();
          PPLX_REQUIRE(sc.world >= 1 && sc.world <= CombineScatter::kMaxPeers &&
                           static_cast<int>(recv.size()) == sc.world && static_cast<int>(flags.size()) == sc.world,
                       "scatter descriptor: peer lists do not match the world size");
          for (int i = 0; i < sc.world; ++i) {
            sc.peer_recv[i] = reinterpret_cast<uint8_t*>(recv[i].cast<uint64_t>());
            sc.peer_flag[i] = reinterpret_cast<uint32_t*>(flags[i].cast<uint64_t>());
          }
          sc.slot_stride = t[3].cast<uint64_t>();
          sc.signal_value = t[6].cast<uint32_t>();
          sc.done_counter = reinterpret_cast<uint32_t*>(t[7].cast<uint64_t>());
          sc.status = reinterpret_cast<const uint32_t*>(t[8].cast<uint64_t>());
        }
        if (p.scale_format == kScalesFp32 && (p.wait_cycles != nullptr || p.trace != nullptr || p.debug_skip != 0)) {
          grouped_fp8_gemm_profiled(p, reinterpret_cast<cudaStream_t>(stream));
        } else {
          grouped_fp8_gemm(p, reinterpret_cast<cudaStream_t>(stream));
        }
      },
      py::arg("a"), py::arg("a_stride"), py::arg("a_scale"), py::arg("a_scale_stride_row"),
      py::arg("a_scale_stride_k"), py::arg("b"), py::arg("b_scale"), py::arg("expert_num_tokens"), py::arg("out"),
      py::arg("out_stride"), py::arg("out_scale"), py::arg("out_scale_stride_row"), py::arg("error_flag"),
      py::arg("num_experts"), py::arg("N"), py::arg("K"), py::arg("expert_padding"), py::arg("max_rows"),
      py::arg("mode"), py::arg("num_ctas"), py::arg("stream"), py::arg("wait_cycles") = 0,
      py::arg("debug_skip") = 0, py::arg("trace") = 0,
      py::arg("scatter") = py::none(), py::arg("tile_rows") = 0, py::arg("scale_format") = 0);
}
