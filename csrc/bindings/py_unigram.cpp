// Python bindings of the Unigram encoder. The reference ships pplx-unigram as a Rust
// crate without a Python binding (python-ext/Cargo.toml:9-15); exposing it here lets the
// differential tests against HuggingFace `tokenizers` run from pytest.
#include <pybind11/pybind11.h>
#include <pybind11/numpy.h>
#include <pybind11/stl.h>

#include "../unigram/engine.h"
#include "../unigram/json.h"
#include "../unigram/unicode.h"

namespace py = pybind11;
using namespace pplx::unigram;

namespace {

struct PyEngine {
  std::shared_ptr<Engine> engine;
  EncodeState state;  // for single-text calls made under the GIL
};

[[noreturn]] void rethrow(const UnigramError& e) {
  switch (e.kind()) {
    case ErrorKind::kIo: throw py::value_error(std::string("io: ") + e.what());
    case ErrorKind::kInvalidConfig: throw py::value_error(std::string("invalid config: ") + e.what());
    case ErrorKind::kUnsupportedConfig:
      throw py::value_error(std::string("unsupported config: ") + e.what());
    default: throw std::runtime_error(std::string("encode failed: ") + e.what());
  }
}

}  // namespace

void bind_unigram(py::module_& m) {
  py::class_<PyEngine>(m, "UnigramEngine")
      .def_static("from_hf_json_path",
                  [](const std::string& path) {
                    try {
                      return PyEngine{Engine::from_hf_json_path(path), {}};
                    } catch (const UnigramError& e) {
                      rethrow(e);
                    }
                  })
      .def_static("from_hf_json_bytes",
                  [](const py::bytes& data) {
                    try {
                      return PyEngine{Engine::from_hf_json_bytes(std::string(data)), {}};
                    } catch (const UnigramError& e) {
                      rethrow(e);
                    }
                  })
      .def_property_readonly("vocab_size", [](const PyEngine& s) { return s.engine->vocab_size(); })
      .def_property_readonly("unk_id", [](const PyEngine& s) { return s.engine->unk_id(); })
      .def_property_readonly("trie_nodes", [](const PyEngine& s) { return s.engine->trie_nodes(); })
      .def_property_readonly("trie_on_huge_pages",
                             [](const PyEngine& s) { return s.engine->trie_on_huge_pages(); })
      .def("encode",
           [](PyEngine& s, const std::string& text) {
             if (!pplx::unicode::is_valid_utf8(text)) throw py::value_error("text is not valid UTF-8");
             try {
               s.engine->encode(text, &s.state);
             } catch (const UnigramError& e) {
               rethrow(e);
             }
             return s.state.tokens;
           },
           py::arg("text"))
      .def("encode_batch",
           [](PyEngine& s, const std::vector<std::string>& texts, int num_threads) {
             for (const std::string& t : texts) {
               if (!pplx::unicode::is_valid_utf8(t)) throw py::value_error("text is not valid UTF-8");
             }
             std::vector<std::string_view> views(texts.begin(), texts.end());
             std::vector<std::vector<TokenId>> out;
             {
               py::gil_scoped_release release;
               try {
                 out = s.engine->encode_batch(views, num_threads);
               } catch (const UnigramError& e) {
                 py::gil_scoped_acquire acquire;
                 rethrow(e);
               }
             }
             return out;
           },
           py::arg("texts"), py::arg("num_threads") = 0)
      .def("encode_batch_flat",
           [](PyEngine& s, const std::vector<std::string>& texts, int num_threads) {
             for (const std::string& t : texts) {
               if (!pplx::unicode::is_valid_utf8(t)) throw py::value_error("text is not valid UTF-8");
             }
             std::vector<std::string_view> views(texts.begin(), texts.end());
             std::vector<std::vector<TokenId>> out;
             {
               py::gil_scoped_release release;
               try {
                 out = s.engine->encode_batch(views, num_threads);
               } catch (const UnigramError& e) {
                 py::gil_scoped_acquire acquire;
                 rethrow(e);
               }
             }
             // two arrays instead of millions of Python integers
             py::array_t<int64_t> offsets(static_cast<py::ssize_t>(out.size() + 1));
             int64_t* off = offsets.mutable_data();
             off[0] = 0;
             for (size_t i = 0; i < out.size(); ++i) off[i + 1] = off[i] + static_cast<int64_t>(out[i].size());
             py::array_t<int32_t> ids(static_cast<py::ssize_t>(off[out.size()]));
             int32_t* dst = ids.mutable_data();
             for (size_t i = 0; i < out.size(); ++i) {
               for (size_t j = 0; j < out[i].size(); ++j) dst[off[i] + static_cast<int64_t>(j)] = static_cast<int32_t>(out[i][j]);
             }
             return py::make_tuple(ids, offsets);
           },
           py::arg("texts"), py::arg("num_threads") = 0,
           "encode_batch with the result as (ids int32 [total], offsets int64 [len(texts) + 1]).")
      .def("normalize",
           [](PyEngine& s, const std::string& text) {
             std::string out;
             s.engine->normalize(text, &out);
             return out;
           })
      .def("split_special", [](PyEngine& s, const std::string& text) {
        std::vector<Segment> segs;
        s.engine->special_matcher().split(text, &segs);
        std::vector<py::tuple> out;
        for (const Segment& g : segs) {
          out.push_back(py::make_tuple(g.start, g.end, g.special ? py::cast(g.special_id) : py::none()));
        }
        return out;
      });

  // The numbers of a flat JSON object as the loader converts them (a test hook).
  m.def("_json_numbers", [](const std::string& text) {
    py::dict out;
    const pplx::json::Value v = pplx::json::parse(text);
    for (const auto& kv : v.as_object()) {
      if (kv.second.is_number()) out[py::str(kv.first)] = kv.second.as_number();
    }
    return out;
  });

  m.def("_grapheme_breaks", [](const std::string& text) {
    std::vector<size_t> ends;
    const uint8_t* p = reinterpret_cast<const uint8_t*>(text.data());
    size_t pos = 0;
    while (pos < text.size()) {
      pos = pplx::unicode::grapheme_end(p, text.size(), pos);
      ends.push_back(pos);
    }
    return ends;
  });
}
