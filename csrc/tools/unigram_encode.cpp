// pplx-unigram-encode <tokenizer.json> <text | @file> [--repeat N] [--threads T]
//
// Prints the token ids of the text and the time per encode; with --threads the input
// file is split into lines that are encoded in parallel and the throughput in MB/s is
// reported. Command-line counterpart of the reference's example binary
// (pplx-unigram/examples/encode.rs:15-57: 1000 encodes of one string, us per encode).
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <sstream>
#include <string>
#include <vector>

#include "../unigram/engine.h"

using namespace pplx::unigram;

int main(int argc, char** argv) {
  if (argc < 3) {
    std::fprintf(stderr, "usage: %s <tokenizer.json> <text | @file> [--repeat N] [--threads T]\n", argv[0]);
    return 2;
  }
  int repeat = 1000, threads = 0;
  for (int i = 3; i + 1 < argc; i += 2) {
    if (std::strcmp(argv[i], "--repeat") == 0) repeat = std::atoi(argv[i + 1]);
    else if (std::strcmp(argv[i], "--threads") == 0) threads = std::atoi(argv[i + 1]);
  }
  try {
    const auto t_load = std::chrono::steady_clock::now();
    std::shared_ptr<Engine> engine = Engine::from_hf_json_path(argv[1]);
    const double load_ms =
        std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t_load).count();
    std::fprintf(stderr, "loaded %zu tokens, %zu trie nodes (%s pages) in %.1f ms\n", engine->vocab_size(),
                 engine->trie_nodes(), engine->trie_on_huge_pages() ? "huge" : "normal", load_ms);
    std::string text = argv[2];
    if (!text.empty() && text[0] == '@') {
      std::ifstream in(text.substr(1), std::ios::binary);
      if (!in) {
        std::fprintf(stderr, "cannot open %s\n", text.c_str() + 1);
        return 1;
      }
      std::ostringstream buf;
      buf << in.rdbuf();
      text = buf.str();
    }
    if (threads > 0) {
      std::vector<std::string_view> lines;
      size_t start = 0;
      const std::string_view all(text);
      while (start < all.size()) {
        size_t nl = all.find('\n', start);
        if (nl == std::string_view::npos) nl = all.size();
        if (nl > start) lines.push_back(all.substr(start, nl - start));
        start = nl + 1;
      }
      size_t tokens = 0;
      const auto t0 = std::chrono::steady_clock::now();
      for (int r = 0; r < std::max(1, repeat); ++r) {
        const auto ids = engine->encode_batch(lines, threads);
        tokens = 0;
        for (const auto& v : ids) tokens += v.size();
      }
      const double secs = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
      const double mb = static_cast<double>(text.size()) * std::max(1, repeat) / 1e6;
      std::printf("%zu lines, %zu tokens, %d threads: %.1f MB/s\n", lines.size(), tokens, threads, mb / secs);
      return 0;
    }
    EncodeState state;
    engine->encode(text, &state);
    for (size_t i = 0; i < state.tokens.size(); ++i) std::printf(i ? " %u" : "%u", state.tokens[i]);
    std::printf("\n");
    const auto t0 = std::chrono::steady_clock::now();
    for (int r = 0; r < repeat; ++r) engine->encode(text, &state);
    const double us = std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - t0).count();
    std::fprintf(stderr, "%d encodes of %zu bytes: %.2f us per encode, %.1f MB/s\n", repeat, text.size(),
                 us / std::max(1, repeat), static_cast<double>(text.size()) * repeat / us);
  } catch (const std::exception& e) {
    std::fprintf(stderr, "error: %s\n", e.what());
    return 1;
  }
  return 0;
}
