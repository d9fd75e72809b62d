#include "trie.h"

#include <sys/mman.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <stdexcept>

namespace pplx::unigram {

namespace {

struct BuildNode {
  int32_t token_id = -1;
  double score = 0.0;
  std::vector<std::pair<uint8_t, uint32_t>> children;  // (byte, build-node index)
};

constexpr size_t kHugePage = 2u << 20;

}  // namespace

VocabTrie::~VocabTrie() { release(); }

void VocabTrie::release() {
  if (nodes_ != nullptr) {
    munmap(nodes_, mapped_bytes_);
    nodes_ = nullptr;
  }
  count_ = 0;
}

VocabTrie::VocabTrie(VocabTrie&& o) noexcept
    : nodes_(o.nodes_), count_(o.count_), mapped_bytes_(o.mapped_bytes_), huge_(o.huge_) {
  o.nodes_ = nullptr;
  o.count_ = 0;
}

VocabTrie& VocabTrie::operator=(VocabTrie&& o) noexcept {
  if (this != &o) {
    release();
    nodes_ = o.nodes_;
    count_ = o.count_;
    mapped_bytes_ = o.mapped_bytes_;
    huge_ = o.huge_;
    o.nodes_ = nullptr;
    o.count_ = 0;
  }
  return *this;
}

VocabTrie VocabTrie::build(const std::vector<std::string>& tokens,
                           const std::vector<double>& scores) {
  if (tokens.size() != scores.size()) throw std::runtime_error("vocab and scores differ in length");
  std::vector<BuildNode> tmp(1);
  for (size_t id = 0; id < tokens.size(); ++id) {
    const std::string& tok = tokens[id];
    if (tok.empty()) throw std::runtime_error("vocab contains an empty token");
    uint32_t cur = 0;
    for (const char ch : tok) {
      const uint8_t b = static_cast<uint8_t>(ch);
      uint32_t next = 0;
      bool found = false;
      for (const auto& c : tmp[cur].children) {
        if (c.first == b) {
          next = c.second;
          found = true;
          break;
        }
      }
      if (!found) {
        next = static_cast<uint32_t>(tmp.size());
        tmp[cur].children.emplace_back(b, next);
        tmp.emplace_back();
      }
      cur = next;
    }
    tmp[cur].token_id = static_cast<int32_t>(id);
    tmp[cur].score = scores[id];
  }

  VocabTrie trie;
  trie.count_ = tmp.size();
  const size_t bytes = trie.count_ * sizeof(TrieNode);
  // Prefer explicit 2 MiB pages; fall back to a normal mapping with a THP hint.
  const size_t huge_bytes = (bytes + kHugePage - 1) / kHugePage * kHugePage;
  void* mem = mmap(nullptr, huge_bytes, PROT_READ | PROT_WRITE,
                   MAP_PRIVATE | MAP_ANONYMOUS | MAP_HUGETLB, -1, 0);
  if (mem != MAP_FAILED) {
    trie.huge_ = true;
    trie.mapped_bytes_ = huge_bytes;
  } else {
    mem = mmap(nullptr, huge_bytes, PROT_READ | PROT_WRITE, MAP_PRIVATE | MAP_ANONYMOUS, -1, 0);
    if (mem == MAP_FAILED) throw std::runtime_error("mmap of the trie failed");
    madvise(mem, huge_bytes, MADV_HUGEPAGE);
    trie.mapped_bytes_ = huge_bytes;
  }
  trie.nodes_ = static_cast<TrieNode*>(mem);

  // Breadth-first numbering: the children of a node get consecutive indices.
  std::vector<uint32_t> order;      // build-node index of final node i
  order.reserve(tmp.size());
  order.push_back(0);
  for (size_t i = 0; i < order.size(); ++i) {
    BuildNode& bn = tmp[order[i]];
    std::sort(bn.children.begin(), bn.children.end());
    TrieNode& n = trie.nodes_[i];
    std::memset(&n, 0, sizeof(n));
    n.token_id = bn.token_id;
    n.score = bn.score;
    n.child_base = static_cast<uint32_t>(order.size());
    for (const auto& c : bn.children) {
      n.bitmap[c.first >> 6] |= 1ull << (c.first & 63);
      order.push_back(c.second);
    }
    uint32_t run = 0;
    for (int w = 0; w < 4; ++w) {
      n.word_rank[w] = static_cast<uint8_t>(run);
      run += static_cast<uint32_t>(__builtin_popcountll(n.bitmap[w]));
    }
  }
  return trie;
}

}  // namespace pplx::unigram
