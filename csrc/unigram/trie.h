// Byte trie over the vocabulary, one 64-byte node per cache line.
//
// A node stores a 256-bit map of the bytes that have a child, the index of its first
// child and the running popcounts of the map's words; the children of a node are stored
// contiguously in byte order, so following byte b is one bit test, one popcount and one
// add. A failed transition is decided inside the parent's line and touches no other
// memory. Terminal nodes carry the token id and its score in the same line.
//
// The reference reaches the same "one line per step" property with a double-array trie
// whose nodes also carry a child bitmap (pplx-unigram/src/trie.rs:19-33,88-194); the
// rank-indexed layout used here needs no slot search at build time and leaves no holes.
#pragma once

#include <cstddef>
#include <cstdint>
#include <string>
#include <vector>

namespace pplx::unigram {

struct alignas(64) TrieNode {
  uint64_t bitmap[4];
  uint32_t child_base;
  int32_t token_id;      // -1: not a token
  double score;
  uint8_t word_rank[4];  // children in bitmap words before word i
  uint8_t pad_[12];

  inline bool has_child(uint8_t b) const { return (bitmap[b >> 6] >> (b & 63)) & 1ull; }
  inline uint32_t child_index(uint8_t b) const {
    const uint64_t below = bitmap[b >> 6] & ((1ull << (b & 63)) - 1ull);
    return child_base + word_rank[b >> 6] + static_cast<uint32_t>(__builtin_popcountll(below));
  }
};
static_assert(sizeof(TrieNode) == 64, "one node per cache line");

class VocabTrie {
 public:
  VocabTrie() = default;
  ~VocabTrie();
  VocabTrie(const VocabTrie&) = delete;
  VocabTrie& operator=(const VocabTrie&) = delete;
  VocabTrie(VocabTrie&& o) noexcept;
  VocabTrie& operator=(VocabTrie&& o) noexcept;

  // Later duplicates of a byte string replace earlier ones; empty strings are rejected.
  static VocabTrie build(const std::vector<std::string>& tokens, const std::vector<double>& scores);

  const TrieNode* nodes() const { return nodes_; }
  size_t size() const { return count_; }
  bool huge_pages() const { return huge_; }

 private:
  void release();
  TrieNode* nodes_ = nullptr;
  size_t count_ = 0;
  size_t mapped_bytes_ = 0;
  bool huge_ = false;
};

}  // namespace pplx::unigram
