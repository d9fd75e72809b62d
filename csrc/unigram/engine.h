// Unigram (SentencePiece-style) tokenizer encoder for HuggingFace tokenizer.json files.
//
// Pipeline: precompiled-charsmap normalisation (with space-run collapse) -> special token
// split -> per text segment: Metaspace -> Viterbi over the vocabulary trie, with one-code-
// point UNK fallback (score = min vocab score - 10) and fusion of adjacent UNKs.
// Same behaviour as the reference's pplx-unigram (pplx-unigram/src/engine.rs:46-165,
// special_tokens.rs:28-127, metaspace.rs:41-59, config.rs:8-127); its public surface
// (`Engine`, `EncodeState`, `Segment`, `Error`: pplx-unigram/src/lib.rs:10-35) maps to
// the classes below. An immutable Engine can be shared by any number of threads, each
// with its own EncodeState; encode_batch() does that with a pool of worker threads.
#pragma once

#include <cstdint>
#include <memory>
#include <stdexcept>
#include <cstring>
#include <string>
#include <string_view>
#include <vector>

#include "precompiled.h"
#include "trie.h"

namespace pplx::unigram {

using TokenId = uint32_t;

enum class ErrorKind { kIo, kInvalidConfig, kUnsupportedConfig, kEncodeFailed };

class UnigramError : public std::runtime_error {
 public:
  UnigramError(ErrorKind kind, const std::string& what) : std::runtime_error(what), kind_(kind) {}
  ErrorKind kind() const { return kind_; }

 private:
  ErrorKind kind_;
};

struct Segment {
  size_t start = 0;
  size_t end = 0;
  bool special = false;
  TokenId special_id = 0;
};

struct SpecialToken {
  TokenId id = 0;
  std::string content;
  bool single_word = false;
  bool lstrip = false;
  bool rstrip = false;
};

// Words seen before and their token ids, per encoding thread. Natural text repeats its words
// (Zipf), and with the text cut into words the best path of a word never depends on its
// neighbours, so a hit replaces the whole Viterbi pass over the word. Open addressing over
// 64-bit hashes with the bytes kept in one arena; bounded: once full, new words are simply
// not remembered.
class WordCache {
 public:
  static constexpr size_t kSlots = 1u << 18;       // power of two; 6 MiB of slots once the first word is kept
  static constexpr size_t kMaxEntries = kSlots / 2;
  static constexpr size_t kMaxWordBytes = 64;
  static constexpr size_t kMaxArenaBytes = 16u << 20;

  struct Entry {
    uint64_t hash = 0;      // 0 = empty slot
    uint32_t key_off = 0;
    uint16_t key_len = 0;
    uint16_t num_tokens = 0;
    uint32_t tok_off = 0;
  };

  // Returns the entry of `word` or nullptr.
  const Entry* find(const uint8_t* word, size_t len, uint64_t hash) const {
    if (slots_.empty()) return nullptr;
    for (size_t i = hash & (kSlots - 1);; i = (i + 1) & (kSlots - 1)) {
      const Entry& e = slots_[i];
      if (e.hash == 0) return nullptr;
      if (e.hash == hash && e.key_len == len && std::memcmp(keys_.data() + e.key_off, word, len) == 0) return &e;
    }
  }
  const TokenId* tokens_of(const Entry& e) const { return toks_.data() + e.tok_off; }
  void insert(const uint8_t* word, size_t len, uint64_t hash, const TokenId* toks, size_t n) {
    if (count_ >= kMaxEntries || keys_.size() + len > kMaxArenaBytes || n > 0xffff) return;
    if (slots_.empty()) slots_.resize(kSlots);
    size_t i = hash & (kSlots - 1);
    while (slots_[i].hash != 0) i = (i + 1) & (kSlots - 1);
    Entry& e = slots_[i];
    e.hash = hash;
    e.key_off = static_cast<uint32_t>(keys_.size());
    e.key_len = static_cast<uint16_t>(len);
    e.num_tokens = static_cast<uint16_t>(n);
    e.tok_off = static_cast<uint32_t>(toks_.size());
    keys_.insert(keys_.end(), word, word + len);
    toks_.insert(toks_.end(), toks, toks + n);
    ++count_;
  }
  // Eight bytes per multiply (a word is mostly one or two steps; a byte-wise FNV chain was the
  // hottest spot of a cache hit). Never 0.
  static uint64_t hash_bytes(const uint8_t* p, size_t n) {
    constexpr uint64_t kMul = 0x9FB21C651E98DF25ull;
    uint64_t h = 0x9E3779B97F4A7C15ull ^ (static_cast<uint64_t>(n) * 0xff51afd7ed558ccdull);
    while (n >= 8) {
      uint64_t v;
      std::memcpy(&v, p, 8);
      h = (h ^ v) * kMul;
      h ^= h >> 32;
      p += 8;
      n -= 8;
    }
    if (n > 0) {
      uint64_t v = 0;
      for (size_t i = 0; i < n; ++i) v |= static_cast<uint64_t>(p[i]) << (8 * i);
      h = (h ^ v) * kMul;
      h ^= h >> 32;
    }
    h *= 0xff51afd7ed558ccdull;
    h ^= h >> 29;
    return h | 1ull;
  }
  size_t size() const { return count_; }

 private:
  std::vector<Entry> slots_;
  std::vector<uint8_t> keys_;
  std::vector<TokenId> toks_;
  size_t count_ = 0;
};

// Scratch buffers of one encoding thread; grow to the longest input seen and are reused.
struct EncodeState {
  std::vector<TokenId> tokens;  // result of the last encode()
  std::string normalized;
  std::string prep;
  std::vector<Segment> segments;
  std::vector<double> best_score;
  std::vector<uint32_t> best_start;
  std::vector<TokenId> best_id;
  std::vector<TokenId> backtrack;
  WordCache words;          // belongs to one engine: do not share a state between engines
  const void* words_owner = nullptr;
};

class SpecialTokenMatcher {
 public:
  SpecialTokenMatcher() = default;
  explicit SpecialTokenMatcher(std::vector<SpecialToken> tokens);
  // Splits `text` into text and special segments (earliest match first; on a tie the
  // longest content wins).
  void split(std::string_view text, std::vector<Segment>* out) const;
  bool empty() const { return tokens_.empty(); }

 private:
  std::vector<SpecialToken> tokens_;
};

class Engine {
 public:
  static std::shared_ptr<Engine> from_hf_json_path(const std::string& path);
  static std::shared_ptr<Engine> from_hf_json_bytes(std::string_view bytes);

  size_t vocab_size() const { return vocab_size_; }
  TokenId unk_id() const { return unk_id_; }
  bool trie_on_huge_pages() const { return trie_.huge_pages(); }
  size_t trie_nodes() const { return trie_.size(); }

  // Encodes valid UTF-8 `text`; the ids are left in state->tokens.
  void encode(std::string_view text, EncodeState* state) const;

  // Encodes many texts with `num_threads` threads (0: hardware concurrency).
  std::vector<std::vector<TokenId>> encode_batch(const std::vector<std::string_view>& texts,
                                                 int num_threads) const;

  // Exposed for tests.
  void normalize(std::string_view text, std::string* out) const { normalizer_.normalize_into(text, out); }
  const SpecialTokenMatcher& special_matcher() const { return special_; }

 private:
  Engine() = default;
  void encode_segment(std::string_view text, EncodeState* state) const;
  void viterbi(const uint8_t* prep, size_t n, EncodeState* state) const;

  PrecompiledNormalizer normalizer_;
  SpecialTokenMatcher special_;
  VocabTrie trie_;
  std::string replacement_;  // UTF-8 of the metaspace replacement character
  bool add_prefix_space_ = true;
  bool split_words_ = true;   // Metaspace "split": encode word by word
  TokenId unk_id_ = 0;
  double unk_score_ = 0.0;
  size_t vocab_size_ = 0;
};

}  // namespace pplx::unigram
