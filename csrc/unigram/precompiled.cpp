#include "precompiled.h"

#include <algorithm>

#include <cstring>
#include <stdexcept>

#include "unicode.h"

namespace pplx::unigram {

std::vector<uint8_t> base64_decode(std::string_view text) {
  static int8_t table[256];
  static bool init = false;
  if (!init) {
    std::memset(table, -1, sizeof(table));
    const char* alphabet = "ABCDEFGHIJKLMNOPQRSTUVWXYZabcdefghijklmnopqrstuvwxyz0123456789+/";
    for (int i = 0; i < 64; ++i) table[static_cast<uint8_t>(alphabet[i])] = static_cast<int8_t>(i);
    init = true;
  }
  std::vector<uint8_t> out;
  out.reserve(text.size() / 4 * 3);
  uint32_t acc = 0;
  int bits = 0;
  size_t pad = 0;
  for (const char ch : text) {
    if (ch == '=') {
      ++pad;
      continue;
    }
    if (ch == '\n' || ch == '\r') continue;
    const int8_t v = table[static_cast<uint8_t>(ch)];
    if (v < 0 || pad > 0) throw std::runtime_error("invalid base64 input");
    acc = (acc << 6) | static_cast<uint32_t>(v);
    bits += 6;
    if (bits >= 8) {
      bits -= 8;
      out.push_back(static_cast<uint8_t>((acc >> bits) & 0xFF));
    }
  }
  if (pad > 2) throw std::runtime_error("invalid base64 padding");
  return out;
}

PrecompiledNormalizer::PrecompiledNormalizer(const std::vector<uint8_t>& blob) {
  if (blob.size() < 4) throw std::runtime_error("precompiled charsmap: blob too short");
  uint32_t trie_bytes;
  std::memcpy(&trie_bytes, blob.data(), 4);
  if (trie_bytes % 4 != 0 || 4ull + trie_bytes > blob.size()) {
    throw std::runtime_error("precompiled charsmap: bad trie size");
  }
  units_.resize(trie_bytes / 4);
  if (trie_bytes > 0) std::memcpy(units_.data(), blob.data() + 4, trie_bytes);   // an empty charsmap has no trie
  normalized_.assign(reinterpret_cast<const char*>(blob.data()) + 4 + trie_bytes,
                     blob.size() - 4 - trie_bytes);
  // ASCII bytes that no charsmap key starts with pass through unchanged whenever they
  // form a grapheme cluster of their own.
  for (int c = 0; c < 128; ++c) {
    const uint8_t b = static_cast<uint8_t>(c);
    size_t len = 0;
    ascii_passthrough_[c] = c != 0 && c != '\r' && transform(&b, 1, &len) == nullptr;
  }
}

PrecompiledNormalizer PrecompiledNormalizer::from_base64(std::string_view b64) {
  return PrecompiledNormalizer(base64_decode(b64));
}

namespace {
// darts-clone unit accessors
inline bool unit_has_leaf(uint32_t u) { return (u >> 8) & 1u; }
inline uint32_t unit_value(uint32_t u) { return u & 0x7FFFFFFFu; }
inline uint32_t unit_label(uint32_t u) { return u & (0x80000000u | 0xFFu); }
inline uint32_t unit_offset(uint32_t u) { return (u >> 10) << ((u & (1u << 9)) >> 6); }
}  // namespace

const char* PrecompiledNormalizer::transform(const uint8_t* chunk, size_t n, size_t* len) const {
  if (units_.empty()) return nullptr;
  const size_t size = units_.size();
  size_t node = 0;
  uint32_t unit = units_[node];
  node ^= unit_offset(unit);
  for (size_t i = 0; i < n; ++i) {
    const uint8_t c = chunk[i];
    if (c == 0) break;
    node ^= c;
    if (node >= size) return nullptr;
    unit = units_[node];
    if (unit_label(unit) != c) return nullptr;
    node ^= unit_offset(unit);
    if (unit_has_leaf(unit)) {
      if (node >= size) return nullptr;
      // first (shortest) match decides
      const size_t index = unit_value(units_[node]);
      if (index >= normalized_.size()) {
        *len = 0;
        return normalized_.data() + normalized_.size();
      }
      const char* start = normalized_.data() + index;
      *len = strnlen(start, normalized_.size() - index);
      return start;
    }
  }
  return nullptr;
}

namespace {

// Appends to a string through a raw pointer (no capacity check per byte) and collapses runs of
// spaces into one, which is the Replace(" {2,}" -> " ") step that follows the charsmap.
struct Collapser {
  std::string* out;
  size_t used = 0;
  bool prev_space = false;
  // room for n more bytes
  inline char* reserve(size_t n) {
    if (used + n > out->size()) out->resize(std::max(out->size() * 2, used + n + 64));
    return out->data() + used;
  }
  inline void push_bytes(const char* p, size_t n) {
    char* w = reserve(n);
    char* const w0 = w;
    bool ps = prev_space;
    for (size_t i = 0; i < n; ++i) {
      const char c = p[i];
      const bool sp = c == ' ';
      *w = c;
      w += (sp && ps) ? 0 : 1;
      ps = sp;
    }
    prev_space = ps;
    used += static_cast<size_t>(w - w0);
  }
  inline void finish() { out->resize(used); }
};

}  // namespace

void PrecompiledNormalizer::normalize_into(std::string_view input, std::string* out) const {
  out->clear();
  out->resize(input.size() + 64);
  const uint8_t* s = reinterpret_cast<const uint8_t*>(input.data());
  const size_t n = input.size();
  Collapser sink{out};
  size_t pos = 0;
  while (pos < n) {
    // Fast path: an unmapped ASCII byte followed by another ASCII byte is a cluster of its own
    // (CR LF is the one ASCII pair that joins; CR always takes the slow path). A run of such
    // bytes is copied in one pass, runs of spaces collapsing into one on the way.
    if (pos + 1 < n && ascii_passthrough_[s[pos]] && s[pos + 1] < 0x80) {
      char* w = sink.reserve(n - pos);
      char* const w0 = w;
      bool ps = sink.prev_space;
      uint8_t c0 = s[pos];
      do {
        const bool sp = c0 == ' ';
        *w = static_cast<char>(c0);
        w += (sp && ps) ? 0 : 1;
        ps = sp;
        ++pos;
        c0 = s[pos];
      } while (pos + 1 < n && ascii_passthrough_[c0] && s[pos + 1] < 0x80);
      sink.prev_space = ps;
      sink.used += static_cast<size_t>(w - w0);
      continue;
    }
    const size_t end = unicode::grapheme_end(s, n, pos);
    const size_t glen = end - pos;
    size_t rlen = 0;
    if (glen < 6) {
      const char* rep = transform(s + pos, glen, &rlen);
      if (rep != nullptr) {
        sink.push_bytes(rep, rlen);
        pos = end;
        continue;
      }
      int first_len = 0;
      unicode::decode(s, n, pos, &first_len);
      if (static_cast<size_t>(first_len) == glen) {
        // a single code point without a mapping: copy it through
        sink.push_bytes(reinterpret_cast<const char*>(s + pos), glen);
        pos = end;
        continue;
      }
    }
    // several code points: look each one up on its own
    size_t p = pos;
    while (p < end) {
      int l = 0;
      unicode::decode(s, n, p, &l);
      const char* rep = transform(s + p, static_cast<size_t>(l), &rlen);
      if (rep != nullptr) sink.push_bytes(rep, rlen);
      else sink.push_bytes(reinterpret_cast<const char*>(s + p), static_cast<size_t>(l));
      p += static_cast<size_t>(l);
    }
    pos = end;
  }
  sink.finish();
}

}  // namespace pplx::unigram
