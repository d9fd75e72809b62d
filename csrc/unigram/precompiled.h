// SentencePiece "precompiled charsmap" normaliser: a darts-clone double array that maps
// byte strings to replacement strings, applied grapheme by grapheme, fused with the
// collapse of space runs. Behaviour matches the reference's NormalizerPipeline
// (pplx-unigram/src/normalizer.rs:15-73), which wraps the spm_precompiled crate: the
// replacement of a chunk is the one of its *shortest* matching prefix.
#pragma once

#include <cstdint>
#include <string>
#include <string_view>
#include <vector>

namespace pplx::unigram {

// Standard base64 (with padding). Throws std::runtime_error on bad input.
std::vector<uint8_t> base64_decode(std::string_view text);

class PrecompiledNormalizer {
 public:
  PrecompiledNormalizer() = default;
  // blob = u32 LE trie size in bytes | trie units (u32 LE) | NUL-separated replacements
  explicit PrecompiledNormalizer(const std::vector<uint8_t>& blob);
  static PrecompiledNormalizer from_base64(std::string_view b64);

  // Replacement for `chunk` or nullptr if no prefix of it is a key; *len gets its size.
  const char* transform(const uint8_t* chunk, size_t n, size_t* len) const;

  // Normalises valid UTF-8 `input` into `out` (cleared first).
  void normalize_into(std::string_view input, std::string* out) const;

  bool empty() const { return units_.empty(); }

 private:
  std::vector<uint32_t> units_;
  std::string normalized_;
  bool ascii_passthrough_[256] = {};   // false from 0x80 up and for CR (CR LF is one cluster)
};

}  // namespace pplx::unigram
