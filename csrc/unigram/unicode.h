// UTF-8 helpers, Unicode property lookup and extended grapheme cluster segmentation
// (UAX #29, rules GB1-GB999 including GB9c and GB11). The reference relies on the
// unicode-segmentation crate for the same job (pplx-unigram/src/normalizer.rs:27-52);
// property data comes from the generated unicode_tables.h.
#pragma once

#include <cstddef>
#include <cstdint>
#include <string_view>

namespace pplx::unicode {

enum GcbClass : uint8_t {
  kOther = 0, kCR, kLF, kControl, kExtend, kZWJ, kRegionalIndicator, kPrepend, kSpacingMark,
  kL, kV, kT, kLV, kLVT,
};

// Packed properties (see gen_unicode_tables.py for the bit layout).
uint16_t properties(uint32_t cp);
inline GcbClass gcb(uint16_t props) { return static_cast<GcbClass>(props & 0xF); }
inline bool is_extended_pictographic(uint16_t props) { return (props >> 4) & 1; }
inline int incb(uint16_t props) { return (props >> 5) & 3; }  // 1 Consonant, 2 Extend, 3 Linker
inline bool is_white_space(uint32_t cp) { return (properties(cp) >> 7) & 1; }
inline bool is_alphanumeric(uint32_t cp) { return (properties(cp) >> 8) & 1; }

// Decodes the code point starting at s[pos] (s must be valid UTF-8); *len gets its
// length in bytes.
inline uint32_t decode(const uint8_t* s, size_t n, size_t pos, int* len) {
  const uint8_t b0 = s[pos];
  if (b0 < 0x80) {
    *len = 1;
    return b0;
  }
  if (b0 < 0xE0 && pos + 1 < n) {
    *len = 2;
    return ((b0 & 0x1Fu) << 6) | (s[pos + 1] & 0x3Fu);
  }
  if (b0 < 0xF0 && pos + 2 < n) {
    *len = 3;
    return ((b0 & 0x0Fu) << 12) | ((s[pos + 1] & 0x3Fu) << 6) | (s[pos + 2] & 0x3Fu);
  }
  if (pos + 3 < n) {
    *len = 4;
    return ((b0 & 0x07u) << 18) | ((s[pos + 1] & 0x3Fu) << 12) | ((s[pos + 2] & 0x3Fu) << 6) |
           (s[pos + 3] & 0x3Fu);
  }
  *len = 1;
  return 0xFFFD;
}

// Code point that ends right before `pos` (pos > 0).
uint32_t decode_before(const uint8_t* s, size_t pos, int* len);

// Byte offset where the extended grapheme cluster starting at `pos` ends.
size_t grapheme_end(const uint8_t* s, size_t n, size_t pos);

// True when `s` is well-formed UTF-8 (no overlongs, no surrogates, <= U+10FFFF).
bool is_valid_utf8(std::string_view s);

}  // namespace pplx::unicode
