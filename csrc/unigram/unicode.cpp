#include "unicode.h"

#include "unicode_tables.h"

namespace pplx::unicode {

uint16_t properties(uint32_t cp) {
  // Printable ASCII carries only the alphanumeric bit; keep it off the binary search.
  if (cp < 0x80) {
    if (cp >= 0x30) {
      const bool alnum = (cp <= 0x39) || (cp >= 0x41 && cp <= 0x5A) || (cp >= 0x61 && cp <= 0x7A);
      if (cp < 0x7F) return alnum ? 0x100 : 0;
    } else if (cp > 0x20) {
      return 0;
    }
  }
  int lo = 0, hi = kNumPropRanges - 1;
  while (lo <= hi) {
    const int mid = (lo + hi) >> 1;
    const PropRange& r = kPropRanges[mid];
    if (cp < r.lo) hi = mid - 1;
    else if (cp > r.hi) lo = mid + 1;
    else return r.props;
  }
  return 0;
}

uint32_t decode_before(const uint8_t* s, size_t pos, int* len) {
  size_t start = pos - 1;
  while (start > 0 && (s[start] & 0xC0) == 0x80 && pos - start < 4) --start;
  int l = 0;
  const uint32_t cp = decode(s, pos, start, &l);
  *len = static_cast<int>(pos - start);
  return cp;
}

size_t grapheme_end(const uint8_t* s, size_t n, size_t pos) {
  if (pos >= n) return n;
  int len = 0;
  uint32_t cp = decode(s, n, pos, &len);
  // Fast path: an ASCII character followed by ASCII forms a cluster on its own, except
  // CR LF. (No ASCII character is Extend, ZWJ, SpacingMark or Prepend.)
  if (cp < 0x80 && pos + 1 < n && s[pos + 1] < 0x80) {
    if (cp == '\r' && s[pos + 1] == '\n') return pos + 2;
    return pos + 1;
  }
  uint16_t props = properties(cp);
  GcbClass prev = gcb(props);
  size_t cur = pos + static_cast<size_t>(len);

  int ri_run = prev == kRegionalIndicator ? 1 : 0;
  // GB11 state: 1 = ExtPict Extend*, 2 = ExtPict Extend* ZWJ
  int pict = is_extended_pictographic(props) ? 1 : 0;
  // GB9c state: 1 = Consonant [Extend Linker]* without Linker, 2 = with a Linker seen
  int conj = incb(props) == 1 ? 1 : 0;

  while (cur < n) {
    cp = decode(s, n, cur, &len);
    props = properties(cp);
    const GcbClass next = gcb(props);
    bool join = false;
    if (prev == kCR && next == kLF) {
      join = true;                                            // GB3
    } else if (prev == kCR || prev == kLF || prev == kControl) {
      join = false;                                           // GB4
    } else if (next == kCR || next == kLF || next == kControl) {
      join = false;                                           // GB5
    } else if (prev == kL && (next == kL || next == kV || next == kLV || next == kLVT)) {
      join = true;                                            // GB6
    } else if ((prev == kLV || prev == kV) && (next == kV || next == kT)) {
      join = true;                                            // GB7
    } else if ((prev == kLVT || prev == kT) && next == kT) {
      join = true;                                            // GB8
    } else if (next == kExtend || next == kZWJ) {
      join = true;                                            // GB9
    } else if (next == kSpacingMark) {
      join = true;                                            // GB9a
    } else if (prev == kPrepend) {
      join = true;                                            // GB9b
    } else if (conj == 2 && incb(props) == 1) {
      join = true;                                            // GB9c
    } else if (pict == 2 && is_extended_pictographic(props)) {
      join = true;                                            // GB11
    } else if (prev == kRegionalIndicator && next == kRegionalIndicator && (ri_run & 1)) {
      join = true;                                            // GB12, GB13
    }
    if (!join) break;

    // advance the rule state over the joined character
    if (next == kRegionalIndicator) ri_run += 1; else ri_run = 0;
    if (is_extended_pictographic(props)) {
      pict = 1;
    } else if (pict == 1 && next == kExtend) {
      pict = 1;
    } else if (pict == 1 && next == kZWJ) {
      pict = 2;
    } else {
      pict = 0;
    }
    const int ic = incb(props);
    if (ic == 1) {
      conj = 1;
    } else if (conj != 0 && ic == 2) {
      // Extend keeps the state
    } else if (conj != 0 && ic == 3) {
      conj = 2;
    } else {
      conj = 0;
    }
    prev = next;
    cur += static_cast<size_t>(len);
  }
  return cur;
}

bool is_valid_utf8(std::string_view sv) {
  const uint8_t* s = reinterpret_cast<const uint8_t*>(sv.data());
  const size_t n = sv.size();
  size_t i = 0;
  while (i < n) {
    const uint8_t b = s[i];
    if (b < 0x80) {
      ++i;
    } else if (b >= 0xC2 && b <= 0xDF) {
      if (i + 1 >= n || (s[i + 1] & 0xC0) != 0x80) return false;
      i += 2;
    } else if (b >= 0xE0 && b <= 0xEF) {
      if (i + 2 >= n || (s[i + 1] & 0xC0) != 0x80 || (s[i + 2] & 0xC0) != 0x80) return false;
      if (b == 0xE0 && s[i + 1] < 0xA0) return false;
      if (b == 0xED && s[i + 1] >= 0xA0) return false;
      i += 3;
    } else if (b >= 0xF0 && b <= 0xF4) {
      if (i + 3 >= n || (s[i + 1] & 0xC0) != 0x80 || (s[i + 2] & 0xC0) != 0x80 ||
          (s[i + 3] & 0xC0) != 0x80) {
        return false;
      }
      if (b == 0xF0 && s[i + 1] < 0x90) return false;
      if (b == 0xF4 && s[i + 1] >= 0x90) return false;
      i += 4;
    } else {
      return false;
    }
  }
  return true;
}

}  // namespace pplx::unicode
