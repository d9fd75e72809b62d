#include "json.h"

#include <cerrno>
#include <cstdlib>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <stdexcept>

namespace pplx::json {

Value Value::make_bool(bool b) {
  Value v;
  v.type_ = Type::kBool;
  v.bool_ = b;
  return v;
}
Value Value::make_number(double d) {
  Value v;
  v.type_ = Type::kNumber;
  v.number_ = d;
  return v;
}
Value Value::make_string(std::string s) {
  Value v;
  v.type_ = Type::kString;
  v.string_ = std::move(s);
  return v;
}
Value Value::make_array(Array a) {
  Value v;
  v.type_ = Type::kArray;
  v.array_ = std::make_shared<Array>(std::move(a));
  return v;
}
Value Value::make_object(Object o) {
  Value v;
  v.type_ = Type::kObject;
  v.object_ = std::make_shared<Object>(std::move(o));
  return v;
}

const Value* Value::find(std::string_view key) const {
  if (type_ != Type::kObject) return nullptr;
  for (const auto& kv : *object_) {
    if (kv.first == key) return &kv.second;
  }
  return nullptr;
}

namespace {

class Parser {
 public:
  explicit Parser(std::string_view text) : p_(text.data()), begin_(text.data()), end_(text.data() + text.size()) {}

  Value run() {
    skip_ws();
    Value v = value(0);
    skip_ws();
    if (p_ != end_) fail("trailing characters after the document");
    return v;
  }

 private:
  [[noreturn]] void fail(const char* what) const {
    throw std::runtime_error(std::string("JSON parse error at byte ") +
                             std::to_string(p_ - begin_) + ": " + what);
  }

  void skip_ws() {
    while (p_ < end_ && (*p_ == ' ' || *p_ == '\n' || *p_ == '\r' || *p_ == '\t')) ++p_;
  }

  bool consume(const char* lit) {
    const size_t n = std::strlen(lit);
    if (static_cast<size_t>(end_ - p_) >= n && std::memcmp(p_, lit, n) == 0) {
      p_ += n;
      return true;
    }
    return false;
  }

  Value value(int depth) {
    if (depth > 256) fail("nesting too deep");
    if (p_ >= end_) fail("unexpected end of input");
    switch (*p_) {
      case '{': return object(depth);
      case '[': return array(depth);
      case '"': return Value::make_string(string());
      case 't':
        if (consume("true")) return Value::make_bool(true);
        fail("bad literal");
      case 'f':
        if (consume("false")) return Value::make_bool(false);
        fail("bad literal");
      case 'n':
        if (consume("null")) return Value();
        fail("bad literal");
      default: return number();
    }
  }

  // Numbers are converted the way Rust's serde_json does without its float_roundtrip feature
  // (what HuggingFace tokenizers and pplx-unigram read vocabularies with): the digits are
  // gathered into a 64-bit significand, converted to double, and scaled by one power of ten.
  // That is up to one unit in the last place away from the correctly rounded value for
  // 16-17 digit literals, and Viterbi ties between equal-score paths are decided by exactly that
  // last bit, so strtod here would make some encodings differ from the originals'.
  static double pow10_table(int k) {
    static const std::vector<double> table = [] {
      std::vector<double> t(309);
      for (int i = 0; i <= 308; ++i) {
        char lit[16];
        std::snprintf(lit, sizeof(lit), "1e%d", i);
        t[static_cast<size_t>(i)] = std::strtod(lit, nullptr);
      }
      return t;
    }();
    return table[static_cast<size_t>(k)];
  }

  static double from_parts(bool positive, uint64_t significand, long long exponent) {
    double f = static_cast<double>(significand);
    for (;;) {
      const long long mag = exponent < 0 ? -exponent : exponent;
      if (mag <= 308) {
        if (exponent >= 0) {
          f *= pow10_table(static_cast<int>(mag));
        } else {
          f /= pow10_table(static_cast<int>(mag));
        }
        break;
      }
      if (f == 0.0) break;
      if (exponent >= 0) return positive ? HUGE_VAL : -HUGE_VAL;
      f /= 1e308;
      exponent += 308;
    }
    return positive ? f : -f;
  }

  Value number() {
    bool positive = true;
    if (p_ < end_ && *p_ == '-') {
      positive = false;
      ++p_;
    }
    if (p_ >= end_ || !(*p_ >= '0' && *p_ <= '9')) fail("expected a value");
    uint64_t significand = 0;
    long long exponent = 0;
    bool saturated = false;   // further digits no longer fit: they only move the exponent
    auto push_digit = [&](unsigned d, bool fractional) {
      const uint64_t max = ~uint64_t{0};
      if (!saturated && (significand >= max / 10 && (significand > max / 10 || d > max % 10))) saturated = true;
      if (saturated) {
        if (!fractional) ++exponent;
        return;
      }
      significand = significand * 10 + d;
      if (fractional) --exponent;
    };
    if (*p_ == '0') {
      ++p_;
      if (p_ < end_ && *p_ >= '0' && *p_ <= '9') fail("malformed number");
    } else {
      while (p_ < end_ && *p_ >= '0' && *p_ <= '9') push_digit(static_cast<unsigned>(*p_++ - '0'), false);
    }
    bool is_float = false;
    if (p_ < end_ && *p_ == '.') {
      ++p_;
      is_float = true;
      if (p_ >= end_ || !(*p_ >= '0' && *p_ <= '9')) fail("malformed number");
      while (p_ < end_ && *p_ >= '0' && *p_ <= '9') push_digit(static_cast<unsigned>(*p_++ - '0'), true);
    }
    if (p_ < end_ && (*p_ == 'e' || *p_ == 'E')) {
      ++p_;
      is_float = true;
      bool exp_positive = true;
      if (p_ < end_ && (*p_ == '+' || *p_ == '-')) exp_positive = *p_++ == '+';
      if (p_ >= end_ || !(*p_ >= '0' && *p_ <= '9')) fail("malformed number");
      long long e = 0;
      while (p_ < end_ && *p_ >= '0' && *p_ <= '9') {
        if (e < 100000) e = e * 10 + (*p_ - '0');
        ++p_;
      }
      exponent += exp_positive ? e : -e;
    }
    if (!is_float && !saturated) {   // an integer literal: exact conversion of the integer
      const double d = static_cast<double>(significand);
      return Value::make_number(positive ? d : -d);
    }
    return Value::make_number(from_parts(positive, significand, exponent));
  }

  static void append_utf8(std::string* out, uint32_t cp) {
    if (cp < 0x80) {
      out->push_back(static_cast<char>(cp));
    } else if (cp < 0x800) {
      out->push_back(static_cast<char>(0xC0 | (cp >> 6)));
      out->push_back(static_cast<char>(0x80 | (cp & 0x3F)));
    } else if (cp < 0x10000) {
      out->push_back(static_cast<char>(0xE0 | (cp >> 12)));
      out->push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F)));
      out->push_back(static_cast<char>(0x80 | (cp & 0x3F)));
    } else {
      out->push_back(static_cast<char>(0xF0 | (cp >> 18)));
      out->push_back(static_cast<char>(0x80 | ((cp >> 12) & 0x3F)));
      out->push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F)));
      out->push_back(static_cast<char>(0x80 | (cp & 0x3F)));
    }
  }

  uint32_t hex4() {
    if (end_ - p_ < 4) fail("truncated \\u escape");
    uint32_t v = 0;
    for (int i = 0; i < 4; ++i) {
      const char c = *p_++;
      v <<= 4;
      if (c >= '0' && c <= '9') v |= static_cast<uint32_t>(c - '0');
      else if (c >= 'a' && c <= 'f') v |= static_cast<uint32_t>(c - 'a' + 10);
      else if (c >= 'A' && c <= 'F') v |= static_cast<uint32_t>(c - 'A' + 10);
      else fail("bad hex digit in \\u escape");
    }
    return v;
  }

  std::string string() {
    ++p_;  // opening quote
    std::string out;
    for (;;) {
      if (p_ >= end_) fail("unterminated string");
      const char* run = p_;
      while (p_ < end_ && *p_ != '"' && *p_ != '\\') {
        if (static_cast<unsigned char>(*p_) < 0x20) fail("control character in string");
        ++p_;
      }
      out.append(run, static_cast<size_t>(p_ - run));
      if (p_ >= end_) fail("unterminated string");
      if (*p_ == '"') {
        ++p_;
        return out;
      }
      ++p_;  // backslash
      if (p_ >= end_) fail("unterminated escape");
      const char c = *p_++;
      switch (c) {
        case '"': out.push_back('"'); break;
        case '\\': out.push_back('\\'); break;
        case '/': out.push_back('/'); break;
        case 'b': out.push_back('\b'); break;
        case 'f': out.push_back('\f'); break;
        case 'n': out.push_back('\n'); break;
        case 'r': out.push_back('\r'); break;
        case 't': out.push_back('\t'); break;
        case 'u': {
          uint32_t cp = hex4();
          if (cp >= 0xD800 && cp <= 0xDBFF) {
            if (end_ - p_ >= 6 && p_[0] == '\\' && p_[1] == 'u') {
              p_ += 2;
              const uint32_t lo = hex4();
              if (lo < 0xDC00 || lo > 0xDFFF) fail("unpaired surrogate");
              cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
            } else {
              fail("unpaired surrogate");
            }
          } else if (cp >= 0xDC00 && cp <= 0xDFFF) {
            fail("unpaired surrogate");
          }
          append_utf8(&out, cp);
          break;
        }
        default: fail("unknown escape");
      }
    }
  }

  Value array(int depth) {
    ++p_;
    Array items;
    skip_ws();
    if (p_ < end_ && *p_ == ']') {
      ++p_;
      return Value::make_array(std::move(items));
    }
    for (;;) {
      skip_ws();
      items.push_back(value(depth + 1));
      skip_ws();
      if (p_ >= end_) fail("unterminated array");
      if (*p_ == ',') {
        ++p_;
        continue;
      }
      if (*p_ == ']') {
        ++p_;
        return Value::make_array(std::move(items));
      }
      fail("expected ',' or ']'");
    }
  }

  Value object(int depth) {
    ++p_;
    Object members;
    skip_ws();
    if (p_ < end_ && *p_ == '}') {
      ++p_;
      return Value::make_object(std::move(members));
    }
    for (;;) {
      skip_ws();
      if (p_ >= end_ || *p_ != '"') fail("expected a member name");
      std::string key = string();
      skip_ws();
      if (p_ >= end_ || *p_ != ':') fail("expected ':'");
      ++p_;
      skip_ws();
      members.emplace_back(std::move(key), value(depth + 1));
      skip_ws();
      if (p_ >= end_) fail("unterminated object");
      if (*p_ == ',') {
        ++p_;
        continue;
      }
      if (*p_ == '}') {
        ++p_;
        return Value::make_object(std::move(members));
      }
      fail("expected ',' or '}'");
    }
  }

  const char* p_;
  const char* begin_;
  const char* end_;
};

}  // namespace

Value parse(std::string_view text) { return Parser(text).run(); }

}  // namespace pplx::json
