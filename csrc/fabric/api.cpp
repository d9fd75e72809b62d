#include "api.h"

#include <chrono>
#include <cstring>
#include <thread>

#include "../core/error.h"

namespace pplx::fabric {

std::string hex_encode(const std::string& bytes) {
  static const char* digits = "0123456789abcdef";
  std::string out;
  out.reserve(bytes.size() * 2);
  for (unsigned char c : bytes) {
    out.push_back(digits[c >> 4]);
    out.push_back(digits[c & 15]);
  }
  return out;
}

std::string hex_decode(const std::string& hex) {
  auto nibble = [](char c) -> int {
    if (c >= '0' && c <= '9') return c - '0';
    if (c >= 'a' && c <= 'f') return c - 'a' + 10;
    if (c >= 'A' && c <= 'F') return c - 'A' + 10;
    return -1;
  };
  if (hex.size() % 2 != 0) throw Error(ErrorKind::kInvalidArgument, "hex string has odd length");
  std::string out;
  out.reserve(hex.size() / 2);
  for (size_t i = 0; i < hex.size(); i += 2) {
    const int hi = nibble(hex[i]), lo = nibble(hex[i + 1]);
    if (hi < 0 || lo < 0) throw Error(ErrorKind::kInvalidArgument, "invalid hex digit");
    out.push_back(static_cast<char>((hi << 4) | lo));
  }
  return out;
}

std::string DomainAddress::to_hex() const { return hex_encode(bytes_); }
DomainAddress DomainAddress::from_hex(const std::string& hex) { return DomainAddress(hex_decode(hex)); }

namespace {
void put_u32(std::string* s, uint32_t v) { s->append(reinterpret_cast<const char*>(&v), 4); }
void put_u64(std::string* s, uint64_t v) { s->append(reinterpret_cast<const char*>(&v), 8); }
template <typename T>
T get(const std::string& s, size_t* off) {
  if (*off + sizeof(T) > s.size()) throw Error(ErrorKind::kInvalidArgument, "truncated descriptor");
  T v;
  std::memcpy(&v, s.data() + *off, sizeof(T));
  *off += sizeof(T);
  return v;
}
constexpr uint32_t kDescMagic = 0x4453524d;  // "MRSD"
}  // namespace

std::string MemoryRegionDescriptor::serialize() const {
  std::string s;
  put_u32(&s, kDescMagic);
  put_u64(&s, ptr);
  put_u32(&s, static_cast<uint32_t>(addr_rkey_list.size()));
  for (const auto& [addr, rkey] : addr_rkey_list) {
    put_u32(&s, static_cast<uint32_t>(addr.bytes().size()));
    s.append(addr.bytes());
    put_u64(&s, rkey);
  }
  return s;
}

MemoryRegionDescriptor MemoryRegionDescriptor::deserialize(const std::string& bytes) {
  size_t off = 0;
  if (get<uint32_t>(bytes, &off) != kDescMagic) {
    throw Error(ErrorKind::kInvalidArgument, "not a memory region descriptor");
  }
  MemoryRegionDescriptor d;
  d.ptr = get<uint64_t>(bytes, &off);
  const uint32_t n = get<uint32_t>(bytes, &off);
  for (uint32_t i = 0; i < n; ++i) {
    const uint32_t len = get<uint32_t>(bytes, &off);
    if (off + len > bytes.size()) throw Error(ErrorKind::kInvalidArgument, "truncated descriptor");
    DomainAddress addr(bytes.substr(off, len));
    off += len;
    const uint64_t rkey = get<uint64_t>(bytes, &off);
    d.addr_rkey_list.emplace_back(std::move(addr), rkey);
  }
  return d;
}

std::string MemoryRegionDescriptor::debug_str() const {
  char buf[64];
  std::snprintf(buf, sizeof(buf), "MemoryRegionDescriptor(ptr=0x%llx, [",
                static_cast<unsigned long long>(ptr));
  std::string s = buf;
  for (size_t i = 0; i < addr_rkey_list.size(); ++i) {
    if (i) s += ", ";
    std::snprintf(buf, sizeof(buf), ":0x%llx",
                  static_cast<unsigned long long>(addr_rkey_list[i].second));
    s += addr_rkey_list[i].first.to_hex() + buf;
  }
  return s + "])";
}

bool ImmCounter::wait(uint32_t target, int64_t deadline_ms) const {
  // Take `target` arrivals out of the counter; if that drives it negative, wait until
  // later arrivals bring it back to zero or above.
  const int64_t old = counter_->fetch_sub(static_cast<int64_t>(target), std::memory_order_acq_rel);
  if (old >= static_cast<int64_t>(target)) return true;
  const auto start = std::chrono::steady_clock::now();
  uint32_t spins = 0;
  while (counter_->load(std::memory_order_acquire) < 0) {
    if (++spins % 1024 == 0) {
      if (deadline_ms >= 0 &&
          std::chrono::steady_clock::now() - start > std::chrono::milliseconds(deadline_ms)) {
        // give the arrivals back so that a retry sees a consistent count
        counter_->fetch_add(static_cast<int64_t>(target), std::memory_order_acq_rel);
        return false;
      }
      std::this_thread::yield();
    }
  }
  return true;
}

}  // namespace pplx::fabric
