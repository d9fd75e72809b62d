#include "shard.h"

#include <algorithm>

namespace pplx::fabric {

std::vector<std::pair<uint64_t, uint64_t>> shard_single_transfer(uint64_t total, size_t num_shards) {
  constexpr uint64_t kMinShard = 8192;
  std::vector<std::pair<uint64_t, uint64_t>> out;
  if (num_shards == 0) return out;
  const uint64_t per = (total / num_shards + kMinShard - 1) / kMinShard * kMinShard;
  uint64_t offset = 0;
  for (size_t i = 0; i < num_shards; ++i) {
    const uint64_t len = std::min(per, total - offset);
    if (len > 0) {
      out.emplace_back(offset, len);
      offset += len;
    } else {
      out.emplace_back(0, 0);
    }
  }
  // total / n rounded *down* before rounding up to 8 KiB can leave a tail: give it to the
  // last shard that carries bytes.
  if (offset < total) {
    for (size_t i = out.size(); i-- > 0;) {
      if (out[i].second > 0 || i == 0) {
        if (out[i].second == 0) out[i].first = offset;
        out[i].second += total - offset;
        break;
      }
    }
  }
  return out;
}

std::vector<std::pair<size_t, size_t>> shard_pages(size_t num_pages, size_t num_shards) {
  std::vector<std::pair<size_t, size_t>> out;
  if (num_shards == 0 || num_pages == 0) return out;
  const size_t base = num_pages / num_shards;
  size_t extra = num_pages % num_shards;
  size_t begin = 0;
  for (size_t i = 0; i < num_shards && begin < num_pages; ++i) {
    size_t n = base + (extra > 0 ? 1 : 0);
    if (extra > 0) --extra;
    if (n == 0) break;
    out.emplace_back(begin, begin + n);
    begin += n;
  }
  return out;
}

}  // namespace pplx::fabric
