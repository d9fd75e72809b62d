// Pure arithmetic for spreading one transfer over several domains (NICs / copy queues).
// Reference: fabric-lib/src/domain_group.rs:209-359,555-595.
#pragma once

#include <cstddef>
#include <cstdint>
#include <utility>
#include <vector>

namespace pplx::fabric {

// Splits `total` bytes into exactly `num_shards` (offset, length) ranges whose lengths are
// multiples of 8 KiB except the last non-empty one. Shards left without bytes are (0, 0):
// a zero-length write must not carry an offset that may sit at the very end of a region.
std::vector<std::pair<uint64_t, uint64_t>> shard_single_transfer(uint64_t total, size_t num_shards);

// Splits `num_pages` page indices into at most `num_shards` contiguous [begin, end) runs of
// nearly equal size (earlier runs get the remainder); empty runs are dropped.
std::vector<std::pair<size_t, size_t>> shard_pages(size_t num_pages, size_t num_shards);

}  // namespace pplx::fabric
