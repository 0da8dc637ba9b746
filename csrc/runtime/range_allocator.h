// First-fit allocator over a byte range with coalescing frees. Pure bookkeeping (no device calls):
// every rank runs the same sequence of alloc / free calls and therefore gets the same offsets,
// which is what makes a buffer addressable on any peer as base[r] + offset.
#pragma once
#include <cstddef>
#include <map>
#include <stdexcept>
#include <string>

namespace fastb {

class RangeAllocator {
 public:
  static constexpr size_t kAlign = 256;
  explicit RangeAllocator(size_t bytes = 0) : bytes_(bytes) {
    if (bytes) free_[0] = bytes;
  }
  size_t capacity() const { return bytes_; }
  size_t in_use() const { return in_use_; }
  size_t live_blocks() const { return taken_.size(); }

  // Offsets are multiples of 256 B; a zero-byte request still gets its own block.
  size_t alloc(size_t bytes) {
    const size_t need = (bytes + kAlign - 1) / kAlign * kAlign + (bytes == 0 ? kAlign : 0);
    for (auto it = free_.begin(); it != free_.end(); ++it) {
      if (it->second < need) continue;
      const size_t off = it->first, left = it->second - need;
      free_.erase(it);
      if (left) free_[off + need] = left;
      taken_[off] = need;
      in_use_ += need;
      return off;
    }
    throw std::runtime_error("out of symmetric memory (asked " + std::to_string(bytes) + " B, in use " + std::to_string(in_use_) + " of " +
                             std::to_string(bytes_) + ")");
  }

  void free(size_t offset) {
    auto it = taken_.find(offset);
    if (it == taken_.end()) throw std::invalid_argument("free of an unknown offset");
    size_t off = it->first, sz = it->second;
    taken_.erase(it);
    in_use_ -= sz;
    auto next = free_.lower_bound(off);
    if (next != free_.end() && off + sz == next->first) { sz += next->second; next = free_.erase(next); }
    if (next != free_.begin()) {
      auto prev = std::prev(next);
      if (prev->first + prev->second == off) { prev->second += sz; return; }
    }
    free_[off] = sz;
  }

  // True when the free list is one block spanning everything (nothing leaked, fully coalesced).
  bool pristine() const { return taken_.empty() && (bytes_ == 0 || (free_.size() == 1 && free_.begin()->second == bytes_)); }

 private:
  size_t bytes_ = 0, in_use_ = 0;
  std::map<size_t, size_t> free_;   // offset -> size
  std::map<size_t, size_t> taken_;  // offset -> size
};

}  // namespace fastb
