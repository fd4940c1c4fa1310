#include "symm_heap.h"

#include <algorithm>
#include <stdexcept>

namespace mb200host {

namespace {
inline int64_t round_up(int64_t v, int64_t a) { return (v + a - 1) / a * a; }
inline bool is_pow2(int64_t v) { return v > 0 && (v & (v - 1)) == 0; }
}  // namespace

SymmHeapAllocator::SymmHeapAllocator(int64_t capacity, int64_t min_align) : capacity_(capacity), min_align_(min_align) {
  if (capacity <= 0 || !is_pow2(min_align)) throw std::invalid_argument("SymmHeapAllocator: bad capacity or alignment");
  reset();
}

void SymmHeapAllocator::reset() {
  free_.clear();
  blocks_.clear();
  free_[0] = capacity_;
  used_ = 0;
}

int64_t SymmHeapAllocator::alloc(int64_t bytes, int64_t align) {
  if (bytes <= 0) return -1;
  if (align <= 0) align = min_align_;
  if (!is_pow2(align)) throw std::invalid_argument("SymmHeapAllocator: alignment must be a power of two");
  align = std::max(align, min_align_);
  const int64_t need = round_up(bytes, min_align_);
  for (auto it = free_.begin(); it != free_.end(); ++it) {
    const int64_t start = it->first, len = it->second;
    const int64_t at = round_up(start, align);
    if (at + need > start + len) continue;
    // split the range: [start, at) stays free, [at, at+need) is the block, the tail stays free
    const int64_t tail = start + len - (at + need);
    free_.erase(it);
    if (at > start) free_[start] = at - start;
    if (tail > 0) free_[at + need] = tail;
    blocks_[at] = need;
    used_ += need;
    return at;
  }
  return -1;
}

bool SymmHeapAllocator::free_block(int64_t offset) {
  auto b = blocks_.find(offset);
  if (b == blocks_.end()) return false;
  int64_t start = b->first, len = b->second;
  blocks_.erase(b);
  used_ -= len;
  // merge with the free range that follows and the one that precedes
  auto next = free_.lower_bound(start);
  if (next != free_.end() && next->first == start + len) {
    len += next->second;
    next = free_.erase(next);
  }
  if (next != free_.begin()) {
    auto prev = std::prev(next);
    if (prev->first + prev->second == start) {
      start = prev->first;
      len += prev->second;
      free_.erase(prev);
    }
  }
  free_[start] = len;
  return true;
}

int64_t SymmHeapAllocator::largest_free() const {
  int64_t best = 0;
  for (const auto& kv : free_) best = std::max(best, kv.second);
  return best;
}

int64_t SymmHeapAllocator::block_size(int64_t offset) const {
  auto b = blocks_.find(offset);
  return b == blocks_.end() ? -1 : b->second;
}

}  // namespace mb200host
