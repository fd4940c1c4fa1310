// Offset allocator of the symmetric heap: one peer-mapped device allocation per rank, carved into
// buffers by this host-side allocator.  It hands out offsets, never pointers, and is deterministic
// (first fit by address, fixed alignment rounding), so ranks that make the same calls in the same
// order get the same offsets: a buffer's address on rank r is that rank's heap base plus the offset,
// and one rendezvous of the heap replaces one per buffer.
#pragma once
#include <cstdint>
#include <map>

namespace mb200host {

class SymmHeapAllocator {
 public:
  explicit SymmHeapAllocator(int64_t capacity, int64_t min_align = 256);
  // offset of a block of at least `bytes` bytes aligned to max(align, min_align) (a power of two);
  // -1 when no free range fits
  int64_t alloc(int64_t bytes, int64_t align = 0);
  // returns the block that starts at `offset` (as given by alloc); false if there is none
  bool free_block(int64_t offset);
  void reset();
  int64_t capacity() const { return capacity_; }
  int64_t used() const { return used_; }
  int64_t largest_free() const;
  int64_t num_blocks() const { return static_cast<int64_t>(blocks_.size()); }
  int64_t block_size(int64_t offset) const;

 private:
  int64_t capacity_, min_align_, used_ = 0;
  std::map<int64_t, int64_t> free_;    // start -> length, non-adjacent
  std::map<int64_t, int64_t> blocks_;  // start -> length of live blocks (start is what alloc returned)
};

}  // namespace mb200host
