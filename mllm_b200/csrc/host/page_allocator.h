// Slot allocator of the paged KV pool (host side).  Slots are token rows of the device pool; slot 0's
// page is reserved as the padding target of CUDA-graph batches.  With page_size > 1 allocation is in
// whole pages (the caller asks for a token count, gets page-aligned runs).  Frees inside a
// begin/end group are collected and merged once.
#pragma once
#include <cstdint>
#include <vector>

namespace mb200host {

class PageAllocator {
 public:
  PageAllocator(int64_t num_slots, int page_size);
  void clear();
  int64_t available() const;
  // n token slots taken from whole pages (the unused tail of the last page is not handed out); false
  // when they do not fit
  bool alloc(int64_t n, std::vector<int64_t>* out);
  void free_slots(const int64_t* slots, int64_t n);
  void group_begin();
  void group_end();
  int page_size() const { return page_size_; }
  int64_t num_slots() const { return num_slots_; }

 private:
  void release_pages(std::vector<int64_t>& pages);
  int64_t num_slots_;
  int page_size_;
  std::vector<int64_t> free_pages_;  // stack; back() is handed out next
  std::vector<int64_t> pending_;
  bool in_group_ = false;
};

}  // namespace mb200host
