#include "host/page_allocator.h"

#include <algorithm>

namespace mb200host {

PageAllocator::PageAllocator(int64_t num_slots, int page_size) : num_slots_(num_slots), page_size_(page_size < 1 ? 1 : page_size) {
  clear();
}

void PageAllocator::clear() {
  const int64_t pages = num_slots_ / page_size_;
  free_pages_.clear();
  free_pages_.reserve(pages);
  // page 0 stays reserved; lowest pages are handed out first
  for (int64_t p = pages - 1; p >= 1; --p) free_pages_.push_back(p);
  pending_.clear();
  in_group_ = false;
}

int64_t PageAllocator::available() const { return static_cast<int64_t>(free_pages_.size() + pending_.size()) * page_size_; }

bool PageAllocator::alloc(int64_t n, std::vector<int64_t>* out) {
  out->clear();
  if (n <= 0) return true;
  const int64_t pages = (n + page_size_ - 1) / page_size_;
  if (static_cast<int64_t>(free_pages_.size()) < pages && !pending_.empty()) release_pages(pending_);
  if (static_cast<int64_t>(free_pages_.size()) < pages) return false;
  out->reserve(pages * page_size_);
  for (int64_t i = 0; i < pages; ++i) {
    const int64_t p = free_pages_.back();
    free_pages_.pop_back();
    for (int j = 0; j < page_size_; ++j) out->push_back(p * page_size_ + j);
  }
  out->resize(n);  // the tail of the last page stays with the caller's run but is not handed out
  return true;
}

void PageAllocator::release_pages(std::vector<int64_t>& pages) {
  std::sort(pages.begin(), pages.end());
  pages.erase(std::unique(pages.begin(), pages.end()), pages.end());
  // keep the stack ordered so that low pages come out first again
  free_pages_.insert(free_pages_.end(), pages.rbegin(), pages.rend());
  std::sort(free_pages_.begin(), free_pages_.end(), [](int64_t a, int64_t b) { return a > b; });
  free_pages_.erase(std::unique(free_pages_.begin(), free_pages_.end()), free_pages_.end());
  pages.clear();
}

void PageAllocator::free_slots(const int64_t* slots, int64_t n) {
  std::vector<int64_t> pages;
  pages.reserve(n / page_size_ + 1);
  for (int64_t i = 0; i < n; ++i) {
    if (slots[i] < page_size_) continue;  // the reserved page is never returned
    pages.push_back(slots[i] / page_size_);  // a page goes back as soon as any of its slots is freed
  }
  if (in_group_) {
    pending_.insert(pending_.end(), pages.begin(), pages.end());
  } else {
    release_pages(pages);
  }
}

void PageAllocator::group_begin() { in_group_ = true; }

void PageAllocator::group_end() {
  in_group_ = false;
  if (!pending_.empty()) release_pages(pending_);
}

}  // namespace mb200host
