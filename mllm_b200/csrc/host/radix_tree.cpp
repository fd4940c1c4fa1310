#include "host/radix_tree.h"

#include <algorithm>
#include <queue>
#include <stdexcept>

namespace mb200host {

RadixTree::RadixTree(int page_size) : page_(page_size < 1 ? 1 : page_size) { reset(); }

void RadixTree::reset() {
  root_ = std::make_unique<RadixNode>();
  root_->id = 0;
  root_->lock_ref = 1;  // the root is never evicted
  by_id_.clear();
  extra_of_.clear();
  by_id_[0] = root_.get();
  next_id_ = 1;
  clock_ = 0;
  evictable_ = protected_ = 0;
}

RadixNode* RadixTree::new_node() {
  auto* n = new RadixNode();
  n->id = next_id_++;
  by_id_[n->id] = n;
  return n;
}

// FNV-1a over the first page of tokens and the namespace key
int64_t RadixTree::child_key(const int64_t* tokens, int64_t extra_key) const {
  uint64_t h = 1469598103934665603ull ^ static_cast<uint64_t>(extra_key);
  for (int i = 0; i < page_; ++i) {
    h ^= static_cast<uint64_t>(tokens[i]);
    h *= 1099511628211ull;
  }
  return static_cast<int64_t>(h);
}

int64_t RadixTree::common_prefix(const std::vector<int64_t>& a, const int64_t* b, int64_t nb) const {
  const int64_t n = std::min<int64_t>(static_cast<int64_t>(a.size()), nb);
  int64_t i = 0;
  while (i < n && a[i] == b[i]) ++i;
  return i / page_ * page_;
}

RadixNode* RadixTree::split(RadixNode* child, int64_t at, int64_t extra_key) {
  // parent -> mid (first `at` tokens) -> child (rest)
  RadixNode* parent = child->parent;
  const int64_t old_key = child_key(child->key.data(), extra_key);
  std::unique_ptr<RadixNode> owned = std::move(parent->children[old_key]);
  RadixNode* mid = new_node();
  mid->parent = parent;
  mid->key.assign(child->key.begin(), child->key.begin() + at);
  mid->value.assign(child->value.begin(), child->value.begin() + at);
  mid->lock_ref = child->lock_ref;
  mid->last_access = child->last_access;
  child->key.erase(child->key.begin(), child->key.begin() + at);
  child->value.erase(child->value.begin(), child->value.begin() + at);
  child->parent = mid;
  mid->children[child_key(child->key.data(), extra_key)] = std::move(owned);
  parent->children[old_key] = std::unique_ptr<RadixNode>(mid);
  extra_of_[mid->id] = extra_key;
  return mid;
}

RadixMatch RadixTree::match_prefix(const int64_t* tokens, int64_t n, int64_t extra_key) {
  RadixMatch out;
  n = n / page_ * page_;
  RadixNode* node = root_.get();
  const uint64_t now = ++clock_;
  node->last_access = now;
  int64_t pos = 0;
  while (pos < n) {
    auto it = node->children.find(child_key(tokens + pos, extra_key));
    if (it == node->children.end()) break;
    RadixNode* child = it->second.get();
    const int64_t m = common_prefix(child->key, tokens + pos, n - pos);
    if (m == 0) break;
    // only the matched part of a partially matched edge counts as used
    if (m < static_cast<int64_t>(child->key.size())) child = split(child, m, extra_key);
    child->last_access = now;
    out.slots.insert(out.slots.end(), child->value.begin(), child->value.end());
    node = child;
    pos += m;
  }
  out.node = node->id;
  return out;
}

int64_t RadixTree::insert(const int64_t* tokens, const int64_t* slots, int64_t n, int64_t extra_key, int64_t* last_node) {
  n = n / page_ * page_;
  RadixNode* node = root_.get();
  const uint64_t now = ++clock_;
  int64_t pos = 0;
  while (pos < n) {
    auto it = node->children.find(child_key(tokens + pos, extra_key));
    if (it == node->children.end()) break;
    RadixNode* child = it->second.get();
    const int64_t m = common_prefix(child->key, tokens + pos, n - pos);
    if (m == 0) break;
    if (m < static_cast<int64_t>(child->key.size())) child = split(child, m, extra_key);
    child->last_access = now;
    node = child;
    pos += m;
  }
  const int64_t matched = pos;
  if (pos < n) {
    RadixNode* leaf = new_node();
    leaf->parent = node;
    leaf->key.assign(tokens + pos, tokens + n);
    leaf->value.assign(slots + pos, slots + n);
    leaf->last_access = now;
    node->children[child_key(tokens + pos, extra_key)] = std::unique_ptr<RadixNode>(leaf);
    extra_of_[leaf->id] = extra_key;
    evictable_ += n - pos;
    node = leaf;
  }
  if (last_node != nullptr) *last_node = node->id;
  return matched;
}

void RadixTree::inc_lock(int64_t id) {
  auto it = by_id_.find(id);
  if (it == by_id_.end()) throw std::invalid_argument("radix tree: unknown node");
  for (RadixNode* n = it->second; n != nullptr && n != root_.get(); n = n->parent) {
    if (n->lock_ref == 0) {
      evictable_ -= static_cast<int64_t>(n->key.size());
      protected_ += static_cast<int64_t>(n->key.size());
    }
    ++n->lock_ref;
  }
}

void RadixTree::dec_lock(int64_t id) {
  auto it = by_id_.find(id);
  if (it == by_id_.end()) throw std::invalid_argument("radix tree: unknown node");
  for (RadixNode* n = it->second; n != nullptr && n != root_.get(); n = n->parent) {
    if (n->lock_ref <= 0) throw std::logic_error("radix tree: lock count underflow");
    if (--n->lock_ref == 0) {
      evictable_ += static_cast<int64_t>(n->key.size());
      protected_ -= static_cast<int64_t>(n->key.size());
    }
  }
}

std::vector<RadixTree::NodeInfo> RadixTree::dump() const {
  std::vector<NodeInfo> out;
  for (const auto& kv : by_id_) {
    const RadixNode* n = kv.second;
    if (n == root_.get()) continue;
    out.push_back({n->id, n->parent->id, n->lock_ref, n->last_access, n->key});
  }
  std::sort(out.begin(), out.end(), [](const NodeInfo& a, const NodeInfo& b) { return a.id < b.id; });
  return out;
}

std::vector<int64_t> RadixTree::evict(int64_t num_tokens) {
  std::vector<int64_t> freed;
  using Item = std::pair<uint64_t, RadixNode*>;
  auto cmp = [](const Item& a, const Item& b) { return a.first > b.first; };
  std::priority_queue<Item, std::vector<Item>, decltype(cmp)> heap(cmp);
  for (auto& kv : by_id_) {
    RadixNode* n = kv.second;
    if (n != root_.get() && n->children.empty() && n->lock_ref == 0) heap.push({n->last_access, n});
  }
  while (static_cast<int64_t>(freed.size()) < num_tokens && !heap.empty()) {
    RadixNode* n = heap.top().second;
    heap.pop();
    freed.insert(freed.end(), n->value.begin(), n->value.end());
    evictable_ -= static_cast<int64_t>(n->key.size());
    RadixNode* parent = n->parent;
    const int64_t extra = extra_of_[n->id];
    const int64_t key = child_key(n->key.data(), extra);
    by_id_.erase(n->id);
    extra_of_.erase(n->id);
    parent->children.erase(key);  // destroys n
    if (parent != root_.get() && parent->children.empty() && parent->lock_ref == 0)
      heap.push({parent->last_access, parent});
  }
  return freed;
}

}  // namespace mb200host
