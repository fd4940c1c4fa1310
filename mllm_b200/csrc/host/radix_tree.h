// Page-aligned radix tree over token ids for KV prefix reuse (host side).  Every edge stores a run
// of token ids (a multiple of page_size long) and the KV slot of each token.  Nodes carry a lock
// count (requests currently reading the prefix); eviction removes unlocked leaves in
// least-recently-used order and returns their slots.  Node handles are integer ids (0 = root).
#pragma once
#include <cstdint>
#include <memory>
#include <unordered_map>
#include <vector>

namespace mb200host {

struct RadixNode {
  int64_t id = 0;
  RadixNode* parent = nullptr;
  std::vector<int64_t> key;     // token ids of the edge leading here
  std::vector<int64_t> value;   // KV slots, same length
  std::unordered_map<int64_t, std::unique_ptr<RadixNode>> children;  // keyed by hash of the first page
  int lock_ref = 0;
  uint64_t last_access = 0;
};

struct RadixMatch {
  std::vector<int64_t> slots;
  int64_t node = 0;
};

class RadixTree {
 public:
  explicit RadixTree(int page_size);
  void reset();
  RadixMatch match_prefix(const int64_t* tokens, int64_t n, int64_t extra_key);
  // inserts tokens -> slots; returns the length of the prefix that was already present and, through
  // last_node, the node that ends the inserted sequence
  int64_t insert(const int64_t* tokens, const int64_t* slots, int64_t n, int64_t extra_key, int64_t* last_node);
  void inc_lock(int64_t node);
  void dec_lock(int64_t node);
  // frees at least num_tokens tokens of unlocked leaves (LRU first); returns their slots
  std::vector<int64_t> evict(int64_t num_tokens);
  int64_t evictable_size() const { return evictable_; }
  int64_t protected_size() const { return protected_; }
  int64_t total_size() const { return evictable_ + protected_; }
  int64_t num_nodes() const { return static_cast<int64_t>(by_id_.size()); }
  // (id, parent id, lock count, last access tick, edge tokens) of every node except the root
  struct NodeInfo {
    int64_t id, parent, lock_ref;
    uint64_t last_access;
    std::vector<int64_t> key;
  };
  std::vector<NodeInfo> dump() const;

 private:
  int64_t child_key(const int64_t* tokens, int64_t extra_key) const;
  int64_t common_prefix(const std::vector<int64_t>& a, const int64_t* b, int64_t nb) const;
  RadixNode* split(RadixNode* child, int64_t at, int64_t extra_key);
  RadixNode* new_node();
  int page_;
  std::unique_ptr<RadixNode> root_;
  std::unordered_map<int64_t, RadixNode*> by_id_;
  std::unordered_map<int64_t, int64_t> extra_of_;  // node id -> extra key of its namespace
  int64_t next_id_ = 1;
  uint64_t clock_ = 0;
  int64_t evictable_ = 0, protected_ = 0;
};

}  // namespace mb200host
