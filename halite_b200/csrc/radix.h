// Host-side serving runtime: a page allocator and a page-granular radix (prefix) tree over token
// ids. Native counterpart of the engine's Python scheduler data structures (the reference keeps
// these in Python: infer/engine/radix_cache.py, infer/engine/memory_pool.py,
// tokainfer/engine/allocator.py). No CUDA here: the tree only hands out page ids.
#pragma once

#include <cstdint>
#include <deque>
#include <unordered_map>
#include <vector>

namespace hb {

class PageAllocator {
 public:
  explicit PageAllocator(int num_pages);           // pages 1..num_pages (0 is the scratch page)
  // Appends n page ids to `out`; returns false (and appends nothing) when fewer are free.
  bool alloc(int n, std::vector<int32_t>& out);
  void free(const std::vector<int32_t>& pages);
  int available() const { return static_cast<int>(free_.size()); }
  int capacity() const { return num_pages_; }
  void clear();

 private:
  int num_pages_;
  std::vector<int32_t> free_;
};

class RadixTree {
 public:
  explicit RadixTree(int page_size);
  void reset();

  // Longest cached prefix in whole pages. Splits a node when the match ends inside it, so the
  // returned node covers exactly the match. Returns the node handle (0 = root).
  int64_t match_prefix(const std::vector<int32_t>& tokens, std::vector<int32_t>& pages_out);
  // Insert whole pages (tokens.size() == pages.size() * page_size). Returns how many leading
  // pages were already cached.
  int insert(const std::vector<int32_t>& tokens, const std::vector<int32_t>& pages);
  void inc_lock_ref(int64_t node);
  void dec_lock_ref(int64_t node);
  // Evict unlocked leaves, least recently used first, until at least n_pages are freed (or
  // nothing evictable is left). Freed page ids are appended to `freed`.
  int evict(int n_pages, std::vector<int32_t>& freed);

  int64_t evictable_pages() const { return evictable_; }
  int64_t protected_pages() const { return protected_; }
  int64_t total_pages() const;
  int64_t node_count() const { return static_cast<int64_t>(live_); }
  int page_size() const { return page_size_; }
  // Throws std::runtime_error when an invariant is broken (tests).
  void sanity_check() const;

 private:
  struct Node {
    int64_t parent = -1;
    std::vector<int32_t> key;     // tokens, size % page_size == 0
    std::vector<int32_t> value;   // page ids
    std::unordered_map<uint64_t, std::vector<int64_t>> children;   // hash of first page -> candidates
    int lock_ref = 0;
    uint64_t last_access = 0;
    bool alive = false;
  };

  uint64_t page_hash(const int32_t* tokens) const;
  int64_t find_child(const Node& node, const int32_t* tokens) const;
  void add_child(int64_t parent, int64_t child);
  void remove_child(int64_t parent, int64_t child);
  int match_pages(const Node& node, const std::vector<int32_t>& tokens, size_t start) const;
  int64_t split(int64_t child, int n_pages);
  int64_t new_node();

  int page_size_;
  std::deque<Node> nodes_;
  std::vector<int64_t> free_nodes_;
  int64_t evictable_ = 0, protected_ = 0;
  size_t live_ = 0;
  uint64_t clock_ = 0;
};

}  // namespace hb
