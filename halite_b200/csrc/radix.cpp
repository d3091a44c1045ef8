#include "radix.h"

#include <algorithm>
#include <queue>
#include <stdexcept>
#include <string>

namespace hb {

// ------------------------------------------------------------------ PageAllocator
PageAllocator::PageAllocator(int num_pages) : num_pages_(num_pages) { clear(); }

void PageAllocator::clear() {
  free_.resize(num_pages_);
  // hand out low page ids first (the back of the vector is popped first)
  for (int i = 0; i < num_pages_; ++i) free_[i] = num_pages_ - i;
}

bool PageAllocator::alloc(int n, std::vector<int32_t>& out) {
  if (n < 0 || n > static_cast<int>(free_.size())) return false;
  out.insert(out.end(), free_.end() - n, free_.end());
  free_.resize(free_.size() - n);
  return true;
}

void PageAllocator::free(const std::vector<int32_t>& pages) { free_.insert(free_.end(), pages.begin(), pages.end()); }

// ------------------------------------------------------------------ RadixTree
RadixTree::RadixTree(int page_size) : page_size_(page_size) {
  if (page_size <= 0) throw std::invalid_argument("page_size must be positive");
  reset();
}

void RadixTree::reset() {
  nodes_.clear();
  free_nodes_.clear();
  nodes_.emplace_back();
  nodes_[0].alive = true;
  nodes_[0].lock_ref = 1;
  evictable_ = protected_ = 0;
  live_ = 1;
  clock_ = 0;
}

int64_t RadixTree::new_node() {
  int64_t id;
  if (!free_nodes_.empty()) {
    id = free_nodes_.back();
    free_nodes_.pop_back();
    nodes_[id] = Node();
  } else {
    id = static_cast<int64_t>(nodes_.size());
    nodes_.emplace_back();
  }
  nodes_[id].alive = true;
  ++live_;
  return id;
}

uint64_t RadixTree::page_hash(const int32_t* t) const {
  uint64_t h = 1469598103934665603ull;            // FNV-1a over the page's tokens
  for (int i = 0; i < page_size_; ++i) {
    h ^= static_cast<uint32_t>(t[i]);
    h *= 1099511628211ull;
  }
  return h;
}

int64_t RadixTree::find_child(const Node& node, const int32_t* tokens) const {
  auto it = node.children.find(page_hash(tokens));
  if (it == node.children.end()) return -1;
  for (int64_t c : it->second)
    if (std::equal(tokens, tokens + page_size_, nodes_[c].key.begin())) return c;
  return -1;
}

void RadixTree::add_child(int64_t parent, int64_t child) {
  nodes_[parent].children[page_hash(nodes_[child].key.data())].push_back(child);
  nodes_[child].parent = parent;
}

void RadixTree::remove_child(int64_t parent, int64_t child) {
  auto& map = nodes_[parent].children;
  auto it = map.find(page_hash(nodes_[child].key.data()));
  if (it == map.end()) return;
  auto& v = it->second;
  v.erase(std::remove(v.begin(), v.end(), child), v.end());
  if (v.empty()) map.erase(it);
}

int RadixTree::match_pages(const Node& node, const std::vector<int32_t>& tokens, size_t start) const {
  const size_t ps = page_size_;
  const size_t limit = std::min(node.key.size(), (tokens.size() - start) / ps * ps);
  size_t n = 0;
  while (n < limit && std::equal(node.key.begin() + n, node.key.begin() + n + ps, tokens.begin() + start + n)) n += ps;
  return static_cast<int>(n / ps);
}

int64_t RadixTree::split(int64_t child_id, int n_pages) {
  const size_t cut = static_cast<size_t>(n_pages) * page_size_;
  const int64_t parent = nodes_[child_id].parent;
  remove_child(parent, child_id);
  const int64_t upper = new_node();
  Node& c = nodes_[child_id];
  Node& u = nodes_[upper];
  u.key.assign(c.key.begin(), c.key.begin() + cut);
  u.value.assign(c.value.begin(), c.value.begin() + n_pages);
  u.lock_ref = c.lock_ref;
  u.last_access = c.last_access;
  c.key.erase(c.key.begin(), c.key.begin() + cut);
  c.value.erase(c.value.begin(), c.value.begin() + n_pages);
  add_child(parent, upper);
  add_child(upper, child_id);
  return upper;
}

int64_t RadixTree::match_prefix(const std::vector<int32_t>& tokens, std::vector<int32_t>& pages) {
  int64_t node = 0;
  size_t pos = 0;
  const uint64_t now = ++clock_;
  while (tokens.size() - pos >= static_cast<size_t>(page_size_)) {
    int64_t child = find_child(nodes_[node], tokens.data() + pos);
    if (child < 0) break;
    nodes_[child].last_access = now;
    const int n = match_pages(nodes_[child], tokens, pos);
    if (static_cast<size_t>(n) * page_size_ < nodes_[child].key.size()) {
      child = split(child, n);
      pages.insert(pages.end(), nodes_[child].value.begin(), nodes_[child].value.end());
      return child;
    }
    pages.insert(pages.end(), nodes_[child].value.begin(), nodes_[child].value.end());
    pos += nodes_[child].key.size();
    node = child;
  }
  return node;
}

int RadixTree::insert(const std::vector<int32_t>& tokens, const std::vector<int32_t>& pages) {
  const size_t ps = page_size_;
  if (tokens.size() != pages.size() * ps) throw std::invalid_argument("insert: tokens must cover whole pages");
  int64_t node = 0;
  size_t pos = 0;
  int shared = 0;
  const uint64_t now = ++clock_;
  while (pos < tokens.size()) {
    int64_t child = find_child(nodes_[node], tokens.data() + pos);
    if (child < 0) {
      const int64_t fresh = new_node();
      Node& f = nodes_[fresh];
      f.key.assign(tokens.begin() + pos, tokens.end());
      f.value.assign(pages.begin() + pos / ps, pages.end());
      f.last_access = now;
      add_child(node, fresh);
      evictable_ += static_cast<int64_t>(f.value.size());
      break;
    }
    nodes_[child].last_access = now;
    const int n = match_pages(nodes_[child], tokens, pos);
    if (static_cast<size_t>(n) * ps < nodes_[child].key.size()) child = split(child, n);
    shared += n;
    pos += static_cast<size_t>(n) * ps;
    node = child;
  }
  return shared;
}

void RadixTree::inc_lock_ref(int64_t node) {
  while (node > 0) {
    Node& n = nodes_[node];
    if (n.lock_ref == 0) {
      evictable_ -= static_cast<int64_t>(n.value.size());
      protected_ += static_cast<int64_t>(n.value.size());
    }
    ++n.lock_ref;
    node = n.parent;
  }
}

void RadixTree::dec_lock_ref(int64_t node) {
  while (node > 0) {
    Node& n = nodes_[node];
    if (n.lock_ref == 1) {
      evictable_ += static_cast<int64_t>(n.value.size());
      protected_ -= static_cast<int64_t>(n.value.size());
    }
    --n.lock_ref;
    node = n.parent;
  }
}

int RadixTree::evict(int n_pages, std::vector<int32_t>& freed) {
  if (n_pages <= 0) return 0;
  using Entry = std::pair<uint64_t, int64_t>;      // (last access, node): oldest first
  std::priority_queue<Entry, std::vector<Entry>, std::greater<Entry>> heap;
  for (int64_t i = 1; i < static_cast<int64_t>(nodes_.size()); ++i) {
    const Node& n = nodes_[i];
    if (n.alive && n.children.empty() && n.lock_ref == 0) heap.emplace(n.last_access, i);
  }
  int count = 0;
  while (count < n_pages && !heap.empty()) {
    const int64_t id = heap.top().second;
    heap.pop();
    Node& n = nodes_[id];
    if (!n.alive || n.lock_ref > 0 || !n.children.empty()) continue;
    freed.insert(freed.end(), n.value.begin(), n.value.end());
    count += static_cast<int>(n.value.size());
    evictable_ -= static_cast<int64_t>(n.value.size());
    const int64_t parent = n.parent;
    remove_child(parent, id);
    n.alive = false;
    n.key.clear();
    n.value.clear();
    free_nodes_.push_back(id);
    --live_;
    const Node& p = nodes_[parent];
    if (parent > 0 && p.children.empty() && p.lock_ref == 0) heap.emplace(p.last_access, parent);
  }
  return count;
}

int64_t RadixTree::total_pages() const {
  int64_t n = 0;
  for (const Node& x : nodes_)
    if (x.alive) n += static_cast<int64_t>(x.value.size());
  return n;
}

void RadixTree::sanity_check() const {
  int64_t ev = 0, pr = 0;
  for (int64_t i = 1; i < static_cast<int64_t>(nodes_.size()); ++i) {
    const Node& n = nodes_[i];
    if (!n.alive) continue;
    if (n.value.empty() || n.key.size() != n.value.size() * page_size_)
      throw std::runtime_error("node " + std::to_string(i) + ": key/value sizes disagree");
    if (n.lock_ref < 0) throw std::runtime_error("negative lock count");
    if (n.parent < 0 || !nodes_[n.parent].alive) throw std::runtime_error("dangling parent");
    if (find_child(nodes_[n.parent], n.key.data()) != i) throw std::runtime_error("parent does not index the child");
    if (n.parent > 0 && n.lock_ref > 0 && nodes_[n.parent].lock_ref < n.lock_ref)
      throw std::runtime_error("child locked more often than its parent");
    (n.lock_ref == 0 ? ev : pr) += static_cast<int64_t>(n.value.size());
  }
  if (ev != evictable_ || pr != protected_) throw std::runtime_error("page counters out of sync");
}

}  // namespace hb
