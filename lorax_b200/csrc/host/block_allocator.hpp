// Paged-KV block bookkeeping of the router.
//
// Behaviour follows the reference router (router/src/block_allocator.rs:146-216 and router/src/radix.rs):
//   * block 0 is reserved (health checks run a one-token prefill on it);
//   * a request needs ceil(tokens / block_size) blocks; with a sliding window only ceil(window / block_size) + 1
//     blocks are held and the slot list cycles over them;
//   * with prefix caching a radix trie -- one root per adapter index, because the KV of the same text differs per
//     adapter -- maps whole blocks of prompt tokens to cached blocks, with reference counts and LRU eviction of
//     unreferenced leaves.
// Not thread safe: the scheduler thread owns it.
#pragma once
#include <algorithm>
#include <cstdint>
#include <map>
#include <memory>
#include <optional>
#include <unordered_map>
#include <vector>

namespace lx {

struct BlockAllocation {
  uint64_t allocation_id = 0;
  std::vector<uint32_t> blocks;
  std::vector<uint32_t> slots;
  uint32_t prefix_len = 0;       // prompt tokens already cached (multiple of block_size)
};

class Allocator {
 public:
  virtual ~Allocator() = default;
  virtual std::optional<BlockAllocation> allocate(uint32_t adapter_index, uint32_t tokens,
                                                  const std::vector<uint32_t>* prefill_tokens) = 0;
  virtual void free(const BlockAllocation& a, uint32_t adapter_index, const std::vector<uint32_t>* all_tokens) = 0;
  virtual size_t free_blocks() const = 0;
};

class SimpleAllocator : public Allocator {
 public:
  SimpleAllocator(uint32_t num_blocks, uint32_t block_size, std::optional<uint32_t> window)
      : block_size_(block_size), window_(window) {
    for (uint32_t b = num_blocks; b-- > 1;) free_.push_back(b);   // block 0 reserved; low ids handed out first
  }
  std::optional<BlockAllocation> allocate(uint32_t, uint32_t tokens, const std::vector<uint32_t>*) override {
    uint32_t required = (tokens + block_size_ - 1) / block_size_;
    uint32_t repeats = 1;
    if (window_) {
      uint32_t tok = std::min(tokens, *window_);
      uint32_t req_w = (tok + block_size_ - 1) / block_size_ + (tokens > *window_ ? 1 : 0);
      repeats = (required + req_w - 1) / std::max(req_w, 1u);
      required = req_w;
    }
    if (required > free_.size()) return std::nullopt;
    BlockAllocation a;
    a.allocation_id = ++next_id_;
    for (uint32_t i = 0; i < required; ++i) { a.blocks.push_back(free_.back()); free_.pop_back(); }
    a.slots.reserve(tokens);
    for (uint32_t rep = 0; rep < repeats && a.slots.size() < tokens; ++rep)
      for (uint32_t b : a.blocks)
        for (uint32_t s = 0; s < block_size_ && a.slots.size() < tokens; ++s) a.slots.push_back(b * block_size_ + s);
    return a;
  }
  void free(const BlockAllocation& a, uint32_t, const std::vector<uint32_t>*) override {
    for (auto it = a.blocks.rbegin(); it != a.blocks.rend(); ++it) free_.push_back(*it);
  }
  size_t free_blocks() const override { return free_.size(); }

 private:
  uint32_t block_size_;
  std::optional<uint32_t> window_;
  std::vector<uint32_t> free_;
  uint64_t next_id_ = 0;
};

// ------------------------------------------------------------------------------------------------ radix
class RadixAllocator : public Allocator {
  struct Node {
    std::vector<uint32_t> key;                       // tokens of this edge (multiple of block_size)
    std::vector<uint32_t> blocks;                    // one per block_size tokens of key
    std::map<uint32_t, std::unique_ptr<Node>> children;   // keyed by the first token of the child's edge... of its first block hash
    Node* parent = nullptr;
    uint32_t ref_count = 0;
    uint64_t last_access = 0;
  };
  struct Live {
    Node* prefix_node = nullptr;     // deepest node referenced by the allocation
    uint32_t cached_blocks = 0;      // leading blocks owned by the trie, not by the allocation
  };

 public:
  RadixAllocator(uint32_t num_blocks, uint32_t block_size) : block_size_(block_size) {
    for (uint32_t b = num_blocks; b-- > 1;) free_.push_back(b);
  }

  std::optional<BlockAllocation> allocate(uint32_t adapter_index, uint32_t tokens, const std::vector<uint32_t>* prefill) override {
    ++clock_;
    Node* root = root_for(adapter_index);
    BlockAllocation a;
    Node* node = root;
    std::vector<uint32_t> cached;
    if (prefill != nullptr) {
      // never match the whole prompt: at least one token must be prefilled to produce logits
      size_t max_match = prefill->empty() ? 0 : ((prefill->size() - 1) / block_size_) * block_size_;
      node = match(root, *prefill, max_match, cached);
    }
    const uint32_t total_blocks = (tokens + block_size_ - 1) / block_size_;
    const uint32_t need = total_blocks > cached.size() ? total_blocks - (uint32_t)cached.size() : 0;
    // hold the matched path before evicting, so eviction cannot take it
    for (Node* n = node; n != nullptr && n != root; n = n->parent) { n->ref_count++; n->last_access = clock_; }
    if (need > free_.size() && !evict(need - free_.size())) {
      for (Node* n = node; n != nullptr && n != root; n = n->parent) n->ref_count--;
      return std::nullopt;
    }
    a.allocation_id = ++next_id_;
    a.blocks = cached;
    for (uint32_t i = 0; i < need; ++i) { a.blocks.push_back(free_.back()); free_.pop_back(); }
    a.prefix_len = (uint32_t)cached.size() * block_size_;
    a.slots.reserve(tokens);
    for (uint32_t b : a.blocks)
      for (uint32_t s = 0; s < block_size_ && a.slots.size() < tokens; ++s) a.slots.push_back(b * block_size_ + s);
    live_[a.allocation_id] = Live{node, (uint32_t)cached.size()};
    return a;
  }

  // all_tokens: prompt + generated tokens whose KV is in the cache; their whole blocks become reusable prefixes.
  void free(const BlockAllocation& a, uint32_t adapter_index, const std::vector<uint32_t>* all_tokens) override {
    ++clock_;
    auto it = live_.find(a.allocation_id);
    if (it == live_.end()) return;
    Live lv = it->second;
    live_.erase(it);
    Node* root = root_for(adapter_index);
    for (Node* n = lv.prefix_node; n != nullptr && n != root; n = n->parent) if (n->ref_count > 0) n->ref_count--;
    size_t inserted_upto = lv.cached_blocks;
    if (all_tokens != nullptr) {
      size_t full = std::min(all_tokens->size() / block_size_, a.blocks.size());
      if (full > lv.cached_blocks) inserted_upto = insert(root, *all_tokens, a.blocks, full);
    }
    // blocks not adopted by the trie go back to the free list (also duplicates of blocks another request cached first)
    for (size_t i = lv.cached_blocks; i < a.blocks.size(); ++i) {
      if (i < inserted_upto && adopted_.count(a.blocks[i])) continue;
      free_.push_back(a.blocks[i]);
    }
  }
  size_t free_blocks() const override { return free_.size(); }
  size_t cached_blocks() const { return adopted_.size(); }

 private:
  Node* root_for(uint32_t adapter) {
    auto& r = roots_[adapter];
    if (!r) r = std::make_unique<Node>();
    return r.get();
  }
  // Walk the trie along `tokens` (at most max_match tokens); appends the blocks of the matched prefix.
  Node* match(Node* root, const std::vector<uint32_t>& tokens, size_t max_match, std::vector<uint32_t>& blocks) {
    Node* node = root;
    size_t pos = 0;
    while (pos + block_size_ <= max_match) {
      auto it = node->children.find(tokens[pos]);
      if (it == node->children.end()) break;
      Node* child = it->second.get();
      size_t common = 0;
      size_t limit = std::min(child->key.size(), max_match - pos);
      while (common < limit && child->key[common] == tokens[pos + common]) ++common;
      common = common / block_size_ * block_size_;
      if (common == 0) break;
      if (common < child->key.size()) child = split(child, common);
      for (uint32_t b : child->blocks) blocks.push_back(b);
      pos += common;
      node = child;
    }
    return node;
  }
  // Split `child` so that a NEW node holding its first `len` tokens sits between it and its parent; `child` itself keeps
  // the rest of the edge.  Live allocations point at `child` and release their references by walking up from it, so the
  // node they know must stay the deepest part; the new head starts with the same count because every one of those walks
  // passes through it.  Returns the head.
  Node* split(Node* child, size_t len) {
    Node* parent = child->parent;
    const uint32_t first = child->key[0];
    std::unique_ptr<Node> owned = std::move(parent->children[first]);
    auto head = std::make_unique<Node>();
    head->key.assign(child->key.begin(), child->key.begin() + len);
    head->blocks.assign(child->blocks.begin(), child->blocks.begin() + len / block_size_);
    head->parent = parent;
    head->ref_count = child->ref_count;
    head->last_access = child->last_access;
    child->key.erase(child->key.begin(), child->key.begin() + len);
    child->blocks.erase(child->blocks.begin(), child->blocks.begin() + len / block_size_);
    child->parent = head.get();
    Node* raw = head.get();
    head->children[child->key[0]] = std::move(owned);
    parent->children[first] = std::move(head);
    return raw;
  }
  // Insert the first `full` blocks of a finished sequence.  Returns how many leading blocks are now owned by the trie
  // (either adopted from this allocation or already present from another one).
  size_t insert(Node* root, const std::vector<uint32_t>& tokens, const std::vector<uint32_t>& blocks, size_t full) {
    Node* node = root;
    size_t pos = 0;
    const size_t end = full * block_size_;
    while (pos < end) {
      auto it = node->children.find(tokens[pos]);
      if (it == node->children.end()) {
        auto leaf = std::make_unique<Node>();
        leaf->key.assign(tokens.begin() + pos, tokens.begin() + end);
        leaf->blocks.assign(blocks.begin() + pos / block_size_, blocks.begin() + full);
        leaf->parent = node;
        leaf->last_access = clock_;
        for (uint32_t b : leaf->blocks) adopted_.insert({b, true});
        node->children[tokens[pos]] = std::move(leaf);
        return full;
      }
      Node* child = it->second.get();
      size_t common = 0;
      size_t limit = std::min(child->key.size(), end - pos);
      while (common < limit && child->key[common] == tokens[pos + common]) ++common;
      common = common / block_size_ * block_size_;
      if (common == 0) return pos / block_size_;       // diverges inside the first block: nothing more to share
      if (common < child->key.size()) child = split(child, common);
      child->last_access = clock_;
      pos += common;
      node = child;
    }
    return full;
  }
  // Drop unreferenced leaves, least recently used first, until `need` blocks were released.
  bool evict(size_t need) {
    size_t released = 0;
    while (released < need) {
      Node* victim = nullptr;
      for (auto& r : roots_) find_lru_leaf(r.second.get(), r.second.get(), victim);
      if (victim == nullptr) return false;
      for (uint32_t b : victim->blocks) { free_.push_back(b); adopted_.erase(b); ++released; }
      Node* parent = victim->parent;
      parent->children.erase(victim->key[0]);
    }
    return true;
  }
  void find_lru_leaf(Node* n, Node* root, Node*& best) {
    if (n != root && n->children.empty() && n->ref_count == 0) {
      if (best == nullptr || n->last_access < best->last_access) best = n;
      return;
    }
    for (auto& kv : n->children) find_lru_leaf(kv.second.get(), root, best);
  }

  uint32_t block_size_;
  std::vector<uint32_t> free_;
  std::unordered_map<uint32_t, std::unique_ptr<Node>> roots_;
  std::unordered_map<uint64_t, Live> live_;
  std::unordered_map<uint32_t, bool> adopted_;      // blocks owned by the trie
  uint64_t next_id_ = 0;
  uint64_t clock_ = 0;
};

inline std::unique_ptr<Allocator> make_allocator(uint32_t num_blocks, uint32_t block_size, std::optional<uint32_t> window,
                                                 bool prefix_caching) {
  if (prefix_caching) return std::make_unique<RadixAllocator>(num_blocks, block_size);
  return std::make_unique<SimpleAllocator>(num_blocks, block_size, window);
}

}  // namespace lx
