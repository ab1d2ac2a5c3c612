// Paged-KV block manager with a radix prefix cache.
//
// The device holds one page pool per layer ([num_pages, 2, kv_heads, page_size, head_dim]); this
// class owns the page ids: a free list, per-page reference counts and generation counters, an LRU
// list of unreferenced pages that still hold a cached prefix, and a trie over whole pages of prompt
// tokens. Sharing is page-granular: a new request reuses the longest run of full pages whose tokens
// match, never a partially filled page (it would have to write into it), and never its whole prompt
// (at least one token must be computed to produce logits). A page enters the trie only once its
// KV has been computed (`mark_computed`, called as prefill chunks finish), so a second request with
// the same prefix can never attend over pages that are reserved but still empty; a request that is
// dropped after a failed step takes its unshared pages out of the cache (`release(id, true)`).
//
// Role of the reference's PagedKVAllocator + RadixPrefixTree (crates/skein_runtime/src/kv/
// allocator.rs:17-308, radix.rs:18-130): same admit / advance / release life cycle, refcounts,
// generation check against stale trie entries and LRU eviction; block tables are handed to the
// kernels instead of assembling contiguous host buffers (kv/paged_cache.rs:30-370).
#pragma once
#include <algorithm>
#include <cstdint>
#include <deque>
#include <list>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

namespace skein {

struct RuntimeError : std::runtime_error { using std::runtime_error::runtime_error; };

struct PageTable {
  uint64_t request_id = 0;
  std::vector<int32_t> pages;
  uint32_t num_tokens = 0;          // tokens whose KV is (or is about to be) in the cache
  uint32_t prefix_hit_tokens = 0;   // tokens served from the prefix cache at admission
  uint32_t registered_pages = 0;    // leading pages that are entered in the trie
  bool no_register = false;         // the prefix cache was cleared while this request was in flight
};

class RadixPrefixTree {
 public:
  RadixPrefixTree(uint32_t page_size, uint32_t max_depth_tokens) : ps_(page_size), max_pages_(max_depth_tokens / page_size) { root_ = std::make_unique<Node>(); }

  // Longest run of full pages of `tokens` present in the trie with a matching page generation.
  // Returns the matched page ids; stale entries (generation mismatch) end the match and are pruned.
  std::vector<int32_t> lookup(const std::vector<int32_t>& tokens, const std::vector<uint64_t>& generations, size_t max_pages) {
    std::vector<int32_t> out;
    Node* n = root_.get();
    const size_t full = std::min({tokens.size() / ps_, (size_t)max_pages_, max_pages});
    for (size_t p = 0; p < full; ++p) {
      auto it = n->children.find(key(tokens, p));
      if (it == n->children.end()) break;
      Node* c = it->second.get();
      if (c->page < 0 || (size_t)c->page >= generations.size() || generations[c->page] != c->generation) {
        n->children.erase(it);  // evicted since it was cached
        break;
      }
      out.push_back(c->page);
      n = c;
    }
    return out;
  }
  // Registers pages[0..n) as holding the first n full pages of `tokens`. Existing nodes keep their page.
  size_t insert(const std::vector<int32_t>& tokens, const std::vector<int32_t>& pages, const std::vector<uint64_t>& generations) {
    Node* n = root_.get();
    const size_t full = std::min({tokens.size() / ps_, pages.size(), (size_t)max_pages_});
    size_t registered = 0;
    for (size_t p = 0; p < full; ++p) {
      auto k = key(tokens, p);
      auto it = n->children.find(k);
      if (it == n->children.end()) {
        auto c = std::make_unique<Node>();
        c->page = pages[p];
        c->generation = generations[pages[p]];
        it = n->children.emplace(std::move(k), std::move(c)).first;
        ++nodes_;
      } else if (it->second->page != pages[p]) {
        Node* c = it->second.get();
        const bool stale = c->page < 0 || (size_t)c->page >= generations.size() || generations[c->page] != c->generation;
        if (!stale) break;  // another request already caches this prefix in a different page; ours stays private
        c->page = pages[p];             // the old page was evicted: the entry now points at ours
        c->generation = generations[pages[p]];
        c->children.clear();
      }
      n = it->second.get();
      ++registered;
    }
    return registered;
  }
  bool holds(const std::vector<int32_t>& tokens, size_t page_idx, int32_t page) const {
    const Node* n = root_.get();
    for (size_t p = 0; p <= page_idx; ++p) {
      auto it = n->children.find(key(tokens, p));
      if (it == n->children.end()) return false;
      n = it->second.get();
    }
    return n->page == page;
  }
  size_t num_nodes() const { return nodes_; }

 private:
  struct Node {
    int32_t page = -1;
    uint64_t generation = 0;
    std::map<std::vector<int32_t>, std::unique_ptr<Node>> children;
  };
  std::vector<int32_t> key(const std::vector<int32_t>& t, size_t p) const { return std::vector<int32_t>(t.begin() + p * ps_, t.begin() + (p + 1) * ps_); }
  uint32_t ps_, max_pages_;
  std::unique_ptr<Node> root_;
  size_t nodes_ = 0;
};

class KvBlockManager {
 public:
  KvBlockManager(uint32_t total_pages, uint32_t page_size, bool prefix_cache = true, uint32_t radix_max_depth = 4096)
      : ps_(page_size), radix_depth_(radix_max_depth), refcount_(total_pages, 0), generation_(total_pages, 0), cached_(total_pages, 0) {
    if (page_size == 0 || total_pages == 0) throw RuntimeError("KV manager needs pages and a page size");
    for (uint32_t p = 0; p < total_pages; ++p) free_.push_back((int32_t)p);
    if (prefix_cache) radix_ = std::make_unique<RadixPrefixTree>(page_size, radix_max_depth);
  }
  static KvBlockManager with_capacity(uint64_t total_kv_bytes, uint64_t bytes_per_token, uint32_t page_size, bool prefix_cache = true) {
    const uint64_t page_bytes = bytes_per_token * page_size;
    if (page_bytes == 0 || total_kv_bytes < page_bytes) throw RuntimeError("KV budget is smaller than one page");
    return KvBlockManager((uint32_t)(total_kv_bytes / page_bytes), page_size, prefix_cache);
  }

  uint32_t page_size() const { return ps_; }
  uint32_t total_pages() const { return (uint32_t)refcount_.size(); }
  uint32_t available_pages() const { return (uint32_t)(free_.size() + lru_.size()); }
  uint32_t in_use_pages() const { return total_pages() - available_pages(); }
  double utilization() const { return (double)in_use_pages() / (double)total_pages(); }
  bool prefix_enabled() const { return (bool)radix_; }
  uint64_t generation_of(int32_t p) const { return generation_.at(p); }
  uint64_t prefix_hit_tokens_total() const { return hit_tokens_total_; }

  uint32_t pages_needed(uint32_t tokens) const { return (tokens + ps_ - 1) / ps_; }
  // Tokens of `prompt` that a new request would get from the prefix cache.
  uint32_t try_prefix_reuse(const std::vector<int32_t>& prompt) {
    if (!radix_ || prompt.empty()) return 0;
    return (uint32_t)(radix_->lookup(prompt, generation_, (prompt.size() - 1) / ps_).size() * ps_);
  }
  bool can_admit(const std::vector<int32_t>& prompt, uint32_t reserve_tokens = 0) {
    const uint32_t hit = try_prefix_reuse(prompt);
    const uint32_t need = pages_needed((uint32_t)prompt.size() + reserve_tokens) - hit / ps_;
    // matched pages sitting in the LRU list stop being "available" once we reference them
    return need <= available_pages_excluding_prefix(prompt, hit);
  }

  PageTable admit(uint64_t request_id, const std::vector<int32_t>& prompt) {
    if (tables_.count(request_id)) throw RuntimeError("request " + std::to_string(request_id) + " is already admitted");
    if (prompt.empty()) throw RuntimeError("empty prompt");
    std::vector<int32_t> matched;
    if (radix_) matched = radix_->lookup(prompt, generation_, (prompt.size() - 1) / ps_);
    const uint32_t need = pages_needed((uint32_t)prompt.size()) - (uint32_t)matched.size();
    if (need > total_pages()) throw RuntimeError("prompt needs " + std::to_string(need) + " pages, the cache has " + std::to_string(total_pages()));
    for (int32_t p : matched) ref(p);
    PageTable pt;
    pt.request_id = request_id;
    pt.pages = matched;
    try {
      for (uint32_t i = 0; i < need; ++i) { int32_t p = allocate_or_evict(); ref(p); pt.pages.push_back(p); }
    } catch (...) {
      for (int32_t p : pt.pages) unref(p);
      throw;
    }
    pt.num_tokens = (uint32_t)prompt.size();
    pt.prefix_hit_tokens = (uint32_t)matched.size() * ps_;
    hit_tokens_total_ += pt.prefix_hit_tokens;
    pt.registered_pages = (uint32_t)matched.size();   // the matched pages already sit in the trie
    tables_[request_id] = pt;
    return pt;
  }
  // The KV of the first `computed_tokens` tokens of `prompt` is now in the request's pages: enter the full
  // pages below that point in the trie. Returns the number of leading pages registered so far.
  uint32_t mark_computed(uint64_t request_id, const std::vector<int32_t>& prompt, uint32_t computed_tokens) {
    auto it = tables_.find(request_id);
    if (it == tables_.end()) throw RuntimeError("unknown request " + std::to_string(request_id));
    PageTable& pt = it->second;
    if (!radix_ || pt.no_register) return pt.registered_pages;
    const uint32_t upto = std::min<uint32_t>(computed_tokens, (uint32_t)prompt.size()) / ps_;
    if (upto <= pt.registered_pages) return pt.registered_pages;
    std::vector<int32_t> pages(pt.pages.begin(), pt.pages.begin() + std::min<size_t>(upto, pt.pages.size()));
    const uint32_t reg = (uint32_t)radix_->insert(prompt, pages, generation_);
    for (uint32_t i = pt.registered_pages; i < reg; ++i) cached_[pt.pages[i]] = 1;
    // a shorter count means another request cached the same prefix in other pages first: ours stay private
    if (reg < upto) pt.no_register = true;
    pt.registered_pages = std::max(pt.registered_pages, reg);
    return pt.registered_pages;
  }
  // Forget every cached prefix (the weights changed): all trie entries become stale, unreferenced cached
  // pages return to the free list, and requests in flight no longer register their pages.
  void clear_prefix_cache() {
    for (size_t p = 0; p < generation_.size(); ++p) { ++generation_[p]; cached_[p] = 0; }
    for (int32_t p : lru_) free_.push_back(p);
    lru_.clear();
    lru_pos_.clear();
    if (radix_) radix_ = std::make_unique<RadixPrefixTree>(ps_, radix_depth_);
    for (auto& kv : tables_) { kv.second.no_register = true; kv.second.registered_pages = 0; }
  }
  // Makes room for `n_new` more tokens; returns the pages that were added to the table.
  std::vector<int32_t> advance(uint64_t request_id, uint32_t n_new) {
    auto it = tables_.find(request_id);
    if (it == tables_.end()) throw RuntimeError("unknown request " + std::to_string(request_id));
    PageTable& pt = it->second;
    const uint32_t next = pt.num_tokens + n_new;
    std::vector<int32_t> added;
    while (pt.pages.size() < pages_needed(next)) {
      int32_t p = allocate_or_evict();
      ref(p);
      pt.pages.push_back(p);
      added.push_back(p);
    }
    pt.num_tokens = next;
    return added;
  }
  // `discard`: the request's step failed, so what its pages hold is not trusted; pages that no other request
  // references leave the prefix cache (generation bump, back to the free list).
  void release(uint64_t request_id, bool discard = false) {
    auto it = tables_.find(request_id);
    if (it == tables_.end()) throw RuntimeError("unknown request " + std::to_string(request_id));
    for (int32_t p : it->second.pages) {
      if (discard && refcount_[p] == 1) { ++generation_[p]; cached_[p] = 0; }
      unref(p);
    }
    tables_.erase(it);
  }
  const PageTable* table(uint64_t request_id) const {
    auto it = tables_.find(request_id);
    return it == tables_.end() ? nullptr : &it->second;
  }
  size_t num_requests() const { return tables_.size(); }

 private:
  uint32_t ps_, radix_depth_;
  std::vector<uint32_t> refcount_;
  std::vector<uint64_t> generation_;
  std::vector<char> cached_;              // page is registered in the trie
  std::deque<int32_t> free_;
  std::list<int32_t> lru_;                // unreferenced pages that still hold a cached prefix (front = oldest)
  std::unordered_map<int32_t, std::list<int32_t>::iterator> lru_pos_;
  std::unique_ptr<RadixPrefixTree> radix_;
  std::map<uint64_t, PageTable> tables_;
  uint64_t hit_tokens_total_ = 0;

  void ref(int32_t p) {
    if (refcount_[p]++ == 0) {
      auto it = lru_pos_.find(p);
      if (it != lru_pos_.end()) { lru_.erase(it->second); lru_pos_.erase(it); }
    }
  }
  void unref(int32_t p) {
    if (refcount_[p] == 0) throw RuntimeError("page " + std::to_string(p) + " released twice");
    if (--refcount_[p] == 0) {
      if (radix_ && cached_[p]) { lru_.push_back(p); lru_pos_[p] = std::prev(lru_.end()); }
      else free_.push_back(p);
    }
  }
  int32_t allocate_or_evict() {
    if (!free_.empty()) { int32_t p = free_.front(); free_.pop_front(); return p; }
    if (!lru_.empty()) {
      int32_t p = lru_.front();
      lru_.pop_front();
      lru_pos_.erase(p);
      ++generation_[p];   // trie entries that point at this page are now stale
      cached_[p] = 0;
      return p;
    }
    throw RuntimeError("KV cache exhausted: all " + std::to_string(total_pages()) + " pages are referenced");
  }
  uint32_t available_pages_excluding_prefix(const std::vector<int32_t>& prompt, uint32_t hit) {
    if (hit == 0 || !radix_) return available_pages();
    uint32_t in_lru = 0;
    for (int32_t p : radix_->lookup(prompt, generation_, (prompt.size() - 1) / ps_)) if (lru_pos_.count(p)) ++in_lru;
    return available_pages() - in_lru;
  }
};

}  // namespace skein
