// Paged KV block manager with a hash-chained prefix cache.
//
// Behaviour follows the reference block layer:
//   * block id 0 is reserved as the padding block and never handed out
//     (xllm/core/framework/block/block_manager_impl.cpp:44-46);
//   * fresh ids are handed out smallest-first (block_manager_impl.cpp:38-62);
//   * blocks are reference counted; a block that only the prefix cache still
//     references is evictable, least-recently-used first
//     (block_manager_impl.cpp:95-125, prefix_cache.cpp:256+);
//   * only full blocks are cached / matched, keys are chained 128-bit hashes
//     (prefix_cache.cpp:31-121,145-206).
// One manager exists per attention-DP rank; BlockManagerPool picks the rank with
// the most free blocks for a new sequence (block_manager_pool.h:92).
#pragma once
#include <algorithm>
#include <cstdint>
#include <list>
#include <stdexcept>
#include <unordered_map>
#include <vector>

#include "hash128.h"

namespace xl {

class BlockManager {
 public:
  BlockManager(int num_blocks, int block_size, bool enable_prefix_cache, uint64_t seed = 1024)
      : num_blocks_(num_blocks), block_size_(block_size), enable_cache_(enable_prefix_cache), seed_(seed),
        ref_(num_blocks, 0), cached_(num_blocks, 0), hash_(num_blocks), lru_pos_(num_blocks) {
    if (num_blocks < 2) throw std::invalid_argument("BlockManager needs at least 2 blocks (block 0 is padding)");
    free_.reserve(num_blocks);
    for (int i = num_blocks - 1; i >= 1; --i) free_.push_back(i);  // back() is the smallest id
  }

  int block_size() const { return block_size_; }
  int num_blocks() const { return num_blocks_; }
  int num_free_blocks() const { return static_cast<int>(free_.size()); }
  int num_blocks_in_prefix_cache() const { return static_cast<int>(lru_.size()); }
  // blocks held by at least one sequence (cache-only blocks are reclaimable, so they count as free capacity)
  int num_used_blocks() const { return num_blocks_ - 1 - num_free_blocks() - num_evictable_; }
  int num_available_blocks() const { return num_free_blocks() + num_evictable_; }
  double utilization() const { return double(num_used_blocks()) / double(num_blocks_ - 1); }
  bool prefix_cache_enabled() const { return enable_cache_; }
  int ref_count(int id) const { return ref_[id]; }
  // Keys that entered / left the prefix cache since the last call (KvCacheEvent of the reference,
  // block_manager_pool.h get_merged_kvcache_event): the service router builds its global prefix index from them.
  void record_cache_events(bool on) { record_events_ = on; }
  std::pair<std::vector<Hash128>, std::vector<Hash128>> take_cache_events() {
    std::pair<std::vector<Hash128>, std::vector<Hash128>> out;
    out.first.swap(stored_events_);
    out.second.swap(removed_events_);
    return out;
  }
  uint64_t match_queries() const { return match_query_blocks_; }
  uint64_t match_hits() const { return match_hit_blocks_; }

  // Allocate n fresh blocks (ref=1 each).  Evicts cache-only blocks when short.
  bool allocate(int n, std::vector<int>& out) {
    if (n <= 0) return true;
    if (num_available_blocks() < n) return false;
    if (num_free_blocks() < n) evict(n - num_free_blocks());
    for (int i = 0; i < n; ++i) {
      int id = free_.back();
      free_.pop_back();
      ref_[id] = 1;
      out.push_back(id);
    }
    return true;
  }

  void add_ref(int id) {
    check(id);
    if (ref_[id] == 1 && cached_[id]) --num_evictable_;
    ++ref_[id];
  }

  // Drop one reference; the block returns to the free list at zero.
  void release(int id) {
    check(id);
    if (ref_[id] <= 0) throw std::logic_error("release of unreferenced block");
    --ref_[id];
    if (ref_[id] == 0) {
      free_.push_back(id);
    } else if (ref_[id] == 1 && cached_[id]) {
      ++num_evictable_;
    }
  }
  void release(const std::vector<int>& ids) {
    for (int id : ids) release(id);
  }

  // Longest cached prefix of `tokens` in whole blocks.  Each returned block gets
  // one more reference (the caller's).  At most max_blocks are matched.
  std::vector<int> match(const int32_t* tokens, int n_tokens, int max_blocks = 1 << 30) {
    std::vector<int> out;
    if (!enable_cache_) return out;
    int full = std::min(n_tokens / block_size_, max_blocks);
    Hash128 prev;
    for (int b = 0; b < full; ++b) {
      Hash128 h = chain_block_hash(b ? &prev : nullptr, tokens + size_t(b) * block_size_, block_size_, seed_);
      ++match_query_blocks_;
      auto it = table_.find(h);
      if (it == table_.end()) break;
      int id = it->second;
      add_ref(id);
      out.push_back(id);
      ++match_hit_blocks_;
      prev = h;
    }
    touch_chain(out);
    return out;
  }

  // Publish the full blocks of a sequence.  Returns how many new blocks entered the cache.
  int insert(const int32_t* tokens, int n_tokens, const std::vector<int>& blocks) {
    if (!enable_cache_) return 0;
    int full = std::min<int>(n_tokens / block_size_, static_cast<int>(blocks.size()));
    Hash128 prev;
    int added = 0;
    std::vector<int> chain;
    for (int b = 0; b < full; ++b) {
      Hash128 h = chain_block_hash(b ? &prev : nullptr, tokens + size_t(b) * block_size_, block_size_, seed_);
      prev = h;
      int id = blocks[b];
      check(id);
      auto it = table_.find(h);
      if (it != table_.end()) {  // content already cached (maybe under another block id): refresh
        chain.push_back(it->second);
        continue;
      }
      if (cached_[id]) continue;  // this block already backs a different key
      table_.emplace(h, id);
      if (record_events_) stored_events_.push_back(h);
      hash_[id] = h;
      cached_[id] = 1;
      lru_.push_back(id);
      lru_pos_[id] = std::prev(lru_.end());
      ++ref_[id];  // the cache's own reference
      ++added;
      chain.push_back(id);
    }
    touch_chain(chain);
    return added;
  }

  // Key under which a cached block is published (zero for a block that is not in the cache).
  Hash128 hash_of(int id) const {
    check(id);
    return cached_[id] ? hash_[id] : Hash128{};
  }

  // How many leading full blocks of `tokens` the cache holds; takes no reference and does not touch the LRU order.
  int count_prefix(const int32_t* tokens, int n_tokens, int max_blocks = 1 << 30) const {
    if (!enable_cache_) return 0;
    int full = std::min(n_tokens / block_size_, max_blocks);
    Hash128 prev;
    int n = 0;
    for (; n < full; ++n) {
      Hash128 h = chain_block_hash(n ? &prev : nullptr, tokens + size_t(n) * block_size_, block_size_, seed_);
      if (table_.find(h) == table_.end()) break;
      prev = h;
    }
    return n;
  }

  // Take the given blocks out of the cache again (their content never arrived).  Only blocks that nobody but the
  // cache references are dropped; returns how many were.
  int drop_cached(const std::vector<int>& ids) {
    int done = 0;
    for (int id : ids) {
      check(id);
      if (!cached_[id] || ref_[id] != 1) continue;
      table_.erase(hash_[id]);
      if (record_events_) removed_events_.push_back(hash_[id]);
      cached_[id] = 0;
      lru_.erase(lru_pos_[id]);
      ref_[id] = 0;
      --num_evictable_;
      free_.push_back(id);
      ++done;
    }
    return done;
  }

  // Evict up to n cache-only blocks, least recently used first.
  int evict(int n) {
    int done = 0;
    for (auto it = lru_.begin(); it != lru_.end() && done < n;) {
      int id = *it;
      if (ref_[id] == 1) {
        table_.erase(hash_[id]);
        if (record_events_) removed_events_.push_back(hash_[id]);
        cached_[id] = 0;
        it = lru_.erase(it);
        ref_[id] = 0;
        --num_evictable_;
        free_.push_back(id);
        ++done;
      } else {
        ++it;
      }
    }
    return done;
  }

 private:
  // Mark the blocks of one prefix chain as most recently used, the chain's tail oldest and its head newest: eviction
  // then shortens a cached prefix from its end instead of cutting off its first block and stranding the rest
  // (the order the reference builds with its push_front / pop_front staging list, prefix_cache.cpp:181-209).
  void touch_chain(const std::vector<int>& chain) {
    for (auto it = chain.rbegin(); it != chain.rend(); ++it) lru_.splice(lru_.end(), lru_, lru_pos_[*it]);
  }
  void check(int id) const {
    if (id <= 0 || id >= num_blocks_) throw std::out_of_range("bad block id");
  }
  int num_blocks_, block_size_;
  bool enable_cache_;
  uint64_t seed_;
  std::vector<int> free_;
  std::vector<int> ref_;
  std::vector<uint8_t> cached_;
  std::vector<Hash128> hash_;
  std::vector<std::list<int>::iterator> lru_pos_;
  std::list<int> lru_;
  std::unordered_map<Hash128, int, Hash128Hasher> table_;
  int num_evictable_ = 0;
  bool record_events_ = false;
  std::vector<Hash128> stored_events_, removed_events_;
  uint64_t match_query_blocks_ = 0, match_hit_blocks_ = 0;
};

class BlockManagerPool {
 public:
  BlockManagerPool(int dp_size, int num_blocks, int block_size, bool enable_prefix_cache, uint64_t seed = 1024) {
    for (int i = 0; i < dp_size; ++i) mgrs_.emplace_back(num_blocks, block_size, enable_prefix_cache, seed);
  }
  int dp_size() const { return static_cast<int>(mgrs_.size()); }
  BlockManager& at(int dp_rank) { return mgrs_.at(dp_rank); }
  const BlockManager& at(int dp_rank) const { return mgrs_.at(dp_rank); }
  int pick_dp_rank() const {
    int best = 0;
    for (int i = 1; i < dp_size(); ++i)
      if (mgrs_[i].num_available_blocks() > mgrs_[best].num_available_blocks()) best = i;
    return best;
  }
  double utilization() const {
    double u = 0;
    for (auto& m : mgrs_) u = std::max(u, m.utilization());
    return u;
  }

 private:
  std::vector<BlockManager> mgrs_;
};

}  // namespace xl
