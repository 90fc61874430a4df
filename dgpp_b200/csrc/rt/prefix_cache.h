// Exact prefix cache over paged KV blocks, keyed by a hash chain of fixed-size token blocks:
//   h_0 = H(seed, ids[0:B]),  h_i = H(h_{i-1}, ids[iB:(i+1)B])      (B = block_tokens, 16 by default)
// An entry maps one chain hash to the physical KV block that holds those B positions; the cache owns
// one reference on the block (taken through the engine) until the entry is evicted.  Lookup walks
// the prompt block by block and returns the longest run of cached blocks, always leaving at least
// one prompt token to prefill so the request still produces its first logits.
//
// Eviction is LRU over entries nobody else references, deepest first among equals, so a chain is
// trimmed from its tail.  Evicted hashes are remembered in a small ghost list for miss explanations.
// Pinned entries (request carried a cache key) are evicted only when nothing else is left.
//
// Hash: FNV-1a 64 over the parent hash bytes then the token ids (little-endian int32).
// (reference behaviour: src/sched/prefix_cache.hpp:1-204 -- exact-match entries, LRU, ghosts, pins;
//  the block-hash chain replaces its cut-position snapshots.)
#pragma once
#include <cstdint>
#include <deque>
#include <functional>
#include <string>
#include <unordered_map>
#include <vector>

namespace dgpp {

constexpr uint64_t kFnvSeed = 0xcbf29ce484222325ull;
constexpr uint64_t kFnvPrime = 0x100000001b3ull;

inline uint64_t fnv1a_bytes(uint64_t h, const void* p, size_t n) {
  const unsigned char* b = static_cast<const unsigned char*>(p);
  for (size_t i = 0; i < n; ++i) {
    h ^= b[i];
    h *= kFnvPrime;
  }
  return h;
}

inline uint64_t chain_hash(uint64_t parent, const int32_t* ids, int n) {
  uint64_t h = fnv1a_bytes(kFnvSeed, &parent, sizeof(parent));
  return fnv1a_bytes(h, ids, sizeof(int32_t) * static_cast<size_t>(n));
}

// Second, independent 64-bit chain over the same blocks (different mixing function and seed).  An entry found under
// the FNV chain hash is only taken when this check value matches too: a prompt crafted to collide FNV-1a would have
// to collide both chains at once to attach another request's blocks.
inline uint64_t check_hash(uint64_t parent, const int32_t* ids, int n) {
  uint64_t h = parent ^ 0x9E3779B97F4A7C15ull;
  for (int i = 0; i < n; ++i) {
    uint64_t x = static_cast<uint64_t>(static_cast<uint32_t>(ids[i])) + 0xD6E8FEB86659FD93ull * static_cast<uint64_t>(i + 1);
    x ^= x >> 32; x *= 0xD6E8FEB86659FD93ull; x ^= x >> 32;
    h = (h ^ x) * 0xFF51AFD7ED558CCDull;
    h ^= h >> 29;
  }
  return h;
}
constexpr uint64_t kCheckSeed = 0x243F6A8885A308D3ull;

struct PrefixHit {
  std::vector<int32_t> blocks;  // physical blocks covering the cached prefix, in order
  int64_t tokens = 0;           // = blocks.size() * block_tokens
  uint64_t last_hash = kFnvSeed;
};

struct PrefixStats {
  int64_t lookups = 0, hits = 0, hit_tokens = 0, miss_tokens = 0, inserts = 0, evictions = 0, ghost_hits = 0;
  int64_t check_rejects = 0;   // entries found under the chain hash whose second hash did not match
};

class PrefixCache {
 public:
  struct Entry {
    int32_t block;
    uint64_t parent;
    int32_t depth;
    int64_t last_use;
    bool pinned;
    uint64_t check;       // check_hash chain value of the prefix ending with this block
  };

  PrefixCache(int block_tokens, int64_t max_entries, int ghost_capacity = 256)
      : block_tokens_(block_tokens), max_entries_(max_entries), ghost_capacity_(ghost_capacity) {}

  int block_tokens() const { return block_tokens_; }
  int64_t size() const { return static_cast<int64_t>(map_.size()); }
  const PrefixStats& stats() const { return stats_; }

  // Longest cached prefix of `ids`, at most n-1 tokens.  Touches the entries it returns.
  PrefixHit lookup(const int32_t* ids, int64_t n, int64_t now) {
    PrefixHit hit;
    ++stats_.lookups;
    uint64_t h = kFnvSeed, c = kCheckSeed;
    const int64_t full = (n - 1) / block_tokens_;
    for (int64_t b = 0; b < full; ++b) {
      const uint64_t hb = chain_hash(h, ids + b * block_tokens_, block_tokens_);
      const uint64_t cb = check_hash(c, ids + b * block_tokens_, block_tokens_);
      auto it = map_.find(hb);
      if (it != map_.end() && it->second.check != cb) {   // same FNV chain value, different tokens: not this prefix
        ++stats_.check_rejects;
        break;
      }
      if (it == map_.end()) {
        if (b == 0 || true) {
          for (uint64_t g : ghosts_)
            if (g == hb) { ++stats_.ghost_hits; break; }
        }
        break;
      }
      it->second.last_use = now;
      hit.blocks.push_back(it->second.block);
      h = hb;
      c = cb;
    }
    hit.tokens = static_cast<int64_t>(hit.blocks.size()) * block_tokens_;
    hit.last_hash = h;
    if (hit.tokens > 0) { ++stats_.hits; stats_.hit_tokens += hit.tokens; }
    stats_.miss_tokens += n - hit.tokens;
    return hit;
  }

  // Publish the first `tokens` positions (rounded down to whole blocks) of a request whose KV lives in
  // `blocks`.  `retain(block)` is called for every block the cache newly references.  Returns the number
  // of new entries.
  int64_t insert(const int32_t* ids, int64_t tokens, const std::vector<int32_t>& blocks, int64_t now, bool pinned,
                 const std::function<void(int32_t)>& retain, const std::function<void(int32_t)>& release) {
    const int64_t full = std::min<int64_t>(tokens / block_tokens_, static_cast<int64_t>(blocks.size()));
    uint64_t h = kFnvSeed, c = kCheckSeed;
    int64_t added = 0;
    for (int64_t b = 0; b < full; ++b) {
      const uint64_t hb = chain_hash(h, ids + b * block_tokens_, block_tokens_);
      const uint64_t cb = check_hash(c, ids + b * block_tokens_, block_tokens_);
      auto it = map_.find(hb);
      if (it != map_.end() && it->second.check != cb) break;   // the slot belongs to another prefix: publish nothing further
      if (it == map_.end()) {
        while (static_cast<int64_t>(map_.size()) >= max_entries_) {
          if (!evict_one(release, /*allow_pinned=*/true, hb)) break;
        }
        if (static_cast<int64_t>(map_.size()) >= max_entries_) break;
        retain(blocks[b]);
        map_.emplace(hb, Entry{blocks[b], h, static_cast<int32_t>(b), now, pinned, cb});
        ++stats_.inserts;
        ++added;
      } else {
        it->second.last_use = now;
        it->second.pinned = it->second.pinned || pinned;
      }
      h = hb;
      c = cb;
    }
    return added;
  }

  // Evict entries until `want_blocks` physical blocks were released or nothing evictable is left.
  // `refcount(block)` tells whether anyone besides the cache holds the block.
  int64_t evict_to_free(int64_t want_blocks, const std::function<int(int32_t)>& refcount,
                        const std::function<void(int32_t)>& release) {
    int64_t freed = 0;
    for (int pass = 0; pass < 2 && freed < want_blocks; ++pass) {
      const bool allow_pinned = pass == 1;
      while (freed < want_blocks) {
        uint64_t victim = 0;
        bool found = false;
        int64_t best_use = 0;
        int32_t best_depth = 0;
        for (const auto& kv : map_) {
          const Entry& e = kv.second;
          if (e.pinned && !allow_pinned) continue;
          if (refcount(e.block) > 1) continue;  // a live request shares it
          if (!found || e.last_use < best_use || (e.last_use == best_use && e.depth > best_depth) ||
              (e.last_use == best_use && e.depth == best_depth && kv.first < victim)) {
            found = true;
            victim = kv.first;
            best_use = e.last_use;
            best_depth = e.depth;
          }
        }
        if (!found) break;
        erase(victim, release);
        ++freed;
      }
    }
    return freed;
  }

  void clear(const std::function<void(int32_t)>& release) {
    for (auto& kv : map_) release(kv.second.block);
    map_.clear();
  }

  // Order-independent digest of the cache content (compared across ranks).
  uint64_t digest() const {
    uint64_t d = 0;
    for (const auto& kv : map_) d ^= fnv1a_bytes(kFnvSeed, &kv.first, sizeof(kv.first)) * (static_cast<uint64_t>(kv.second.block) + 1);
    return d ^ static_cast<uint64_t>(map_.size());
  }

 private:
  bool evict_one(const std::function<void(int32_t)>& release, bool allow_pinned, uint64_t keep) {
    uint64_t victim = 0;
    bool found = false;
    int64_t best_use = 0;
    int32_t best_depth = 0;
    for (const auto& kv : map_) {
      const Entry& e = kv.second;
      if (kv.first == keep) continue;
      if (e.pinned && !allow_pinned) continue;
      if (!found || e.last_use < best_use || (e.last_use == best_use && e.depth > best_depth) ||
          (e.last_use == best_use && e.depth == best_depth && kv.first < victim)) {
        found = true;
        victim = kv.first;
        best_use = e.last_use;
        best_depth = e.depth;
      }
    }
    if (!found) return false;
    erase(victim, release);
    return true;
  }
  void erase(uint64_t h, const std::function<void(int32_t)>& release) {
    auto it = map_.find(h);
    if (it == map_.end()) return;
    release(it->second.block);
    map_.erase(it);
    ++stats_.evictions;
    ghosts_.push_back(h);
    while (static_cast<int>(ghosts_.size()) > ghost_capacity_) ghosts_.pop_front();
  }

  int block_tokens_;
  int64_t max_entries_;
  int ghost_capacity_;
  std::unordered_map<uint64_t, Entry> map_;
  std::deque<uint64_t> ghosts_;
  PrefixStats stats_;
};

}  // namespace dgpp
