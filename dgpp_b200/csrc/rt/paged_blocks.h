// Block bookkeeping of the paged KV pool: LIFO free list, per-block reference counts (prefix sharing)
// and a generation number per block that changes every time the block is handed out again, so a stale
// (block, generation) reference can be recognised.
// (reference behaviour: src/engine/paged_blocks.hpp:1-215.)
#pragma once
#include <cstdint>
#include <stdexcept>
#include <vector>

namespace dgpp {

class PagedBlockTable {
 public:
  explicit PagedBlockTable(int num_blocks) : ref_(num_blocks, 0), gen_(num_blocks, 0) {
    free_.reserve(num_blocks);
    for (int b = num_blocks - 1; b >= 0; --b) free_.push_back(b);
  }
  int num_blocks() const { return static_cast<int>(ref_.size()); }
  int free_count() const { return static_cast<int>(free_.size()); }
  // Returns -1 when the pool is exhausted.
  int alloc() {
    if (free_.empty()) return -1;
    const int b = free_.back();
    free_.pop_back();
    ref_[b] = 1;
    ++gen_[b];
    return b;
  }
  void retain(int b) {
    check(b);
    if (ref_[b] <= 0) throw std::runtime_error("retain of a free block");
    ++ref_[b];
  }
  void release(int b) {
    check(b);
    if (ref_[b] <= 0) throw std::runtime_error("release of a free block");
    if (--ref_[b] == 0) free_.push_back(b);
  }
  int refcount(int b) const { check(b); return ref_[b]; }
  uint32_t generation(int b) const { check(b); return gen_[b]; }

 private:
  void check(int b) const {
    if (b < 0 || b >= static_cast<int>(ref_.size())) throw std::out_of_range("block id out of range");
  }
  std::vector<int> free_;
  std::vector<int> ref_;
  std::vector<uint32_t> gen_;
};

}  // namespace dgpp
