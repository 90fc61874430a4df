// Deterministic stand-in for a model engine: real block accounting (PagedBlockTable, shared prefix
// blocks, refcounts) and a token function that depends only on the request's token history, so
// scheduler / prefix-cache / service tests can check exact token streams without a GPU.
// The next token after a sequence t_0..t_{n-1} is  mix(hash(t_0..t_{n-1})) % vocab; the engine also
// verifies that every position it is asked to decode has its KV "written" (a per-block fill count),
// which catches scheduler bugs such as skipped prefill chunks or wrong prefix attachment.
// (same idea as the FakeEngine of tests/host/scheduler_test.cpp:53 in the reference.)
#pragma once
#include <stdexcept>
#include <vector>

#include "rt/paged_blocks.h"
#include "rt/scheduler.h"

namespace dgpp {

class FakeEngine : public SchedulerEngine {
 public:
  FakeEngine(int slots, int block_tokens, int64_t blocks, int64_t max_context, int vocab, int tokens_per_step = 1)
      : table_(static_cast<int>(blocks)), block_tokens_(block_tokens), max_context_(max_context), vocab_(vocab),
        tokens_per_step_(tokens_per_step), slots_(static_cast<size_t>(slots)),
        block_hash_(static_cast<size_t>(blocks), 0), block_fill_(static_cast<size_t>(blocks), 0) {}

  int max_concurrent() const override { return static_cast<int>(slots_.size()); }
  int block_tokens() const override { return block_tokens_; }
  int64_t total_blocks() const override { return table_.num_blocks(); }
  int64_t free_blocks() const override { return table_.free_count(); }
  int64_t max_context() const override { return max_context_; }
  int max_tokens_per_step() const override { return tokens_per_step_; }

  bool reserve(int slot, int64_t tokens) override {
    S& s = slots_.at(slot);
    const int64_t need = (tokens + block_tokens_ - 1) / block_tokens_;
    if (need - static_cast<int64_t>(s.blocks.size()) > table_.free_count()) return false;
    while (static_cast<int64_t>(s.blocks.size()) < need) {
      const int b = table_.alloc();
      block_fill_[b] = 0;
      block_hash_[b] = 0;
      s.blocks.push_back(b);
    }
    return true;
  }
  void attach_prefix(int slot, const std::vector<int32_t>& blocks) override {
    S& s = slots_.at(slot);
    if (!s.blocks.empty()) throw std::runtime_error("attach_prefix on a non-empty slot");
    for (int32_t b : blocks) {
      if (block_fill_[b] != block_tokens_) throw std::runtime_error("attached block is not full");
      table_.retain(b);
      s.blocks.push_back(b);
    }
    s.filled = static_cast<int64_t>(blocks.size()) * block_tokens_;
    s.hash = blocks.empty() ? kFnvSeed : block_hash_[blocks.back()];
    s.history_from_prefix = true;
  }
  int32_t prefill(int slot, const int32_t* tokens, int64_t pos, int64_t count, bool last) override {
    S& s = slots_.at(slot);
    if (pos != s.filled) throw std::runtime_error("prefill position does not continue the filled prefix");
    ++prefill_calls;
    prefill_tokens += count;
    for (int64_t i = 0; i < count; ++i) feed(s, tokens[i]);
    return last ? next_token(s) : -1;
  }
  std::vector<std::vector<int32_t>> step_batch(const std::vector<int>& slots) override {
    ++decode_passes;
    std::vector<std::vector<int32_t>> out;
    for (int slot : slots) {
      S& s = slots_.at(slot);
      std::vector<int32_t> toks;
      for (int k = 0; k < tokens_per_step_; ++k) {
        // the previously emitted token is fed now (its KV gets written), then the next one is picked
        feed(s, s.pending);
        toks.push_back(next_token(s));
      }
      out.push_back(toks);
    }
    return out;
  }
  bool mixed_step(const PrefillPiece& piece, const std::vector<int>& slots, int32_t* first,
                  std::vector<std::vector<int32_t>>* out) override {
    if (!mixed) return false;
    ++mixed_calls;
    *out = step_batch(slots);
    *first = prefill(piece.slot, piece.tokens, piece.pos, piece.count, piece.last);
    --decode_passes;          // one engine call, counted as mixed
    --prefill_calls;
    return true;
  }
  std::vector<int32_t> slot_blocks(int slot) const override { return slots_.at(slot).blocks; }
  void retain_block(int32_t b) override { table_.retain(b); }
  void release_block(int32_t b) override { table_.release(b); }
  int block_refcount(int32_t b) const override { return table_.refcount(b); }
  void close(int slot) override {
    S& s = slots_.at(slot);
    for (int32_t b : s.blocks) table_.release(b);
    s = S();
  }

  int64_t prefill_calls = 0, prefill_tokens = 0, decode_passes = 0, mixed_calls = 0;
  bool mixed = false;            // answer mixed_step (tests of the scheduler's mixed pass)

  // The token stream a request must produce, independent of scheduling (oracle for tests).
  static std::vector<int32_t> expected(const std::vector<int32_t>& prompt, int64_t n, int vocab) {
    uint64_t h = kFnvSeed;
    for (int32_t t : prompt) h = fnv1a_bytes(h, &t, sizeof(t));
    std::vector<int32_t> out;
    for (int64_t i = 0; i < n; ++i) {
      const int32_t t = pick(h, vocab);
      out.push_back(t);
      h = fnv1a_bytes(h, &t, sizeof(t));
    }
    return out;
  }

 private:
  struct S {
    std::vector<int32_t> blocks;
    int64_t filled = 0;       // positions whose KV is written
    uint64_t hash = kFnvSeed; // hash of all tokens fed so far
    int32_t pending = -1;     // token emitted but not yet fed
    bool history_from_prefix = false;
  };
  static int32_t pick(uint64_t h, int vocab) {
    h ^= h >> 33;
    h *= 0xff51afd7ed558ccdull;
    h ^= h >> 33;
    return static_cast<int32_t>(h % static_cast<uint64_t>(vocab));
  }
  void feed(S& s, int32_t tok) {
    const int64_t blk = s.filled / block_tokens_;
    if (blk >= static_cast<int64_t>(s.blocks.size())) throw std::runtime_error("write beyond reserved blocks");
    const int32_t b = s.blocks[blk];
    if (table_.refcount(b) > 1 && block_fill_[b] == block_tokens_)
      throw std::runtime_error("write into a shared full block");
    s.hash = fnv1a_bytes(s.hash, &tok, sizeof(tok));
    ++block_fill_[b];
    ++s.filled;
    if (block_fill_[b] == block_tokens_) block_hash_[b] = s.hash;
  }
  int32_t next_token(S& s) {
    s.pending = pick(s.hash, vocab_);
    return s.pending;
  }

  PagedBlockTable table_;
  int block_tokens_;
  int64_t max_context_;
  int vocab_;
  int tokens_per_step_;
  std::vector<S> slots_;
  std::vector<uint64_t> block_hash_;
  std::vector<int> block_fill_;
};

}  // namespace dgpp
