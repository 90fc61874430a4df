// Continuous-batching scheduler with a deterministic tick.
//
// One tick does, in this order:
//   1. cancel sweep            -- requests flagged by the service are retired ("cancelled")
//   2. reservation growth      -- (grow-on-demand policy) decoders about to cross a block boundary get a
//                                 block; when the pool is dry the youngest request is shed back to the queue
//   3. admission               -- FIFO by arrival while a slot and blocks are free; prefix-cache lookup
//                                 shares cached blocks, LRU entries are evicted to make room
//   4. prefill                 -- chunked and resumable, at most `prefill_budget` prompt tokens per tick
//                                 (idle / busy budgets); the last chunk yields the first token
//   5. one decode pass         -- all requests in decode state step together
//   6. retirement              -- eos / length / stop-token / cancelled / error; finished prompts are
//                                 published to the prefix cache
// Every decision is a pure function of the submitted request stream and the engine's answers, so two
// ranks fed the same stream make the same decisions; an FNV-1a digest of the op stream is kept for
// cross-rank checks.
// (behavioural spec: src/sched/scheduler.cpp:1500-1958 tick/quantum, admission 683, retire 1292;
//  src/sched/scheduler.hpp:57-560 engine contract, 637-680 admission policies, 1197-1257 observer.)
#pragma once
#include <algorithm>
#include <cstdint>
#include <deque>
#include <functional>
#include <map>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include "rt/prefix_cache.h"

namespace dgpp {

// What the scheduler needs from an execution engine.  Slots are 0 .. max_concurrent()-1.
class SchedulerEngine {
 public:
  virtual ~SchedulerEngine() = default;
  virtual int max_concurrent() const = 0;
  virtual int block_tokens() const = 0;            // tokens per KV block
  virtual int64_t total_blocks() const = 0;
  virtual int64_t free_blocks() const = 0;
  virtual int64_t max_context() const = 0;         // longest sequence a slot can hold
  // Make slot own blocks covering `tokens` positions (after any attached prefix).  false = pool exhausted.
  virtual bool reserve(int slot, int64_t tokens) = 0;
  // How many of the matched cached blocks (a prefix of `blocks`) the engine can resume from.  Engines whose state is
  // more than KV blocks (recurrent layers) keep state snapshots only at some block boundaries and answer with the
  // longest prefix that ends on one; the default is all of them.
  virtual int64_t usable_prefix(const std::vector<int32_t>& blocks) const { return static_cast<int64_t>(blocks.size()); }
  // Share cached blocks as the first blocks of an empty slot.
  virtual void attach_prefix(int slot, const std::vector<int32_t>& blocks) = 0;
  // Run prompt tokens [pos, pos+count) of the slot.  Returns the first generated token when `last`, else -1.
  virtual int32_t prefill(int slot, const int32_t* tokens, int64_t pos, int64_t count, bool last) = 0;
  // Several readers in ONE engine call (group prefill): pieces of different slots, each a run of consecutive prompt
  // positions.  Returns, per piece, the first generated token when the piece is `last`, else -1.  The default runs the
  // pieces one after the other; an engine that can carry rows of several requests in one pass overrides it (the weights
  // are then read once for all of them).
  struct PrefillPiece {
    int slot;
    const int32_t* tokens;
    int64_t pos, count;
    bool last;
  };
  virtual std::vector<int32_t> prefill_group(const std::vector<PrefillPiece>& pieces) {
    std::vector<int32_t> out;
    out.reserve(pieces.size());
    for (const auto& p : pieces) out.push_back(prefill(p.slot, p.tokens, p.pos, p.count, p.last));
    return out;
  }
  // One decode pass; result[i] holds the new tokens of slots[i] (one, or several with speculative decoding).
  virtual std::vector<std::vector<int32_t>> step_batch(const std::vector<int>& slots) = 0;
  // Mixed pass: the rows of one prefill piece and one decode step of `slots` in ONE engine call (the weights are read
  // once, the decoders do not wait behind the reader's chunk).  Returns false when the engine has no such pass for
  // these requests; the scheduler then runs the piece and the decode pass one after the other.  *first: the piece's
  // first generated token when it is `last`, else -1; (*out)[i]: the new tokens of slots[i].
  virtual bool mixed_step(const PrefillPiece& piece, const std::vector<int>& slots, int32_t* first,
                          std::vector<std::vector<int32_t>>* out) {
    (void)piece; (void)slots; (void)first; (void)out;
    return false;
  }
  virtual int max_tokens_per_step() const { return 1; }
  // Physical blocks of a slot, in position order (for publishing to the prefix cache).
  virtual std::vector<int32_t> slot_blocks(int slot) const = 0;
  virtual void retain_block(int32_t block) = 0;
  virtual void release_block(int32_t block) = 0;
  virtual int block_refcount(int32_t block) const = 0;
  // Drop the slot's blocks and state.
  // Called once when request `id` is admitted into `slot`, before its first prefill chunk: the engine binds the
  // request's sampling parameters, grammar and token-count row to the slot.
  virtual void open(int slot, const std::string& id) { (void)slot; (void)id; }
  virtual void close(int slot) = 0;
};

enum class RetireReason { Eos, Length, Stop, Cancelled, Error, Shed };

inline const char* retire_name(RetireReason r) {
  switch (r) {
    case RetireReason::Eos: return "stop";
    case RetireReason::Length: return "length";
    case RetireReason::Stop: return "stop";
    case RetireReason::Cancelled: return "cancelled";
    case RetireReason::Error: return "error";
    case RetireReason::Shed: return "shed";
  }
  return "?";
}

struct SchedRequest {
  std::string id;
  std::vector<int32_t> prompt;
  int64_t max_tokens = 16;
  std::vector<int32_t> eos_ids;
  std::vector<int32_t> stop_ids;     // single-token stops handled here; stop strings live above
  bool ignore_eos = false;
  bool prefix_cache = true;
  std::string cache_key;             // non-empty: pin published blocks
};

class SchedulerObserver {
 public:
  virtual ~SchedulerObserver() = default;
  virtual void on_admit(const std::string& id, int slot, int64_t cached_tokens) { (void)id; (void)slot; (void)cached_tokens; }
  virtual void on_token(const std::string& id, int32_t token, int64_t index) { (void)id; (void)token; (void)index; }
  virtual void on_retire(const std::string& id, RetireReason why, int64_t generated) { (void)id; (void)why; (void)generated; }
};

enum class AdmissionPolicy { FullReserve, GrowOnDemand };

struct SchedulerConfig {
  AdmissionPolicy policy = AdmissionPolicy::FullReserve;
  int64_t prefill_budget_idle = 4096;   // prompt tokens per tick when nobody is decoding
  int64_t prefill_budget_busy = 1024;   // ... when decoders are waiting for their pass
  int64_t prefill_chunk = 2048;         // largest single engine call
  bool prefix_cache = true;
  int64_t prefix_min_tokens = 16;
  int64_t prefix_max_entries = 1 << 20;
  int64_t grow_margin_tokens = 1;       // grow-on-demand keeps this many positions reserved ahead
  // Group prefill: the readers of a tick are planned together and handed to the engine in calls of up to
  // `prefill_group_max` pieces whose tokens sum to at most `prefill_chunk` (oldest reader first, every reader gets an
  // equal share of what the budget leaves before the leftovers go to the oldest).  1 = one reader per engine call.
  int prefill_group_max = 1;
  // Mixed passes: while requests are decoding, the oldest reader's next chunk rides in the same engine call as their
  // decode step (engines without such a pass keep the two calls).  At most `prefill_budget_busy` prompt tokens.
  bool mixed_pass = false;
};

struct SchedMeters {
  int64_t ticks = 0, admitted = 0, retired = 0, shed = 0, decode_passes = 0, decode_tokens = 0;
  int64_t prefill_tokens = 0, prefill_calls = 0, prefix_hit_tokens = 0, cancelled = 0;
  int64_t queue_peak = 0, active_peak = 0;
  int64_t mixed_passes = 0;      // engine calls that carried a prefill piece and a decode step together
};

class Scheduler {
 public:
  Scheduler(SchedulerEngine* engine, SchedulerConfig cfg, SchedulerObserver* obs = nullptr)
      : eng_(engine), cfg_(cfg), obs_(obs),
        cache_(engine->block_tokens(), cfg.prefix_max_entries),
        slots_(static_cast<size_t>(engine->max_concurrent())) {}

  ~Scheduler() {
    cache_.clear([this](int32_t b) { eng_->release_block(b); });
  }

  void submit(SchedRequest req) {
    fold("submit", req.id, static_cast<int64_t>(req.prompt.size()));
    Pending p;
    p.req = std::move(req);
    p.arrival = next_arrival_++;
    queue_.push_back(std::move(p));
    meters_.queue_peak = std::max<int64_t>(meters_.queue_peak, static_cast<int64_t>(queue_.size()));
  }

  void cancel(const std::string& id) { cancels_.push_back(id); }

  bool idle() const { return queue_.empty() && active_count() == 0; }
  int active_count() const {
    int n = 0;
    for (const auto& s : slots_) n += s.live ? 1 : 0;
    return n;
  }
  int64_t queued() const { return static_cast<int64_t>(queue_.size()); }
  const SchedMeters& meters() const { return meters_; }
  const PrefixStats& prefix_stats() const { return cache_.stats(); }
  uint64_t op_digest() const { return digest_; }
  uint64_t prefix_digest() const { return cache_.digest(); }
  int64_t now() const { return meters_.ticks; }

  // Returns the number of tokens produced in this tick.
  int64_t tick() {
    ++meters_.ticks;
    int64_t produced = 0;
    sweep_cancels();
    if (cfg_.policy == AdmissionPolicy::GrowOnDemand) grow_reservations();
    admit();
    tick_prefill_used_ = 0;
    const bool decoded = cfg_.mixed_pass && mixed_pass(&produced);
    produced += advance_prefills();
    if (!decoded) produced += decode_pass();
    meters_.active_peak = std::max<int64_t>(meters_.active_peak, active_count());
    return produced;
  }

  // Convenience: tick until everything submitted has retired (bounded by max_ticks).
  int64_t run(int64_t max_ticks = 1 << 30) {
    int64_t total = 0;
    for (int64_t t = 0; t < max_ticks && !idle(); ++t) total += tick();
    return total;
  }

 private:
  struct Pending {
    SchedRequest req;
    int64_t arrival = 0;
    std::vector<int32_t> generated;  // non-empty when a shed request comes back
  };
  enum class Phase { Prefill, Decode };
  struct Slot {
    bool live = false;
    Phase phase = Phase::Prefill;
    SchedRequest req;
    int64_t arrival = 0;
    std::vector<int32_t> tokens;     // prompt followed by generated tokens
    int64_t prompt_len = 0;          // length of the sequence to prefill (prompt + regenerated tail after a shed)
    int64_t prefilled = 0;           // positions whose KV is in the cache
    int64_t generated = 0;
    int64_t reserved = 0;            // positions covered by reserved blocks
    int64_t cached = 0;              // positions attached from the prefix cache
    int64_t already_emitted = 0;     // tokens a shed request had emitted before (not re-reported)
  };

  void fold(const char* op, const std::string& id, int64_t v) {
    digest_ = fnv1a_bytes(digest_, op, strlen_(op));
    digest_ = fnv1a_bytes(digest_, id.data(), id.size());
    digest_ = fnv1a_bytes(digest_, &v, sizeof(v));
  }
  static size_t strlen_(const char* s) { size_t n = 0; while (s[n]) ++n; return n; }

  int64_t blocks_for(int64_t tokens) const {
    const int64_t b = eng_->block_tokens();
    return (tokens + b - 1) / b;
  }

  void sweep_cancels() {
    for (const std::string& id : cancels_) {
      bool found = false;
      for (size_t s = 0; s < slots_.size(); ++s) {
        if (slots_[s].live && slots_[s].req.id == id) {
          retire(static_cast<int>(s), RetireReason::Cancelled);
          found = true;
          break;
        }
      }
      if (!found) {
        for (auto it = queue_.begin(); it != queue_.end(); ++it) {
          if (it->req.id == id) {
            fold("cancel_queued", id, 0);
            if (obs_) obs_->on_retire(id, RetireReason::Cancelled, static_cast<int64_t>(it->generated.size()));
            ++meters_.cancelled;
            queue_.erase(it);
            break;
          }
        }
      }
    }
    cancels_.clear();
  }

  // Youngest live request goes back to the head of the queue, keeping what it generated so far.
  bool shed_youngest(int except_slot) {
    int victim = -1;
    for (size_t s = 0; s < slots_.size(); ++s) {
      if (!slots_[s].live || static_cast<int>(s) == except_slot) continue;
      if (victim < 0 || slots_[s].arrival > slots_[victim].arrival) victim = static_cast<int>(s);
    }
    if (victim < 0) return false;
    Slot& v = slots_[victim];
    Pending p;
    p.req = v.req;
    p.arrival = v.arrival;
    p.generated.assign(v.tokens.begin() + static_cast<int64_t>(v.req.prompt.size()), v.tokens.end());
    fold("shed", v.req.id, v.generated);
    ++meters_.shed;
    eng_->close(victim);
    v = Slot();
    // keep FIFO order by arrival
    auto pos = queue_.begin();
    while (pos != queue_.end() && pos->arrival < p.arrival) ++pos;
    queue_.insert(pos, std::move(p));
    return true;
  }

  bool ensure_reserved(int s, int64_t tokens) {
    Slot& sl = slots_[s];
    if (tokens <= sl.reserved) return true;
    for (;;) {
      if (eng_->reserve(s, tokens)) {
        sl.reserved = blocks_for(tokens) * eng_->block_tokens();
        return true;
      }
      const int64_t need = blocks_for(tokens) - blocks_for(sl.reserved);
      const int64_t freed = cache_.evict_to_free(
          need, [this](int32_t b) { return eng_->block_refcount(b); }, [this](int32_t b) { eng_->release_block(b); });
      if (freed > 0) continue;
      return false;
    }
  }

  void grow_reservations() {
    // oldest first, so the youngest is the one that finds the pool dry
    std::vector<int> order;
    for (size_t s = 0; s < slots_.size(); ++s)
      if (slots_[s].live && slots_[s].phase == Phase::Decode) order.push_back(static_cast<int>(s));
    std::sort(order.begin(), order.end(), [this](int a, int b) { return slots_[a].arrival < slots_[b].arrival; });
    for (int s : order) {
      if (!slots_[s].live) continue;
      const int64_t want = static_cast<int64_t>(slots_[s].tokens.size()) + cfg_.grow_margin_tokens +
                           eng_->max_tokens_per_step() - 1;
      while (slots_[s].live && !ensure_reserved(s, want)) {
        if (!shed_youngest(s)) {
          retire(s, RetireReason::Error);
          break;
        }
      }
    }
  }

  int free_slot() const {
    for (size_t s = 0; s < slots_.size(); ++s)
      if (!slots_[s].live) return static_cast<int>(s);
    return -1;
  }

  void admit() {
    while (!queue_.empty()) {
      const int s = free_slot();
      if (s < 0) return;
      Pending& p = queue_.front();
      const int64_t seq_len = static_cast<int64_t>(p.req.prompt.size() + p.generated.size());
      const int64_t remaining = p.req.max_tokens - static_cast<int64_t>(p.generated.size());
      const int64_t total = seq_len + std::max<int64_t>(remaining, 1);
      if (seq_len == 0 || total > eng_->max_context()) {
        fold("reject", p.req.id, total);
        if (obs_) obs_->on_retire(p.req.id, RetireReason::Error, 0);
        queue_.pop_front();
        continue;
      }
      Slot sl;
      sl.live = true;
      sl.req = p.req;
      sl.arrival = p.arrival;
      sl.tokens = p.req.prompt;
      sl.tokens.insert(sl.tokens.end(), p.generated.begin(), p.generated.end());
      sl.prompt_len = seq_len;
      sl.generated = static_cast<int64_t>(p.generated.size());
      sl.already_emitted = sl.generated;
      // prefix lookup (over the sequence to prefill)
      PrefixHit hit;
      if (cfg_.prefix_cache && sl.req.prefix_cache && seq_len >= cfg_.prefix_min_tokens)
        hit = cache_.lookup(sl.tokens.data(), seq_len, meters_.ticks);
      if (hit.tokens > 0) {
        const int64_t keep = std::max<int64_t>(0, std::min<int64_t>(eng_->usable_prefix(hit.blocks), static_cast<int64_t>(hit.blocks.size())));
        if (keep < static_cast<int64_t>(hit.blocks.size())) {
          hit.blocks.resize(static_cast<size_t>(keep));
          hit.tokens = keep * eng_->block_tokens();
        }
      }
      slots_[s] = std::move(sl);
      Slot& cur = slots_[s];
      if (hit.tokens > 0) {
        eng_->attach_prefix(s, hit.blocks);
        cur.cached = cur.prefilled = cur.reserved = hit.tokens;
      }
      const int64_t want = cfg_.policy == AdmissionPolicy::FullReserve
                               ? total + eng_->max_tokens_per_step() - 1
                               : seq_len + cfg_.grow_margin_tokens + eng_->max_tokens_per_step() - 1;   // (a request may
                               // finish its prefill and take its first decode pass in the tick that admitted it)
      if (!ensure_reserved(s, want)) {
        // not enough blocks even after evicting the prefix cache: wait for a retirement
        eng_->close(s);
        slots_[s] = Slot();
        if (active_count() == 0) {
          // nothing will ever free blocks: the request cannot run
          fold("reject", queue_.front().req.id, want);
          if (obs_) obs_->on_retire(queue_.front().req.id, RetireReason::Error, 0);
          queue_.pop_front();
          continue;
        }
        return;
      }
      fold("admit", cur.req.id, (static_cast<int64_t>(s) << 40) | hit.tokens);
      ++meters_.admitted;
      meters_.prefix_hit_tokens += hit.tokens;
      eng_->open(s, cur.req.id);
      if (obs_) obs_->on_admit(cur.req.id, s, hit.tokens);
      queue_.pop_front();
    }
  }

  // The oldest reader's next chunk together with one decode step of everybody who is decoding.  True when the engine
  // ran the mixed pass (the tick then needs no decode pass of its own); the chunk counts against the tick's budget.
  bool mixed_pass(int64_t* produced) {
    std::vector<int> batch;
    int reader = -1;
    for (size_t s = 0; s < slots_.size(); ++s) {
      if (!slots_[s].live) continue;
      if (slots_[s].phase == Phase::Decode) batch.push_back(static_cast<int>(s));
      else if (slots_[s].phase == Phase::Prefill && (reader < 0 || slots_[s].arrival < slots_[reader].arrival))
        reader = static_cast<int>(s);
    }
    if (batch.empty() || reader < 0) return false;
    Slot& sl = slots_[reader];
    const int64_t left = sl.prompt_len - sl.prefilled;
    const int64_t n = std::min<int64_t>({left, cfg_.prefill_budget_busy, cfg_.prefill_chunk});
    if (n <= 0) return false;
    const SchedulerEngine::PrefillPiece piece{reader, sl.tokens.data() + sl.prefilled, sl.prefilled, n, n == left};
    int32_t first = -1;
    std::vector<std::vector<int32_t>> out;
    if (!eng_->mixed_step(piece, batch, &first, &out) || out.size() != batch.size()) return false;
    ++meters_.mixed_passes;
    ++meters_.prefill_calls;
    ++meters_.decode_passes;
    fold("prefill", sl.req.id, (sl.prefilled << 20) | n);
    meters_.prefill_tokens += n;
    sl.prefilled += n;
    tick_prefill_used_ += n;
    // the decoders first (their tokens were computed against the state before this pass), then the reader's first token
    int64_t got = 0;
    for (size_t i = 0; i < batch.size(); ++i) {
      const int s = batch[i];
      slots_[s].prefilled = static_cast<int64_t>(slots_[s].tokens.size());
      for (int32_t t : out[i]) {
        if (!slots_[s].live) break;
        got += accept_token(s, t) ? 1 : 0;
      }
    }
    meters_.decode_tokens += got;
    if (piece.last) {
      sl.phase = Phase::Decode;
      publish(reader, sl.prompt_len);
      got += accept_token(reader, first) ? 1 : 0;
    }
    *produced += got;
    return true;
  }

  int64_t advance_prefills() {
    bool decoders = false;
    for (const auto& s : slots_) decoders |= s.live && s.phase == Phase::Decode;
    int64_t budget = (decoders ? cfg_.prefill_budget_busy : cfg_.prefill_budget_idle) - tick_prefill_used_;
    int64_t produced = 0;
    // oldest reader first
    std::vector<int> order;
    for (size_t s = 0; s < slots_.size(); ++s)
      if (slots_[s].live && slots_[s].phase == Phase::Prefill) order.push_back(static_cast<int>(s));
    std::sort(order.begin(), order.end(), [this](int a, int b) { return slots_[a].arrival < slots_[b].arrival; });
    if (cfg_.prefill_group_max > 1 && order.size() > 1) return advance_prefill_group(order, budget);
    for (int s : order) {
      while (budget > 0 && slots_[s].live && slots_[s].phase == Phase::Prefill) {
        Slot& sl = slots_[s];
        const int64_t left = sl.prompt_len - sl.prefilled;
        const int64_t n = std::min<int64_t>({left, budget, cfg_.prefill_chunk});
        const bool last = n == left;
        const int32_t tok = eng_->prefill(s, sl.tokens.data() + sl.prefilled, sl.prefilled, n, last);
        fold("prefill", sl.req.id, (sl.prefilled << 20) | n);
        ++meters_.prefill_calls;
        meters_.prefill_tokens += n;
        sl.prefilled += n;
        budget -= n;
        if (last) {
          sl.phase = Phase::Decode;
          publish(s, sl.prompt_len);
          produced += accept_token(s, tok) ? 1 : 0;
        }
      }
      if (budget <= 0) break;
    }
    return produced;
  }

  // Readers in `order` (oldest first) advance together: per engine call at most prefill_group_max pieces and
  // prefill_chunk tokens; a call's token room is split evenly over its readers, what is left goes to the readers
  // closest to the end of their prompt, so a long prompt cannot starve the short ones behind it.
  int64_t advance_prefill_group(const std::vector<int>& order, int64_t budget) {
    int64_t produced = 0;
    for (;;) {
      std::vector<int> readers;
      for (int s : order)
        if (slots_[s].live && slots_[s].phase == Phase::Prefill &&
            static_cast<int>(readers.size()) < cfg_.prefill_group_max) readers.push_back(s);
      int64_t room = std::min<int64_t>(budget, cfg_.prefill_chunk);
      if (readers.empty() || room <= 0) break;
      // even shares, then the leftovers to the oldest readers that still have prompt left
      std::vector<int64_t> take(readers.size(), 0);
      const int64_t share = std::max<int64_t>(1, room / static_cast<int64_t>(readers.size()));
      int64_t used = 0;
      for (size_t i = 0; i < readers.size() && used < room; ++i) {
        const Slot& sl = slots_[readers[i]];
        take[i] = std::min<int64_t>({sl.prompt_len - sl.prefilled, share, room - used});
        used += take[i];
      }
      // leftovers: the reader closest to the end of its prompt first (it reaches its first token in this call), age
      // breaks ties
      std::vector<size_t> by_need(readers.size());
      for (size_t i = 0; i < by_need.size(); ++i) by_need[i] = i;
      std::stable_sort(by_need.begin(), by_need.end(), [&](size_t a, size_t b) {
        const Slot& x = slots_[readers[a]];
        const Slot& y = slots_[readers[b]];
        return x.prompt_len - x.prefilled - take[a] < y.prompt_len - y.prefilled - take[b];
      });
      for (size_t k = 0; k < by_need.size() && used < room; ++k) {
        const size_t i = by_need[k];
        const Slot& sl = slots_[readers[i]];
        const int64_t more = std::min<int64_t>(sl.prompt_len - sl.prefilled - take[i], room - used);
        take[i] += more;
        used += more;
      }
      std::vector<SchedulerEngine::PrefillPiece> pieces;
      std::vector<int> who;
      for (size_t i = 0; i < readers.size(); ++i) {
        if (take[i] <= 0) continue;
        const Slot& sl = slots_[readers[i]];
        pieces.push_back({readers[i], sl.tokens.data() + sl.prefilled, sl.prefilled, take[i],
                          take[i] == sl.prompt_len - sl.prefilled});
        who.push_back(readers[i]);
      }
      if (pieces.empty()) break;
      const std::vector<int32_t> firsts = eng_->prefill_group(pieces);
      ++meters_.prefill_calls;
      for (size_t i = 0; i < pieces.size(); ++i) {
        const int s = who[i];
        Slot& sl = slots_[s];
        fold("prefill", sl.req.id, (sl.prefilled << 20) | pieces[i].count);
        meters_.prefill_tokens += pieces[i].count;
        sl.prefilled += pieces[i].count;
        budget -= pieces[i].count;
        if (pieces[i].last) {
          sl.phase = Phase::Decode;
          publish(s, sl.prompt_len);
          produced += accept_token(s, firsts[i]) ? 1 : 0;
        }
      }
    }
    return produced;
  }

  int64_t decode_pass() {
    std::vector<int> batch;
    for (size_t s = 0; s < slots_.size(); ++s)
      if (slots_[s].live && slots_[s].phase == Phase::Decode) batch.push_back(static_cast<int>(s));
    if (batch.empty()) return 0;
    ++meters_.decode_passes;
    const auto out = eng_->step_batch(batch);
    int64_t produced = 0;
    for (size_t i = 0; i < batch.size(); ++i) {
      const int s = batch[i];
      slots_[s].prefilled = static_cast<int64_t>(slots_[s].tokens.size());
      for (int32_t t : out[i]) {
        if (!slots_[s].live) break;
        produced += accept_token(s, t) ? 1 : 0;
      }
    }
    meters_.decode_tokens += produced;
    return produced;
  }

  // Appends a token; returns true when it was delivered (not a swallowed eos/stop).
  bool accept_token(int s, int32_t tok) {
    Slot& sl = slots_[s];
    const bool is_eos = !sl.req.ignore_eos &&
                        std::find(sl.req.eos_ids.begin(), sl.req.eos_ids.end(), tok) != sl.req.eos_ids.end();
    const bool is_stop = std::find(sl.req.stop_ids.begin(), sl.req.stop_ids.end(), tok) != sl.req.stop_ids.end();
    if (is_eos || is_stop) {
      fold("eos", sl.req.id, tok);
      retire(s, is_eos ? RetireReason::Eos : RetireReason::Stop);
      return false;
    }
    sl.tokens.push_back(tok);
    ++sl.generated;
    fold("token", sl.req.id, tok);
    if (obs_ && sl.generated > sl.already_emitted) obs_->on_token(sl.req.id, tok, sl.generated - 1);
    if (sl.generated >= sl.req.max_tokens) retire(s, RetireReason::Length);
    return true;
  }

  void publish(int s, int64_t tokens) {
    Slot& sl = slots_[s];
    if (!cfg_.prefix_cache || !sl.req.prefix_cache || tokens < cfg_.prefix_min_tokens) return;
    const auto blocks = eng_->slot_blocks(s);
    cache_.insert(
        sl.tokens.data(), tokens, blocks, meters_.ticks, !sl.req.cache_key.empty(),
        [this](int32_t b) { eng_->retain_block(b); }, [this](int32_t b) { eng_->release_block(b); });
  }

  void retire(int s, RetireReason why) {
    Slot& sl = slots_[s];
    // positions whose KV is complete: everything but the last token (never fed back through the model)
    if (why != RetireReason::Error && why != RetireReason::Cancelled && sl.phase == Phase::Decode)
      publish(s, std::min<int64_t>(sl.prefilled, static_cast<int64_t>(sl.tokens.size())));
    fold("retire", sl.req.id, static_cast<int64_t>(why));
    ++meters_.retired;
    if (why == RetireReason::Cancelled) ++meters_.cancelled;
    if (obs_) obs_->on_retire(sl.req.id, why, sl.generated);
    eng_->close(s);
    sl = Slot();
  }

  SchedulerEngine* eng_;
  SchedulerConfig cfg_;
  SchedulerObserver* obs_;
  PrefixCache cache_;
  std::vector<Slot> slots_;
  std::deque<Pending> queue_;
  std::vector<std::string> cancels_;
  SchedMeters meters_;
  int64_t tick_prefill_used_ = 0;      // prompt tokens a mixed pass already took out of this tick's budget
  int64_t next_arrival_ = 0;
  uint64_t digest_ = kFnvSeed;
};

}  // namespace dgpp
