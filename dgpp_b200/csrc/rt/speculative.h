// Speculative decoding control (host side): drafts from an n-gram lookup over the request's own tokens, an
// adaptive verify schedule, and the accept / rollback transaction around one verify pass.
//
// One speculative step for a request:
//   1. draft    k tokens d[0..k) are proposed (lookup drafter here; an MTP head or a draft model plug in the same way)
//   2. verify   the target model runs ONE pass over the rows [last, d0, .., d(k-1)] (k + 1 rows, causal) and picks a
//               token for each row: t[0..k]
//   3. judge    accepted = longest prefix with d[i] == t[i]; the step emits d[0..accepted) followed by t[accepted]
//               (the target's own token after the accepted prefix), i.e. accepted + 1 tokens, all of them exactly
//               the tokens plain greedy decoding would have produced
//   4. commit   the KV / recurrent state of the rejected rows is rolled back: positions >= base + accepted + 1 are
//               discarded (paged KV: the length is cut; recurrent layers: restore the snapshot taken before the
//               pass and replay the accepted rows)
// The schedule shrinks the draft when acceptance is poor and widens it when drafts keep landing.
// (reference counterparts: src/engine/speculative.hpp, verify_schedule.hpp, lookup_draft.hpp; lines 1934-2123 of its top-level design document.)
#pragma once
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <unordered_map>
#include <vector>

namespace dgpp {
namespace spec {

// Proposes the continuation that followed the most recent earlier occurrence of the current suffix.
class LookupDraft {
 public:
  explicit LookupDraft(int min_ngram = 2, int max_ngram = 4) : min_n_(min_ngram), max_n_(max_ngram) {}

  void reset() { tokens_.clear(); index_.clear(); }
  void append(const std::vector<int32_t>& toks) { for (int32_t t : toks) push(t); }
  void push(int32_t t) {
    tokens_.push_back(t);
    const int64_t n = static_cast<int64_t>(tokens_.size());
    // index the n-grams that END at the previous token: their continuation (this token) is now known
    for (int g = min_n_; g <= max_n_; ++g) {
      if (n - 1 < g) break;
      index_[key(n - 1 - g, g)] = n - 1;    // position of the continuation; later occurrences overwrite earlier ones
    }
  }
  // Up to `k` draft tokens; empty when no earlier occurrence of the suffix exists.
  std::vector<int32_t> propose(int k) const {
    std::vector<int32_t> out;
    const int64_t n = static_cast<int64_t>(tokens_.size());
    for (int g = max_n_; g >= min_n_ && out.empty(); --g) {
      if (n < g) continue;
      auto it = index_.find(key(n - g, g));
      if (it == index_.end()) continue;
      for (int64_t p = it->second; p < n && static_cast<int>(out.size()) < k; ++p) out.push_back(tokens_[p]);
    }
    return out;
  }
  size_t size() const { return tokens_.size(); }

 private:
  uint64_t key(int64_t start, int g) const {
    uint64_t h = 1469598103934665603ull ^ static_cast<uint64_t>(g);
    for (int i = 0; i < g; ++i) {
      h ^= static_cast<uint32_t>(tokens_[start + i]);
      h *= 1099511628211ull;
    }
    return h;
  }
  int min_n_, max_n_;
  std::vector<int32_t> tokens_;
  std::unordered_map<uint64_t, int64_t> index_;
};

// Draft length controller: exponential moving average of accepted / proposed.
class VerifySchedule {
 public:
  VerifySchedule(int min_draft = 0, int max_draft = 7, int start = 3) : min_(min_draft), max_(max_draft), cur_(start) {}
  int draft_len() const { return cur_; }
  double acceptance() const { return ema_; }
  void observe(int proposed, int accepted) {
    if (proposed <= 0) return;
    const double rate = static_cast<double>(accepted) / proposed;
    ema_ = seen_ ? 0.8 * ema_ + 0.2 * rate : rate;
    seen_ = true;
    if (accepted == proposed && cur_ < max_) ++cur_;            // everything landed: try one more
    else if (ema_ < 0.3 && cur_ > min_) --cur_;                 // mostly wasted rows: draft less
    ++steps_;
    proposed_ += proposed;
    accepted_ += accepted;
  }
  int64_t steps() const { return steps_; }
  int64_t proposed_total() const { return proposed_; }
  int64_t accepted_total() const { return accepted_; }

 private:
  int min_, max_, cur_;
  double ema_ = 0.0;
  bool seen_ = false;
  int64_t steps_ = 0, proposed_ = 0, accepted_ = 0;
};

// Verify depth from the drafter's own confidence.  A drafter that emits, per draft position, a logit c_i of "this draft
// survives given that the ones before it did" lets the engine decide how many of the block's drafts are worth a verify
// row: with p_i = scale / (1 + exp(-c_i)) and S_i = p_1 .. p_i (non-increasing), verifying k drafts commits
// 1 + S_1 + .. + S_k tokens in expectation and costs base + (1 + k) rows of time.  Throughput over a whole run is a
// ratio of sums, whose optimum (Dinkelbach) is a linear trade per step at one multiplier lambda = the throughput the
// run achieves (tokens per ms): draft i is verified while S_i > lambda * row_ms, and the first one that fails ends the
// prefix.  lambda is tracked here as a moving average of committed tokens over MODELLED step time (base + rows * row,
// never a clock: every rank must derive the same depth from the same replicated inputs) and is never allowed below the
// rate of a plain one-token step, 1 / (base + row).  The depth changes how many rows a step verifies, never which
// tokens it emits.
class ConfidenceDepth {
 public:
  ConfidenceDepth(double base_ms, double row_ms, double ema = 0.1)
      : base_(base_ms), row_(row_ms), ema_(ema), floor_(base_ms + row_ms > 0.0 ? 1.0 / (base_ms + row_ms) : 0.0),
        lambda_(floor_) {}

  double lambda() const { return lambda_; }
  double floor() const { return floor_; }

  // One request: leading drafts to verify, 0 .. conf.size().  accept_scale < 1 for a sampled request whose drafts are
  // arg-max tokens (they are accepted with the target's probability of the draft, not whenever they are the arg-max).
  int depth(const std::vector<float>& conf, double accept_scale = 1.0) const {
    const double limit = lambda_ * row_;
    double survive = 1.0;
    int k = 0;
    for (size_t i = 0; i < conf.size(); ++i) {
      survive *= accept_scale / (1.0 + std::exp(-static_cast<double>(conf[i])));
      if (!(survive > limit)) break;
      k = static_cast<int>(i) + 1;
    }
    return k;
  }

  // A batch that replays ONE graph for all its requests shares one depth: a further position costs one row per request
  // and yields the sum of their survivals there, so it is kept while the MEAN survival beats lambda * row.
  int depth_batch(const std::vector<std::vector<float>>& conf, const std::vector<double>& accept_scale = {}) const {
    if (conf.empty()) return 0;
    size_t block = conf[0].size();
    for (const auto& c : conf) block = std::min(block, c.size());
    const double limit = lambda_ * row_;
    std::vector<double> survive(conf.size(), 1.0);
    int k = 0;
    for (size_t i = 0; i < block; ++i) {
      double sum = 0.0;
      for (size_t s = 0; s < conf.size(); ++s) {
        const double scale = s < accept_scale.size() ? accept_scale[s] : 1.0;
        survive[s] *= scale / (1.0 + std::exp(-static_cast<double>(conf[s][i])));
        sum += survive[s];
      }
      if (!(sum / static_cast<double>(conf.size()) > limit)) break;
      k = static_cast<int>(i) + 1;
    }
    return k;
  }

  // After a step that ran `rows` verify rows in all and committed `committed` tokens in all.
  void observe(int committed, int rows) {
    const double t = base_ + static_cast<double>(rows) * row_;
    if (!(t > 0.0) || committed < 0) return;
    lambda_ += ema_ * (static_cast<double>(committed) / t - lambda_);
    if (lambda_ < floor_) lambda_ = floor_;
  }

 private:
  double base_, row_, ema_, floor_, lambda_;
};

struct Verdict {
  int accepted = 0;                 // draft tokens kept
  std::vector<int32_t> emitted;     // accepted draft tokens + the target's token after them
  int64_t keep_length = 0;          // sequence length (positions) that stays committed after the step
};

// Greedy judgement of one verify pass.  base = tokens committed before the pass (the row of `last` sits at
// position base - 1 + 1 ... the pass wrote positions base .. base + k).  target has k + 1 picks.
inline Verdict judge(int64_t base, const std::vector<int32_t>& draft, const std::vector<int32_t>& target,
                     const std::vector<int32_t>& stop_ids = {}, int64_t budget = -1) {
  Verdict v;
  const int k = static_cast<int>(draft.size());
  while (v.accepted < k && v.accepted < static_cast<int>(target.size()) && draft[v.accepted] == target[v.accepted]) ++v.accepted;
  for (int i = 0; i < v.accepted; ++i) v.emitted.push_back(draft[i]);
  if (v.accepted < static_cast<int>(target.size())) v.emitted.push_back(target[v.accepted]);
  // a stop token or the token budget cuts the emission (and with it the accepted rows)
  size_t cut = v.emitted.size();
  for (size_t i = 0; i < v.emitted.size(); ++i)
    if (std::find(stop_ids.begin(), stop_ids.end(), v.emitted[i]) != stop_ids.end()) { cut = i + 1; break; }
  if (budget >= 0 && static_cast<int64_t>(cut) > budget) cut = static_cast<size_t>(budget);
  v.emitted.resize(cut);
  v.accepted = std::min<int>(v.accepted, static_cast<int>(cut));
  // rows whose KV stays: the input row (position base) and the accepted draft rows
  v.keep_length = base + 1 + std::min<int64_t>(v.accepted, cut ? static_cast<int64_t>(cut) - 1 : 0);
  return v;
}

}  // namespace spec
}  // namespace dgpp
