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
// (reference counterparts: src/engine/speculative.hpp, verify_schedule.hpp, lookup_draft.hpp; the reference tree's own DESIGN.md:1934-2123.)
#pragma once
#include <algorithm>
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
