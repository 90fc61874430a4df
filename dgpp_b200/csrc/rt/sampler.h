// Host oracle of the token sampler.  The device sampler (csrc/kernels/sample.cu) implements the same steps
// with the same deterministic math, so both produce identical tokens for identical inputs.
//
// Order of operations for one row of logits:
//   1. penalties over the request's token counts: repetition (divide positive / multiply negative logits of
//      seen tokens), presence (subtract once), frequency (subtract count times)
//   2. logit_bias, then the grammar mask (disallowed ids -> -inf)
//   3. temperature == 0 (or top_p == 0): greedy, ties to the lowest token id
//   4. z = logits / temperature; row-wide (max, sum exp) over fixed 256-wide chunks folded pairwise
//   5. candidates = a prefix of the canonical order (value descending, id ascending), 128 wide at first
//   6. top_k / min_p / top_p / draw on that prefix (common/sampler_core.h); when the prefix cannot resolve the
//      draw it is widened: 1,024 -> 8,192 -> 65,536 -> the whole vocabulary
//   7. u = uniform01(seed, position)
// Log-probabilities describe the filtered, renormalised distribution when temperature > 0 and the raw
// distribution when temperature == 0.
// Sharded vocabularies: each rank reports its top candidates and a slice log-sum-exp computed over fixed
// 256-wide chunks and folded pairwise; slices are merged in ascending rank order (merge_logsumexp).
// (behavioural spec: src/sample/sampler.hpp:378-1422 and lines 2125-2296 of its top-level design document, both in the reference tree.)
#pragma once
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <limits>
#include <map>
#include <utility>
#include <vector>

#include "common/det_math.h"
#include "common/sampler_core.h"

namespace dgpp {
namespace sample {

struct Params {
  float temperature = 0.f;
  int top_k = 0;          // 0 = off
  float top_p = 1.f;
  float min_p = 0.f;
  float repetition_penalty = 1.f;
  float presence_penalty = 0.f;
  float frequency_penalty = 0.f;
  uint64_t seed = 0;
  int top_logprobs = 0;   // how many alternatives to report
  std::map<int32_t, float> logit_bias;
};

struct Result {
  int32_t token = -1;
  float logprob = 0.f;
  std::vector<std::pair<int32_t, float>> top;  // (token, logprob), best first
  int candidates_used = 0;                     // width of the candidate prefix that resolved the draw
};

constexpr int kLseChunk = 256;

// log-sum-exp of a slice: per-chunk (max, sum) in index order, then a pairwise tree over the chunks.
inline std::pair<float, float> slice_max_sum(const float* x, int64_t n) {
  std::vector<std::pair<float, float>> parts;
  for (int64_t c = 0; c < n; c += kLseChunk) {
    const int64_t e = std::min<int64_t>(n, c + kLseChunk);
    float m = -std::numeric_limits<float>::infinity();
    for (int64_t i = c; i < e; ++i) m = x[i] > m ? x[i] : m;
    float s = 0.f;
    if (m > -std::numeric_limits<float>::infinity())
      for (int64_t i = c; i < e; ++i) s = s + det::exp(x[i] - m);
    parts.emplace_back(m, s);
  }
  while (parts.size() > 1) {
    std::vector<std::pair<float, float>> next;
    for (size_t i = 0; i + 1 < parts.size(); i += 2) {
      const auto& a = parts[i];
      const auto& b = parts[i + 1];
      const float m = a.first > b.first ? a.first : b.first;
      float s = 0.f;
      if (m > -std::numeric_limits<float>::infinity())
        s = a.second * det::exp(a.first - m) + b.second * det::exp(b.first - m);
      next.emplace_back(m, s);
    }
    if (parts.size() & 1) next.push_back(parts.back());
    parts.swap(next);
  }
  if (parts.empty()) return {-std::numeric_limits<float>::infinity(), 0.f};
  return parts[0];
}
inline float slice_logsumexp(const float* x, int64_t n) {
  const auto ms = slice_max_sum(x, n);
  return ms.second > 0.f ? ms.first + det::log(ms.second) : -std::numeric_limits<float>::infinity();
}
// Fold per-rank (max, sum) pairs in ascending rank order.
inline float merge_logsumexp(const std::vector<std::pair<float, float>>& slices) {
  float m = -std::numeric_limits<float>::infinity();
  for (const auto& s : slices) m = s.first > m ? s.first : m;
  if (!(m > -std::numeric_limits<float>::infinity())) return m;
  float sum = 0.f;
  for (const auto& s : slices) sum = sum + s.second * det::exp(s.first - m);
  return m + det::log(sum);
}

inline void apply_penalties(std::vector<float>& l, const Params& p, const std::map<int32_t, int>& counts,
                            const std::vector<uint8_t>* allowed) {
  for (const auto& kv : counts) {
    if (kv.first < 0 || kv.first >= static_cast<int32_t>(l.size()) || kv.second <= 0) continue;
    float v = l[kv.first];
    if (p.repetition_penalty != 1.f) v = v > 0.f ? v / p.repetition_penalty : v * p.repetition_penalty;
    v = v - p.presence_penalty;
    v = v - p.frequency_penalty * static_cast<float>(kv.second);
    l[kv.first] = v;
  }
  for (const auto& kv : p.logit_bias)
    if (kv.first >= 0 && kv.first < static_cast<int32_t>(l.size())) l[kv.first] = l[kv.first] + kv.second;
  if (allowed)
    for (size_t i = 0; i < l.size(); ++i)
      if (!(*allowed)[i]) l[i] = -std::numeric_limits<float>::infinity();
}

inline int32_t argmax_lowest(const std::vector<float>& l) {
  int32_t best = 0;
  for (int32_t i = 1; i < static_cast<int32_t>(l.size()); ++i)
    if (l[i] > l[best]) best = i;
  return best;
}

inline Result sample(const std::vector<float>& logits, const Params& p, const std::map<int32_t, int>& counts,
                     uint64_t position, const std::vector<uint8_t>* allowed = nullptr, int candidates = 128) {
  std::vector<float> l = logits;
  apply_penalties(l, p, counts, allowed);
  Result r;
  const bool greedy = p.temperature <= 0.f || p.top_p <= 0.f;
  auto fill_top = [&](const std::vector<std::pair<float, int32_t>>& cand, float lse) {
    for (int i = 0; i < p.top_logprobs && i < static_cast<int>(cand.size()); ++i)
      r.top.emplace_back(cand[i].second, cand[i].first - lse);
  };
  if (greedy) {
    r.token = argmax_lowest(l);
    const float lse = slice_logsumexp(l.data(), static_cast<int64_t>(l.size()));
    r.logprob = l[r.token] - lse;
    if (p.top_logprobs > 0) {
      std::vector<std::pair<float, int32_t>> cand;
      for (int32_t i = 0; i < static_cast<int32_t>(l.size()); ++i) cand.emplace_back(l[i], i);
      const size_t k = std::min<size_t>(cand.size(), static_cast<size_t>(p.top_logprobs));
      std::partial_sort(cand.begin(), cand.begin() + k, cand.end(), [](const auto& a, const auto& b) {
        return a.first != b.first ? a.first > b.first : a.second < b.second;
      });
      cand.resize(k);
      fill_top(cand, lse);
    }
    return r;
  }
  const float inv_t = 1.f / p.temperature;
  std::vector<float> z(l.size());
  int64_t n_total = 0;
  for (size_t i = 0; i < l.size(); ++i) {
    z[i] = l[i] > -std::numeric_limits<float>::infinity() ? l[i] * inv_t : l[i];
    if (l[i] > -std::numeric_limits<float>::infinity()) ++n_total;
  }
  if (n_total == 0) { r.token = 0; return r; }
  const auto ms = slice_max_sum(z.data(), static_cast<int64_t>(z.size()));
  std::vector<std::pair<float, int32_t>> all;
  all.reserve(static_cast<size_t>(n_total));
  for (int32_t i = 0; i < static_cast<int32_t>(z.size()); ++i)
    if (l[i] > -std::numeric_limits<float>::infinity()) all.emplace_back(z[i], i);
  auto order = [](const std::pair<float, int32_t>& a, const std::pair<float, int32_t>& b) {
    return a.first != b.first ? a.first > b.first : a.second < b.second;
  };
  Filter f;
  f.temperature = p.temperature; f.top_k = p.top_k; f.top_p = p.top_p; f.min_p = p.min_p;
  const float u = det::uniform01(p.seed, position);
  // candidate prefix, widened until the draw resolves (the device sampler stops at its first width and asks the
  // host for the rest)
  const int64_t widths[5] = {candidates, 1024, 8192, 65536, n_total};
  size_t sorted = 0;
  for (int64_t w : widths) {
    const size_t c = static_cast<size_t>(std::min<int64_t>(std::max<int64_t>(w, 1), n_total));
    if (c <= sorted && c < static_cast<size_t>(n_total)) continue;
    if (c > sorted) {
      std::partial_sort(all.begin(), all.begin() + c, all.end(), order);
      sorted = c;
    }
    std::vector<float> pc(c);
    for (size_t i = 0; i < c; ++i) pc[i] = det::exp(all[i].first - ms.first);
    const Decision d = decide(pc.data(), static_cast<int>(c), n_total, ms.second, f, u);
    if (!d.resolved) continue;
    const float lse = ms.first + det::log(d.total);
    r.token = all[d.pick].second;
    r.logprob = all[d.pick].first - lse;
    r.candidates_used = static_cast<int>(c);
    all.resize(std::min<size_t>(c, static_cast<size_t>(d.keep)));
    fill_top(all, lse);
    return r;
  }
  r.token = all[0].second;  // unreachable: the full width always resolves
  return r;
}

// Greedy verification of a draft: accepted = length of the longest prefix where the target's pick after
// accepting draft[0..i) equals draft[i]; the token emitted after the accepted prefix is target[accepted].
inline int judge_verify(const std::vector<int32_t>& draft, const std::vector<int32_t>& target_picks) {
  int acc = 0;
  while (acc < static_cast<int>(draft.size()) && acc < static_cast<int>(target_picks.size()) &&
         draft[acc] == target_picks[acc])
    ++acc;
  return acc;
}

// Sampled verification (ratio rule): accept draft token d with probability min(1, P(d) / Q(d)); on rejection
// the replacement is drawn from the residual (P - Q)+ renormalised.  Returns (accepted?, token).
inline std::pair<bool, int32_t> spec_accept_ratio(const std::vector<float>& target_prob,
                                                  const std::vector<float>& draft_prob, int32_t draft_token,
                                                  uint64_t seed, uint64_t position) {
  const float pt = target_prob[draft_token], qd = draft_prob[draft_token];
  const float u = det::uniform01(seed, position * 2);
  if (qd <= 0.f || u * qd < pt) return {true, draft_token};
  float total = 0.f;
  for (size_t i = 0; i < target_prob.size(); ++i) {
    const float d = target_prob[i] - draft_prob[i];
    if (d > 0.f) total = total + d;
  }
  if (total <= 0.f) return {false, draft_token};
  const float v = det::uniform01(seed, position * 2 + 1) * total;
  float cum = 0.f;
  int32_t last = draft_token;
  for (size_t i = 0; i < target_prob.size(); ++i) {
    const float d = target_prob[i] - draft_prob[i];
    if (d > 0.f) {
      cum = cum + d;
      last = static_cast<int32_t>(i);
      if (v < cum) return {false, last};
    }
  }
  return {false, last};
}

}  // namespace sample
}  // namespace dgpp
