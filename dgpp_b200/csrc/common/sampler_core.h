// The filter-and-draw step of the sampler, shared verbatim by the host oracle and the device kernel.
//
// Inputs: the row's candidates p[i] = exp(z[i] - m), z = logits / temperature, in canonical order (value descending, token id
// ascending), the number of tokens with a finite logit in the whole vocabulary (n_total), and the row-wide
// (max m, sum s of exp(z - m)) computed over fixed 256-wide chunks folded pairwise.  The candidate list is a
// PREFIX of the full canonical order; the step either resolves the draw inside that prefix or reports that a
// longer prefix is needed (the caller widens: 128 -> 1,024 -> 8,192 -> 65,536 -> everything).
//
//   top_k   : the distribution is the first k candidates, total = their sum in canonical order
//             (k beyond the prefix: widen).  Without top_k the total is the row-wide sum s.
//   min_p   : keep the prefix with p >= min_p * p[0]; total = sum of the kept prefix
//   top_p   : keep the shortest prefix whose mass reaches top_p * total; total = sum of that prefix
//   draw    : walk the kept prefix until u * total < cumulative sum
// All sums run in canonical order with plain float adds; exp is det::exp.
// (behavioural spec: src/sample/sampler.hpp and lines 2125-2296 of its top-level design document, both in the reference tree.)
#pragma once
#include <stdint.h>

#include "common/det_math.h"

namespace dgpp {
namespace sample {

struct Filter {
  float temperature;
  int top_k;      // 0 = off
  float top_p;    // 1 = off
  float min_p;    // 0 = off
};

struct Decision {
  int resolved;   // 0: the candidate prefix is too short
  int pick;       // index into the candidate list
  int keep;       // size of the final support (may exceed n_cand only when unfiltered)
  float total;    // mass of the final support, in units of exp(z - m)
};

// p[i] = det::exp(z[i] - m) of the candidate prefix (computed by the caller, in parallel on the device).
DGPP_HD Decision decide(const float* p, int n_cand, int64_t n_total, float s, const Filter& f, float u) {
  Decision d;
  d.resolved = 0; d.pick = 0; d.keep = 0; d.total = 0.f;
  if (n_cand <= 0 || n_total <= 0) return d;
  int64_t keep = n_total;
  float total = s;
  if (f.top_k > 0 && f.top_k < n_total) {
    if (f.top_k > n_cand) return d;
    keep = f.top_k;
    total = 0.f;
    for (int i = 0; i < f.top_k; ++i) total = total + p[i];
  }
  if (f.min_p > 0.f) {
    const float thr = f.min_p * p[0];
    const int lim = keep < n_cand ? static_cast<int>(keep) : n_cand;
    int k = 0;
    while (k < lim && p[k] >= thr) ++k;
    if (k == lim && lim < keep) return d;   // every candidate passed and more exist
    keep = k > 1 ? k : 1;
    total = 0.f;
    for (int i = 0; i < keep; ++i) total = total + p[i];
  }
  if (f.top_p < 1.f) {
    const float want = f.top_p * total;
    const int lim = keep < n_cand ? static_cast<int>(keep) : n_cand;
    float cum = 0.f;
    int k = 0;
    bool reached = false;
    while (k < lim) {
      cum = cum + p[k];
      ++k;
      if (cum >= want) { reached = true; break; }
    }
    if (!reached && lim < keep) return d;
    keep = k > 1 ? k : 1;
    total = 0.f;
    for (int i = 0; i < keep; ++i) total = total + p[i];
  }
  const float uu = u * total;
  const int lim = keep < n_cand ? static_cast<int>(keep) : n_cand;
  float cum = 0.f;
  int pick = -1;
  for (int i = 0; i < lim; ++i) {
    cum = cum + p[i];
    if (uu < cum) { pick = i; break; }
  }
  if (pick < 0) {
    if (lim < keep) return d;               // the draw falls beyond the prefix
    pick = lim - 1;                         // rounding left u * total at the very end of the support
  }
  d.resolved = 1;
  d.pick = pick;
  d.keep = static_cast<int>(keep < 0x7fffffff ? keep : 0x7fffffff);
  d.total = total;
  return d;
}

// Penalties + bias for one token (mask handled by the caller): repetition, presence, frequency, then bias.
DGPP_HD float adjust_logit(float v, int count, float repetition, float presence, float frequency, float bias) {
  if (count > 0) {
    if (repetition != 1.f) v = v > 0.f ? v / repetition : v * repetition;
    v = v - presence;
    v = v - frequency * static_cast<float>(count);
  }
  return v + bias;
}

}  // namespace sample
}  // namespace dgpp
