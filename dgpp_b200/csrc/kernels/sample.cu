// Device sampler: the steps of the host oracle (rt/sampler.h) with the same deterministic math, so both pick the
// same token for the same inputs.  Built with --fmad=false (no contraction), like the oracle.
//
//   sample_prepare_kernel  grid (chunks of 256, rows): penalties from the request's token-count row, logit_bias,
//                          grammar mask, temperature -> z (fp32 scratch); per-chunk (max, sum exp) in index order
//   sample_select_kernel   grid (rows), 1024 threads: pairwise fold of the chunk partials (the oracle's tree),
//                          greedy rows: argmax with ties to the lowest id; sampled rows: exact top-C candidates by
//                          an 8-pass radix select on the 64-bit key (ordered float bits, ~id), bitonic sort into
//                          canonical order, probabilities in parallel, then ONE thread runs the shared
//                          filter-and-draw step (common/sampler_core.h).  A row whose draw does not resolve inside
//                          the C-wide prefix is flagged; the host finishes it with the oracle's wider prefixes.
//   count kernels          per-slot token count rows for the penalties
// (reference counterparts: src/kernels/sample_pick.cu:247,321,500,1276,1903,1930.)
#include <math.h>
#include <string.h>

#include "common/common.h"
#include "common/det_math.h"
#include "common/ptx.cuh"
#include "common/sampler_core.h"

namespace dgpp {

constexpr int kChunk = 256;          // the oracle's kLseChunk
constexpr int kSelThreads = 1024;
constexpr int kMaxCand = 256;
constexpr int kMaxTop = 20;
constexpr int kMaxBias = 512;

struct SampleRow {
  float temperature, top_p, min_p;
  float repetition, presence, frequency;
  int top_k, top_logprobs;
  int slot;            // row of the count table, -1: no penalties
  int n_bias;          // entries of this row in the bias lists
  unsigned long long seed, position;
};

struct SampleArgs {
  const float* logits;       // [rows, ld]
  int64_t ld;
  const SampleRow* rows;     // [rows]
  const int32_t* counts;     // [slots, vocab] or null
  const int32_t* bias_ids;   // [rows, kMaxBias] or null
  const float* bias_vals;
  const uint32_t* mask;      // [rows, ceil(vocab / 32)] allowed bits, or null
  float* z;                  // [rows, vocab] scratch
  float2* parts;             // [rows, chunks] (max, sum)
  int32_t* out_token;        // [rows]
  float* out_logprob;        // [rows]
  int32_t* out_flags;        // [rows]: 1 resolved, 0 needs the host's wider prefix
  int32_t* out_top_ids;      // [rows, kMaxTop]
  float* out_top_lp;         // [rows, kMaxTop]
  int32_t* out_top_n;        // [rows]
  int vocab, chunks, candidates;
  // Vocabulary-sharded head: this rank holds ids [id_base, id_base + vocab) of a `vocab_total`-wide vocabulary (the count
  // table, the bias lists and the mask are indexed by global id).  local_only: stop after the slice's candidate table
  // (tp_cand [rows, candidates] keys, descending), its (max, sum) pair (tp_ms) and its support size (tp_nt);
  // sample_merge_kernel folds the ranks' tables.
  int id_base, vocab_total, local_only;
  unsigned long long* tp_cand;
  float2* tp_ms;
  int32_t* tp_nt;
};

__device__ __forceinline__ float neg_inf() { return det::bits_to_f(0xff800000u); }

__global__ void __launch_bounds__(kChunk) sample_prepare_kernel(SampleArgs a) {
  __shared__ float zs[kChunk];
  __shared__ int32_t b_ids[kMaxBias];
  __shared__ float b_vals[kMaxBias];
  pdl_wait();
  const int row = blockIdx.y, c = blockIdx.x, tid = threadIdx.x;
  const SampleRow r = a.rows[row];
  const int i = c * kChunk + tid;
  const int nb = a.bias_ids ? min(r.n_bias, kMaxBias) : 0;
  for (int j = tid; j < nb; j += kChunk) {
    b_ids[j] = a.bias_ids[static_cast<size_t>(row) * kMaxBias + j];
    b_vals[j] = a.bias_vals[static_cast<size_t>(row) * kMaxBias + j];
  }
  __syncthreads();
  float v = neg_inf();
  if (i < a.vocab) {
    v = a.logits[static_cast<size_t>(row) * a.ld + i];
    const int gid = i + a.id_base;
    const int cnt = (a.counts && r.slot >= 0) ? a.counts[static_cast<size_t>(r.slot) * a.vocab_total + gid] : 0;
    float bias = 0.f;
    bool has_bias = false;
    for (int j = 0; j < nb; ++j)
      if (b_ids[j] == gid) { bias = bias + b_vals[j]; has_bias = true; }
    if (cnt > 0 || has_bias) v = sample::adjust_logit(v, cnt, r.repetition, r.presence, r.frequency, bias);
    if (a.mask && !((a.mask[static_cast<size_t>(row) * ((a.vocab_total + 31) / 32) + (gid >> 5)] >> (gid & 31)) & 1u)) v = neg_inf();
    const bool greedy = r.temperature <= 0.f || r.top_p <= 0.f;
    if (!greedy && v > neg_inf()) v = v * (1.f / r.temperature);
    a.z[static_cast<size_t>(row) * a.vocab + i] = v;
  }
  zs[tid] = v;
  __syncthreads();
  if (tid == 0) {
    const int n = min(kChunk, a.vocab - c * kChunk);
    float m = neg_inf();
    for (int j = 0; j < n; ++j) m = zs[j] > m ? zs[j] : m;
    float s = 0.f;
    if (m > neg_inf())
      for (int j = 0; j < n; ++j) s = s + det::exp(zs[j] - m);
    a.parts[static_cast<size_t>(row) * a.chunks + c] = make_float2(m, s);
  }
}

__device__ __forceinline__ uint32_t ordered_bits(float f) {
  const uint32_t u = det::f_to_bits(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ unsigned long long cand_key(float z, int id) {
  return (static_cast<unsigned long long>(ordered_bits(z)) << 32) | (0xffffffffu - static_cast<uint32_t>(id));
}
__device__ __forceinline__ float key_value(unsigned long long k) {
  const uint32_t o = static_cast<uint32_t>(k >> 32);
  return det::bits_to_f((o & 0x80000000u) ? (o & 0x7fffffffu) : ~o);
}
__device__ __forceinline__ int key_id(unsigned long long k) { return static_cast<int>(0xffffffffu - static_cast<uint32_t>(k)); }

__global__ void __launch_bounds__(kSelThreads) sample_select_kernel(SampleArgs a) {
  extern __shared__ __align__(16) unsigned char smem[];
  float2* tree = reinterpret_cast<float2*>(smem);                                   // [chunks]
  __shared__ unsigned long long cand[kMaxCand];
  __shared__ float prob[kMaxCand];
  __shared__ uint32_t hist[256];
  __shared__ unsigned long long sel_prefix;
  __shared__ int sel_k, n_cand_s, n_total_s;
  __shared__ unsigned long long best_s[kSelThreads / 32];
  pdl_wait();
  const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  const SampleRow r = a.rows[row];
  const float* z = a.z + static_cast<size_t>(row) * a.vocab;
  // ---- pairwise fold of the chunk partials: level by level, the oracle's order
  for (int i = tid; i < a.chunks; i += kSelThreads) tree[i] = a.parts[static_cast<size_t>(row) * a.chunks + i];
  if (tid == 0) n_total_s = 0;
  __syncthreads();
  int n = a.chunks;
  while (n > 1) {
    const int half = n / 2;
    float2 mine;
    bool have = false;
    if (tid < half) {
      const float2 x = tree[2 * tid], y = tree[2 * tid + 1];
      const float m = x.x > y.x ? x.x : y.x;
      float s = 0.f;
      if (m > neg_inf()) s = x.y * det::exp(x.x - m) + y.y * det::exp(y.x - m);
      mine = make_float2(m, s);
      have = true;
    } else if (tid == half && (n & 1)) {
      mine = tree[n - 1];
      have = true;
    }
    __syncthreads();
    if (have) tree[tid] = mine;
    __syncthreads();
    n = half + (n & 1);
  }
  const float m_all = tree[0].x, s_all = tree[0].y;
  // ---- support size and greedy argmax in one sweep
  int fin = 0;
  unsigned long long best = 0ull;
  for (int i = tid; i < a.vocab; i += kSelThreads) {
    const float v = z[i];
    if (v > neg_inf()) ++fin;
    const unsigned long long k = cand_key(v, i + a.id_base);
    best = k > best ? k : best;
  }
  for (int o = 16; o > 0; o >>= 1) {
    fin += __shfl_xor_sync(0xffffffffu, fin, o);
    const unsigned long long ob = __shfl_xor_sync(0xffffffffu, best, o);
    best = ob > best ? ob : best;
  }
  if (lane == 0) { atomicAdd(&n_total_s, fin); best_s[wid] = best; }
  __syncthreads();
  const int n_total = n_total_s;
  const bool greedy = r.temperature <= 0.f || r.top_p <= 0.f;
  const int want_top = min(r.top_logprobs, kMaxTop);
  int C = greedy ? want_top : min(max(a.candidates, 1), kMaxCand);
  if (a.local_only) C = min(max(a.candidates, 1), kMaxCand);      // the merge decides what it needs
  C = min(C, a.vocab);
  if (greedy && tid == 0 && !a.local_only) {
    unsigned long long b = best_s[0];
    for (int w = 1; w < kSelThreads / 32; ++w) b = best_s[w] > b ? best_s[w] : b;
    const float lse = s_all > 0.f ? m_all + det::log(s_all) : neg_inf();
    a.out_token[row] = key_id(b);
    a.out_logprob[row] = key_value(b) - lse;
    a.out_flags[row] = 1;
    a.out_top_n[row] = 0;
  }
  if (C == 0) return;
  if (!greedy || a.local_only) C = min(C, max(n_total, 1));
  // ---- exact top-C by radix select on the 64-bit key (keys are unique: no ties)
  if (tid == 0) { sel_prefix = 0ull; sel_k = C; n_cand_s = 0; }
  __syncthreads();
  for (int pass = 0; pass < 8; ++pass) {
    const int shift = 56 - 8 * pass;
    for (int i = tid; i < 256; i += kSelThreads) hist[i] = 0;
    __syncthreads();
    const unsigned long long prefix = sel_prefix;
    for (int i = tid; i < a.vocab; i += kSelThreads) {
      const unsigned long long k = cand_key(z[i], i + a.id_base);
      if (pass == 0 || (k >> (shift + 8)) == prefix) atomicAdd(&hist[(k >> shift) & 255], 1u);
    }
    __syncthreads();
    if (tid == 0) {
      int k = sel_k;
      int b = 255;
      uint32_t cum = 0;
      for (; b > 0; --b) {
        if (cum + hist[b] >= static_cast<uint32_t>(k)) break;
        cum += hist[b];
      }
      sel_k = k - static_cast<int>(cum);
      sel_prefix = (prefix << 8) | static_cast<unsigned long long>(b);
    }
    __syncthreads();
  }
  const unsigned long long thr = sel_prefix;   // the C-th largest key
  for (int i = tid; i < a.vocab; i += kSelThreads) {
    const unsigned long long k = cand_key(z[i], i + a.id_base);
    if (k >= thr) {
      const int at = atomicAdd(&n_cand_s, 1);
      if (at < kMaxCand) cand[at] = k;
    }
  }
  __syncthreads();
  const int nc = min(n_cand_s, C);
  for (int i = tid; i < kMaxCand; i += kSelThreads)
    if (i >= nc) cand[i] = 0ull;
  __syncthreads();
  // bitonic sort, descending
  for (int size = 2; size <= kMaxCand; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      if (tid < kMaxCand) {
        const int j = tid ^ stride;
        if (j > tid) {
          const unsigned long long x = cand[tid], y = cand[j];
          const bool desc = (tid & size) == 0;
          if (desc ? (x < y) : (x > y)) { cand[tid] = y; cand[j] = x; }
        }
      }
      __syncthreads();
    }
  }
  if (a.local_only) {
    // the slice's table: keys in descending order (0 = empty entry), its (max, sum) and its support size
    if (tid < a.candidates) a.tp_cand[static_cast<size_t>(row) * a.candidates + tid] = tid < nc ? cand[tid] : 0ull;
    if (tid == 0) {
      a.tp_ms[row] = make_float2(m_all, s_all);
      a.tp_nt[row] = n_total;
    }
    return;
  }
  if (tid < kMaxCand) prob[tid] = tid < nc ? det::exp(key_value(cand[tid]) - m_all) : 0.f;
  __syncthreads();
  if (tid != 0) return;
  if (greedy) {
    const float lse = s_all > 0.f ? m_all + det::log(s_all) : neg_inf();
    const int nt = min(nc, want_top);
    for (int i = 0; i < nt; ++i) {
      a.out_top_ids[row * kMaxTop + i] = key_id(cand[i]);
      a.out_top_lp[row * kMaxTop + i] = key_value(cand[i]) - lse;
    }
    a.out_top_n[row] = nt;
    return;
  }
  sample::Filter f;
  f.temperature = r.temperature; f.top_k = r.top_k; f.top_p = r.top_p; f.min_p = r.min_p;
  const float u = det::uniform01(r.seed, r.position);
  const sample::Decision d = sample::decide(prob, nc, n_total, s_all, f, u);
  a.out_flags[row] = d.resolved;
  a.out_top_n[row] = 0;
  if (!d.resolved) {
    a.out_token[row] = nc > 0 ? key_id(cand[0]) : 0;
    a.out_logprob[row] = 0.f;
    return;
  }
  const float lse = m_all + det::log(d.total);
  a.out_token[row] = key_id(cand[d.pick]);
  a.out_logprob[row] = key_value(cand[d.pick]) - lse;
  const int nt = min(min(nc, d.keep), want_top);
  for (int i = 0; i < nt; ++i) {
    a.out_top_ids[row * kMaxTop + i] = key_id(cand[i]);
    a.out_top_lp[row * kMaxTop + i] = key_value(cand[i]) - lse;
  }
  a.out_top_n[row] = nt;
}

// Fold of the ranks' slice tables (vocabulary-sharded head): g_cand [world, rows, cands] keys, g_ms [world, rows] (max, sum),
// g_nt [world, rows] support sizes, all in rank order.  The (max, sum) pairs are merged in ascending rank order (the
// oracle's merge_logsumexp), the candidate lists are merged by one bitonic sort (the global top-C is a subset of the
// union of the slices' top-C), then the same filter-and-draw step as the unsharded kernel runs.  Every rank runs this
// on identical inputs and draws the same token.
constexpr int kMergeMax = 2048;    // world * candidates
__global__ void __launch_bounds__(kSelThreads) sample_merge_kernel(SampleArgs a, const unsigned long long* __restrict__ g_cand,
                                                                   const float2* __restrict__ g_ms, const int32_t* __restrict__ g_nt,
                                                                   int world, int rows) {
  __shared__ unsigned long long keys[kMergeMax];
  __shared__ float prob[kMaxCand];
  pdl_wait();
  const int row = blockIdx.x, tid = threadIdx.x;
  const SampleRow r = a.rows[row];
  const int per = a.candidates, n_in = world * per;
  for (int i = tid; i < kMergeMax; i += kSelThreads)
    keys[i] = i < n_in ? g_cand[(static_cast<size_t>(i / per) * rows + row) * per + i % per] : 0ull;
  __syncthreads();
  for (int size = 2; size <= kMergeMax; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int i = tid; i < kMergeMax; i += kSelThreads) {
        const int j = i ^ stride;
        if (j > i) {
          const unsigned long long x = keys[i], y = keys[j];
          const bool desc = (i & size) == 0;
          if (desc ? (x < y) : (x > y)) { keys[i] = y; keys[j] = x; }
        }
      }
      __syncthreads();
    }
  }
  // slice (max, sum) pairs in ascending rank order
  float m_all = neg_inf();
  for (int w = 0; w < world; ++w) {
    const float m = g_ms[static_cast<size_t>(w) * rows + row].x;
    m_all = m > m_all ? m : m_all;
  }
  float s_all = 0.f;
  int n_total = 0;
  for (int w = 0; w < world; ++w) {
    const float2 ms = g_ms[static_cast<size_t>(w) * rows + row];
    if (m_all > neg_inf() && ms.x > neg_inf()) s_all = s_all + ms.y * det::exp(ms.x - m_all);
    n_total += g_nt[static_cast<size_t>(w) * rows + row];
  }
  const bool greedy = r.temperature <= 0.f || r.top_p <= 0.f;
  const int want_top = min(r.top_logprobs, kMaxTop);
  int C = min(min(max(a.candidates, 1), kMaxCand), max(n_total, 1));
  int nc = 0;
  for (int i = 0; i < C; ++i) nc += keys[i] != 0ull ? 1 : 0;       // (uniform over the threads)
  if (tid < kMaxCand) prob[tid] = tid < nc ? det::exp(key_value(keys[tid]) - m_all) : 0.f;
  __syncthreads();
  if (tid != 0) return;
  if (greedy) {
    const float lse = s_all > 0.f ? m_all + det::log(s_all) : neg_inf();
    a.out_token[row] = nc > 0 ? key_id(keys[0]) : 0;
    a.out_logprob[row] = nc > 0 ? key_value(keys[0]) - lse : 0.f;
    a.out_flags[row] = 1;
    const int nt = min(nc, want_top);
    for (int i = 0; i < nt; ++i) {
      a.out_top_ids[row * kMaxTop + i] = key_id(keys[i]);
      a.out_top_lp[row * kMaxTop + i] = key_value(keys[i]) - lse;
    }
    a.out_top_n[row] = nt;
    return;
  }
  sample::Filter f;
  f.temperature = r.temperature; f.top_k = r.top_k; f.top_p = r.top_p; f.min_p = r.min_p;
  const float u = det::uniform01(r.seed, r.position);
  const sample::Decision d = sample::decide(prob, nc, n_total, s_all, f, u);
  a.out_flags[row] = d.resolved;
  a.out_top_n[row] = 0;
  if (!d.resolved) {
    a.out_token[row] = nc > 0 ? key_id(keys[0]) : 0;
    a.out_logprob[row] = 0.f;
    return;
  }
  const float lse = m_all + det::log(d.total);
  a.out_token[row] = key_id(keys[d.pick]);
  a.out_logprob[row] = key_value(keys[d.pick]) - lse;
  const int nt = min(min(nc, d.keep), want_top);
  for (int i = 0; i < nt; ++i) {
    a.out_top_ids[row * kMaxTop + i] = key_id(keys[i]);
    a.out_top_lp[row * kMaxTop + i] = key_value(keys[i]) - lse;
  }
  a.out_top_n[row] = nt;
}

// counts[slot][ids[i]] += delta for i < n (prompt ingestion, one generated token, speculative rollback).
__global__ void count_tokens_kernel(int32_t* counts, int vocab, int slot, const int32_t* ids, int n, int delta) {
  pdl_wait();
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const int id = ids[i];
    if (id >= 0 && id < vocab) atomicAdd(&counts[static_cast<size_t>(slot) * vocab + id], delta);
  }
}
// Per decode step: counts[slots[r]][tokens[r]] += 1 for every sampled row.
__global__ void count_step_kernel(int32_t* counts, int vocab, const SampleRow* rows, const int32_t* tokens, int n) {
  pdl_wait();
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r < n && rows[r].slot >= 0 && tokens[r] >= 0 && tokens[r] < vocab)
    atomicAdd(&counts[static_cast<size_t>(rows[r].slot) * vocab + tokens[r]], 1);
}

}  // namespace dgpp

using namespace dgpp;

DGPP_API int dgpp_sample_row_bytes() { return static_cast<int>(sizeof(SampleRow)); }
DGPP_API int dgpp_sample_limits(int* out) {
  out[0] = kMaxCand; out[1] = kMaxTop; out[2] = kMaxBias; out[3] = kChunk;
  return 0;
}

// z: [rows, vocab] floats, parts: [rows, ceil(vocab / 256)] float2.  Outputs as in SampleArgs.
DGPP_API int dgpp_sample(const void* logits, int64_t ld, const void* row_params, const void* counts, const void* bias_ids,
                         const void* bias_vals, const void* mask, void* z, void* parts, void* out_token,
                         void* out_logprob, void* out_flags, void* out_top_ids, void* out_top_lp, void* out_top_n,
                         int rows, int vocab, int candidates, cudaStream_t st) {
  DGPP_REQUIRE(rows >= 0 && vocab > 0, "sample: bad sizes rows %d vocab %d", rows, vocab);
  DGPP_REQUIRE(candidates >= 1 && candidates <= kMaxCand, "sample: candidates %d outside 1..%d", candidates, kMaxCand);
  if (rows == 0) return 0;
  SampleArgs a;
  a.logits = static_cast<const float*>(logits);
  a.ld = ld;
  a.rows = static_cast<const SampleRow*>(row_params);
  a.counts = static_cast<const int32_t*>(counts);
  a.bias_ids = static_cast<const int32_t*>(bias_ids);
  a.bias_vals = static_cast<const float*>(bias_vals);
  a.mask = static_cast<const uint32_t*>(mask);
  a.z = static_cast<float*>(z);
  a.parts = static_cast<float2*>(parts);
  a.out_token = static_cast<int32_t*>(out_token);
  a.out_logprob = static_cast<float*>(out_logprob);
  a.out_flags = static_cast<int32_t*>(out_flags);
  a.out_top_ids = static_cast<int32_t*>(out_top_ids);
  a.out_top_lp = static_cast<float*>(out_top_lp);
  a.out_top_n = static_cast<int32_t*>(out_top_n);
  a.vocab = vocab;
  a.chunks = dgpp_ceil_div(vocab, kChunk);
  a.candidates = candidates;
  a.id_base = 0; a.vocab_total = vocab; a.local_only = 0;
  a.tp_cand = nullptr; a.tp_ms = nullptr; a.tp_nt = nullptr;
  DGPP_REQUIRE(a.chunks <= 2 * kSelThreads, "sample: vocabulary %d too large for the chunk tree", vocab);
  sample_prepare_kernel<<<dim3(a.chunks, rows), kChunk, 0, st>>>(a);
  DGPP_CUDA_OK(cudaGetLastError());
  sample_select_kernel<<<rows, kSelThreads, static_cast<size_t>(a.chunks) * sizeof(float2), st>>>(a);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

// Vocabulary-sharded head, step 1 (every rank, on its slice [id_base, id_base + vocab) of vocab_total ids): penalties,
// bias, mask, temperature, then the slice's candidate table.  cand: [rows, candidates] uint64, ms: [rows] float2,
// nt: [rows] int32.  The caller gathers the three tables over the ranks (rank order) and runs dgpp_sample_merge.
DGPP_API int dgpp_sample_local(const void* logits, int64_t ld, const void* row_params, const void* counts, const void* bias_ids,
                               const void* bias_vals, const void* mask, void* z, void* parts, void* cand, void* ms, void* nt,
                               int rows, int vocab, int id_base, int vocab_total, int candidates, cudaStream_t st) {
  DGPP_REQUIRE(rows >= 0 && vocab > 0 && id_base >= 0 && id_base + vocab <= vocab_total, "sample_local: bad slice %d + %d of %d",
               id_base, vocab, vocab_total);
  DGPP_REQUIRE(candidates >= 1 && candidates <= kMaxCand, "sample_local: candidates %d outside 1..%d", candidates, kMaxCand);
  if (rows == 0) return 0;
  SampleArgs a;
  memset(&a, 0, sizeof(a));
  a.logits = static_cast<const float*>(logits);
  a.ld = ld;
  a.rows = static_cast<const SampleRow*>(row_params);
  a.counts = static_cast<const int32_t*>(counts);
  a.bias_ids = static_cast<const int32_t*>(bias_ids);
  a.bias_vals = static_cast<const float*>(bias_vals);
  a.mask = static_cast<const uint32_t*>(mask);
  a.z = static_cast<float*>(z);
  a.parts = static_cast<float2*>(parts);
  a.vocab = vocab;
  a.chunks = dgpp_ceil_div(vocab, kChunk);
  a.candidates = candidates;
  a.id_base = id_base; a.vocab_total = vocab_total; a.local_only = 1;
  a.tp_cand = static_cast<unsigned long long*>(cand);
  a.tp_ms = static_cast<float2*>(ms);
  a.tp_nt = static_cast<int32_t*>(nt);
  DGPP_REQUIRE(a.chunks <= 2 * kSelThreads, "sample_local: slice %d too large for the chunk tree", vocab);
  sample_prepare_kernel<<<dim3(a.chunks, rows), kChunk, 0, st>>>(a);
  DGPP_CUDA_OK(cudaGetLastError());
  sample_select_kernel<<<rows, kSelThreads, static_cast<size_t>(a.chunks) * sizeof(float2), st>>>(a);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

// Step 2 (every rank, identical inputs): g_cand [world, rows, candidates], g_ms [world, rows], g_nt [world, rows].
DGPP_API int dgpp_sample_merge(const void* row_params, const void* g_cand, const void* g_ms, const void* g_nt, void* out_token,
                               void* out_logprob, void* out_flags, void* out_top_ids, void* out_top_lp, void* out_top_n, int rows,
                               int world, int candidates, cudaStream_t st) {
  DGPP_REQUIRE(world >= 1 && candidates >= 1 && candidates <= kMaxCand && world * candidates <= kMergeMax,
               "sample_merge: %d ranks x %d candidates exceed %d", world, candidates, kMergeMax);
  if (rows == 0) return 0;
  SampleArgs a;
  memset(&a, 0, sizeof(a));
  a.rows = static_cast<const SampleRow*>(row_params);
  a.out_token = static_cast<int32_t*>(out_token);
  a.out_logprob = static_cast<float*>(out_logprob);
  a.out_flags = static_cast<int32_t*>(out_flags);
  a.out_top_ids = static_cast<int32_t*>(out_top_ids);
  a.out_top_lp = static_cast<float*>(out_top_lp);
  a.out_top_n = static_cast<int32_t*>(out_top_n);
  a.candidates = candidates;
  sample_merge_kernel<<<rows, kSelThreads, 0, st>>>(a, static_cast<const unsigned long long*>(g_cand), static_cast<const float2*>(g_ms),
                                                    static_cast<const int32_t*>(g_nt), world, rows);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

DGPP_API int dgpp_sample_count_tokens(void* counts, int vocab, int slot, const void* ids, int n, int delta, cudaStream_t st) {
  if (n <= 0) return 0;
  count_tokens_kernel<<<dgpp_ceil_div(n, 256) > 64 ? 64 : dgpp_ceil_div(n, 256), 256, 0, st>>>(
      static_cast<int32_t*>(counts), vocab, slot, static_cast<const int32_t*>(ids), n, delta);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

DGPP_API int dgpp_sample_count_step(void* counts, int vocab, const void* row_params, const void* tokens, int n, cudaStream_t st) {
  if (n <= 0) return 0;
  count_step_kernel<<<dgpp_ceil_div(n, 128), 128, 0, st>>>(static_cast<int32_t*>(counts), vocab,
                                                            static_cast<const SampleRow*>(row_params),
                                                            static_cast<const int32_t*>(tokens), n);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}
