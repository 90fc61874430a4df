// Multi-head latent attention (absorbed form) over a paged latent cache, dense or sparse, plus the sparse
// attention index: lightning-indexer scores and exact top-k selection.
//
// Cache: one latent row per token, [dc latent | dr rotary key] bf16, shared by every head.  With the key
// up-projection absorbed into the query (q_abs = W_uk^T q_nope) a head's score is q_abs . c_t + q_rot . k_rot_t and
// its output is the probability-weighted latent sum (the value up-projection is applied afterwards).
//
//   mla_decode_kernel     grid (kv splits, rows, head groups of 8): a CTA stages 32-token latent tiles in shared
//                         memory (rows padded against bank conflicts); warp = one head: lane = token for the
//                         scores, lane = 16 latent dims for the output; online softmax; split partials are merged
//                         by mla_combine_kernel in ascending split order.  With `sel` the tokens come from a
//                         per-row index list (sparse attention) instead of the whole context.
//   dsa_index_kernel      index score of every cached token for a row: sum_h w[h] * relu(q_idx[h] . k_idx[t])
//   topk_select_kernel    exact top-k token positions of a score row (ties to the lower position): 8-pass radix
//                         select on the 64-bit key (ordered float bits, ~position), output ascending
// (reference counterparts: src/kernels/dsa.cu latent decode / indexer / top-k, src/models/dsa_layer.cu.)
#include <math.h>

#include "common/common.h"
#include "common/dtypes.cuh"
#include "common/ptx.cuh"

namespace dgpp {

constexpr int kMlaThreads = 256;
constexpr int kMlaHeads = 8;       // heads per CTA (one warp each)
constexpr int kMlaTile = 32;       // tokens per tile

struct MlaArgs {
  const bf16* q;            // [rows, heads, dc + dr] absorbed query
  const bf16* cache;        // [blocks, page, dc + dr]
  const int32_t* block_table;   // [requests, max_blocks]
  const int32_t* row_req;   // [rows]
  const int32_t* positions; // [rows] position of the row's own token (already in the cache)
  const int32_t* sel;       // [rows, sel_stride] selected token positions (ascending, -1 padded) or null
  float* part_ml;           // [rows, heads, splits, 2]
  float* part_acc;          // [rows, heads, splits, dc]
  bf16* out;                // [rows, heads, dc]
  int rows, heads, dc, dr, page, max_blocks, splits, sel_stride;
  float scale;
};

template <int DC, int DR>
__global__ void __launch_bounds__(kMlaThreads) mla_decode_kernel(MlaArgs a) {
  constexpr int D = DC + DR, DP = D + 2;              // padded row (bank-conflict free for lane = token)
  constexpr int PER = DC / 32;                        // output dims per lane
  extern __shared__ __align__(16) unsigned char smem[];
  bf16* tile = reinterpret_cast<bf16*>(smem);                          // [kMlaTile][DP]
  float* qs = reinterpret_cast<float*>(tile + kMlaTile * DP);          // [kMlaHeads][D]
  __shared__ int tok_s[kMlaTile];
  pdl_wait();
  const int split = blockIdx.x, row = blockIdx.y, hg = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  const int head = hg * kMlaHeads + wid;
  const bool head_ok = head < a.heads;
  const int req = a.row_req[row], pos = a.positions[row];
  for (int i = tid; i < kMlaHeads * D; i += kMlaThreads) {
    const int h = hg * kMlaHeads + i / D;
    qs[i] = h < a.heads ? bf16_to_f32(a.q[(static_cast<size_t>(row) * a.heads + h) * D + i % D]) : 0.f;
  }
  // token range of this split: over the context, or over the selection list
  int n_tok = pos + 1;
  const int32_t* sel = a.sel ? a.sel + static_cast<size_t>(row) * a.sel_stride : nullptr;
  if (sel) {
    n_tok = 0;   // count of valid entries (list is -1 padded); every thread counts the same
    for (int i = 0; i < a.sel_stride; ++i) n_tok += (sel[i] >= 0 && sel[i] <= pos) ? 1 : 0;
  }
  const int tiles = (n_tok + kMlaTile - 1) / kMlaTile;
  const int per = (tiles + a.splits - 1) / a.splits;
  const int t_begin = split * per, t_end = min(tiles, t_begin + per);
  float m = -INFINITY, l = 0.f, acc[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) acc[i] = 0.f;
  for (int tl = t_begin; tl < t_end; ++tl) {
    __syncthreads();
    if (tid < kMlaTile) {
      const int idx = tl * kMlaTile + tid;
      int tok = -1;
      if (idx < n_tok) tok = sel ? sel[idx] : idx;      // list entries beyond `pos` were not counted: lists are ascending
      tok_s[tid] = tok;
    }
    __syncthreads();
    // stage the tile: 16-byte vectors, D / 8 per token
    for (int i = tid; i < kMlaTile * (D / 8); i += kMlaThreads) {
      const int t = i / (D / 8), v = i % (D / 8);
      const int tok = tok_s[t];
      uint4 x = make_uint4(0, 0, 0, 0);
      if (tok >= 0) {
        const int blk = a.block_table[static_cast<size_t>(req) * a.max_blocks + tok / a.page];
        x = *reinterpret_cast<const uint4*>(a.cache + (static_cast<size_t>(blk) * a.page + tok % a.page) * D + v * 8);
      }
      // padded rows are only 4-byte aligned: store as four words
      uint32_t* dst = reinterpret_cast<uint32_t*>(tile + t * DP + v * 8);
      dst[0] = x.x; dst[1] = x.y; dst[2] = x.z; dst[3] = x.w;
    }
    __syncthreads();
    if (!head_ok) continue;
    // scores: lane = token
    const bf16* tr = tile + lane * DP;
    const float* qh = qs + wid * D;
    float s = 0.f;
#pragma unroll 8
    for (int d = 0; d < D; d += 2) {
      const bf162 c2 = *reinterpret_cast<const bf162*>(tr + d);
      s = fmaf(__bfloat162float(c2.x), qh[d], s);
      s = fmaf(__bfloat162float(c2.y), qh[d + 1], s);
    }
    const bool valid = tok_s[lane] >= 0;
    s = valid ? s * a.scale : -INFINITY;
    float tm = s;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, o));
    const float mn = fmaxf(m, tm);
    const float corr = m == -INFINITY ? 0.f : __expf(m - mn);
    const float p = valid ? __expf(s - mn) : 0.f;
    float ps = p;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
    l = l * corr + ps;
    m = mn;
#pragma unroll
    for (int i = 0; i < PER; ++i) acc[i] *= corr;
    // output: lane = PER consecutive latent dims, tokens in order
    for (int t = 0; t < kMlaTile; ++t) {
      const float pt = __shfl_sync(0xffffffffu, p, t);
      if (pt == 0.f) continue;
      const bf16* cr = tile + t * DP + lane * PER;
#pragma unroll
      for (int i = 0; i < PER; i += 2) {
        const bf162 c2 = *reinterpret_cast<const bf162*>(cr + i);
        acc[i] = fmaf(pt, __bfloat162float(c2.x), acc[i]);
        acc[i + 1] = fmaf(pt, __bfloat162float(c2.y), acc[i + 1]);
      }
    }
  }
  if (!head_ok) return;
  if (a.splits == 1) {
    const float inv = l > 0.f ? 1.f / l : 0.f;
    bf16* o = a.out + (static_cast<size_t>(row) * a.heads + head) * DC + lane * PER;
#pragma unroll
    for (int i = 0; i < PER; ++i) o[i] = f32_to_bf16(acc[i] * inv);
  } else {
    const size_t pi = (static_cast<size_t>(row) * a.heads + head) * a.splits + split;
    float* pa = a.part_acc + pi * DC + lane * PER;
#pragma unroll
    for (int i = 0; i < PER; ++i) pa[i] = acc[i];
    if (lane == 0) { a.part_ml[pi * 2] = m; a.part_ml[pi * 2 + 1] = l; }
  }
}

__global__ void mla_combine_kernel(const float* __restrict__ part_ml, const float* __restrict__ part_acc,
                                   bf16* __restrict__ out, int splits, int dc) {
  pdl_wait();
  const size_t rh = blockIdx.x;
  float mm = -INFINITY;
  for (int s = 0; s < splits; ++s) mm = fmaxf(mm, part_ml[(rh * splits + s) * 2]);
  for (int d = threadIdx.x; d < dc; d += blockDim.x) {
    float ll = 0.f, acc = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float ms = part_ml[(rh * splits + s) * 2];
      const float c = ms == -INFINITY ? 0.f : __expf(ms - mm);
      ll += part_ml[(rh * splits + s) * 2 + 1] * c;
      acc += part_acc[(rh * splits + s) * dc + d] * c;
    }
    out[rh * dc + d] = f32_to_bf16(ll > 0.f ? acc / ll : 0.f);
  }
}

// scores[row, t] = sum_h w[row, h] * relu(q[row, h, :] . k[t, :]) for t <= position; -inf beyond.
// k: paged [blocks, page, di] bf16.  grid (ceil(max_ctx / 256), rows); thread = token.
struct IndexArgs {
  const bf16* q;        // [rows, hi, di]
  const float* w;       // [rows, hi]
  const bf16* k;        // [blocks, page, di]
  const int32_t* block_table;
  const int32_t* row_req;
  const int32_t* positions;
  float* scores;        // [rows, ld]
  int rows, hi, di, page, max_blocks, ld;
};

__global__ void __launch_bounds__(256) dsa_index_kernel(IndexArgs a) {
  extern __shared__ __align__(16) unsigned char smem[];
  float* qs = reinterpret_cast<float*>(smem);        // [hi][di]
  float* ws = qs + a.hi * a.di;                      // [hi]
  pdl_wait();
  const int row = blockIdx.y, t = blockIdx.x * 256 + threadIdx.x;
  for (int i = threadIdx.x; i < a.hi * a.di; i += 256) qs[i] = bf16_to_f32(a.q[static_cast<size_t>(row) * a.hi * a.di + i]);
  for (int i = threadIdx.x; i < a.hi; i += 256) ws[i] = a.w[static_cast<size_t>(row) * a.hi + i];
  __syncthreads();
  if (t >= a.ld) return;
  const int pos = a.positions[row];
  float out = -INFINITY;
  if (t <= pos) {
    const int blk = a.block_table[static_cast<size_t>(a.row_req[row]) * a.max_blocks + t / a.page];
    const bf16* kr = a.k + (static_cast<size_t>(blk) * a.page + t % a.page) * a.di;
    out = 0.f;
    for (int h = 0; h < a.hi; ++h) {
      float s = 0.f;
      for (int d = 0; d < a.di; d += 8) {
        Pack16 kv;
        kv.u = *reinterpret_cast<const uint4*>(kr + d);
#pragma unroll
        for (int j = 0; j < 8; ++j) s = fmaf(bf16_to_f32(kv.h[j]), qs[h * a.di + d + j], s);
      }
      out = fmaf(ws[h], fmaxf(s, 0.f), out);
    }
  }
  a.scores[static_cast<size_t>(row) * a.ld + t] = out;
}

__device__ __forceinline__ unsigned long long topk_key(float z, int id) {
  const uint32_t u = __float_as_uint(z);
  const uint32_t o = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
  return (static_cast<unsigned long long>(o) << 32) | (0xffffffffu - static_cast<uint32_t>(id));
}

// out[row, 0..k): positions of the k best scores among scores[row, 0..n_row), ascending, padded with -1 when the
// row has fewer than k finite scores.  One CTA of 1024 threads per row.
__global__ void __launch_bounds__(1024) topk_select_kernel(const float* __restrict__ scores, int64_t ld,
                                                           const int32_t* __restrict__ n_valid, int32_t* __restrict__ out,
                                                           int k) {
  __shared__ uint32_t hist[256];
  __shared__ unsigned long long prefix_s;
  __shared__ int need_s, fill_s;
  pdl_wait();
  const int row = blockIdx.x, tid = threadIdx.x;
  const float* z = scores + static_cast<size_t>(row) * ld;
  const int n = n_valid[row] + 1;                      // positions 0 .. pos
  int32_t* o = out + static_cast<size_t>(row) * k;
  if (n <= k) {                                        // everything is selected
    for (int i = tid; i < k; i += blockDim.x) o[i] = i < n ? i : -1;
    return;
  }
  if (tid == 0) { prefix_s = 0ull; need_s = k; fill_s = 0; }
  __syncthreads();
  const int lane = tid & 31, wid = tid >> 5;
  unsigned long long thr = 0ull;
  for (int pass = 0; pass < 8; ++pass) {
    const int shift = 56 - 8 * pass;
    for (int i = tid; i < 256; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    const unsigned long long prefix = prefix_s;
    // histogram of this digit over the keys that still match the prefix; the lanes of a warp that hit the same bin
    // send ONE add (score rows are far from uniform in their leading digits: without this the first passes serialise)
    for (int c0 = 0; c0 < n; c0 += blockDim.x) {
      const int i = c0 + tid;
      int bin = -1;
      if (i < n) {
        const unsigned long long key = topk_key(z[i], i);
        if (pass == 0 || (key >> (shift + 8)) == prefix) bin = static_cast<int>((key >> shift) & 255);
      }
      const unsigned peers = __match_any_sync(0xffffffffu, bin);
      if (bin >= 0 && lane == __ffs(peers) - 1) atomicAdd(&hist[bin], static_cast<uint32_t>(__popc(peers)));
    }
    __syncthreads();
    if (tid == 0) {
      int need = need_s, bsel = 255;
      uint32_t cum = 0;
      for (; bsel > 0; --bsel) {
        if (cum + hist[bsel] >= static_cast<uint32_t>(need)) break;
        cum += hist[bsel];
      }
      need_s = need - static_cast<int>(cum);
      prefix_s = (prefix << 8) | static_cast<unsigned long long>(bsel);
      // every key of the chosen bin is needed: the lowest key with this prefix is the threshold, no digit below matters
      fill_s = (hist[bsel] == static_cast<uint32_t>(need_s)) ? 1 : 0;
    }
    __syncthreads();
    thr = prefix_s << shift;
    if (fill_s) break;
  }
  // ascending output without a sort: warp w owns the contiguous positions [w * seg, (w + 1) * seg); it counts its
  // selected positions, the counts are scanned once, then it writes them in order from its base
  __shared__ int warp_cnt[32];
  const int warps = blockDim.x >> 5;
  const int seg = ((n + warps - 1) / warps + 31) & ~31;
  const int lo = wid * seg, hi = min(n, lo + seg);
  int cnt = 0;
  for (int c0 = lo; c0 < hi; c0 += 32) {
    const int i = c0 + lane;
    cnt += __popc(__ballot_sync(0xffffffffu, i < hi && topk_key(z[i], i) >= thr));
  }
  if (lane == 0) warp_cnt[wid] = cnt;
  __syncthreads();
  int before = 0;
  for (int w = 0; w < wid; ++w) before += warp_cnt[w];
  for (int c0 = lo; c0 < hi; c0 += 32) {
    const int i = c0 + lane;
    const bool take = i < hi && topk_key(z[i], i) >= thr;
    const unsigned ballot = __ballot_sync(0xffffffffu, take);
    const int at = before + __popc(ballot & ((1u << lane) - 1u));
    if (take && at < k) o[at] = i;
    before += __popc(ballot);
  }
}

template <int DC, int DR>
static int launch_mla(const MlaArgs& a, cudaStream_t st) {
  constexpr int D = DC + DR;
  const size_t smem = static_cast<size_t>(kMlaTile) * (D + 2) * 2 + static_cast<size_t>(kMlaHeads) * D * 4;
  static bool attr = false;
  if (!attr) {
    DGPP_CUDA_OK(cudaFuncSetAttribute(mla_decode_kernel<DC, DR>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      static_cast<int>(smem)));
    attr = true;
  }
  dim3 grid(a.splits, a.rows, dgpp_ceil_div(a.heads, kMlaHeads));
  mla_decode_kernel<DC, DR><<<grid, kMlaThreads, smem, st>>>(a);
  DGPP_CUDA_OK(cudaGetLastError());
  if (a.splits > 1) {
    mla_combine_kernel<<<a.rows * a.heads, 256, 0, st>>>(a.part_ml, a.part_acc, a.out, a.splits, DC);
    DGPP_CUDA_OK(cudaGetLastError());
  }
  return 0;
}

}  // namespace dgpp

using namespace dgpp;

// Scratch for splits > 1: part_ml rows*heads*splits*2 floats, part_acc rows*heads*splits*dc floats.
DGPP_API int dgpp_mla_decode(const void* q, const void* cache, const void* block_table, const void* row_req,
                             const void* positions, const void* sel, int sel_stride, void* part_ml, void* part_acc,
                             void* out, int rows, int heads, int dc, int dr, int page, int max_blocks, int splits,
                             float scale, cudaStream_t st) {
  DGPP_REQUIRE(splits >= 1 && (splits == 1 || (part_ml && part_acc)), "mla_decode: scratch required when splits > 1");
  if (rows == 0) return 0;
  MlaArgs a;
  a.q = static_cast<const bf16*>(q);
  a.cache = static_cast<const bf16*>(cache);
  a.block_table = static_cast<const int32_t*>(block_table);
  a.row_req = static_cast<const int32_t*>(row_req);
  a.positions = static_cast<const int32_t*>(positions);
  a.sel = static_cast<const int32_t*>(sel);
  a.part_ml = static_cast<float*>(part_ml);
  a.part_acc = static_cast<float*>(part_acc);
  a.out = static_cast<bf16*>(out);
  a.rows = rows; a.heads = heads; a.dc = dc; a.dr = dr; a.page = page; a.max_blocks = max_blocks; a.splits = splits;
  a.sel_stride = sel_stride; a.scale = scale;
  if (dc == 512 && dr == 64) return launch_mla<512, 64>(a, st);
  if (dc == 256 && dr == 64) return launch_mla<256, 64>(a, st);
  if (dc == 128 && dr == 32) return launch_mla<128, 32>(a, st);
  dgpp_set_error("mla_decode: latent %d + rotary %d unsupported (512+64, 256+64, 128+32)", dc, dr);
  return -1;
}

DGPP_API int dgpp_dsa_index(const void* q, const void* w, const void* k, const void* block_table, const void* row_req,
                            const void* positions, void* scores, int rows, int hi, int di, int page, int max_blocks,
                            int ld, cudaStream_t st) {
  DGPP_REQUIRE(di % 8 == 0 && hi >= 1, "dsa_index: bad index geometry %d x %d", hi, di);
  if (rows == 0) return 0;
  IndexArgs a;
  a.q = static_cast<const bf16*>(q); a.w = static_cast<const float*>(w); a.k = static_cast<const bf16*>(k);
  a.block_table = static_cast<const int32_t*>(block_table);
  a.row_req = static_cast<const int32_t*>(row_req);
  a.positions = static_cast<const int32_t*>(positions);
  a.scores = static_cast<float*>(scores);
  a.rows = rows; a.hi = hi; a.di = di; a.page = page; a.max_blocks = max_blocks; a.ld = ld;
  const size_t smem = static_cast<size_t>(hi) * di * 4 + static_cast<size_t>(hi) * 4;
  DGPP_REQUIRE(smem <= 48 * 1024, "dsa_index: %d heads x %d dims exceed shared memory", hi, di);
  dsa_index_kernel<<<dim3(dgpp_ceil_div(ld, 256), rows), 256, smem, st>>>(a);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

DGPP_API int dgpp_topk_select(const void* scores, int64_t ld, const void* positions, void* out, int rows, int k,
                              cudaStream_t st) {
  DGPP_REQUIRE(k >= 1, "topk_select: k must be positive");
  if (rows == 0) return 0;
  topk_select_kernel<<<rows, 1024, 0, st>>>(static_cast<const float*>(scores), ld,
                                            static_cast<const int32_t*>(positions), static_cast<int32_t*>(out), k);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}
