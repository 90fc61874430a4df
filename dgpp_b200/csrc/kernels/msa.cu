// Block-sparse attention index (the selection half of block-sparse GQA; the attention half is the block-selection
// form of the paged decode kernel).  Every token stores one index key of DI values; every kv head owns one index
// query head.  A (row, index head) scores each block of `sel_block` tokens by the largest query-key product among
// the block's visible tokens, always keeps the block that holds the row's own position, and keeps the `topk` best
// blocks in all (ties go to the lower block id).  The list comes out in ascending block order, -1 padded.
//
//   msa_index_prep    per-head RMSNorm (optionally 1 + w) and partial rotary embedding of the index queries and the
//                     index key of every row, in place; the key is appended to the paged index cache
//                     [blocks, page, DI] bf16 (same block table as the KV cache)
//   msa_index_select  block scores (one warp per sparse block, all index heads of a row at once, keys staged
//                     through shared memory with coalesced 16-byte loads), then the pick, one CTA per (index head, row)
//
// Pooled-key form (one list per row, shared by every kv head): the index keys are appended raw; when a block of
// `kpool` tokens completes, its keys are averaged once (fp32 mean, one bf16 rounding), normalised, rotated at the
// block's first position and stored as the block's compressed key.  A row scores every complete visible block
// b < (pos + 1) / kpool by sum over index heads of relu(<q_h, c_b>) / sqrt(DI), keeps the `select_k` best (all of
// them when there are no more than that; ties to the lower id) and always appends its own incomplete block.
//   qsa_compress      compressed keys of the blocks that complete at the rows of this pass
//   qsa_select        scores + selection, one CTA per row; the list is written once per kv head
// (reference counterparts: src/kernels/minimax.hpp minimax_norm_rope, minimax_index_append, minimax_index_score,
//  minimax_index_select; src/models/minimax/reference.cpp select_blocks is the arithmetic contract.)
#include <math.h>

#include "common/common.h"
#include "common/dtypes.cuh"
#include "common/ptx.cuh"

namespace dgpp {

struct MsaPrepParams {
  bf16* iqk;                   // [rows, (ih + 1) * DI]: index query heads, then the index key
  const int32_t* positions;    // [rows]
  const int32_t* row_req;      // [rows]
  const int32_t* block_table;  // [requests, max_blocks]
  const float* inv_freq;       // [rot_dim / 2]
  const bf16* q_norm_w;        // [DI] or null
  const bf16* k_norm_w;        // [DI] or null
  bf16* index_cache;           // [blocks, page, DI]
  int rows, ih, rot_dim, page, max_blocks, one_plus_w;
  int raw_key;                 // 1: the key is appended as it is (no norm, no rotation): pooled later
  float eps;
};

// One warp per (row, head); element j of lane l is dim l + 32 j.
template <int DI>
__global__ void __launch_bounds__(128) msa_index_prep_kernel(MsaPrepParams p) {
  pdl_wait();
  constexpr int PER = DI / 32;
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int heads = p.ih + 1;
  if (warp >= p.rows * heads) return;
  const int row = warp / heads, head = warp % heads;
  const bool is_key = head == p.ih;
  bf16* src = p.iqk + (static_cast<size_t>(row) * heads + head) * DI;
  float v[PER];
#pragma unroll
  for (int j = 0; j < PER; ++j) v[j] = bf16_to_f32(src[lane + 32 * j]);
  const bf16* nw = is_key ? p.k_norm_w : p.q_norm_w;
  const int pos = p.positions[row];
  if (is_key && p.raw_key) {
    const int blk = p.block_table[static_cast<size_t>(p.row_req[row]) * p.max_blocks + pos / p.page];
    bf16* dst = p.index_cache + (static_cast<size_t>(blk) * p.page + pos % p.page) * DI;
#pragma unroll
    for (int j = 0; j < PER; ++j) dst[lane + 32 * j] = f32_to_bf16(v[j]);
    return;
  }
  if (nw != nullptr) {
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < PER; ++j) ss += v[j] * v[j];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float rstd = rsqrtf(ss / DI + p.eps);
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      float g = bf16_to_f32(nw[lane + 32 * j]);
      if (p.one_plus_w) g += 1.f;
      v[j] = bf16_to_f32(f32_to_bf16(bf16_to_f32(f32_to_bf16(v[j] * rstd)) * g));
    }
  }
  const int half = p.rot_dim / 2;
  float r[PER];
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int a = lane + 32 * j;
    const int pd = a < half ? a + half : (a < p.rot_dim ? a - half : a);      // rotate-half partner
    float partner = 0.f;
#pragma unroll
    for (int jj = 0; jj < PER; ++jj) {
      const float cand = __shfl_sync(0xffffffffu, v[jj], pd & 31);
      if ((pd >> 5) == jj) partner = cand;
    }
    if (a < p.rot_dim) {
      float sn, cs;
      sincosf(static_cast<float>(pos) * p.inv_freq[a < half ? a : a - half], &sn, &cs);
      r[j] = a < half ? v[j] * cs - partner * sn : v[j] * cs + partner * sn;
    } else {
      r[j] = v[j];
    }
  }
#pragma unroll
  for (int j = 0; j < PER; ++j) src[lane + 32 * j] = f32_to_bf16(r[j]);
  if (!is_key) return;
  const int blk = p.block_table[static_cast<size_t>(p.row_req[row]) * p.max_blocks + pos / p.page];
  bf16* dst = p.index_cache + (static_cast<size_t>(blk) * p.page + pos % p.page) * DI;
#pragma unroll
  for (int j = 0; j < PER; ++j) dst[lane + 32 * j] = f32_to_bf16(r[j]);
}

struct MsaSelectParams {
  const bf16* iqk;             // [rows, iqk_stride]: index query head h at column h * DI
  int64_t iqk_stride;
  const bf16* index_cache;     // [blocks, page, DI]
  const int32_t* block_table;
  const int32_t* row_req;
  const int32_t* positions;
  int32_t* sel;                // [rows, ih, topk]
  float* scores;               // [rows, ih, max_sel] block scores (workspace of the two-kernel selection; the row's own
                               // block holds its real score here, the pick treats it as +inf)
  int rows, ih, page, max_blocks, sel_block, topk, max_sel;
};

constexpr int kMsaThreads = 256;
constexpr int kMsaMaxTopk = 64;

// Block-wide (kMsaThreads threads): the `keep` largest of sc[0 .. nblk) (ties to the lower index; taken entries are
// overwritten with -inf), then `extra` (a block id, or -1 for none) appended, the whole list in ascending order, -1
// padded to out_k entries, written `copies` times `copy_stride` entries apart.  chosen holds kMsaMaxTopk + 1 ints.
__device__ __forceinline__ void msa_topk_write(float* sc, int nblk, int keep, int extra, int* chosen, float* wv, int* wi,
                                               int32_t* out, int out_k, int copies, int copy_stride) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int r = 0; r < keep; ++r) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int b = threadIdx.x; b < nblk; b += kMsaThreads) {
      const float s = sc[b];
      if (s > -INFINITY && (s > bv || (s == bv && b < bi) || bi == 0x7fffffff)) { bv = s; bi = b; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
    }
    if (lane == 0) { wv[warp] = bv; wi[warp] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
      float fv = wv[0];
      int fi = wi[0];
      for (int w = 1; w < kMsaThreads / 32; ++w) {
        if (wi[w] != 0x7fffffff && (fi == 0x7fffffff || wv[w] > fv || (wv[w] == fv && wi[w] < fi))) { fv = wv[w]; fi = wi[w]; }
      }
      chosen[r] = fi;
      if (fi != 0x7fffffff) sc[fi] = -INFINITY;
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    // ascending order (a handful of entries: insertion sort), then the -1 padding
    int n = 0;
    for (int r = 0; r < keep; ++r)
      if (chosen[r] != 0x7fffffff) chosen[n++] = chosen[r];
    if (extra >= 0) chosen[n++] = extra;
    for (int i = 1; i < n; ++i) {
      const int v = chosen[i];
      int j = i - 1;
      while (j >= 0 && chosen[j] > v) { chosen[j + 1] = chosen[j]; --j; }
      chosen[j + 1] = v;
    }
    for (int c = 0; c < copies; ++c)
      for (int r = 0; r < out_k; ++r) out[static_cast<size_t>(c) * copy_stride + r] = r < n ? chosen[r] : -1;
  }
}

constexpr int kMsaScoreWarps = 4;      // sparse blocks per CTA of the score kernel (one per warp)
constexpr int kMsaMaxIndexHeads = 8;

// Block scores.  grid (ceil(max_sel / kMsaScoreWarps), rows), kMsaScoreWarps warps: warp w scores sparse block
// blockIdx.x * kMsaScoreWarps + w of the row for every index head at once (each key is read once).  32 tokens at a
// time travel through shared memory with 16-byte coalesced loads; lane t then owns token t of the tile and runs the
// dot products of all heads against it (queries are broadcast reads).  scores [rows, ih, max_sel].
template <int DI>
__global__ void __launch_bounds__(kMsaScoreWarps * 32) msa_index_score_kernel(MsaSelectParams p) {
  constexpr int ROW = DI + 8;                    // padded tile row (bf16): 16-byte reads of 32 lanes spread over the banks
  extern __shared__ __align__(16) unsigned char msa_smem[];
  float* q_s = reinterpret_cast<float*>(msa_smem);                                   // [ih][DI]
  bf16* tiles = reinterpret_cast<bf16*>(msa_smem + static_cast<size_t>(p.ih) * DI * sizeof(float));
  pdl_wait();
  const int row = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pos = p.positions[row];
  const int nblk = min(pos / p.sel_block + 1, p.max_sel);
  if (blockIdx.x * kMsaScoreWarps >= nblk) return;
  for (int i = threadIdx.x; i < p.ih * DI; i += kMsaScoreWarps * 32)
    q_s[i] = bf16_to_f32(p.iqk[static_cast<size_t>(row) * p.iqk_stride + i]);
  __syncthreads();
  const int b = blockIdx.x * kMsaScoreWarps + warp;
  if (b >= nblk) return;
  bf16* tile = tiles + static_cast<size_t>(warp) * 32 * ROW;
  const int32_t* bt = p.block_table + static_cast<size_t>(p.row_req[row]) * p.max_blocks;
  float mx[kMsaMaxIndexHeads];
#pragma unroll
  for (int h = 0; h < kMsaMaxIndexHeads; ++h) mx[h] = -INFINITY;
  const int t_end = min((b + 1) * p.sel_block, pos + 1);
  for (int t0 = b * p.sel_block; t0 < t_end; t0 += 32) {
    const int n = min(32, t_end - t0);
    // n tokens x (DI / 8) chunks of 16 bytes, consecutive lanes on consecutive chunks of a token
    for (int i = lane; i < n * (DI / 8); i += 32) {
      const int tt = i / (DI / 8), c = i % (DI / 8);
      const int t = t0 + tt;
      const uint4 v = reinterpret_cast<const uint4*>(
          p.index_cache + (static_cast<size_t>(bt[t / p.page]) * p.page + t % p.page) * DI)[c];
      *reinterpret_cast<uint4*>(tile + tt * ROW + c * 8) = v;
    }
    __syncwarp();
    if (lane < n) {
      float s[kMsaMaxIndexHeads];
#pragma unroll
      for (int h = 0; h < kMsaMaxIndexHeads; ++h) s[h] = 0.f;
#pragma unroll 4
      for (int c = 0; c < DI / 8; ++c) {
        Pack16 kb;
        kb.u = *reinterpret_cast<const uint4*>(tile + lane * ROW + c * 8);
        float kf[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) kf[j] = bf16_to_f32(kb.h[j]);
#pragma unroll
        for (int h = 0; h < kMsaMaxIndexHeads; ++h) {
          if (h < p.ih) {
#pragma unroll
            for (int j = 0; j < 8; ++j) s[h] = fmaf(q_s[h * DI + c * 8 + j], kf[j], s[h]);
          }
        }
      }
#pragma unroll
      for (int h = 0; h < kMsaMaxIndexHeads; ++h) mx[h] = fmaxf(mx[h], s[h]);
    }
    __syncwarp();
  }
#pragma unroll
  for (int h = 0; h < kMsaMaxIndexHeads; ++h) {
    if (h < p.ih) {
      float v = mx[h];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
      if (lane == 0) p.scores[(static_cast<size_t>(row) * p.ih + h) * p.max_sel + b] = v;
    }
  }
}

// Selection from the block scores.  grid (ih, rows).
__global__ void __launch_bounds__(kMsaThreads) msa_index_pick_kernel(MsaSelectParams p) {
  extern __shared__ float sc[];                  // [max_sel]
  __shared__ float wv[kMsaThreads / 32];
  __shared__ int wi[kMsaThreads / 32];
  __shared__ int chosen[kMsaMaxTopk + 1];
  pdl_wait();
  const int h = blockIdx.x, row = blockIdx.y;
  const int pos = p.positions[row];
  const int nblk = min(pos / p.sel_block + 1, p.max_sel);
  const float* src = p.scores + (static_cast<size_t>(row) * p.ih + h) * p.max_sel;
  for (int b = threadIdx.x; b < nblk; b += kMsaThreads) sc[b] = b == nblk - 1 ? INFINITY : src[b];   // own block always kept
  __syncthreads();
  msa_topk_write(sc, nblk, min(p.topk, nblk), -1, chosen, wv, wi,
                 p.sel + (static_cast<size_t>(row) * p.ih + h) * p.topk, p.topk, 1, 0);
}

struct QsaCompressParams {
  const bf16* raw_cache;       // [blocks, page, DI] raw index keys (page == kpool)
  bf16* comp_cache;            // [blocks, DI] one compressed key per block
  const int32_t* positions;
  const int32_t* row_req;
  const int32_t* block_table;
  const float* inv_freq;
  const bf16* k_norm_w;        // [DI] or null
  int rows, kpool, rot_dim, max_blocks, one_plus_w;
  float eps;
};

// One warp per row; rows that do not complete a block leave at once.
template <int DI>
__global__ void __launch_bounds__(128) qsa_compress_kernel(QsaCompressParams p) {
  pdl_wait();
  constexpr int PER = DI / 32;
  const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= p.rows) return;
  const int pos = p.positions[row];
  if ((pos + 1) % p.kpool != 0) return;
  const int b = pos / p.kpool;
  const int blk = p.block_table[static_cast<size_t>(p.row_req[row]) * p.max_blocks + b];
  const bf16* src = p.raw_cache + static_cast<size_t>(blk) * p.kpool * DI;
  float v[PER];
#pragma unroll
  for (int j = 0; j < PER; ++j) v[j] = 0.f;
  for (int t = 0; t < p.kpool; ++t)
#pragma unroll
    for (int j = 0; j < PER; ++j) v[j] += bf16_to_f32(src[static_cast<size_t>(t) * DI + lane + 32 * j]);
#pragma unroll
  for (int j = 0; j < PER; ++j) v[j] = bf16_to_f32(f32_to_bf16(v[j] / static_cast<float>(p.kpool)));
  if (p.k_norm_w != nullptr) {
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < PER; ++j) ss += v[j] * v[j];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float rstd = rsqrtf(ss / DI + p.eps);
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      float g = bf16_to_f32(p.k_norm_w[lane + 32 * j]);
      if (p.one_plus_w) g += 1.f;
      v[j] = bf16_to_f32(f32_to_bf16(bf16_to_f32(f32_to_bf16(v[j] * rstd)) * g));
    }
  }
  const int half = p.rot_dim / 2;
  const int first = b * p.kpool;                 // the block's first position
  bf16* dst = p.comp_cache + static_cast<size_t>(blk) * DI;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int a = lane + 32 * j;
    const int pd = a < half ? a + half : (a < p.rot_dim ? a - half : a);
    float partner = 0.f;
#pragma unroll
    for (int jj = 0; jj < PER; ++jj) {
      const float cand = __shfl_sync(0xffffffffu, v[jj], pd & 31);
      if ((pd >> 5) == jj) partner = cand;
    }
    float r = v[j];
    if (a < p.rot_dim) {
      float sn, cs;
      sincosf(static_cast<float>(first) * p.inv_freq[a < half ? a : a - half], &sn, &cs);
      r = a < half ? v[j] * cs - partner * sn : v[j] * cs + partner * sn;
    }
    dst[a] = f32_to_bf16(r);
  }
}

struct QsaSelectParams {
  const bf16* iqk;             // [rows, iqk_stride]: index query head h at column h * DI
  int64_t iqk_stride;
  const bf16* comp_cache;      // [blocks, DI]
  const int32_t* block_table;
  const int32_t* row_req;
  const int32_t* positions;
  int32_t* sel;                // [rows, copies, select_k + 1]
  float* scores;               // optional [rows, max_sel]
  int rows, ih, max_blocks, kpool, select_k, max_sel, copies;
};

// grid (rows), kMsaThreads threads
template <int DI>
__global__ void __launch_bounds__(kMsaThreads) qsa_select_kernel(QsaSelectParams p) {
  extern __shared__ float sc[];                  // [max_sel]
  __shared__ float wv[kMsaThreads / 32];
  __shared__ int wi[kMsaThreads / 32];
  __shared__ int chosen[kMsaMaxTopk + 1];
  pdl_wait();
  const int row = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pos = p.positions[row];
  const int visible = min((pos + 1) / p.kpool, p.max_sel);          // complete blocks
  const int tail = (pos + 1) % p.kpool != 0 ? pos / p.kpool : -1;   // the row's own incomplete block
  const int32_t* bt = p.block_table + static_cast<size_t>(p.row_req[row]) * p.max_blocks;
  const bf16* q = p.iqk + static_cast<size_t>(row) * p.iqk_stride;
  const float inv = rsqrtf(static_cast<float>(DI));
  for (int b = warp; b < visible; b += kMsaThreads / 32) {
    const bf16* c = p.comp_cache + static_cast<size_t>(bt[b]) * DI;
    float cv[DI / 32];
#pragma unroll
    for (int j = 0; j < DI / 32; ++j) cv[j] = bf16_to_f32(c[lane + 32 * j]);
    float total = 0.f;
    for (int h = 0; h < p.ih; ++h) {                                 // ascending heads: a fixed summation order
      float s = 0.f;
#pragma unroll
      for (int j = 0; j < DI / 32; ++j) s = fmaf(bf16_to_f32(q[h * DI + lane + 32 * j]), cv[j], s);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      total += fmaxf(s, 0.f);
    }
    if (lane == 0) sc[b] = total * inv;
  }
  __syncthreads();
  if (p.scores != nullptr)
    for (int b = threadIdx.x; b < visible; b += kMsaThreads) p.scores[static_cast<size_t>(row) * p.max_sel + b] = sc[b];
  __syncthreads();
  msa_topk_write(sc, visible, min(p.select_k, visible), tail, chosen, wv, wi,
                 p.sel + static_cast<size_t>(row) * p.copies * (p.select_k + 1), p.select_k + 1, p.copies, p.select_k + 1);
}

}  // namespace dgpp

using namespace dgpp;

DGPP_API int dgpp_msa_index_prep(void* iqk, const void* positions, const void* row_req, const void* block_table,
                                 const void* inv_freq, const void* q_norm_w, const void* k_norm_w, void* index_cache,
                                 int rows, int ih, int di, int rot_dim, int page, int max_blocks, float eps,
                                 int one_plus_w, int raw_key, cudaStream_t st) {
  DGPP_REQUIRE(di == 64 || di == 128, "msa_index_prep: index width %d not in {64, 128}", di);
  DGPP_REQUIRE(rot_dim >= 2 && rot_dim <= di && rot_dim % 2 == 0, "msa_index_prep: bad rotary width %d", rot_dim);
  DGPP_REQUIRE(ih >= 1 && page >= 1, "msa_index_prep: bad geometry");
  if (rows == 0) return 0;
  MsaPrepParams p;
  p.iqk = static_cast<bf16*>(iqk);
  p.positions = static_cast<const int32_t*>(positions);
  p.row_req = static_cast<const int32_t*>(row_req);
  p.block_table = static_cast<const int32_t*>(block_table);
  p.inv_freq = static_cast<const float*>(inv_freq);
  p.q_norm_w = static_cast<const bf16*>(q_norm_w);
  p.k_norm_w = static_cast<const bf16*>(k_norm_w);
  p.index_cache = static_cast<bf16*>(index_cache);
  p.rows = rows; p.ih = ih; p.rot_dim = rot_dim; p.page = page; p.max_blocks = max_blocks; p.one_plus_w = one_plus_w;
  p.raw_key = raw_key;
  p.eps = eps;
  const int warps = rows * (ih + 1);
  const int grid = dgpp_ceil_div(warps, 4);
  if (di == 64) msa_index_prep_kernel<64><<<grid, 128, 0, st>>>(p);
  else msa_index_prep_kernel<128><<<grid, 128, 0, st>>>(p);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

DGPP_API int dgpp_msa_index_select(const void* iqk, int64_t iqk_stride, const void* index_cache,
                                   const void* block_table, const void* row_req, const void* positions, void* sel,
                                   void* scores, int rows, int ih, int di, int page, int max_blocks, int sel_block,
                                   int topk, int max_sel, cudaStream_t st) {
  DGPP_REQUIRE(di == 64 || di == 128, "msa_index_select: index width %d not in {64, 128}", di);
  DGPP_REQUIRE(topk >= 1 && topk <= kMsaMaxTopk, "msa_index_select: topk %d outside 1..%d", topk, kMsaMaxTopk);
  DGPP_REQUIRE(sel_block >= 1 && max_sel >= 1 && max_sel <= 8192, "msa_index_select: %d blocks of %d tokens unsupported",
               max_sel, sel_block);
  DGPP_REQUIRE(ih >= 1 && ih <= kMsaMaxIndexHeads && rows <= 65535, "msa_index_select: %d index heads (1..%d) / %d rows",
               ih, kMsaMaxIndexHeads, rows);
  DGPP_REQUIRE(scores != nullptr, "msa_index_select: the block-score workspace [rows, ih, max_sel] is required");
  if (rows == 0) return 0;
  MsaSelectParams p;
  p.iqk = static_cast<const bf16*>(iqk);
  p.iqk_stride = iqk_stride;
  p.index_cache = static_cast<const bf16*>(index_cache);
  p.block_table = static_cast<const int32_t*>(block_table);
  p.row_req = static_cast<const int32_t*>(row_req);
  p.positions = static_cast<const int32_t*>(positions);
  p.sel = static_cast<int32_t*>(sel);
  p.scores = static_cast<float*>(scores);
  p.rows = rows; p.ih = ih; p.page = page; p.max_blocks = max_blocks; p.sel_block = sel_block; p.topk = topk;
  p.max_sel = max_sel;
  // scores, then the pick
  const size_t smem_score = static_cast<size_t>(ih) * di * sizeof(float) +
                            static_cast<size_t>(kMsaScoreWarps) * 32 * (di + 8) * sizeof(bf16);
  dim3 grid_score(dgpp_ceil_div(max_sel, kMsaScoreWarps), rows);
  if (di == 64) msa_index_score_kernel<64><<<grid_score, kMsaScoreWarps * 32, smem_score, st>>>(p);
  else msa_index_score_kernel<128><<<grid_score, kMsaScoreWarps * 32, smem_score, st>>>(p);
  DGPP_CUDA_OK(cudaGetLastError());
  msa_index_pick_kernel<<<dim3(ih, rows), kMsaThreads, static_cast<size_t>(max_sel) * sizeof(float), st>>>(p);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

DGPP_API int dgpp_qsa_compress(const void* raw_cache, void* comp_cache, const void* positions, const void* row_req,
                               const void* block_table, const void* inv_freq, const void* k_norm_w, int rows, int di,
                               int kpool, int rot_dim, int max_blocks, float eps, int one_plus_w, cudaStream_t st) {
  DGPP_REQUIRE(di == 64 || di == 128, "qsa_compress: index width %d not in {64, 128}", di);
  DGPP_REQUIRE(kpool >= 1 && rot_dim >= 2 && rot_dim <= di && rot_dim % 2 == 0, "qsa_compress: bad geometry");
  if (rows == 0) return 0;
  QsaCompressParams p;
  p.raw_cache = static_cast<const bf16*>(raw_cache);
  p.comp_cache = static_cast<bf16*>(comp_cache);
  p.positions = static_cast<const int32_t*>(positions);
  p.row_req = static_cast<const int32_t*>(row_req);
  p.block_table = static_cast<const int32_t*>(block_table);
  p.inv_freq = static_cast<const float*>(inv_freq);
  p.k_norm_w = static_cast<const bf16*>(k_norm_w);
  p.rows = rows; p.kpool = kpool; p.rot_dim = rot_dim; p.max_blocks = max_blocks; p.one_plus_w = one_plus_w;
  p.eps = eps;
  const int grid = dgpp_ceil_div(rows, 4);
  if (di == 64) qsa_compress_kernel<64><<<grid, 128, 0, st>>>(p);
  else qsa_compress_kernel<128><<<grid, 128, 0, st>>>(p);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

// sel: int32 [rows, copies, select_k + 1]; scores: optional fp32 [rows, max_sel].
DGPP_API int dgpp_qsa_select(const void* iqk, int64_t iqk_stride, const void* comp_cache, const void* block_table,
                             const void* row_req, const void* positions, void* sel, void* scores, int rows, int ih,
                             int di, int max_blocks, int kpool, int select_k, int max_sel, int copies, cudaStream_t st) {
  DGPP_REQUIRE(di == 64 || di == 128, "qsa_select: index width %d not in {64, 128}", di);
  DGPP_REQUIRE(select_k >= 1 && select_k <= kMsaMaxTopk, "qsa_select: select_k %d outside 1..%d", select_k, kMsaMaxTopk);
  DGPP_REQUIRE(kpool >= 1 && max_sel >= 1 && max_sel <= 8192 && copies >= 1 && ih >= 1, "qsa_select: bad geometry");
  if (rows == 0) return 0;
  QsaSelectParams p;
  p.iqk = static_cast<const bf16*>(iqk);
  p.iqk_stride = iqk_stride;
  p.comp_cache = static_cast<const bf16*>(comp_cache);
  p.block_table = static_cast<const int32_t*>(block_table);
  p.row_req = static_cast<const int32_t*>(row_req);
  p.positions = static_cast<const int32_t*>(positions);
  p.sel = static_cast<int32_t*>(sel);
  p.scores = static_cast<float*>(scores);
  p.rows = rows; p.ih = ih; p.max_blocks = max_blocks; p.kpool = kpool; p.select_k = select_k; p.max_sel = max_sel;
  p.copies = copies;
  const size_t smem = static_cast<size_t>(max_sel) * sizeof(float);
  if (di == 64) qsa_select_kernel<64><<<rows, kMsaThreads, smem, st>>>(p);
  else qsa_select_kernel<128><<<rows, kMsaThreads, smem, st>>>(p);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}
