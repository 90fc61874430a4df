// Absorbed multi-head latent attention on the tensor cores (tcgen05 kind::f16, bf16 operands) over the paged latent cache.
//
// One CTA serves one query row (a decode token, or one row of a prefill chunk), one group of up to 32 heads and one KV
// split, and walks its token range in tiles of 128.  A latent tile [128 tokens, dc + dr] is fetched ONCE by TMA (as
// (dc + dr) / 64 column blocks of [128, 64] bf16 with the 128-byte swizzle) and feeds both products:
//
//   MMA1   S^T[token, head]  = C_tile[128, dc + dr] . Q[head, dc + dr]^T          A = the tile read K-major
//   softmax (thread = token): scores in log2 units, column maxima by shuffle + shared memory, p = 2^(s - m)
//   MMA2   O^T[d, head]      = C_tile^T[d, 128 tokens] . P[head, 128 tokens]^T    A = the same tile read MN-major,
//                                                                                  dc / 128 blocks of 128 latent dims
//   accumulate (thread = latent dim of each block): o = (o + O^T) * 2^(m_old - m_new)
//
// The tile is single buffered (147 KB at dc + dr = 576): the PV product of tile i must retire before tile i + 1 lands.
// S^T, P and O^T are double buffered, so the fold of tile i overlaps the load of tile i + 1.
// Warps: 0 = TMA producer (walks the block table), 1 = MMA issuer / TMEM owner, 2..5 = softmax and accumulation.
// Every wait is bounded (status code + clean exit).  Split partials use the layout of mla.cu and its combine kernel.
// (reference counterparts: src/kernels/dsa.cu:2502 attn_flash_kernel, latent decode kernels of the same file.)
#include <cuda.h>
#include <math.h>
#include <string.h>

#include "common/common.h"
#include "common/dtypes.cuh"
#include "common/ptx.cuh"
#include "kernels/gemm_common.cuh"

namespace dgpp {

constexpr int kMtThreads = 192;
constexpr int kMtTile = 128;   // tokens per tile
constexpr int kMtNQ = 32;      // head columns per CTA
constexpr int kMtBlk = kMtTile * 128;   // 16 KB: one 64-element column block of the latent tile

struct MlaTcParams {
  const bf16* q;               // [rows, heads, dc + dr] absorbed query, rotary part rotated
  const bf16* cache;           // [blocks, page, dc + dr] (the sparse form gathers rows itself)
  const int32_t* sel;          // sparse form: [rows, sel_stride] selected token positions, ascending, -1 padded
  int sel_stride;
  const int32_t* block_table;  // [requests, max_blocks]
  const int32_t* row_req;      // [rows]
  const int32_t* positions;    // [rows] position of the row's own token (already in the cache)
  float* part_ml;              // [rows, heads, splits, 2]   (max in natural-log units, sum)
  float* part_acc;             // [rows, heads, splits, dc]
  bf16* out;                   // [rows, heads, dc]
  DeviceStatus* status;
  int rows, heads, page, max_blocks, splits;
  float scale;
};

// SPARSE: the tokens of a tile come from the row's selection list instead of consecutive positions; the four softmax
// warps (idle while a tile loads: it is single buffered) gather them, thread = token: 72 16-byte chunks of the token's
// latent row into the swizzled column blocks, then a proxy fence and one arrival per warp on the tile barrier.
template <int DC, int DR, bool SPARSE>
__global__ void __launch_bounds__(kMtThreads, 1)
mla_decode_tc_kernel(const __grid_constant__ CUtensorMap tmC, MlaTcParams p) {
  constexpr int D = DC + DR;
  constexpr int KB = D / 64;     // column blocks of the tile and of Q
  constexpr int MB = DC / 128;   // 128-dim output blocks
  static_assert(D % 64 == 0 && DC % 128 == 0 && MB <= 4, "latent geometry");
  constexpr int kTileBytes = KB * kMtBlk;
  constexpr int kQBlk = kMtNQ * 128;     // 4 KB: [32 heads, 64 elements]
  extern __shared__ __align__(1024) unsigned char smem_dyn[];
  unsigned char* sp = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  unsigned char* sC = sp;  sp += kTileBytes;
  unsigned char* sQ = sp;  sp += KB * kQBlk;
  unsigned char* sP = sp;  sp += 2 * 2 * kQBlk;       // [buffer][64-token block][32 heads x 128 B]
  float* red = reinterpret_cast<float*>(sp);   sp += 2 * 4 * kMtNQ * sizeof(float);   // [buffer][warp][head] tile maxima
  float* mrun = reinterpret_cast<float*>(sp);  sp += 2 * kMtNQ * sizeof(float);       // [buffer][head] running maxima
  float* corr = reinterpret_cast<float*>(sp);  sp += 2 * kMtNQ * sizeof(float);       // [buffer][head] 2^(m_old - m_new)
  float* lred = reinterpret_cast<float*>(sp);  sp += 4 * kMtNQ * sizeof(float);       // [warp][head] probability mass
  float* flags = reinterpret_cast<float*>(sp); sp += 2 * 4 * sizeof(float);           // [buffer][warp] 1 = this warp gave up
  uint64_t* c_full = reinterpret_cast<uint64_t*>(sp);
  uint64_t* c_empty = c_full + 1;
  uint64_t* s_full = c_empty + 1;   // [2]
  uint64_t* p_full = s_full + 2;    // [2]
  uint64_t* o_full = p_full + 2;    // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_full + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int split = blockIdx.x, row = blockIdx.y, hg = blockIdx.z;
  const int req = p.row_req[row];
  int len = p.positions[row] + 1;
  const int32_t* sel = nullptr;
  if (SPARSE) {
    // listed tokens at or before the row's own position (lists are ascending, so they form a prefix of the list)
    sel = p.sel + static_cast<size_t>(row) * p.sel_stride;
    int n = 0;
    for (int i0 = 0; i0 < p.sel_stride; i0 += kMtThreads) {
      const int i = i0 + threadIdx.x;
      n += __syncthreads_count(i < p.sel_stride && sel[i] >= 0 && sel[i] < len);
    }
    len = n;
  }
  const int total_tiles = (len + kMtTile - 1) / kMtTile;
  const int per = (total_tiles + p.splits - 1) / p.splits;
  const int tile_begin = split * per;
  const int ntiles = max(0, min(total_tiles, tile_begin + per) - tile_begin);
  const int32_t* bt = p.block_table + static_cast<size_t>(req) * p.max_blocks;
  const int nheads = min(kMtNQ, p.heads - hg * kMtNQ);

  if (threadIdx.x == 0) {
    mbar_init(c_full, SPARSE ? 4 : 1); mbar_init(c_empty, 1);
    for (int i = 0; i < 2; ++i) { mbar_init(&s_full[i], 1); mbar_init(&p_full[i], 4); mbar_init(&o_full[i], 1); }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmC);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  pdl_wait();
  // ---- the group's query rows as the B operand of MMA1: KB blocks of [32 heads, 64 elements], 128-byte swizzle
  if (warp >= 2) {
    const int t = threadIdx.x - 64;
    constexpr int kChunks = D / 8;   // 16-byte chunks per head
    for (int i = t; i < kMtNQ * kChunks; i += 128) {
      const int h = i / kChunks, c = i % kChunks;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (h < nheads)
        v = *reinterpret_cast<const uint4*>(p.q + (static_cast<size_t>(row) * p.heads + hg * kMtNQ + h) * D + c * 8);
      *reinterpret_cast<uint4*>(sQ + (c >> 3) * kQBlk + h * 128 + (((c & 7) ^ (h & 7)) << 4)) = v;
    }
    if (t < kMtNQ) { mrun[kMtNQ + t] = -INFINITY; mrun[t] = -INFINITY; }
    fence_proxy_async_smem();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s = tmem_base;         // 2 x 32 columns
  const uint32_t tmem_o = tmem_base + 64;    // 2 x MB x 32 columns

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (dense form)
    if (!SPARSE && elect_one()) {
      const int ppt = kMtTile / p.page;
      for (int i = 0; i < ntiles; ++i) {
        if (!wait_bar(c_empty, (i & 1) ^ 1)) { report(p.status, kTimeoutStageEmpty, 51); *abort_flag = 1; break; }
        mbar_expect_tx(c_full, kTileBytes);
        const int page0 = (tile_begin + i) * kMtTile / p.page;
        for (int pg = 0; pg < ppt; ++pg) {
          const int pi = min(page0 + pg, p.max_blocks - 1);
          const int r0 = bt[pi] * p.page;
#pragma unroll
          for (int kb = 0; kb < KB; ++kb)
            tma_load_2d(sC + kb * kMtBlk + pg * p.page * 128, &tmC, kb * 64, r0, c_full);
        }
        if (*abort_flag) break;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc1 = umma_idesc_f16(128, kMtNQ, 1u, 1u);                // tile (K-major) x Q (K-major)
      constexpr uint32_t idesc2 = umma_idesc_f16(128, kMtNQ, 1u, 1u) | (1u << 15);   // tile^T (MN-major A) x P (K-major)
      const uint32_t c_addr = smem_u32(sC), q_addr = smem_u32(sQ);
      auto mma2 = [&](int j) {
        const int b = j & 1;
        const uint32_t p_addr = smem_u32(sP + b * 2 * kQBlk);
#pragma unroll
        for (int mb = 0; mb < MB; ++mb)
#pragma unroll
          for (int k = 0; k < kMtTile / 16; ++k)   // 16 tokens per step: two 8-row groups of the tile, 32 bytes of P
            umma_f16(tmem_o + (b * MB + mb) * kMtNQ, umma_desc_sw128_mn(c_addr + 2 * mb * kMtBlk + k * 2048, kMtBlk),
                     umma_desc_sw128(p_addr + (k >> 2) * kQBlk + (k & 3) * 32), idesc2, k > 0 ? 1u : 0u);
        umma_commit(&o_full[b]);
        umma_commit(c_empty);
      };
      bool ok = true;
      for (int i = 0; i < ntiles && ok; ++i) {
        const int b = i & 1;
        if (!wait_bar(c_full, i & 1)) { report(p.status, kTimeoutTmaFull, 52); *abort_flag = 1; ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int kb = 0; kb < KB; ++kb)
#pragma unroll
          for (int k = 0; k < 4; ++k)   // 16 elements (32 bytes) per step
            umma_f16(tmem_s + b * kMtNQ, umma_desc_sw128(c_addr + kb * kMtBlk + k * 32),
                     umma_desc_sw128(q_addr + kb * kQBlk + k * 32), idesc1, (kb > 0 || k > 0) ? 1u : 0u);
        umma_commit(&s_full[b]);
        // the tile is single buffered: its PV product follows as soon as the probabilities are written
        if (!wait_bar(&p_full[b], (i >> 1) & 1)) { report(p.status, kTimeoutConvert, 53); *abort_flag = 1; ok = false; break; }
        tc_fence_after();
        mma2(i);
        if (*abort_flag) ok = false;
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + accumulation (warps 2..5)
    const int quad = warp & 3;
    const int idx = quad * 32 + lane;        // token lane for S^T, latent-dim lane for O^T
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const int wslot = warp - 2;
    const float sm = p.scale * 1.4426950408889634f;  // scores in log2 units
    float l_thr[kMtNQ];
    float o_acc[MB][kMtNQ];
#pragma unroll
    for (int c = 0; c < kMtNQ; ++c) {
      l_thr[c] = 0.f;
#pragma unroll
      for (int mb = 0; mb < MB; ++mb) o_acc[mb][c] = 0.f;
    }
    auto fold = [&](int j) -> bool {   // o += O^T of tile j (both halves of the head columns)
      const int bp = j & 1;
      if (!wait_bar(&o_full[bp], (j >> 1) & 1)) return false;
      tc_fence_after();
#pragma unroll
      for (int mb = 0; mb < MB; ++mb) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t oc[16];
          tmem_ld_x16(tmem_o + (bp * MB + mb) * kMtNQ + half * 16 + lane_addr, oc);
          tmem_ld_wait();
#pragma unroll
          for (int c = 0; c < 16; ++c) o_acc[mb][half * 16 + c] += __uint_as_float(oc[c]);
        }
      }
      return true;
    };
    bool ok = true;
    for (int i = 0; i < ntiles; ++i) {
      const int b = i & 1;
      const int t = (tile_begin + i) * kMtTile + idx;
      const bool valid = t < len;
      if (SPARSE) {
        if (wait_bar(c_empty, (i & 1) ^ 1)) {
          // a warp gathers its 32 tokens one after the other: lanes take the 72 chunks of a token's row in turns, so the
          // row is read with coalesced 512-byte requests; four tokens are in flight at a time
          const int my_tok = valid ? sel[t] : -1;
#pragma unroll 1
          for (int t4 = 0; t4 < 32; t4 += 4) {
            uint4 v[4][3];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int tok = __shfl_sync(0xffffffffu, my_tok, t4 + u);
              const uint4* src = tok >= 0 ? reinterpret_cast<const uint4*>(
                                                p.cache + (static_cast<size_t>(bt[tok / p.page]) * p.page + tok % p.page) * D)
                                          : nullptr;
#pragma unroll
              for (int j = 0; j < 3; ++j) {
                const int c = lane + 32 * j;
                v[u][j] = (src != nullptr && c < D / 8) ? src[c] : make_uint4(0u, 0u, 0u, 0u);   // unlisted rows: zeros (0 x NaN)
              }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int r = quad * 32 + t4 + u;
#pragma unroll
              for (int j = 0; j < 3; ++j) {
                const int c = lane + 32 * j;
                if (c < D / 8)
                  *reinterpret_cast<uint4*>(sC + (c >> 3) * kMtBlk + r * 128 + (((c & 7) ^ (r & 7)) << 4)) = v[u][j];
              }
            }
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(c_full);
        } else {
          report(p.status, kTimeoutStageEmpty, 57);
          *abort_flag = 1;
        }
      }
      bool okw = ok && wait_bar(&s_full[b], (i >> 1) & 1);
      if (!okw && ok) { report(p.status, kTimeoutAccum, 54); *abort_flag = 1; }
      tc_fence_after();
      float s[kMtNQ];
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t raw[16];
        tmem_ld_x16(tmem_s + b * kMtNQ + half * 16 + lane_addr, raw);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 16; ++c) s[half * 16 + c] = valid ? __uint_as_float(raw[c]) * sm : -INFINITY;
      }
      float* rp = red + (b * 4 + wslot) * kMtNQ;
#pragma unroll
      for (int c = 0; c < kMtNQ; ++c) {
        float mx = s[c];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        if (lane == 0) rp[c] = mx;
      }
      if (lane == 0) flags[b * 4 + wslot] = (okw && !*abort_flag) ? 0.f : 1.f;
      asm volatile("bar.sync 1, 128;" ::: "memory");
      // a failed wait must not leave the other warps alone at the barriers: all four read the verdicts and leave together
      if (flags[b * 4] + flags[b * 4 + 1] + flags[b * 4 + 2] + flags[b * 4 + 3] != 0.f) { ok = false; break; }
      const float* r0 = red + b * 4 * kMtNQ;
      const float* m_prev = mrun + (b ^ 1) * kMtNQ;
      unsigned char* pbuf = sP + b * 2 * kQBlk + (idx >> 6) * kQBlk;
      const uint32_t pbyte = (idx & 63) * 2;
#pragma unroll
      for (int c = 0; c < kMtNQ; ++c) {
        const float mt = fmaxf(fmaxf(r0[c], r0[kMtNQ + c]), fmaxf(r0[2 * kMtNQ + c], r0[3 * kMtNQ + c]));
        const float mo = m_prev[c];
        const float mn = fmaxf(mo, mt);
        const float cr = (mo == -INFINITY) ? 0.f : exp2f(mo - mn);
        const float pv = (valid && mn > -INFINITY) ? exp2f(s[c] - mn) : 0.f;
        l_thr[c] = l_thr[c] * cr + pv;
        if (idx == c) { mrun[b * kMtNQ + c] = mn; corr[b * kMtNQ + c] = cr; }
        // P[head c][token idx]: row c of the 64-token block, 2 bytes at the token's column (128-byte swizzle)
        *reinterpret_cast<bf16*>(pbuf + c * 128 + ((((pbyte >> 4) ^ (c & 7)) << 4) | (pbyte & 15))) = f32_to_bf16(pv);
      }
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[b]);
      asm volatile("bar.sync 1, 128;" ::: "memory");   // corr[b] / mrun[b] visible to all four warps
      // fold the previous tile's O^T (taken relative to the previous maxima), then rescale to this tile's maxima
      if (i > 0 && !fold(i - 1)) {
        report(p.status, kTimeoutAccum, 55);
        *abort_flag = 1;   // agreed on at the next tile's barrier
      }
      const float* cb = corr + b * kMtNQ;
#pragma unroll
      for (int c = 0; c < kMtNQ; ++c) {
        const float cr = cb[c];
#pragma unroll
        for (int mb = 0; mb < MB; ++mb) o_acc[mb][c] *= cr;
      }
    }
    bool done = ok && !*abort_flag;
    if (done && ntiles > 0 && !fold(ntiles - 1)) {
      report(p.status, kTimeoutAccum, 56);
      *abort_flag = 1;
      done = false;
    }
    // total probability mass per head: sum the per-thread partials
#pragma unroll
    for (int c = 0; c < kMtNQ; ++c) {
      float l = l_thr[c];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
      if (lane == 0) lred[wslot * kMtNQ + c] = l;
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (done) {
      const float* m_fin = mrun + ((ntiles > 0 ? (ntiles - 1) & 1 : 0)) * kMtNQ;
#pragma unroll
      for (int c = 0; c < kMtNQ; ++c) {
        if (c < nheads) {
          const float l = lred[c] + lred[kMtNQ + c] + lred[2 * kMtNQ + c] + lred[3 * kMtNQ + c];
          const size_t rh = static_cast<size_t>(row) * p.heads + hg * kMtNQ + c;
          if (p.splits == 1) {
            const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
            for (int mb = 0; mb < MB; ++mb) p.out[rh * DC + mb * 128 + idx] = f32_to_bf16(o_acc[mb][c] * inv);
          } else {
            const size_t pi = rh * p.splits + split;
#pragma unroll
            for (int mb = 0; mb < MB; ++mb) p.part_acc[pi * DC + mb * 128 + idx] = o_acc[mb][c];
            if (idx == 0) {
              // running max is kept in log2 units; the combine kernel works in natural-log units
              p.part_ml[pi * 2] = ntiles > 0 ? m_fin[c] * 0.6931471805599453f : -INFINITY;
              p.part_ml[pi * 2 + 1] = l;
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, 512);
}

__global__ void mla_tc_combine_kernel(const float* __restrict__ part_ml, const float* __restrict__ part_acc,
                                      bf16* __restrict__ out, int splits, int dc) {
  pdl_wait();
  const size_t rh = blockIdx.x;
  float mm = -INFINITY;
  for (int s = 0; s < splits; ++s) mm = fmaxf(mm, part_ml[(rh * splits + s) * 2]);
  for (int d = threadIdx.x; d < dc; d += blockDim.x) {
    float ll = 0.f, acc = 0.f;
    for (int s = 0; s < splits; ++s) {   // ascending split order
      const float ms = part_ml[(rh * splits + s) * 2];
      const float c = ms == -INFINITY ? 0.f : __expf(ms - mm);
      ll += part_ml[(rh * splits + s) * 2 + 1] * c;
      acc += part_acc[(rh * splits + s) * dc + d] * c;
    }
    out[rh * dc + d] = f32_to_bf16(ll > 0.f ? acc / ll : 0.f);
  }
}

}  // namespace dgpp

using namespace dgpp;

// Absorbed latent attention on the tensor cores, dense or over per-row selection lists (sel [rows, sel_stride] int32).  cache: [num_blocks, page, dc + dr] bf16 pages; q: [rows, heads,
// dc + dr]; out: [rows, heads, dc].  dc = 512, dr = 64; page in {16, 32, 64, 128}.  Rows of a prefill chunk are simply
// rows whose positions differ (the causal limit is the row's own position).
DGPP_API int dgpp_mla_decode_tc(const void* q, const void* cache, const void* block_table, const void* row_req,
                                const void* positions, const void* sel, int sel_stride, void* part_ml, void* part_acc,
                                void* out, int rows, int heads, int dc, int dr, int page, int max_blocks, int num_blocks,
                                int splits, float scale, cudaStream_t st) {
  DGPP_REQUIRE(dc == 512 && dr == 64, "mla_decode_tc: latent geometry %d + %d (512 + 64 only)", dc, dr);
  DGPP_REQUIRE(page == 16 || page == 32 || page == 64 || page == 128, "mla_decode_tc: page %d unsupported", page);
  DGPP_REQUIRE(splits >= 1 && (splits == 1 || (part_ml && part_acc)), "mla_decode_tc: scratch required for splits");
  DGPP_REQUIRE(out != nullptr && heads >= 1, "mla_decode_tc: bad arguments");
  if (rows == 0) return 0;
  MlaTcParams p;
  p.q = static_cast<const bf16*>(q);
  p.cache = static_cast<const bf16*>(cache);
  p.sel = static_cast<const int32_t*>(sel);
  p.sel_stride = sel_stride;
  p.block_table = static_cast<const int32_t*>(block_table);
  p.row_req = static_cast<const int32_t*>(row_req);
  p.positions = static_cast<const int32_t*>(positions);
  p.part_ml = static_cast<float*>(part_ml);
  p.part_acc = static_cast<float*>(part_acc);
  p.out = static_cast<bf16*>(out);
  p.status = device_status_ptr();
  p.rows = rows; p.heads = heads; p.page = page; p.max_blocks = max_blocks; p.splits = splits; p.scale = scale;
  const int D = dc + dr;
  CUtensorMap tC;
  if (make_tmap_2d(&tC, cache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, D, static_cast<uint64_t>(num_blocks) * page,
                   static_cast<uint64_t>(D) * 2, 64, page, CU_TENSOR_MAP_SWIZZLE_128B))
    return -1;
  constexpr int KB = 576 / 64;
  constexpr size_t smem = 1024 + KB * kMtBlk + KB * kMtNQ * 128 + 4 * kMtNQ * 128 + (2 * 4 + 2 + 2 + 4) * kMtNQ * 4 + 2 * 4 * 4 +
                          8 * 8 + 64;
  static_assert(smem <= 227 * 1024, "mla_decode_tc: shared memory over the per-CTA limit");
  static bool attr = false;
  if (!attr) {
    DGPP_CUDA_OK(cudaFuncSetAttribute(mla_decode_tc_kernel<512, 64, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      static_cast<int>(smem)));
    DGPP_CUDA_OK(cudaFuncSetAttribute(mla_decode_tc_kernel<512, 64, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      static_cast<int>(smem)));
    attr = true;
  }
  dim3 grid(splits, rows, dgpp_ceil_div(heads, kMtNQ));
  if (sel) mla_decode_tc_kernel<512, 64, true><<<grid, kMtThreads, smem, st>>>(tC, p);
  else mla_decode_tc_kernel<512, 64, false><<<grid, kMtThreads, smem, st>>>(tC, p);
  DGPP_CUDA_OK(cudaGetLastError());
  if (splits > 1) {
    mla_tc_combine_kernel<<<rows * heads, 256, 0, st>>>(p.part_ml, p.part_acc, p.out, splits, dc);
    DGPP_CUDA_OK(cudaGetLastError());
  }
  return 0;
}
