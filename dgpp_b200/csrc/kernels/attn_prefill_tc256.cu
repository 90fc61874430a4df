// Causal flash attention for prefill at head_dim 256 over the paged FP8 KV cache, on tcgen05 (kind::f8f6f4).
//
// Same arithmetic as the head_dim-128 kernel (attn_prefill_tc.cu): one CTA = one query head x 128 consecutive query
// positions; Q and P are carried as two e4m3 terms, K / V go from the cache pages to the tensor core untouched.  A
// 256-wide head is two 128-byte halves everywhere (tiles are [rows, 128 B] with the 128-byte swizzle, half 0 then half 1):
//
//   MMA1   S[q, t]        = sum over halves, terms of Q[q, half] . K[t, half]^T       16 MMAs of 128 x 128 x 32
//   MMA2   O[q, half]     = sum over terms of P[q, t] . V[t, half]                     16 MMAs of 128 x 128 x 32
//
// A thread cannot hold 256 output accumulators, so the softmax runs on TWO sets of four warps.  Both sets own all 128
// query rows (thread = row).  Set s computes the scores / probabilities of token columns [64 s, 64 s + 64) of every tile
// and accumulates output half s (128 fp32 registers).  Per tile the sets exchange their partial row maxima through
// shared memory (one 256-thread named barrier); the row sums stay per set and are added once at the end.
//
// Shared memory: Q 64 KB, P 32 KB, K ring 2 x 32 KB, V 1 x 32 KB (V of tile i + 1 is fetched while the softmax of tile
// i + 1 runs, after the PV product of tile i has retired), token scales in a ring of 4.
// Warps: 0 = TMA producer, 1 = MMA issuer / TMEM owner (512 columns: S 2 x 128, O 256), 2..5 = set 0, 6..9 = set 1.
// Every wait is bounded (status code + clean exit).
// (reference counterparts: src/kernels/full_attn.cu:442,679,983 prefill kernels at head_dim 256.)
#include <cuda.h>
#include <math.h>
#include <string.h>

#include "common/common.h"
#include "common/dtypes.cuh"
#include "common/ptx.cuh"
#include "kernels/gemm_common.cuh"

namespace dgpp {

constexpr int kA2Threads = 320;
constexpr int kA2Tile = 128;          // tokens per tile, query rows per CTA
constexpr int kA2Half = kA2Tile * 128;  // 16 KB: one 128-byte half of a 128-row tile
constexpr int kA2KStages = 2;
constexpr int kA2ScaleSlots = 4;

struct AttnPrefill256Params {
  const bf16* q;            // [T, q_stride]: head h at column h * 256 (already rotated)
  int64_t q_stride;
  const float* k_scale;     // [blocks, hkv, page]
  const float* v_scale;
  const int32_t* block_table;  // row of this request
  bf16* out;                // [T, hq * 256]
  DeviceStatus* status;
  int T, pos0, hq, hkv, page, max_blocks, window;
  float scale;
};

__device__ __forceinline__ uint32_t sw128_o2(uint32_t row, uint32_t byte_in_row) {
  return row * 128u + ((((byte_in_row >> 4) ^ (row & 7u)) << 4) | (byte_in_row & 15u));
}

// Row maximum of raw score * k_scale over 64 token columns starting at `col0` (thread = query row).
template <bool kMask>
__device__ __forceinline__ float half_row_max(uint32_t taddr, const float* ks, int col0, int t0, int my_pos, int my_first) {
  float mt = -INFINITY;
#pragma unroll 1
  for (int c0 = col0; c0 < col0 + 64; c0 += 16) {
    uint32_t raw[16];
    tmem_ld_x16(taddr + c0, raw);
    tmem_ld_wait();
#pragma unroll
    for (int q4 = 0; q4 < 4; ++q4) {
      const float4 k4 = *reinterpret_cast<const float4*>(ks + c0 + q4 * 4);
      const float kk[4] = {k4.x, k4.y, k4.z, k4.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float sv = __uint_as_float(raw[q4 * 4 + j]) * kk[j];
        if (kMask) {
          const int t = t0 + c0 + q4 * 4 + j;
          mt = fmaxf(mt, (t <= my_pos && t >= my_first) ? sv : -INFINITY);
        } else {
          mt = fmaxf(mt, sv);
        }
      }
    }
  }
  return mt;
}

// Probabilities of 64 token columns: p = 2^(raw * k_scale * sm - m); P = p * v_scale * c_tile as two e4m3 terms in row r
// of the swizzled A operand (term 2 one tile further).  Returns the row sum of p over these columns.
template <bool kMask>
__device__ __forceinline__ float half_probs(uint32_t taddr, const float* ks, const float* vs, unsigned char* sP, int r,
                                            int col0, float sm, float neg_m, float c_tile, int t0, int my_pos, int my_first) {
  float lsum = 0.f;
#pragma unroll 1
  for (int c0 = col0; c0 < col0 + 64; c0 += 16) {
    uint32_t raw[16];
    tmem_ld_x16(taddr + c0, raw);
    tmem_ld_wait();
    Pack16 a, bq;
#pragma unroll
    for (int q4 = 0; q4 < 4; ++q4) {
      const float4 k4 = *reinterpret_cast<const float4*>(ks + c0 + q4 * 4);
      const float4 v4 = *reinterpret_cast<const float4*>(vs + c0 + q4 * 4);
      const float kk[4] = {k4.x, k4.y, k4.z, k4.w};
      const float vv[4] = {v4.x, v4.y, v4.z, v4.w};
      float pw[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float e = fmaf(__uint_as_float(raw[q4 * 4 + j]) * kk[j], sm, neg_m);
        if (kMask) {
          const int t = t0 + c0 + q4 * 4 + j;
          e = (t <= my_pos && t >= my_first) ? e : -INFINITY;
        }
        const float pv = fast_exp2(e);
        lsum += pv;
        pw[j] = pv * (vv[j] * c_tile);
      }
      f32x2_to_e4m3x2_two_term(pw[0], pw[1], a.s[q4 * 2], bq.s[q4 * 2]);
      f32x2_to_e4m3x2_two_term(pw[2], pw[3], a.s[q4 * 2 + 1], bq.s[q4 * 2 + 1]);
    }
    *reinterpret_cast<uint4*>(sP + sw128_o2(r, c0)) = a.u;
    *reinterpret_cast<uint4*>(sP + kA2Half + sw128_o2(r, c0)) = bq.u;
  }
  return lsum;
}

__global__ void __launch_bounds__(kA2Threads, 1)
attn_prefill_tc256_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                          AttnPrefill256Params p) {
  constexpr int D = 256;
  constexpr int kTileBytes = kA2Tile * D;  // 32 KB: both halves
  extern __shared__ __align__(1024) unsigned char smem_dyn[];
  unsigned char* sp = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  unsigned char* sQ = sp;  sp += 2 * kTileBytes;             // [term][half][128 rows x 128 B]
  unsigned char* sP = sp;  sp += 2 * kA2Half;                // [term][128 rows x 128 B]
  unsigned char* sK = sp;  sp += kA2KStages * kTileBytes;    // [stage][half][128 tokens x 128 B]
  unsigned char* sV = sp;  sp += kTileBytes;                 // [half][128 tokens x 128 B]
  float* sKs = reinterpret_cast<float*>(sp);  sp += kA2ScaleSlots * kA2Tile * sizeof(float);
  float* sVs = reinterpret_cast<float*>(sp);  sp += kA2ScaleSlots * kA2Tile * sizeof(float);
  float* rowmax = reinterpret_cast<float*>(sp);  sp += 2 * 2 * kA2Tile * sizeof(float);   // [parity][set][row]
  float* red = reinterpret_cast<float*>(sp);  sp += 2 * 16 * sizeof(float);               // [parity][8 v-scale maxima, 8 flags]
  uint64_t* k_full = reinterpret_cast<uint64_t*>(sp);
  uint64_t* k_empty = k_full + kA2KStages;
  uint64_t* v_full = k_empty + kA2KStages;   // [1]
  uint64_t* v_empty = v_full + 1;            // [1]
  uint64_t* s_full = v_empty + 1;            // [2]
  uint64_t* p_full = s_full + 2;             // [1]
  uint64_t* o_full = p_full + 1;             // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.y, kvh = head / (p.hq / p.hkv);
  const int row0 = blockIdx.x * kA2Tile;                      // first chunk row of this CTA
  const int rows = min(kA2Tile, p.T - row0);
  const int last_pos = p.pos0 + row0 + rows - 1;
  const int first_pos = p.pos0 + row0;
  const int first_tok = (p.window > 0 && first_pos + 1 > p.window) ? first_pos + 1 - p.window : 0;
  const int base = first_tok & ~(kA2Tile - 1);
  const int ntiles = (last_pos + 1 - base + kA2Tile - 1) / kA2Tile;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kA2KStages; ++i) { mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1); }
    mbar_init(v_full, 1); mbar_init(v_empty, 1);
    mbar_init(&s_full[0], 1); mbar_init(&s_full[1], 1);
    mbar_init(p_full, 8);
    mbar_init(o_full, 1);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  pdl_wait();
  // ---- quantise the query rows into two e4m3 terms: thread (set, row) converts half `set` of its row; the row scale is
  //      the maximum over both halves (exchanged through shared memory)
  const int set = warp >= 6 ? 1 : 0;
  const int quad = warp & 3;                 // the TMEM lane quadrant this warp may read: warp % 4
  const int r = quad * 32 + lane;
  float q_scale = 1.f;
  if (warp >= 2) {
    float v[128];
    float amax = 0.f;
    if (r < rows) {
      const uint4* src = reinterpret_cast<const uint4*>(p.q + static_cast<size_t>(row0 + r) * p.q_stride + head * D + set * 128);
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        Pack16 x;
        x.u = src[c];
#pragma unroll
        for (int j = 0; j < 8; ++j) { v[c * 8 + j] = bf16_to_f32(x.h[j]); amax = fmaxf(amax, fabsf(v[c * 8 + j])); }
      }
    } else {
#pragma unroll
      for (int j = 0; j < 128; ++j) v[j] = 0.f;
    }
    rowmax[set * kA2Tile + r] = amax;
    asm volatile("bar.sync 3, 256;" ::: "memory");
    amax = fmaxf(amax, rowmax[(set ^ 1) * kA2Tile + r]);
    q_scale = amax > 0.f ? amax / 448.f : 1.f;
    const float inv = 1.f / q_scale;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      Pack16 a, b;
#pragma unroll
      for (int j = 0; j < 8; ++j)
        f32x2_to_e4m3x2_two_term(v[c * 16 + 2 * j] * inv, v[c * 16 + 2 * j + 1] * inv, a.s[j], b.s[j]);
      *reinterpret_cast<uint4*>(sQ + set * kA2Half + sw128_o2(r, c * 16)) = a.u;
      *reinterpret_cast<uint4*>(sQ + kTileBytes + set * kA2Half + sw128_o2(r, c * 16)) = b.u;
    }
    fence_proxy_async_smem();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s = tmem_base;          // 2 x 128 columns
  const uint32_t tmem_o = tmem_base + 256;    // 2 halves x 128 columns

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer: K_0, then (K_{i+1}, V_i) per tile
    if (elect_one()) {
      const int ppt = kA2Tile / p.page;
      auto load_k = [&](int i) -> bool {
        const int s = i % kA2KStages, slot = i % kA2ScaleSlots;
        if (!wait_bar(&k_empty[s], ((i / kA2KStages) & 1) ^ 1)) { report(p.status, kTimeoutStageEmpty, 41); *abort_flag = 1; return false; }
        mbar_expect_tx(&k_full[s], kTileBytes + 2 * kA2Tile * sizeof(float));
        const int page0 = (base + i * kA2Tile) / p.page;
        for (int pg = 0; pg < ppt; ++pg) {
          const int pi = min(page0 + pg, p.max_blocks - 1);
          const int r0 = (p.block_table[pi] * p.hkv + kvh) * p.page;
          tma_load_2d(sK + s * kTileBytes + pg * p.page * 128, &tmK, 0, r0, &k_full[s]);
          tma_load_2d(sK + s * kTileBytes + kA2Half + pg * p.page * 128, &tmK, 128, r0, &k_full[s]);
          bulk_load_1d(sKs + slot * kA2Tile + pg * p.page, p.k_scale + r0, p.page * sizeof(float), &k_full[s]);
          bulk_load_1d(sVs + slot * kA2Tile + pg * p.page, p.v_scale + r0, p.page * sizeof(float), &k_full[s]);
        }
        return true;
      };
      auto load_v = [&](int i) -> bool {
        if (!wait_bar(v_empty, (i & 1) ^ 1)) { report(p.status, kTimeoutStageEmpty, 42); *abort_flag = 1; return false; }
        mbar_expect_tx(v_full, kTileBytes);
        const int page0 = (base + i * kA2Tile) / p.page;
        for (int pg = 0; pg < ppt; ++pg) {
          const int pi = min(page0 + pg, p.max_blocks - 1);
          const int r0 = (p.block_table[pi] * p.hkv + kvh) * p.page;
          tma_load_2d(sV + pg * p.page * 128, &tmV, 0, r0, v_full);
          tma_load_2d(sV + kA2Half + pg * p.page * 128, &tmV, 128, r0, v_full);
        }
        return true;
      };
      bool ok = ntiles > 0 && load_k(0);
      for (int i = 0; i < ntiles && ok; ++i) {
        if (i + 1 < ntiles) ok = load_k(i + 1);
        if (ok) ok = load_v(i);
        if (*abort_flag) ok = false;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc1 = umma_idesc_f8(128, 128, 0u, 0u);                 // Q (K-major) x K (K-major)
      constexpr uint32_t idesc2 = umma_idesc_f8(128, 128, 0u, 0u) | (1u << 16);    // P (K-major) x V (MN-major B)
      const uint32_t q_addr = smem_u32(sQ), p_addr = smem_u32(sP), v_addr = smem_u32(sV);
      auto mma2 = [&](int j) -> bool {
        if (!wait_bar(v_full, j & 1)) { report(p.status, kTimeoutTmaFull, 43); *abort_flag = 1; return false; }
        tc_fence_after();
#pragma unroll
        for (int hf = 0; hf < 2; ++hf)
#pragma unroll
          for (int term = 0; term < 2; ++term)
#pragma unroll
            for (int k = 0; k < 4; ++k)  // 32 tokens per step: P advances 32 bytes, V advances 32 token rows
              umma_f8f6f4(tmem_o + hf * 128, umma_desc_sw128(p_addr + term * kA2Half + k * 32),
                          umma_desc_sw128(v_addr + hf * kA2Half + k * 4096), idesc2, (term > 0 || k > 0) ? 1u : 0u);
        umma_commit(o_full);
        umma_commit(v_empty);
        return true;
      };
      bool ok = true;
      for (int i = 0; i < ntiles && ok; ++i) {
        const int s = i % kA2KStages, b = i & 1;
        if (!wait_bar(&k_full[s], (i / kA2KStages) & 1)) { report(p.status, kTimeoutTmaFull, 44); *abort_flag = 1; ok = false; break; }
        tc_fence_after();
        const uint32_t k_addr = smem_u32(sK + s * kTileBytes);
#pragma unroll
        for (int term = 0; term < 2; ++term)
#pragma unroll
          for (int k = 0; k < 8; ++k)   // 32 bytes of the head per step, half k / 4
            umma_f8f6f4(tmem_s + b * 128, umma_desc_sw128(q_addr + term * kTileBytes + (k >> 2) * kA2Half + (k & 3) * 32),
                        umma_desc_sw128(k_addr + (k >> 2) * kA2Half + (k & 3) * 32), idesc1, (term > 0 || k > 0) ? 1u : 0u);
        umma_commit(&s_full[b]);
        umma_commit(&k_empty[s]);
        if (i > 0) {
          if (!wait_bar(p_full, (i - 1) & 1)) { report(p.status, kTimeoutConvert, 45); *abort_flag = 1; ok = false; break; }
          tc_fence_after();
          ok = mma2(i - 1);
        }
        if (*abort_flag) ok = false;
      }
      if (ok && ntiles > 0) {
        if (wait_bar(p_full, (ntiles - 1) & 1)) {
          tc_fence_after();
          mma2(ntiles - 1);
        } else {
          report(p.status, kTimeoutConvert, 46);
          *abort_flag = 1;
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + accumulation: thread = (set, query row)
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const int wslot = warp - 2;               // 0..7
    const int col0 = set * 64;                // this set's token columns of every tile
    const int my_pos = p.pos0 + row0 + r;
    const int my_first = (p.window > 0 && my_pos + 1 > p.window) ? my_pos + 1 - p.window : 0;
    const float sm = p.scale * 1.4426950408889634f * q_scale;
    float m_run = -INFINITY, l_run = 0.f, inv_c_prev = 0.f;
    float o[128];
#pragma unroll
    for (int j = 0; j < 128; ++j) o[j] = 0.f;
    bool ok = true;
    for (int i = 0; i < ntiles; ++i) {
      const int b = i & 1, slot = i % kA2ScaleSlots;
      bool okw = ok && wait_bar(&s_full[b], (i >> 1) & 1);
      if (!okw && ok) { report(p.status, kTimeoutAccum, 47); *abort_flag = 1; }
      tc_fence_after();
      const float* ks = sKs + slot * kA2Tile;
      const float* vs = sVs + slot * kA2Tile;
      const int t0 = base + i * kA2Tile;
      float* rr = red + b * 16;
      {
        // tile-wide max of the V scales (fixes the range of the e4m3 P operand); every warp covers 32 of the tokens twice over
        float vm = (t0 + r <= last_pos) ? vs[r] : 0.f;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) vm = fmaxf(vm, __shfl_xor_sync(0xffffffffu, vm, off));
        if (lane == 0) { rr[wslot] = vm; rr[8 + wslot] = (okw && !*abort_flag) ? 0.f : 1.f; }
      }
      // pass 1: maximum of the scaled, masked scores over this set's 64 columns; the other set's half comes through shared
      // memory.  Warp-uniform choice of the masked form: tcgen05.ld is .sync.aligned.
      const bool full = __all_sync(0xffffffffu, (t0 + col0 + 63 <= my_pos) && (t0 + col0 >= my_first)) != 0;
      const float mh = full ? half_row_max<false>(tmem_s + b * 128 + lane_addr, ks, col0, t0, my_pos, my_first)
                            : half_row_max<true>(tmem_s + b * 128 + lane_addr, ks, col0, t0, my_pos, my_first);
      rowmax[(b * 2 + set) * kA2Tile + r] = mh;
      asm volatile("bar.sync 3, 256;" ::: "memory");
      if (rr[8] + rr[9] + rr[10] + rr[11] + rr[12] + rr[13] + rr[14] + rr[15] != 0.f) { ok = false; break; }
      const float vmax = fmaxf(fmaxf(fmaxf(rr[0], rr[1]), fmaxf(rr[2], rr[3])), fmaxf(fmaxf(rr[4], rr[5]), fmaxf(rr[6], rr[7])));
      const float c_tile = vmax > 0.f ? 256.f / vmax : 0.f;
      const float mt = fmaxf(mh, rowmax[(b * 2 + (set ^ 1)) * kA2Tile + r]);
      const float mn = fmaxf(m_run, mt * sm);   // sm > 0: scaling commutes with the maximum
      const float corr = (m_run == -INFINITY) ? 0.f : fast_exp2(m_run - mn);
      m_run = mn;
      // the previous tile's PV product is folded in before P is overwritten: this set's output half
      if (i > 0) {
        if (__all_sync(0xffffffffu, wait_bar(o_full, (i - 1) & 1))) {
          tc_fence_after();
#pragma unroll
          for (int c0 = 0; c0 < 128; c0 += 16) {
            uint32_t raw[16];
            tmem_ld_x16(tmem_o + set * 128 + lane_addr + c0, raw);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j) o[c0 + j] += __uint_as_float(raw[j]) * inv_c_prev;
          }
        } else {
          report(p.status, kTimeoutAccum, 48);
          *abort_flag = 1;   // agreed on at the next tile's barrier
        }
      }
#pragma unroll
      for (int j = 0; j < 128; ++j) o[j] *= corr;
      // pass 2: probabilities of this set's columns -> two e4m3 terms of P (row r of the A operand)
      const float neg_m = (mn == -INFINITY) ? 0.f : -mn;
      const float lsum = full ? half_probs<false>(tmem_s + b * 128 + lane_addr, ks, vs, sP, r, col0, sm, neg_m, c_tile, t0, my_pos, my_first)
                              : half_probs<true>(tmem_s + b * 128 + lane_addr, ks, vs, sP, r, col0, sm, neg_m, c_tile, t0, my_pos, my_first);
      l_run = l_run * corr + lsum;
      inv_c_prev = c_tile > 0.f ? 1.f / c_tile : 0.f;
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    bool done = ok && !*abort_flag && ntiles > 0;
    if (done) {
      if (__all_sync(0xffffffffu, wait_bar(o_full, (ntiles - 1) & 1))) {
        tc_fence_after();
#pragma unroll
        for (int c0 = 0; c0 < 128; c0 += 16) {
          uint32_t raw[16];
          tmem_ld_x16(tmem_o + set * 128 + lane_addr + c0, raw);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) o[c0 + j] += __uint_as_float(raw[j]) * inv_c_prev;
        }
      } else {
        report(p.status, kTimeoutAccum, 49);
        *abort_flag = 1;
        done = false;
      }
    }
    // total probability mass of a row = the two sets' sums (both carry the same running maximum)
    rowmax[set * kA2Tile + r] = l_run;
    asm volatile("bar.sync 3, 256;" ::: "memory");
    const float l_all = l_run + rowmax[(set ^ 1) * kA2Tile + r];
    if (done && r < rows) {
      const float inv_l = l_all > 0.f ? 1.f / l_all : 0.f;
      uint4* dst = reinterpret_cast<uint4*>(p.out + (static_cast<size_t>(row0 + r) * p.hq + head) * D + set * 128);
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        Pack16 x;
#pragma unroll
        for (int j = 0; j < 8; ++j) x.h[j] = f32_to_bf16(o[c * 8 + j] * inv_l);
        dst[c] = x.u;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, 512);
}

}  // namespace dgpp

using namespace dgpp;

// Causal attention of T chunk rows (positions pos0 .. pos0 + T - 1 of the request whose block-table row is
// `block_table_row`) against the FP8 paged cache, which must already hold those positions.  head_dim 256.
DGPP_API int dgpp_attn_prefill_tc256(const void* q, int64_t q_stride, const void* k_cache, const void* v_cache,
                                     const void* k_scale, const void* v_scale, const void* block_table_row, void* out,
                                     int T, int pos0, int hq, int hkv, int d, int page, int max_blocks, int num_blocks,
                                     float scale, int window, cudaStream_t st) {
  DGPP_REQUIRE(d == 256, "attn_prefill_tc256: head_dim %d != 256", d);
  DGPP_REQUIRE(hkv > 0 && hq % hkv == 0, "attn_prefill_tc256: bad head grouping %d/%d", hq, hkv);
  DGPP_REQUIRE(page == 16 || page == 32 || page == 64 || page == 128, "attn_prefill_tc256: page %d unsupported", page);
  DGPP_REQUIRE(q_stride % 8 == 0, "attn_prefill_tc256: q row stride %lld must be a multiple of 8", (long long)q_stride);
  if (T == 0) return 0;
  AttnPrefill256Params p;
  p.q = static_cast<const bf16*>(q);
  p.q_stride = q_stride;
  p.k_scale = static_cast<const float*>(k_scale);
  p.v_scale = static_cast<const float*>(v_scale);
  p.block_table = static_cast<const int32_t*>(block_table_row);
  p.out = static_cast<bf16*>(out);
  p.status = device_status_ptr();
  p.T = T; p.pos0 = pos0; p.hq = hq; p.hkv = hkv; p.page = page; p.max_blocks = max_blocks; p.window = window;
  p.scale = scale;
  const uint64_t total_rows = static_cast<uint64_t>(num_blocks) * hkv * page;
  CUtensorMap tK, tV;
  if (make_tmap_2d(&tK, k_cache, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, 256, total_rows, 256, 128, page, CU_TENSOR_MAP_SWIZZLE_128B))
    return -1;
  if (make_tmap_2d(&tV, v_cache, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, 256, total_rows, 256, 128, page, CU_TENSOR_MAP_SWIZZLE_128B))
    return -1;
  constexpr size_t smem = 1024 + 2 * kA2Tile * 256 + 2 * kA2Half + (kA2KStages + 1) * kA2Tile * 256 +
                          2 * kA2ScaleSlots * kA2Tile * 4 + 2 * 2 * kA2Tile * 4 + 2 * 16 * 4 + (2 * kA2KStages + 6) * 8 + 64;
  static_assert(smem <= 227 * 1024, "attn_prefill_tc256: shared memory over the per-CTA limit");
  static bool attr = false;
  if (!attr) {
    DGPP_CUDA_OK(cudaFuncSetAttribute(attn_prefill_tc256_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      static_cast<int>(smem)));
    attr = true;
  }
  dim3 grid(dgpp_ceil_div(T, kA2Tile), hq);
  attn_prefill_tc256_kernel<<<grid, kA2Threads, smem, st>>>(tK, tV, p);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}
