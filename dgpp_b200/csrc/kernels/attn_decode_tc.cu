// Flash-decoding over the paged FP8 KV cache on the tensor cores (tcgen05 kind::f8f6f4): the e4m3
// cache bytes go HBM -> TMA -> shared memory -> tensor core untouched; no thread converts K or V.
//
// One CTA serves one (batch row, kv head, KV split) and walks its KV range in tiles of 128 tokens:
//
//   MMA1   S^T[token, col]   = K_tile[128 tokens, d] . Qq[col, d]^T         (tokens are the TMEM lanes)
//   softmax (thread = token): s = S^T * q_scale[h] * k_scale[token] * sm_scale, running max per head,
//           p = exp(s - m), per-thread partial sums of p, P = p * v_scale[token] * c_tile
//   MMA2   O^T[d, col]       = V_tile^T[d, 128 tokens] . Pq[col, tokens]^T  (V read as an MN-major operand)
//   accumulate (thread = d): o[h] = (o[h] + O^T / c_tile) * exp(m_old - m_new)
//
// bf16-grade operands from 8-bit tensor-core inputs: q and P are split into two e4m3 terms
// (x ~= x1 + x2 / 16, x2 = e4m3(16 * (x - x1))), which occupy columns h and 8 + h of the N = 16 wide
// B operand; their products are summed in fp32 after the MMA, so the 3-bit e4m3 mantissa of q / P
// costs ~2^-8 relative error instead of 2^-4.  K and V are exact (they are stored as e4m3).
//
// Warps: 0 = TMA producer (walks the block table), 1 = MMA issuer / TMEM owner, 2..5 = softmax and
// accumulation (128 threads).  S^T, O^T and the P operand are double buffered so MMA1 of tile i + 1
// overlaps the softmax of tile i.  Every wait is bounded (status code + clean exit).
// Partials (m, l, acc) use the layout of attn_decode.cu and are merged by the same combine kernel.
// Block-selection form (sel [rows, hkv, sel_k], see attn_decode.cu): the CTA walks the concatenation of the listed
// blocks as one virtual sequence; the producer and the scale loads translate virtual positions to cache positions
// (sel_block is a multiple of the page, so a page never straddles two listed blocks).
// (reference counterparts: src/kernels/full_attn.cu:163,1234 decode row / block-decode kernels, mma.sync m16n8k32.)
#include <cuda.h>
#include <math.h>
#include <string.h>

#include "common/common.h"
#include "common/dtypes.cuh"
#include "common/ptx.cuh"
#include "kernels/gemm_common.cuh"

namespace dgpp {

constexpr int kAdThreads = 192;
constexpr int kAdTile = 128;      // tokens per tile
constexpr int kAdStages = 3;
constexpr int kAdCols = 16;       // 2 terms x 8 head slots

struct AttnTcParams {
  const bf16* q;
  int64_t q_stride;
  const float* k_scale;
  const float* v_scale;
  const int32_t* block_table;
  const int32_t* row_req;
  const int32_t* positions;
  float* part_ml;
  float* part_acc;
  bf16* out;
  DeviceStatus* status;
  int rows, hq, hkv, page, max_blocks, splits, window;
  float scale;
  const int32_t* sel;     // optional block selection, null = dense
  int sel_k, sel_block;
};

__device__ __forceinline__ uint32_t sw128_byte(uint32_t row, uint32_t byte_in_row) {
  return row * 128u + ((((byte_in_row >> 4) ^ (row & 7u)) << 4) | (byte_in_row & 15u));
}

// G = query heads per kv head (<= 8); D = head_dim, 128 or 256.  A 256-wide head is handled as two 128-byte halves:
// K / V / q tiles hold half 0 then half 1 (each [rows, 128 B], 128-byte swizzle), MMA1 runs 8 k-steps over both
// halves, MMA2 writes one 16-column accumulator per half and thread `idx` owns output dims idx and 128 + idx.
template <int G, int D>
__global__ void __launch_bounds__(kAdThreads, 1)
attn_decode_tc_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                      AttnTcParams p) {
  constexpr int NH = D / 128;          // 128-byte halves of a head
  constexpr int kHalf = kAdTile * 128;  // 16 KB: one half of a K or V tile
  constexpr int kStage = kAdTile * D;
  constexpr int kTmemCols = NH == 1 ? 64 : 128;
  extern __shared__ __align__(1024) unsigned char smem_dyn[];
  unsigned char* sp = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  unsigned char* sK = sp;  sp += kAdStages * kStage;
  unsigned char* sV = sp;  sp += kAdStages * kStage;
  unsigned char* sQ = sp;  sp += NH * kAdCols * 128;   // 2 KB per half
  unsigned char* sP = sp;  sp += 2 * kAdCols * 128;    // 2 x 2 KB
  float* red = reinterpret_cast<float*>(sp);  sp += 2 * 4 * 12 * sizeof(float);   // [parity][warp][G + 1 (+pad)]
  float* redl = reinterpret_cast<float*>(sp); sp += 4 * 8 * sizeof(float);
  uint64_t* kv_full = reinterpret_cast<uint64_t*>(sp);
  uint64_t* kv_empty = kv_full + kAdStages;
  uint64_t* s_full = kv_empty + kAdStages;   // [2]
  uint64_t* p_full = s_full + 2;             // [2]
  uint64_t* o_full = p_full + 2;             // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_full + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kvh = blockIdx.x, split = blockIdx.y, row = blockIdx.z;
  const int req = p.row_req[row];
  const int pos_row = p.positions[row];
  int len = pos_row + 1;
  const int32_t* sl = nullptr;
  int sel_n = 0;
  if (p.sel != nullptr) {
    // the list is the previous kernel's output: nothing of it may be read before that kernel has finished
    pdl_wait();
    sl = p.sel + (static_cast<size_t>(row) * p.hkv + kvh) * p.sel_k;
    for (int j = 0; j < p.sel_k; ++j) sel_n += sl[j] >= 0 ? 1 : 0;
    len = sel_n > 0 ? (sel_n - 1) * p.sel_block + pos_row % p.sel_block + 1 : 0;   // every listed block is full but the last
  }
  // virtual position -> cache position (identity without a selection; clamped into the listed blocks and to the row's
  // own position, so that padding tokens of the last tile still address pages the request owns)
  auto cache_pos = [&](int v) {
    if (sl == nullptr) return v;
    const int vb = max(0, min(v / p.sel_block, sel_n - 1));
    return min(sl[vb] * p.sel_block + v % p.sel_block, pos_row);
  };
  const int first = (p.window > 0 && len > p.window) ? len - p.window : 0;
  const int base = first & ~(kAdTile - 1);
  const int total_tiles = (len - base + kAdTile - 1) / kAdTile;
  const int per = (total_tiles + p.splits - 1) / p.splits;
  const int tile_begin = split * per;
  const int ntiles = max(0, min(total_tiles, tile_begin + per) - tile_begin);
  const int32_t* bt = p.block_table + static_cast<size_t>(req) * p.max_blocks;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kAdStages; ++i) { mbar_init(&kv_full[i], 1); mbar_init(&kv_empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&s_full[i], 1); mbar_init(&p_full[i], 4); mbar_init(&o_full[i], 1); }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  pdl_wait();
  // ---- quantise q of this kv head's G query heads into two e4m3 terms (B operand of MMA1)
  float q_scale[G];
  if (warp >= 2) {
    const int d = threadIdx.x - 64;  // 0..127
#pragma unroll
    for (int h = 0; h < G; ++h) {
      float a = 0.f;
#pragma unroll
      for (int hf = 0; hf < NH; ++hf)
        a = fmaxf(a, fabsf(bf16_to_f32(p.q[static_cast<size_t>(row) * p.q_stride + (kvh * G + h) * D + hf * 128 + d])));
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
      if (lane == 0) redl[(warp - 2) * 8 + h] = a;
    }
  }
  __syncthreads();
  if (warp >= 2) {
    const int d = threadIdx.x - 64;
#pragma unroll
    for (int h = 0; h < 8; ++h) {
      float sc = 1.f;
      if (h < G) {
        const float am = fmaxf(fmaxf(redl[h], redl[8 + h]), fmaxf(redl[16 + h], redl[24 + h]));
        sc = am > 0.f ? am / 448.f : 1.f;
        q_scale[h < G ? h : 0] = sc;
      }
#pragma unroll
      for (int hf = 0; hf < NH; ++hf) {
        uint8_t b1 = 0, b2 = 0;
        if (h < G) {
          const float v = bf16_to_f32(p.q[static_cast<size_t>(row) * p.q_stride + (kvh * G + h) * D + hf * 128 + d]) / sc;
          b1 = f32_to_e4m3(v);
          b2 = f32_to_e4m3((v - e4m3_value_f32(v)) * 16.f);   // residual against the VALUE of b1 (no fp8 decode of b1)
        }
        sQ[hf * kAdCols * 128 + sw128_byte(h, d)] = b1;
        sQ[hf * kAdCols * 128 + sw128_byte(8 + h, d)] = b2;
      }
    }
    fence_proxy_async_smem();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s = tmem_base;        // 2 x 16 columns
  const uint32_t tmem_o = tmem_base + 32;   // 2 x NH x 16 columns

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      const int ppt = kAdTile / p.page;  // pages per tile
      for (int i = 0; i < ntiles; ++i) {
        const int s = i % kAdStages;
        if (!wait_bar(&kv_empty[s], ((i / kAdStages) & 1) ^ 1)) { report(p.status, kTimeoutStageEmpty, 21); *abort_flag = 1; break; }
        mbar_expect_tx(&kv_full[s], 2 * kStage);
        const int page0 = (base + (tile_begin + i) * kAdTile) / p.page;
        for (int pg = 0; pg < ppt; ++pg) {
          const int pi = min(sl == nullptr ? page0 + pg : cache_pos((page0 + pg) * p.page) / p.page, p.max_blocks - 1);
          const int blk = bt[pi];
          const int r0 = (blk * p.hkv + kvh) * p.page;
#pragma unroll
          for (int hf = 0; hf < NH; ++hf) {
            tma_load_2d(sK + s * kStage + hf * kHalf + pg * p.page * 128, &tmK, hf * 128, r0, &kv_full[s]);
            tma_load_2d(sV + s * kStage + hf * kHalf + pg * p.page * 128, &tmV, hf * 128, r0, &kv_full[s]);
          }
        }
        if (*abort_flag) break;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      // kind::f8f6f4, e4m3 x e4m3 -> fp32.  MMA1: A = K (K-major).  MMA2: A = V (MN-major, bit 15).
      constexpr uint32_t idesc1 = umma_idesc_f8(128, kAdCols, 0u, 0u);
      constexpr uint32_t idesc2 = umma_idesc_f8(128, kAdCols, 0u, 0u) | (1u << 15);
      const uint32_t q_addr = smem_u32(sQ);
      auto mma2 = [&](int j) {
        const int s = j % kAdStages, b = j & 1;
        const uint32_t v_addr = smem_u32(sV + s * kStage);
        const uint32_t p_addr = smem_u32(sP + b * kAdCols * 128);
#pragma unroll
        for (int hf = 0; hf < NH; ++hf)
#pragma unroll
          for (int k = 0; k < 4; ++k)  // 32 tokens per step: 4 groups of 8 token rows (1024 bytes each)
            umma_f8f6f4(tmem_o + (b * NH + hf) * 16, umma_desc_sw128(v_addr + hf * kHalf + k * 4096),
                        umma_desc_sw128(p_addr + k * 32), idesc2, k > 0 ? 1u : 0u);
        umma_commit(&o_full[b]);
        umma_commit(&kv_empty[s]);
      };
      bool ok = true;
      for (int i = 0; i < ntiles && ok; ++i) {
        const int s = i % kAdStages, b = i & 1;
        if (!wait_bar(&kv_full[s], (i / kAdStages) & 1)) { report(p.status, kTimeoutTmaFull, 22); *abort_flag = 1; ok = false; break; }
        tc_fence_after();
        const uint32_t k_addr = smem_u32(sK + s * kStage);
#pragma unroll
        for (int k = 0; k < 4 * NH; ++k)  // 32 bytes of d per step, half k / 4
          umma_f8f6f4(tmem_s + b * 16, umma_desc_sw128(k_addr + (k >> 2) * kHalf + (k & 3) * 32),
                      umma_desc_sw128(q_addr + (k >> 2) * kAdCols * 128 + (k & 3) * 32), idesc1, k > 0 ? 1u : 0u);
        umma_commit(&s_full[b]);
        if (i > 0) {
          if (!wait_bar(&p_full[(i - 1) & 1], ((i - 1) >> 1) & 1)) { report(p.status, kTimeoutConvert, 23); *abort_flag = 1; ok = false; break; }
          tc_fence_after();
          mma2(i - 1);
        }
        if (*abort_flag) ok = false;
      }
      if (ok && ntiles > 0) {
        const int j = ntiles - 1;
        if (wait_bar(&p_full[j & 1], (j >> 1) & 1)) {
          tc_fence_after();
          mma2(j);
        } else {
          report(p.status, kTimeoutConvert, 24);
          *abort_flag = 1;
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + accumulation (warps 2..5)
    const int quad = warp & 3;
    const int idx = quad * 32 + lane;        // token lane for S^T, head-dim lane for O^T
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const int wslot = warp - 2;
    const float sm = p.scale * 1.4426950408889634f;  // scores in log2 units
    float m_run[G], l_thr[G], o_acc[NH][G];
#pragma unroll
    for (int h = 0; h < G; ++h) {
      m_run[h] = -INFINITY; l_thr[h] = 0.f;
#pragma unroll
      for (int hf = 0; hf < NH; ++hf) o_acc[hf][h] = 0.f;
    }
    float inv_c_prev = 0.f;
    bool ok = true;
    // token scales of the first tile
    auto load_scales = [&](int i, float& ks, float& vs, bool& valid) {
      const int t = base + (tile_begin + i) * kAdTile + idx;
      valid = t >= first && t < len;
      const int tc = cache_pos(max(0, min(t, len - 1)));
      const int pi = min(tc / p.page, p.max_blocks - 1);
      const size_t tok = (static_cast<size_t>(bt[pi]) * p.hkv + kvh) * p.page + tc % p.page;
      ks = p.k_scale[tok];
      vs = valid ? p.v_scale[tok] : 0.f;
    };
    float ks_n = 0.f, vs_n = 0.f;
    bool valid_n = false;
    if (ntiles > 0) load_scales(0, ks_n, vs_n, valid_n);
    for (int i = 0; i < ntiles; ++i) {
      const int b = i & 1;
      const float ks = ks_n, vs = vs_n;
      const bool valid = valid_n;
      if (i + 1 < ntiles) load_scales(i + 1, ks_n, vs_n, valid_n);
      // a failed wait must not leave the other softmax warps alone at the named barrier below: every warp
      // publishes its verdict next to the tile maxima and all four leave the loop together
      bool okw = ok && wait_bar(&s_full[b], (i >> 1) & 1);
      if (!okw && ok) { report(p.status, kTimeoutAccum, 25); *abort_flag = 1; }
      tc_fence_after();
      uint32_t c[16];
      if (okw) {
        tmem_ld_x16(tmem_s + b * 16 + lane_addr, c);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) c[j] = 0;
      }
      float s[G];
      float* rp = red + (b * 4 + wslot) * 12;
#pragma unroll
      for (int h = 0; h < G; ++h) {
        const float raw = (__uint_as_float(c[h]) + __uint_as_float(c[8 + h]) * 0.0625f) * q_scale[h] * ks * sm;
        s[h] = valid ? raw : -INFINITY;
        float mx = s[h];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        if (lane == 0) rp[h] = mx;
      }
      {
        float vm = vs;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) vm = fmaxf(vm, __shfl_xor_sync(0xffffffffu, vm, o));
        if (lane == 0) {
          rp[G] = vm;
          rp[11] = (okw && !*abort_flag) ? 0.f : 1.f;
        }
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      const float* r0 = red + (b * 4) * 12;
      if (r0[11] + r0[12 + 11] + r0[24 + 11] + r0[36 + 11] != 0.f) { ok = false; break; }
      const float vmax = fmaxf(fmaxf(r0[G], r0[12 + G]), fmaxf(r0[24 + G], r0[36 + G]));
      const float c_tile = vmax > 0.f ? 256.f / vmax : 0.f;
      float corr[G];
      uint8_t pb1[8], pb2[8];
#pragma unroll
      for (int h = 0; h < 8; ++h) { pb1[h] = 0; pb2[h] = 0; }
#pragma unroll
      for (int h = 0; h < G; ++h) {
        const float mt = fmaxf(fmaxf(r0[h], r0[12 + h]), fmaxf(r0[24 + h], r0[36 + h]));
        const float mn = fmaxf(m_run[h], mt);
        corr[h] = (m_run[h] == -INFINITY) ? 0.f : exp2f(m_run[h] - mn);
        const float pv = (valid && mn > -INFINITY) ? exp2f(s[h] - mn) : 0.f;
        l_thr[h] = l_thr[h] * corr[h] + pv;
        m_run[h] = mn;
        const float pw = pv * vs * c_tile;
        pb1[h] = f32_to_e4m3(pw);
        pb2[h] = f32_to_e4m3((pw - e4m3_value_f32(pw)) * 16.f);
      }
      unsigned char* pbuf = sP + b * kAdCols * 128;
#pragma unroll
      for (int h = 0; h < 8; ++h) {
        pbuf[sw128_byte(h, idx)] = pb1[h];
        pbuf[sw128_byte(8 + h, idx)] = pb2[h];
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[b]);
      // fold the previous tile's O^T into the running output, then apply this tile's correction
      if (i > 0) {
        const int bp = (i - 1) & 1;
        if (wait_bar(&o_full[bp], ((i - 1) >> 1) & 1)) {
          tc_fence_after();
#pragma unroll
          for (int hf = 0; hf < NH; ++hf) {
            uint32_t oc[16];
            tmem_ld_x16(tmem_o + (bp * NH + hf) * 16 + lane_addr, oc);
            tmem_ld_wait();
#pragma unroll
            for (int h = 0; h < G; ++h)
              o_acc[hf][h] += (__uint_as_float(oc[h]) + __uint_as_float(oc[8 + h]) * 0.0625f) * inv_c_prev;
          }
        } else {
          report(p.status, kTimeoutAccum, 26);
          *abort_flag = 1;  // agreed on at the next tile's barrier
        }
      }
#pragma unroll
      for (int h = 0; h < G; ++h)
#pragma unroll
        for (int hf = 0; hf < NH; ++hf) o_acc[hf][h] *= corr[h];
      inv_c_prev = c_tile > 0.f ? 1.f / c_tile : 0.f;
      tc_fence_before();
    }
    if (ok && !*abort_flag && ntiles > 0) {
      const int j = ntiles - 1, bp = j & 1;
      if (wait_bar(&o_full[bp], (j >> 1) & 1)) {
        tc_fence_after();
#pragma unroll
        for (int hf = 0; hf < NH; ++hf) {
          uint32_t oc[16];
          tmem_ld_x16(tmem_o + (bp * NH + hf) * 16 + lane_addr, oc);
          tmem_ld_wait();
#pragma unroll
          for (int h = 0; h < G; ++h)
            o_acc[hf][h] += (__uint_as_float(oc[h]) + __uint_as_float(oc[8 + h]) * 0.0625f) * inv_c_prev;
        }
      } else {
        report(p.status, kTimeoutAccum, 27);
        *abort_flag = 1;
      }
    }
    // total probability mass per head: sum the per-thread partials
    asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll
    for (int h = 0; h < G; ++h) {
      float l = l_thr[h];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
      if (lane == 0) redl[wslot * 8 + h] = l;
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll
    for (int h = 0; h < G; ++h) {
      const float l = redl[h] + redl[8 + h] + redl[16 + h] + redl[24 + h];
      const int hh = kvh * G + h;
      if (p.splits == 1) {
#pragma unroll
        for (int hf = 0; hf < NH; ++hf)
          p.out[(static_cast<size_t>(row) * p.hq + hh) * D + hf * 128 + idx] = f32_to_bf16(l > 0.f ? o_acc[hf][h] / l : 0.f);
      } else {
        const size_t pi = (static_cast<size_t>(row) * p.hq + hh) * p.splits + split;
#pragma unroll
        for (int hf = 0; hf < NH; ++hf) p.part_acc[pi * D + hf * 128 + idx] = o_acc[hf][h];
        if (idx == 0) {
          // running max is kept in log2 units; the combine kernel works in natural-log units
          p.part_ml[pi * 2] = m_run[h] * 0.6931471805599453f;
          p.part_ml[pi * 2 + 1] = l;
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
}

__global__ void attn_tc_combine_kernel(const float* __restrict__ part_ml, const float* __restrict__ part_acc,
                                       bf16* __restrict__ out, int splits) {
  pdl_wait();
  const size_t rh = blockIdx.x;
  const int d = threadIdx.x;
  const int D = blockDim.x;
  float mm = -INFINITY;
  for (int s = 0; s < splits; ++s) mm = fmaxf(mm, part_ml[(rh * splits + s) * 2]);
  float ll = 0.f, a = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float ms = part_ml[(rh * splits + s) * 2];
    const float c = ms == -INFINITY ? 0.f : __expf(ms - mm);
    ll += part_ml[(rh * splits + s) * 2 + 1] * c;
    a += part_acc[(rh * splits + s) * D + d] * c;
  }
  out[rh * D + d] = f32_to_bf16(ll > 0.f ? a / ll : 0.f);
}

template <int G, int D>
static int launch_attn_tc(const CUtensorMap& tK, const CUtensorMap& tV, const AttnTcParams& p, cudaStream_t st) {
  constexpr size_t smem = 1024 + 2 * kAdStages * kAdTile * D + kAdCols * 128 * (2 + D / 128) + 2 * 4 * 12 * 4 + 4 * 8 * 4 +
                          (2 * kAdStages + 6) * 8 + 64;
  static_assert(smem <= 227 * 1024, "attn_decode_tc: shared memory over the per-CTA limit");
  static bool attr = false;
  if (!attr) {
    DGPP_CUDA_OK(cudaFuncSetAttribute(attn_decode_tc_kernel<G, D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      static_cast<int>(smem)));
    attr = true;
  }
  dim3 grid(p.hkv, p.splits, p.rows);
  attn_decode_tc_kernel<G, D><<<grid, kAdThreads, smem, st>>>(tK, tV, p);
  DGPP_CUDA_OK(cudaGetLastError());
  if (p.splits > 1 && p.out != nullptr) {   // out == nullptr: the caller folds the partials itself (dgpp_attn_combine_quant)
    attn_tc_combine_kernel<<<p.rows * p.hq, D, 0, st>>>(p.part_ml, p.part_acc, p.out, p.splits);
    DGPP_CUDA_OK(cudaGetLastError());
  }
  return 0;
}

}  // namespace dgpp

using namespace dgpp;

// Tensor-core decode attention over an FP8 paged cache; head_dim 128 or 256, hq / hkv <= 8, page in {16, 32, 64, 128}.
// num_blocks = blocks in the pool (extent of the TMA descriptors).
DGPP_API int dgpp_attn_decode_tc(const void* q, int64_t q_stride, const void* k_cache, const void* v_cache,
                                 const void* k_scale, const void* v_scale, const void* block_table,
                                 const void* row_req, const void* positions, void* part_ml, void* part_acc,
                                 void* out, int rows, int hq, int hkv, int d, int page, int max_blocks,
                                 int num_blocks, int splits, float scale, int window, const void* sel, int sel_k,
                                 int sel_block, cudaStream_t st) {
  DGPP_REQUIRE(d == 128 || d == 256, "attn_decode_tc: head_dim %d (128 or 256)", d);
  DGPP_REQUIRE(sel == nullptr || (sel_k >= 1 && sel_block >= page && sel_block % page == 0 && window == 0),
               "attn_decode_tc: a block selection needs sel_k >= 1, blocks of whole pages (%d / %d) and no window", sel_block,
               page);
  DGPP_REQUIRE(hkv > 0 && hq % hkv == 0 && hq / hkv <= 8, "attn_decode_tc: unsupported head grouping %d/%d", hq, hkv);
  DGPP_REQUIRE(page == 16 || page == 32 || page == 64 || page == 128, "attn_decode_tc: page %d unsupported", page);
  DGPP_REQUIRE(splits >= 1 && (splits == 1 || (part_ml && part_acc)), "attn_decode_tc: scratch required for splits");
  DGPP_REQUIRE(out != nullptr || splits > 1, "attn_decode_tc: an output buffer is required without splits");
  if (rows == 0) return 0;
  AttnTcParams p;
  p.q = static_cast<const bf16*>(q);
  p.q_stride = q_stride;
  p.k_scale = static_cast<const float*>(k_scale);
  p.v_scale = static_cast<const float*>(v_scale);
  p.block_table = static_cast<const int32_t*>(block_table);
  p.row_req = static_cast<const int32_t*>(row_req);
  p.positions = static_cast<const int32_t*>(positions);
  p.part_ml = static_cast<float*>(part_ml);
  p.part_acc = static_cast<float*>(part_acc);
  p.out = static_cast<bf16*>(out);
  p.status = device_status_ptr();
  p.rows = rows; p.hq = hq; p.hkv = hkv; p.page = page; p.max_blocks = max_blocks; p.splits = splits;
  p.window = window; p.scale = scale;
  p.sel = static_cast<const int32_t*>(sel);
  p.sel_k = sel_k; p.sel_block = sel_block;
  const uint64_t total_rows = static_cast<uint64_t>(num_blocks) * hkv * page;
  CUtensorMap tK, tV;
  if (make_tmap_2d(&tK, k_cache, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, d, total_rows, d, 128, page,
                   CU_TENSOR_MAP_SWIZZLE_128B))
    return -1;
  if (make_tmap_2d(&tV, v_cache, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, d, total_rows, d, 128, page,
                   CU_TENSOR_MAP_SWIZZLE_128B))
    return -1;
  if (d == 256) {
    switch (hq / hkv) {
      case 1: return launch_attn_tc<1, 256>(tK, tV, p, st);
      case 2: return launch_attn_tc<2, 256>(tK, tV, p, st);
      case 4: return launch_attn_tc<4, 256>(tK, tV, p, st);
      case 8: return launch_attn_tc<8, 256>(tK, tV, p, st);
    }
  } else {
    switch (hq / hkv) {
      case 1: return launch_attn_tc<1, 128>(tK, tV, p, st);
      case 2: return launch_attn_tc<2, 128>(tK, tV, p, st);
      case 4: return launch_attn_tc<4, 128>(tK, tV, p, st);
      case 5: return launch_attn_tc<5, 128>(tK, tV, p, st);
      case 8: return launch_attn_tc<8, 128>(tK, tV, p, st);
    }
  }
  dgpp_set_error("attn_decode_tc: group size %d at head_dim %d not instantiated", hq / hkv, d);
  return -1;
}
