// Causal flash attention for prefill over the paged FP8 KV cache, on tcgen05 (kind::f8f6f4).
//
// One CTA = one query head x 128 consecutive query positions of one request.  K / V tiles of 128 tokens come
// from the cache pages by TMA exactly as stored (e4m3 bytes); nothing converts them:
//
//   MMA1   S[q, t]  = (Q1 + Q2)[q, d] . K[t, d]^T          Q split into two e4m3 terms (A operand, K-major)
//   softmax (thread = query row): s = S * q_scale[q] * k_scale[t] * sm_scale, causal mask, running max / sum,
//           P[q, t] = p * v_scale[t] * c_tile split into two e4m3 terms, written as the next A operand
//   MMA2   O_tile[q, d] = (P1 + P2)[q, t] . V[t, d]        V is the B operand read MN-major (d contiguous)
//   accumulate (thread = query row, 128 fp32 registers): o = o * corr + O_tile / c_tile
//
// S is double buffered in TMEM so MMA1 of tile i + 1 overlaps the softmax of tile i; the PV product of tile i
// runs while the softmax threads exponentiate tile i + 1.  Both splits keep ~2^-8 relative operand error
// (e4m3 value + e4m3 residual), K and V are exact.
// Warps: 0 = TMA producer (pages + their scales), 1 = MMA issuer / TMEM owner, 2..5 = softmax (one row each).
// (reference counterparts: src/kernels/full_attn.cu:442,679,983 tile / TMA / fp8-compute prefill kernels.)
#include <cuda.h>
#include <math.h>
#include <string.h>

#include "common/common.h"
#include "common/dtypes.cuh"
#include "common/ptx.cuh"
#include "kernels/gemm_common.cuh"

namespace dgpp {

constexpr int kApThreads = 192;
constexpr int kApTile = 128;
constexpr int kApStages = 3;

struct AttnPrefillParams {
  const bf16* q;            // [T, q_stride]: head h at column h * 128 (already rotated)
  int64_t q_stride;
  const float* k_scale;     // [blocks, hkv, page]
  const float* v_scale;
  const int32_t* block_table;  // row of this request
  bf16* out;                // [T, hq * 128]
  DeviceStatus* status;
  int T, pos0, hq, hkv, page, max_blocks, window;
  float scale;
};

__device__ __forceinline__ uint32_t sw128_off(uint32_t row, uint32_t byte_in_row) {
  return row * 128u + ((((byte_in_row >> 4) ^ (row & 7u)) << 4) | (byte_in_row & 15u));
}

// Row maximum of raw score * k_scale over one 128-token tile (thread = query row, scores read from TMEM).
template <bool kMask>
__device__ __forceinline__ float tile_row_max(uint32_t taddr, const float* ks, int t0, int my_pos, int my_first) {
  float mt = -INFINITY;
#pragma unroll 2
  for (int c0 = 0; c0 < kApTile; c0 += 16) {
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

// Probabilities of one tile: p = 2^(raw * k_scale * sm - m); P = p * v_scale * c_tile as two e4m3 terms written
// to row r of the swizzled A operand (term 2 one tile further).  Returns the row sum of p.
template <bool kMask>
__device__ __forceinline__ float tile_probs(uint32_t taddr, const float* ks, const float* vs, unsigned char* sP, int r,
                                            float sm, float neg_m, float c_tile, int t0, int my_pos, int my_first) {
  float lsum = 0.f;
#pragma unroll 2
  for (int c0 = 0; c0 < kApTile; c0 += 16) {
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
    *reinterpret_cast<uint4*>(sP + sw128_off(r, c0)) = a.u;
    *reinterpret_cast<uint4*>(sP + kApTile * 128 + sw128_off(r, c0)) = bq.u;
  }
  return lsum;
}

__global__ void __launch_bounds__(kApThreads, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                       AttnPrefillParams p) {
  constexpr int D = 128;
  constexpr int kTileBytes = kApTile * D;  // 16 KB
  extern __shared__ __align__(1024) unsigned char smem_dyn[];
  unsigned char* sp = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  unsigned char* sQ = sp;  sp += 2 * kTileBytes;             // Q1, Q2
  unsigned char* sP = sp;  sp += 2 * kTileBytes;             // P1, P2
  unsigned char* sK = sp;  sp += kApStages * kTileBytes;
  unsigned char* sV = sp;  sp += kApStages * kTileBytes;
  float* sKs = reinterpret_cast<float*>(sp);  sp += kApStages * kApTile * sizeof(float);
  float* sVs = reinterpret_cast<float*>(sp);  sp += kApStages * kApTile * sizeof(float);
  float* red = reinterpret_cast<float*>(sp);  sp += 2 * 8 * sizeof(float);
  uint64_t* kv_full = reinterpret_cast<uint64_t*>(sp);
  uint64_t* kv_empty = kv_full + kApStages;
  uint64_t* s_full = kv_empty + kApStages;   // [2]
  uint64_t* p_full = s_full + 2;             // [1]
  uint64_t* o_full = p_full + 1;             // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.y, kvh = head / (p.hq / p.hkv);
  const int row0 = blockIdx.x * kApTile;                      // first chunk row of this CTA
  const int rows = min(kApTile, p.T - row0);
  const int last_pos = p.pos0 + row0 + rows - 1;
  const int first_pos = p.pos0 + row0;
  const int first_tok = (p.window > 0 && first_pos + 1 > p.window) ? first_pos + 1 - p.window : 0;
  const int base = first_tok & ~(kApTile - 1);
  const int ntiles = (last_pos + 1 - base + kApTile - 1) / kApTile;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kApStages; ++i) { mbar_init(&kv_full[i], 1); mbar_init(&kv_empty[i], 1); }
    mbar_init(&s_full[0], 1); mbar_init(&s_full[1], 1);
    mbar_init(p_full, 4);
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
  // ---- quantise this CTA's query rows into two e4m3 terms (thread = row)
  float q_scale = 1.f;
  if (warp >= 2) {
    const int r = (warp & 3) * 32 + lane;   // the TMEM lane quadrant this warp may read: warp % 4
    float v[D];
    float amax = 0.f;
    if (r < rows) {
      const uint4* src = reinterpret_cast<const uint4*>(p.q + static_cast<size_t>(row0 + r) * p.q_stride + head * D);
#pragma unroll
      for (int c = 0; c < D / 8; ++c) {
        Pack16 x;
        x.u = src[c];
#pragma unroll
        for (int j = 0; j < 8; ++j) { v[c * 8 + j] = bf16_to_f32(x.h[j]); amax = fmaxf(amax, fabsf(v[c * 8 + j])); }
      }
    } else {
#pragma unroll
      for (int j = 0; j < D; ++j) v[j] = 0.f;
    }
    q_scale = amax > 0.f ? amax / 448.f : 1.f;
    const float inv = 1.f / q_scale;
#pragma unroll
    for (int c = 0; c < D / 16; ++c) {
      Pack16 a, b;
#pragma unroll
      for (int j = 0; j < 8; ++j)
        f32x2_to_e4m3x2_two_term(v[c * 16 + 2 * j] * inv, v[c * 16 + 2 * j + 1] * inv, a.s[j], b.s[j]);
      *reinterpret_cast<uint4*>(sQ + sw128_off(r, c * 16)) = a.u;
      *reinterpret_cast<uint4*>(sQ + kTileBytes + sw128_off(r, c * 16)) = b.u;
    }
    fence_proxy_async_smem();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s = tmem_base;          // 2 x 128 columns
  const uint32_t tmem_o = tmem_base + 256;    // 128 columns

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      const int ppt = kApTile / p.page;
      for (int i = 0; i < ntiles; ++i) {
        const int s = i % kApStages;
        if (!wait_bar(&kv_empty[s], ((i / kApStages) & 1) ^ 1)) { report(p.status, kTimeoutStageEmpty, 31); *abort_flag = 1; break; }
        mbar_expect_tx(&kv_full[s], 2 * kTileBytes + 2 * kApTile * sizeof(float));
        const int page0 = (base + i * kApTile) / p.page;
        for (int pg = 0; pg < ppt; ++pg) {
          const int pi = min(page0 + pg, p.max_blocks - 1);
          const int blk = p.block_table[pi];
          const int r0 = (blk * p.hkv + kvh) * p.page;
          tma_load_2d(sK + s * kTileBytes + pg * p.page * D, &tmK, 0, r0, &kv_full[s]);
          tma_load_2d(sV + s * kTileBytes + pg * p.page * D, &tmV, 0, r0, &kv_full[s]);
          bulk_load_1d(sKs + s * kApTile + pg * p.page, p.k_scale + r0, p.page * sizeof(float), &kv_full[s]);
          bulk_load_1d(sVs + s * kApTile + pg * p.page, p.v_scale + r0, p.page * sizeof(float), &kv_full[s]);
        }
        if (*abort_flag) break;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc1 = umma_idesc_f8(128, 128, 0u, 0u);                 // Q (K-major) x K (K-major)
      constexpr uint32_t idesc2 = umma_idesc_f8(128, 128, 0u, 0u) | (1u << 16);    // P (K-major) x V (MN-major B)
      const uint32_t q_addr = smem_u32(sQ), p_addr = smem_u32(sP);
      auto mma2 = [&](int j) {
        const int s = j % kApStages;
        const uint32_t v_addr = smem_u32(sV + s * kTileBytes);
#pragma unroll
        for (int term = 0; term < 2; ++term)
#pragma unroll
          for (int k = 0; k < 4; ++k)  // 32 tokens per step: P advances 32 bytes, V advances 32 token rows
            umma_f8f6f4(tmem_o, umma_desc_sw128(p_addr + term * kTileBytes + k * 32), umma_desc_sw128(v_addr + k * 4096),
                        idesc2, (term > 0 || k > 0) ? 1u : 0u);
        umma_commit(o_full);
        umma_commit(&kv_empty[s]);
      };
      bool ok = true;
      for (int i = 0; i < ntiles && ok; ++i) {
        const int s = i % kApStages, b = i & 1;
        if (!wait_bar(&kv_full[s], (i / kApStages) & 1)) { report(p.status, kTimeoutTmaFull, 32); *abort_flag = 1; ok = false; break; }
        tc_fence_after();
        const uint32_t k_addr = smem_u32(sK + s * kTileBytes);
#pragma unroll
        for (int term = 0; term < 2; ++term)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_f8f6f4(tmem_s + b * 128, umma_desc_sw128(q_addr + term * kTileBytes + k * 32), umma_desc_sw128(k_addr + k * 32),
                        idesc1, (term > 0 || k > 0) ? 1u : 0u);
        umma_commit(&s_full[b]);
        if (i > 0) {
          if (!wait_bar(p_full, (i - 1) & 1)) { report(p.status, kTimeoutConvert, 33); *abort_flag = 1; ok = false; break; }
          tc_fence_after();
          mma2(i - 1);
        }
        if (*abort_flag) ok = false;
      }
      if (ok && ntiles > 0) {
        if (wait_bar(p_full, (ntiles - 1) & 1)) {
          tc_fence_after();
          mma2(ntiles - 1);
        } else {
          report(p.status, kTimeoutConvert, 34);
          *abort_flag = 1;
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + accumulation (thread = query row)
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const int my_pos = p.pos0 + row0 + r;
    const int my_first = (p.window > 0 && my_pos + 1 > p.window) ? my_pos + 1 - p.window : 0;
    const float sm = p.scale * 1.4426950408889634f * q_scale;
    float m_run = -INFINITY, l_run = 0.f, inv_c_prev = 0.f;
    float o[D];
#pragma unroll
    for (int j = 0; j < D; ++j) o[j] = 0.f;
    bool ok = true;
    for (int i = 0; i < ntiles; ++i) {
      const int s = i % kApStages, b = i & 1;
      bool okw = ok && wait_bar(&s_full[b], (i >> 1) & 1);
      if (!okw && ok) { report(p.status, kTimeoutAccum, 35); *abort_flag = 1; }
      tc_fence_after();
      const float* ks = sKs + s * kApTile;
      const float* vs = sVs + s * kApTile;
      const int t0 = base + i * kApTile;
      // tile-wide max of the V scales (fixes the range of the e4m3 P operand)
      {
        float vm = (t0 + r <= last_pos) ? vs[r] : 0.f;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) vm = fmaxf(vm, __shfl_xor_sync(0xffffffffu, vm, off));
        if (lane == 0) { red[(i & 1) * 8 + quad] = vm; red[(i & 1) * 8 + 4 + quad] = (okw && !*abort_flag) ? 0.f : 1.f; }
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      const float* rr = red + (i & 1) * 8;
      if (rr[4] + rr[5] + rr[6] + rr[7] != 0.f) { ok = false; break; }
      const float vmax = fmaxf(fmaxf(rr[0], rr[1]), fmaxf(rr[2], rr[3]));
      const float c_tile = vmax > 0.f ? 256.f / vmax : 0.f;
      // pass 1: row maximum of the scaled, masked scores (the scores are re-read from TMEM in pass 2 instead of
      // being kept in 128 registers next to the 128 output accumulators)
      // warp-uniform choice: tcgen05.ld is .sync.aligned, every lane of the warp must take the same path
      const bool full = __all_sync(0xffffffffu, (t0 + kApTile - 1 <= my_pos) && (t0 >= my_first)) != 0;
      const float mt = full ? tile_row_max<false>(tmem_s + b * 128 + lane_addr, ks, t0, my_pos, my_first)
                            : tile_row_max<true>(tmem_s + b * 128 + lane_addr, ks, t0, my_pos, my_first);
      const float mn = fmaxf(m_run, mt * sm);   // sm > 0: scaling commutes with the maximum
      const float corr = (m_run == -INFINITY) ? 0.f : fast_exp2(m_run - mn);
      m_run = mn;
      float lsum = 0.f;
      // the previous tile's PV product must be folded in before P is overwritten
      if (i > 0) {
        if (__all_sync(0xffffffffu, wait_bar(o_full, (i - 1) & 1))) {
          tc_fence_after();
#pragma unroll
          for (int c0 = 0; c0 < D; c0 += 16) {
            uint32_t raw[16];
            tmem_ld_x16(tmem_o + lane_addr + c0, raw);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j) o[c0 + j] += __uint_as_float(raw[j]) * inv_c_prev;
          }
        } else {
          report(p.status, kTimeoutAccum, 36);
          *abort_flag = 1;
        }
      }
#pragma unroll
      for (int j = 0; j < D; ++j) o[j] *= corr;
      // pass 2: probabilities -> two e4m3 terms of P (row r of the A operand)
      const float neg_m = (mn == -INFINITY) ? 0.f : -mn;
      lsum = full ? tile_probs<false>(tmem_s + b * 128 + lane_addr, ks, vs, sP, r, sm, neg_m, c_tile, t0, my_pos, my_first)
                  : tile_probs<true>(tmem_s + b * 128 + lane_addr, ks, vs, sP, r, sm, neg_m, c_tile, t0, my_pos, my_first);
      l_run = l_run * corr + lsum;
      inv_c_prev = c_tile > 0.f ? 1.f / c_tile : 0.f;
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    if (ok && !*abort_flag && ntiles > 0) {
      if (__all_sync(0xffffffffu, wait_bar(o_full, (ntiles - 1) & 1))) {
        tc_fence_after();
#pragma unroll
        for (int c0 = 0; c0 < D; c0 += 16) {
          uint32_t raw[16];
          tmem_ld_x16(tmem_o + lane_addr + c0, raw);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) o[c0 + j] += __uint_as_float(raw[j]) * inv_c_prev;
        }
      } else {
        report(p.status, kTimeoutAccum, 37);
        *abort_flag = 1;
      }
    }
    if (r < rows) {
      const float inv_l = l_run > 0.f ? 1.f / l_run : 0.f;
      uint4* dst = reinterpret_cast<uint4*>(p.out + (static_cast<size_t>(row0 + r) * p.hq + head) * D);
#pragma unroll
      for (int c = 0; c < D / 8; ++c) {
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
// `block_table_row`) against the FP8 paged cache, which must already hold those positions.  head_dim 128.
DGPP_API int dgpp_attn_prefill_tc(const void* q, int64_t q_stride, const void* k_cache, const void* v_cache,
                                  const void* k_scale, const void* v_scale, const void* block_table_row, void* out,
                                  int T, int pos0, int hq, int hkv, int d, int page, int max_blocks, int num_blocks,
                                  float scale, int window, cudaStream_t st) {
  DGPP_REQUIRE(d == 128, "attn_prefill_tc: head_dim %d != 128", d);
  DGPP_REQUIRE(hkv > 0 && hq % hkv == 0, "attn_prefill_tc: bad head grouping %d/%d", hq, hkv);
  DGPP_REQUIRE(page == 16 || page == 32 || page == 64 || page == 128, "attn_prefill_tc: page %d unsupported", page);
  if (T == 0) return 0;
  AttnPrefillParams p;
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
  if (make_tmap_2d(&tK, k_cache, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, 128, total_rows, 128, 128, page, CU_TENSOR_MAP_SWIZZLE_128B))
    return -1;
  if (make_tmap_2d(&tV, v_cache, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, 128, total_rows, 128, 128, page, CU_TENSOR_MAP_SWIZZLE_128B))
    return -1;
  constexpr size_t smem = 1024 + (4 + 2 * kApStages) * kApTile * 128 + 2 * kApStages * kApTile * 4 + 64 +
                          (2 * kApStages + 4) * 8 + 64;
  static bool attr = false;
  if (!attr) {
    DGPP_CUDA_OK(cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      static_cast<int>(smem)));
    attr = true;
  }
  dim3 grid(dgpp_ceil_div(T, kApTile), hq);
  attn_prefill_tc_kernel<<<grid, kApThreads, smem, st>>>(tK, tV, p);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}
