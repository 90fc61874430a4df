// Linear layer on the 5th-generation tensor cores:   C[T, N] = alpha * X[T, K] . W[N, K]^T
//
// The weight tile is always the UMMA "A" operand (128 weight rows = 128 TMEM lanes) and the
// activation rows are the "B" operand (BN = 16..256 tokens = TMEM columns), so the same kernel
// serves decode (a handful of rows, pure weight streaming) and prefill (thousands of rows).
// Accumulators are fp32 in TMEM; inputs to tcgen05.mma are 16-bit floats.
//
// Weight sources (WMODE):
//   0  bf16 [N, K]                      TMA (128B swizzle) straight into the MMA stage
//   1  NVFP4: e2m1 pairs [N, K/2] + e4m3 scale per 16 [N, K/16]
//        TMA brings the packed bytes and their scales as stored; eight converter warps expand
//        them into a 16-bit K-major swizzled stage (exact: e2m1 * e4m3 fits 16-bit floats), the
//        fp32 tensor scale is `alpha` in the epilogue.  No dequantised copy ever reaches HBM.
//   2  FP8 e4m3 [N, K] with one fp32 scale per 128x128 block [N/128, K/128]
//        converter warps write bf16(e4m3 * scale).
//   3  MXFP4: e2m1 pairs + e8m0 scale per 32 [N, K/32]   (scales read with plain loads)
//   4  MXFP8: e4m3 [N, K] + e8m0 scale per 32 [N, K/32]   bf16(e4m3 * 2^e) is exact
//   5  int8 and 6 int4 (two per byte, low nibble first): offset-binary codes (code - 128 / code - 8) with one bf16
//        scale per 64 [N, K/64]; converter warps write bf16(int * scale)
//   7  BF12: a lossless 12-bit resident form of a bf16 matrix.  A weight's sign + mantissa byte is stored as is
//        ([N, K] bytes); its exponent becomes a 4-bit code against a per-row base ([N, K/2] nibbles, low nibble =
//        even column).  Code 15 escapes to a per-row, column-sorted side table holding the true bf16 bits (a few
//        weights in ten thousand fall outside a window of 15 exponents).  TMA streams both planes as stored (0.75
//        of the bf16 bytes), converter warps rebuild the exact bf16 bits in the MMA stage, so the result is bitwise
//        the bf16 kernel's.
//
// Warp roles (320 threads): warp 0 = TMA producer, warp 1 = MMA issuer + TMEM owner,
// warps 2..9 = converters (quantised modes), warps 2..5 = epilogue (TMEM -> registers -> global).
// Split-K: grid.z CTAs write fp32 partials to a workspace; the last CTA to arrive on a tile's
// counter folds them in ascending split order (deterministic) and resets the counter.
//
// Every wait is bounded; on expiry the kernel records a status code, unwinds and frees TMEM.
// (reference counterparts: src/kernels/moe_w4a4.cu:476 dense_w4a4_tma_kernel, src/kernels/fp4w_gemm.cu:71,
//  src/kernels/fp8w_gemm.cu:84, src/kernels/gemm_cublaslt.cpp -- all mma.sync / library there.)
#include <cuda.h>
#include <dlfcn.h>
#include <string.h>

#include "common/common.h"
#include "common/dtypes.cuh"
#include "common/ptx.cuh"
#include "kernels/gemm_common.cuh"
#include "kernels/comm.cuh"

namespace dgpp {

constexpr int kBM = 128;          // weight rows per CTA (UMMA M)
constexpr int kBK = 64;           // K elements per MMA stage (one 128-byte swizzle row of 16-bit values)
constexpr int kGemmThreads = 320;
constexpr int kConvWarps = 8;

struct GemmParams {
  float alpha;
  bf16* out;               // [T, ldc] bf16 (may be null when out32 is set)
  float* out32;            // [T, ldc] fp32 (optional)
  const bf16* resid;       // optional residual added in the epilogue: out = bf16(resid + bf16(alpha*acc))
  float* ws;               // split-K partials [splits, T, N] fp32
  uint32_t* counters;      // split-K tile counters [n_tiles * m_tiles], zero at rest
  const float* blk_scale;  // WMODE 2: [ceil(N/128), K/128] fp32
  const uint8_t* sf_plain; // WMODE 3 / 4: e8m0 scales [N, K/32]
  const bf16* sf_bf16;     // WMODE 5 / 6: bf16 scales [N, K/64]
  const uint8_t* bf12_base;   // WMODE 7: exponent window base per row [N]
  const uint32_t* bf12_rows;  // WMODE 7: [N + 1] first escape of each row
  const uint32_t* bf12_esc;   // WMODE 7: (column << 16) | bf16 bits, column-sorted within a row
  DeviceStatus* status;
  int T, N, K, ldc;
  int kb_per_split;        // k64 blocks per split
  // Reduce-scatter push (tensor-parallel o_proj / down_proj at prefill sizes): the finished bf16 tile goes into slot
  // `rank` of the rank that owns the tile's tokens (token tiles are dealt in runs of tiles_per_rank) and that
  // owner's arrival counter of (this rank, token tile) is bumped; dgpp_comm_rs_ag folds and redistributes.
  int push, tiles_per_rank;
  // All-gather mode (the consumer side of the sequence-parallel boundary): the activations are the normed rows that
  // rs_norm_push_kernel of every rank stored into this rank's region, token tile t in slot owner(t) of the current
  // parity.  tmB is then a 3-D map [K, T, 2 * world slots]; a CTA takes its token tile in an order that starts with
  // this rank's own tiles, and its producer warp waits (bounded) for the owner's flag before the first load.
  int ag;
  CommState comm;
};

template <int BN>
struct GemmSmem {
  static constexpr int kStageB = BN * 128;                 // bytes
  static constexpr int kStageA = kBM * 128;                // 16 KB
  static constexpr int kStageRaw = kBM * 128;              // 16 KB packed fp4 (256 K per row) / fp8 (128 K per row)
  static constexpr int kStageSf = kBM * 16;                // 2 KB
  static constexpr int kStageEx = kBM * 64;                // 8 KB exponent nibbles of 128 K per row (BF12)
};

// True bf16 bits of an escaped BF12 weight: binary search of the row's column-sorted side table.
__device__ __forceinline__ uint32_t bf12_escape(const uint32_t* __restrict__ esc, uint32_t lo, uint32_t hi, uint32_t col) {
  while (lo < hi) {
    const uint32_t mid = (lo + hi) >> 1, v = __ldg(esc + mid), c = v >> 16;
    if (c == col) return v & 0xFFFFu;
    if (c < col) lo = mid + 1; else hi = mid;
  }
  return 0u;   // not listed (cannot happen for an encoder-produced matrix): a zero weight
}

// WMODE: 0 bf16, 1 nvfp4, 2 fp8 block, 3 mxfp4, 4 mxfp8 (e4m3 + e8m0 per 32), 5 int8 and 6 int4 (offset-binary codes,
// bf16 scale per 64).  Byte-per-element sources (2, 4, 5) stage 128 K per raw row, nibble sources (1, 3, 6) 256 K.
// Converted operands are bf16 (kind::f16 requires A and B
// to have the same 16-bit type; mixing an f16 A with a bf16 B is an illegal instruction on sm_100a).
template <int BN, int WMODE, int SB, int SA, int SR>
__global__ void __launch_bounds__(kGemmThreads, (WMODE != 0 && BN <= 32) ? 2 : 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA,   // bf16 weights, or packed raw weights (uint8)
               const __grid_constant__ CUtensorMap tmB,   // activations bf16 [T, K]
               const __grid_constant__ CUtensorMap tmSf,  // NVFP4 scales (uint8) [N, K/16]
               GemmParams p) {
  using L = GemmSmem<BN>;
  constexpr bool kQuant = WMODE != 0;
  extern __shared__ __align__(1024) unsigned char smem_dyn[];
  // carve shared memory (all tile bases 1024-byte aligned)
  unsigned char* sp = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  unsigned char* sB = sp;                   sp += SB * L::kStageB;
  unsigned char* sA = sp;                   sp += (kQuant ? SA : SB) * L::kStageA;
  unsigned char* sRaw = sp;                 sp += kQuant ? SR * L::kStageRaw : 0;
  unsigned char* sSf = sp;                  sp += (WMODE == 1) ? SR * L::kStageSf : (WMODE == 7 ? SR * L::kStageEx : 0);
  uint64_t* bars = reinterpret_cast<uint64_t*>(sp);
  uint64_t* b_full = bars;                  // [SB]
  uint64_t* b_empty = b_full + SB;          // [SB]
  uint64_t* a_full = b_empty + SB;          // [SA]
  uint64_t* a_empty = a_full + SA;          // [SA]
  uint64_t* raw_full = a_empty + SA;        // [SR]
  uint64_t* raw_empty = raw_full + SR;      // [SR]
  uint64_t* acc_full = raw_empty + SR;      // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* last_flag = const_cast<int*>(abort_flag) + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * kBM;
  int my = blockIdx.y;
  if (p.ag) my = (min(p.comm.rank * p.tiles_per_rank, static_cast<int>(gridDim.y)) + static_cast<int>(blockIdx.y)) % static_cast<int>(gridDim.y);
  const int m0 = my * BN;
  const int split = blockIdx.z, splits = gridDim.z;
  const int num_kb_total = p.K / kBK;
  const int kb_begin = split * p.kb_per_split;
  const int kb_end = min(num_kb_total, kb_begin + p.kb_per_split);
  const int nkb = max(0, kb_end - kb_begin);
  constexpr uint32_t kTmemCols = BN < 32 ? 32 : BN;

  if (threadIdx.x == 0) {
    for (int i = 0; i < SB; ++i) { mbar_init(&b_full[i], 1); mbar_init(&b_empty[i], 1); }
    for (int i = 0; i < SA; ++i) { mbar_init(&a_full[i], kConvWarps); mbar_init(&a_empty[i], 1); }
    for (int i = 0; i < SR; ++i) { mbar_init(&raw_full[i], 1); mbar_init(&raw_empty[i], kConvWarps); }
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    *last_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    if (WMODE == 1 || WMODE == 7) tma_prefetch_desc(&tmSf);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      int ag_z = 0;
      bool ag_waited = !p.ag;
      for (int i = 0; i < nkb; ++i) {
        const int kb = kb_begin + i;
        if (kQuant) {
          // raw weight stage: WMODE 1/3 cover 256 K (4 k64 blocks), WMODE 2 covers 128 K (2 k64 blocks)
          constexpr bool kByteSrc = WMODE == 2 || WMODE == 4 || WMODE == 5 || WMODE == 7;
          constexpr int kSubs = kByteSrc ? 2 : 4;
          if (i % kSubs == 0) {
            const int r = i / kSubs, sr = r % SR;
            if (!wait_bar(&raw_empty[sr], ((r / SR) & 1) ^ 1)) { report(p.status, kTimeoutStageEmpty, 1); *abort_flag = 1; break; }
            const uint32_t bytes = L::kStageRaw + (WMODE == 1 ? L::kStageSf : (WMODE == 7 ? L::kStageEx : 0));
            mbar_expect_tx(&raw_full[sr], bytes);
            // packed bytes: x in bytes. fp4: kb*32 bytes; fp8: kb*64 bytes
            const int xb = kByteSrc ? kb * 64 : kb * 32;
            tma_load_2d(sRaw + sr * L::kStageRaw, &tmA, xb, n0, &raw_full[sr]);
            if (WMODE == 1) tma_load_2d(sSf + sr * L::kStageSf, &tmSf, kb * 4, n0, &raw_full[sr]);
            if (WMODE == 7) tma_load_2d(sSf + sr * L::kStageEx, &tmSf, kb * 32, n0, &raw_full[sr]);
          }
        }
        const int sb = i % SB;
        if (!wait_bar(&b_empty[sb], ((i / SB) & 1) ^ 1)) { report(p.status, kTimeoutStageEmpty, 2); *abort_flag = 1; break; }
        mbar_expect_tx(&b_full[sb], L::kStageB + (kQuant ? 0 : L::kStageA));
        if (!ag_waited) {
          // the weight stages above are already in flight; only the activation tile waits for its owner
          const uint32_t epoch = *p.comm.epoch;
          const int parity = epoch & 1;
          const int owner = min(my / p.tiles_per_rank, p.comm.world - 1);
          ag_z = parity * p.comm.world + owner;
          if (owner != p.comm.rank && !wait_flag(ag_flag(p.comm, p.comm.rank, parity, my, 0), epoch)) {
            report(p.status, kTimeoutPeerFlag, 500 + owner);
            *abort_flag = 1;
            break;
          }
          asm volatile("fence.proxy.async;" ::: "memory");     // the peer's stores, acquired above, before the bulk reads
          ag_waited = true;
        }
        if (p.ag) tma_load_3d(sB + sb * L::kStageB, &tmB, kb * kBK, m0, ag_z, &b_full[sb]);
        else tma_load_2d(sB + sb * L::kStageB, &tmB, kb * kBK, m0, &b_full[sb]);
        if (!kQuant) tma_load_2d(sA + sb * L::kStageA, &tmA, kb * kBK, n0, &b_full[sb]);
        if (*abort_flag) break;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc_f16(kBM, BN, 1u, 1u);
      for (int i = 0; i < nkb; ++i) {
        const int sb = i % SB;
        if (!wait_bar(&b_full[sb], (i / SB) & 1)) { report(p.status, kTimeoutTmaFull, 3); *abort_flag = 1; break; }
        uint32_t a_addr;
        if (kQuant) {
          const int sa = i % SA;
          if (!wait_bar(&a_full[sa], (i / SA) & 1)) { report(p.status, kTimeoutConvert, 4); *abort_flag = 1; break; }
          a_addr = smem_u32(sA + sa * L::kStageA);
        } else {
          a_addr = smem_u32(sA + sb * L::kStageA);
        }
        tc_fence_after();
        const uint32_t b_addr = smem_u32(sB + sb * L::kStageB);
#pragma unroll
        for (int kk = 0; kk < kBK / 16; ++kk) {
          umma_f16(tmem_base, umma_desc_sw128(a_addr + kk * 32), umma_desc_sw128(b_addr + kk * 32), idesc,
                   (i > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(&b_empty[sb]);
        if (kQuant) umma_commit(&a_empty[i % SA]);
        if (*abort_flag) break;
      }
      umma_commit(acc_full);
    }
  } else if (kQuant) {
    // ------------------------------------------------------------------ converters (warps 2..9)
    const int ct = threadIdx.x - 64;       // 0..255
    const int row = ct >> 1, half = ct & 1;
    constexpr bool kByteSrc = WMODE == 2 || WMODE == 4 || WMODE == 5 || WMODE == 7;
    constexpr int kSubs = kByteSrc ? 2 : 4;
    uint32_t bf12_b = 0, esc_lo = 0, esc_hi = 0;
    if (WMODE == 7) {
      const int nrow = min(n0 + row, p.N - 1);
      bf12_b = p.bf12_base[nrow];
      esc_lo = p.bf12_rows[nrow];
      esc_hi = p.bf12_rows[nrow + 1];
    }
    for (int i = 0; i < nkb; ++i) {
      const int r = i / kSubs, sub = i % kSubs, sr = r % SR, sa = i % SA;
      bool ok = true;
      if (sub == 0) ok = wait_bar(&raw_full[sr], (r / SR) & 1);
      if (ok) ok = wait_bar(&a_empty[sa], ((i / SA) & 1) ^ 1);
      if (!ok) { report(p.status, kTimeoutTmaFull, 5); *abort_flag = 1; break; }
      const unsigned char* raw = sRaw + sr * L::kStageRaw + row * 128;
      unsigned char* dst = sA + sa * L::kStageA + row * 128;
      const int kb = kb_begin + i;
      if (WMODE == 6) {
        // packed int4, offset binary: 32 weights = 16 bytes at logical chunk (sub*2 + half); one bf16 scale per 64
        const int cl = sub * 2 + half;
        Pack16 w;
        w.u = *reinterpret_cast<const uint4*>(raw + ((cl ^ (row & 7)) << 4));
        const int nrow = min(n0 + row, p.N - 1);
        const float sc = bf16_to_f32(p.sf_bf16[static_cast<size_t>(nrow) * (p.K / 64) + kb]);
        Pack16 o[4];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int lo = static_cast<int>(w.b[j] & 15) - 8, hi = static_cast<int>(w.b[j] >> 4) - 8;
          bf162 v = __floats2bfloat162_rn(static_cast<float>(lo) * sc, static_cast<float>(hi) * sc);
          o[j >> 2].w[j & 3] = *reinterpret_cast<uint32_t*>(&v);
        }
#pragma unroll
        for (int c = 0; c < 4; ++c)
          *reinterpret_cast<uint4*>(dst + (((half * 4 + c) ^ (row & 7)) << 4)) = o[c].u;
      } else if (WMODE == 7) {
        // this k64 block: sign+mantissa bytes [sub*64, +64) of the raw row and nibble bytes [sub*32, +32) of the
        // exponent row; the thread rebuilds its 32 weights (bytes half*32.., nibble bytes half*16..)
        Pack16 e;
        e.u = *reinterpret_cast<const uint4*>(sSf + sr * L::kStageEx + row * 64 + sub * 32 + half * 16);
        Pack16 o[4];
#pragma unroll
        for (int c2 = 0; c2 < 2; ++c2) {
          const int cl = sub * 4 + half * 2 + c2;
          Pack16 w;
          w.u = *reinterpret_cast<const uint4*>(raw + ((cl ^ (row & 7)) << 4));
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const uint32_t s0 = w.b[2 * j], s1 = w.b[2 * j + 1], eb = e.b[c2 * 8 + j];
            const uint32_t e0 = eb & 15u, e1 = eb >> 4;
            uint32_t lo = ((s0 & 0x80u) << 8) | ((bf12_b + e0) << 7) | (s0 & 0x7Fu);
            uint32_t hi = ((s1 & 0x80u) << 8) | ((bf12_b + e1) << 7) | (s1 & 0x7Fu);
            if (e0 == 15u || e1 == 15u) {
              const uint32_t col = static_cast<uint32_t>(kb) * 64 + half * 32 + c2 * 16 + 2 * j;
              if (e0 == 15u) lo = bf12_escape(p.bf12_esc, esc_lo, esc_hi, col);
              if (e1 == 15u) hi = bf12_escape(p.bf12_esc, esc_lo, esc_hi, col + 1);
            }
            o[c2 * 2 + (j >> 2)].w[j & 3] = lo | (hi << 16);
          }
        }
#pragma unroll
        for (int c = 0; c < 4; ++c)
          *reinterpret_cast<uint4*>(dst + (((half * 4 + c) ^ (row & 7)) << 4)) = o[c].u;
      } else if (WMODE == 1 || WMODE == 3) {
        // 32 weights = 16 packed bytes at logical 16-byte chunk (sub*2 + half) of the swizzled 128-byte row
        const int cl = sub * 2 + half;
        Pack16 w;
        w.u = *reinterpret_cast<const uint4*>(raw + ((cl ^ (row & 7)) << 4));
        float s0f, s1f;
        if (WMODE == 1) {
          const unsigned char* sf = sSf + sr * L::kStageSf + row * 16 + sub * 4 + half * 2;
          s0f = e4m3_to_f32(sf[0]);
          s1f = e4m3_to_f32(sf[1]);
        } else {
          const int nrow = min(n0 + row, p.N - 1);
          const uint8_t e = p.sf_plain[static_cast<size_t>(nrow) * (p.K / 32) + kb * 2 + half];
          s0f = s1f = e8m0_to_f32(e);
        }
        Pack16 o[4];
        {
          // f16 bits >> 3 read as bf16 equal value * 2^-112; fold 2^112 into the (exact) bf16 scale
          const bf162 s0 = __float2bfloat162_rn(s0f * 5.192296858534828e33f);
          const bf162 s1 = __float2bfloat162_rn(s1f * 5.192296858534828e33f);
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            __half2 h = e2m1x2_to_h2(w.b[j]);
            const uint32_t hb = *reinterpret_cast<uint32_t*>(&h);
            uint32_t bb = ((hb & 0x7FFF7FFFu) >> 3) | (hb & 0x80008000u);
            bf162 v = __hmul2(*reinterpret_cast<bf162*>(&bb), j < 8 ? s0 : s1);
            o[j >> 2].w[j & 3] = *reinterpret_cast<uint32_t*>(&v);
          }
        }
#pragma unroll
        for (int c = 0; c < 4; ++c)
          *reinterpret_cast<uint4*>(dst + (((half * 4 + c) ^ (row & 7)) << 4)) = o[c].u;
      } else {
        // FP8: 128-byte raw row holds 128 K; this k64 block is bytes [sub*64, sub*64+64); thread takes 32 of them
        // (this thread's 32 elements are one e8m0 group of 32, half of a bf16-scale group of 64)
        float sc;
        if (WMODE == 2) {
          sc = p.blk_scale[static_cast<size_t>(blockIdx.x) * (p.K / 128) + (kb >> 1)];
        } else {
          const int nrow = min(n0 + row, p.N - 1);
          sc = WMODE == 4 ? e8m0_to_f32(p.sf_plain[static_cast<size_t>(nrow) * (p.K / 32) + kb * 2 + half])
                          : bf16_to_f32(p.sf_bf16[static_cast<size_t>(nrow) * (p.K / 64) + kb]);
        }
        Pack16 o[4];
#pragma unroll
        for (int c2 = 0; c2 < 2; ++c2) {
          const int cl = sub * 4 + half * 2 + c2;
          Pack16 w;
          w.u = *reinterpret_cast<const uint4*>(raw + ((cl ^ (row & 7)) << 4));
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            float2 f;
            if (WMODE == 5) {
              f.x = static_cast<float>(static_cast<int>(w.b[2 * j]) - 128);
              f.y = static_cast<float>(static_cast<int>(w.b[2 * j + 1]) - 128);
            } else {
              f = __half22float2(e4m3x2_to_h2(w.s[j]));
            }
            bf162 v = __floats2bfloat162_rn(f.x * sc, f.y * sc);
            o[c2 * 2 + (j >> 2)].w[j & 3] = *reinterpret_cast<uint32_t*>(&v);
          }
        }
#pragma unroll
        for (int c = 0; c < 4; ++c)
          *reinterpret_cast<uint4*>(dst + (((half * 4 + c) ^ (row & 7)) << 4)) = o[c].u;
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&a_full[sa]);
        if (sub == kSubs - 1 || i == nkb - 1) mbar_arrive(&raw_empty[sr]);
      }
      if (*abort_flag) break;
    }
  }

  // ------------------------------------------------------------------ epilogue (warps 2..5)
  if (warp >= 2 && warp < 6) {
    const int q = warp & 3;  // TMEM lane quadrant this warp may read
    const bool ok = nkb > 0 ? wait_bar(acc_full, 0) : true;
    if (!ok) { report(p.status, kTimeoutAccum, 6); *abort_flag = 1; }
    tc_fence_after();
    const int n = n0 + q * 32 + lane;
    const int cols = min(BN, p.T - m0);
    uint32_t push_epoch = 0;
    int push_owner = 0;
    bf16* push_dst = nullptr;
    if (p.push) {
      push_epoch = *p.comm.epoch + 1;
      push_owner = min(static_cast<int>(blockIdx.y) / p.tiles_per_rank, p.comm.world - 1);
      push_dst = reinterpret_cast<bf16*>(payload(p.comm, push_owner, push_epoch & 1, p.comm.rank));
    }
    if (ok && !*abort_flag) {
      float* wsp = splits > 1 ? p.ws + (static_cast<size_t>(split) * p.T + m0) * p.N : nullptr;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 16) {
        if (c0 >= cols) break;
        uint32_t r[16];
        if (nkb > 0) {
          tmem_ld_x16(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + c0, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) r[j] = 0;
        }
        if (n < p.N) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int m = c0 + j;
            if (m < cols) {
              const float v = __uint_as_float(r[j]);
              if (splits > 1) {
                wsp[static_cast<size_t>(m) * p.N + n] = v;
              } else if (p.push) {
                // stage the tile in shared memory (the operand rings are idle once the accumulator is complete) so
                // that the peer stores below are 16-byte vectors in 256-byte runs instead of 2-byte scalars
                reinterpret_cast<bf16*>(sB)[m * kBM + (q * 32 + lane)] = f32_to_bf16(v * p.alpha);
              } else {
                const size_t o = static_cast<size_t>(m0 + m) * p.ldc + n;
                float y = v * p.alpha;
                if (p.out32) p.out32[o] = y;
                if (p.out) {
                  if (p.resid) y = bf16_to_f32(p.resid[o]) + bf16_to_f32(f32_to_bf16(y));
                  p.out[o] = f32_to_bf16(y);
                }
              }
            }
          }
        }
      }
    }
    if (p.push) {
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (ok && !*abort_flag) {
        const int et = static_cast<int>(threadIdx.x) - 64;            // 0..127 over the four epilogue warps
        const uint4* tile = reinterpret_cast<const uint4*>(sB);
        for (int cidx = et; cidx < cols * (kBM / 8); cidx += 128) {
          const int m = cidx / (kBM / 8), seg = cidx % (kBM / 8);
          st_v4_global(push_dst + static_cast<size_t>(m0 + m) * p.N + n0 + seg * 8, tile[m * (kBM / 8) + seg]);
        }
      }
      // make the tile visible at system scope, then count it in at the owner (also after a failed wait: the owner's
      // bounded wait reports the missing data through the status block of THIS rank, not by stalling there)
      __threadfence_system();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (warp == 2 && lane == 0)
        red_release_sys_add(rs_counter(p.comm, push_owner, push_epoch & 1, p.comm.rank, blockIdx.y), 1u);
    }
    if (splits > 1) {
      // publish partials, elect the last CTA of this tile, fold in ascending split order
      __threadfence();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (warp == 2 && lane == 0) {
        const uint32_t prev = atomicAdd(&p.counters[blockIdx.y * gridDim.x + blockIdx.x], 1u);
        *last_flag = (prev == static_cast<uint32_t>(splits - 1)) ? 1 : 0;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (*last_flag) {
        __threadfence();
        if (n < p.N) {
          // 4 rows x 4 splits of partials are requested together and added in ascending split order (the sum of a
          // plain loop, without one L2 round trip per (row, split))
          for (int mb = 0; mb < cols; mb += 4) {
            float acc[4];
#pragma unroll
            for (int mm = 0; mm < 4; ++mm) acc[mm] = 0.f;
            for (int s0 = 0; s0 < splits; s0 += 4) {
              float t[4][4];
#pragma unroll
              for (int mm = 0; mm < 4; ++mm) {
#pragma unroll
                for (int ss = 0; ss < 4; ++ss) {
                  const bool live = mb + mm < cols && s0 + ss < splits;
                  t[mm][ss] = live ? __ldcg(p.ws + (static_cast<size_t>(s0 + ss) * p.T + m0 + mb + mm) * p.N + n) : 0.f;
                }
              }
#pragma unroll
              for (int mm = 0; mm < 4; ++mm) {
#pragma unroll
                for (int ss = 0; ss < 4; ++ss) acc[mm] += t[mm][ss];
              }
            }
#pragma unroll
            for (int mm = 0; mm < 4; ++mm) {
              const int m = mb + mm;
              if (m >= cols) break;
              const size_t o = static_cast<size_t>(m0 + m) * p.ldc + n;
              float y = acc[mm] * p.alpha;
              if (p.out32) p.out32[o] = y;
              if (p.out) {
                if (p.resid) y = bf16_to_f32(p.resid[o]) + bf16_to_f32(f32_to_bf16(y));
                p.out[o] = f32_to_bf16(y);
              }
            }
          }
        }
        if (warp == 2 && lane == 0) p.counters[blockIdx.y * gridDim.x + blockIdx.x] = 0;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
}

// ---------------------------------------------------------------------------------- host side
template <int BN, int WMODE>
struct GemmCfg {
  static constexpr bool kQuant = WMODE != 0;
  // ring depths: deep raw prefetch for small BN (weight streaming), wide B ring for large BN
  static constexpr int kBf16Depth = (200 * 1024) / (BN * 128 + kBM * 128);
  // Quantised weights with a small token tile run two CTAs per SM (<= 113 KB each): the second CTA hides
  // the converter <-> tensor-core handshakes of the first while both keep HBM requests in flight.
  // (BF12 carries an 8 KB exponent plane per raw stage; its B ring is shallower to stay under two CTAs per SM)
  static constexpr int SB = !kQuant ? (kBf16Depth > 8 ? 8 : kBf16Depth)
                            : WMODE == 7 && BN <= 32 ? (BN <= 16 ? 6 : 3)
                                    : (BN <= 16 ? 8 : (BN <= 32 ? 6 : (BN <= 64 ? 8 : (BN <= 128 ? 6 : 4))));
  static constexpr int SA = kQuant ? (BN <= 32 ? 3 : (BN <= 128 ? 4 : 3)) : 1;
  static constexpr int SR = kQuant ? (BN <= 32 ? 2 : (BN <= 64 ? 4 : 2)) : 1;
  static constexpr size_t smem() {
    size_t s = 1024;  // alignment slack
    s += static_cast<size_t>(SB) * BN * 128;
    s += static_cast<size_t>(kQuant ? SA : SB) * kBM * 128;
    if (kQuant) s += static_cast<size_t>(SR) * kBM * 128;
    if (WMODE == 1) s += static_cast<size_t>(SR) * kBM * 16;
    if (WMODE == 7) s += static_cast<size_t>(SR) * kBM * 64;
    s += (2 * SB + 2 * SA + 2 * SR + 1) * 8 + 64;
    return s;
  }
};

template <int BN, int WMODE>
static int launch_gemm(const CUtensorMap& tA, const CUtensorMap& tB, const CUtensorMap& tSf, const GemmParams& p,
                       int splits, cudaStream_t st) {
  using C = GemmCfg<BN, WMODE>;
  auto kern = gemm_tc_kernel<BN, WMODE, C::SB, C::SA, C::SR>;
  static bool attr = false;
  constexpr size_t smem = C::smem();
  static_assert(smem <= 227 * 1024, "shared memory budget exceeded");
  if (!attr) {
    DGPP_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    attr = true;
  }
  dim3 grid(dgpp_ceil_div(p.N, kBM), dgpp_ceil_div(p.T, BN), splits);
  kern<<<grid, kGemmThreads, smem, st>>>(tA, tB, tSf, p);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

}  // namespace dgpp

using namespace dgpp;

// Scratch sizes for split-K: ws = splits * T * N floats; counters = ceil(N/128) * ceil(T/BN) uint32 (zeroed once).
//
// wmode: 0 bf16, 1 nvfp4, 2 fp8-block, 3 mxfp4, 4 mxfp8, 5 int8 g64, 6 int4 g64, 7 bf12.   a_f16 is ignored (ABI
// stability).  bf12: w = sign+mantissa bytes [N, K]; w_scale = one buffer holding, each 16-byte aligned and in this
// order, the exponent nibbles [N, K/2], the row bases [N], the escape row starts [N + 1] uint32 and the escapes.
// bn: token tile (16, 32, 64, 128, 256).  splits >= 1; K/64 blocks are divided evenly (4-block aligned for fp4).
static int gemm_tc_impl(int wmode, int a_f16, int bn, const void* x, int64_t x_stride, const void* w,
                        const void* w_scale, float alpha, void* out, void* out32, const void* resid, int ldc,
                        int T, int N, int K, int splits, void* ws, void* counters, void* comm_push, cudaStream_t st,
                        void* comm_ag = nullptr) {
  DGPP_REQUIRE(T >= 1 && N >= 1, "gemm_tc: empty problem");
  DGPP_REQUIRE(K % 64 == 0, "gemm_tc: K %d must be a multiple of 64", K);
  const bool nibble_src = wmode == 1 || wmode == 3 || wmode == 6;
  const bool byte_src = wmode == 2 || wmode == 4 || wmode == 5 || wmode == 7;
  if (nibble_src) DGPP_REQUIRE(K % 256 == 0, "gemm_tc: 4-bit weights need K %% 256 == 0 (K=%d)", K);
  if (byte_src) DGPP_REQUIRE(K % 128 == 0, "gemm_tc: 8-bit weights need K %% 128 == 0 (K=%d)", K);
  DGPP_REQUIRE(splits >= 1, "gemm_tc: splits must be >= 1");
  DGPP_REQUIRE(splits == 1 || (ws && counters), "gemm_tc: split-K needs workspace and counters");
  DGPP_REQUIRE(out || out32 || comm_push, "gemm_tc: no output");
  GemmParams p;
  p.push = 0;
  p.ag = 0;
  p.tiles_per_rank = 1;
  if (comm_ag) {
    const DgppComm* c = static_cast<const DgppComm*>(comm_ag);
    DGPP_REQUIRE(!comm_push, "gemm_tc: all-gather input and reduce-scatter push are separate calls");
    DGPP_REQUIRE(dgpp_ceil_div(T, bn) <= kCommMaxCtas, "gemm_tc ag: %d rows in tiles of %d exceed %d token tiles", T, bn, kCommMaxCtas);
    DGPP_REQUIRE(static_cast<size_t>(T) * K * 2 <= c->st.slot_bytes, "gemm_tc ag: %d x %d exceeds the slot", T, K);
    p.ag = 1;
    p.comm = c->st;
    p.tiles_per_rank = dgpp_ceil_div(dgpp_ceil_div(T, bn), c->st.world);
  }
  if (comm_push) {
    const DgppComm* c = static_cast<const DgppComm*>(comm_push);
    DGPP_REQUIRE(splits == 1, "gemm_tc push: split-K is not combined with the reduce-scatter push");
    DGPP_REQUIRE(N % 128 == 0, "gemm_tc push: N %d must be a multiple of 128", N);
    DGPP_REQUIRE(dgpp_ceil_div(T, bn) <= kCommMaxCtas, "gemm_tc push: %d rows in tiles of %d exceed %d token tiles", T, bn, kCommMaxCtas);
    DGPP_REQUIRE(static_cast<size_t>(T) * N * 2 <= c->st.slot_bytes, "gemm_tc push: %d x %d exceeds the slot", T, N);
    p.push = 1;
    p.comm = c->st;
    p.tiles_per_rank = dgpp_ceil_div(dgpp_ceil_div(T, bn), c->st.world);
  }
  p.alpha = alpha;
  p.out = static_cast<bf16*>(out);
  p.out32 = static_cast<float*>(out32);
  p.resid = static_cast<const bf16*>(resid);
  p.ws = static_cast<float*>(ws);
  p.counters = static_cast<uint32_t*>(counters);
  p.blk_scale = wmode == 2 ? static_cast<const float*>(w_scale) : nullptr;
  p.sf_plain = (wmode == 3 || wmode == 4) ? static_cast<const uint8_t*>(w_scale) : nullptr;
  p.sf_bf16 = (wmode == 5 || wmode == 6) ? static_cast<const bf16*>(w_scale) : nullptr;
  p.bf12_base = nullptr; p.bf12_rows = nullptr; p.bf12_esc = nullptr;
  if (wmode == 7) {
    DGPP_REQUIRE(w_scale != nullptr && K <= 65536, "gemm_tc: bf12 needs its side buffer and K <= 65536");
    auto up16 = [](size_t v) { return (v + 15) & ~size_t(15); };
    const uint8_t* aux = static_cast<const uint8_t*>(w_scale);
    const size_t off_base = up16(static_cast<size_t>(N) * (K / 2));
    const size_t off_rows = off_base + up16(static_cast<size_t>(N));
    const size_t off_esc = off_rows + up16((static_cast<size_t>(N) + 1) * 4);
    p.bf12_base = aux + off_base;
    p.bf12_rows = reinterpret_cast<const uint32_t*>(aux + off_rows);
    p.bf12_esc = reinterpret_cast<const uint32_t*>(aux + off_esc);
  }
  p.status = device_status_ptr();
  p.T = T; p.N = N; p.K = K; p.ldc = ldc;
  const int num_kb = K / 64;
  const int align = nibble_src ? 4 : (byte_src ? 2 : 1);
  int per = dgpp_ceil_div(num_kb, splits);
  per = dgpp_ceil_div(per, align) * align;
  p.kb_per_split = per;
  splits = dgpp_ceil_div(num_kb, per);

  CUtensorMap tA, tB, tSf;
  memset(&tSf, 0, sizeof(tSf));
  if (comm_ag) {
    // [K, T, 2 * world] over this rank's payload slots: z = parity * world + owner
    const DgppComm* c = static_cast<const DgppComm*>(comm_ag);
    if (make_tmap_3d(&tB, c->st.peers[c->st.rank], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, T, 2 * c->st.world,
                     static_cast<uint64_t>(K) * 2, c->st.slot_bytes, 64, bn, CU_TENSOR_MAP_SWIZZLE_128B))
      return -1;
  } else if (make_tmap_2d(&tB, x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, T, x_stride * 2, 64, bn, CU_TENSOR_MAP_SWIZZLE_128B))
    return -1;
  if (wmode == 0) {
    if (make_tmap_2d(&tA, w, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, N, static_cast<uint64_t>(K) * 2, 64, kBM,
                     CU_TENSOR_MAP_SWIZZLE_128B))
      return -1;
  } else if (byte_src) {
    if (make_tmap_2d(&tA, w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, K, N, K, 128, kBM, CU_TENSOR_MAP_SWIZZLE_128B))
      return -1;
    if (wmode == 7 &&
        make_tmap_2d(&tSf, w_scale, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, K / 2, N, K / 2, 64, kBM,
                     CU_TENSOR_MAP_SWIZZLE_NONE))
      return -1;
  } else {
    if (make_tmap_2d(&tA, w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, K / 2, N, K / 2, 128, kBM, CU_TENSOR_MAP_SWIZZLE_128B))
      return -1;
    if (wmode == 1 &&
        make_tmap_2d(&tSf, w_scale, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, K / 16, N, K / 16, 16, kBM,
                     CU_TENSOR_MAP_SWIZZLE_NONE))
      return -1;
  }
#define DGPP_GEMM_BN(BNV)                                                       \
  if (bn == BNV) {                                                              \
    if (wmode == 0) return launch_gemm<BNV, 0>(tA, tB, tSf, p, splits, st);      \
    if (wmode == 1) return launch_gemm<BNV, 1>(tA, tB, tSf, p, splits, st);      \
    if (wmode == 2) return launch_gemm<BNV, 2>(tA, tB, tSf, p, splits, st);      \
    if (wmode == 3) return launch_gemm<BNV, 3>(tA, tB, tSf, p, splits, st);      \
    if (wmode == 4) return launch_gemm<BNV, 4>(tA, tB, tSf, p, splits, st);      \
    if (wmode == 5) return launch_gemm<BNV, 5>(tA, tB, tSf, p, splits, st);      \
    if (wmode == 6) return launch_gemm<BNV, 6>(tA, tB, tSf, p, splits, st);      \
    if (wmode == 7) return launch_gemm<BNV, 7>(tA, tB, tSf, p, splits, st);      \
  }
  DGPP_GEMM_BN(16) DGPP_GEMM_BN(32) DGPP_GEMM_BN(64) DGPP_GEMM_BN(128) DGPP_GEMM_BN(256)
#undef DGPP_GEMM_BN
  dgpp_set_error("gemm_tc: unsupported bn %d / wmode %d", bn, wmode);
  return -1;
}

DGPP_API int dgpp_gemm_tc(int wmode, int a_f16, int bn, const void* x, int64_t x_stride, const void* w,
                          const void* w_scale, float alpha, void* out, void* out32, const void* resid, int ldc,
                          int T, int N, int K, int splits, void* ws, void* counters, cudaStream_t st) {
  return gemm_tc_impl(wmode, a_f16, bn, x, x_stride, w, w_scale, alpha, out, out32, resid, ldc, T, N, K, splits, ws,
                      counters, nullptr, st);
}

// Same GEMM whose activations are the normed rows of the sequence-parallel all-gather (dgpp_comm_rs_norm_push of every
// rank, same token tile bn): x is not read; token tiles wait for their owner's flag inside the kernel.
DGPP_API int dgpp_gemm_tc_ag(int wmode, int a_f16, int bn, void* comm_ag, const void* w, const void* w_scale, float alpha,
                             void* out, void* out32, int ldc, int T, int N, int K, int splits, void* ws, void* counters,
                             cudaStream_t st) {
  DGPP_REQUIRE(comm_ag != nullptr, "gemm_tc_ag: communicator required");
  return gemm_tc_impl(wmode, a_f16, bn, nullptr, K, w, w_scale, alpha, out, out32, nullptr, ldc, T, N, K, splits, ws, counters,
                      nullptr, st, comm_ag);
}

// Same GEMM with the reduce-scatter push epilogue (see GemmParams::push); pair with dgpp_comm_rs_ag(comm, x, T, N, bn).
DGPP_API int dgpp_gemm_tc_push(int wmode, int a_f16, int bn, const void* x, int64_t x_stride, const void* w,
                               const void* w_scale, float alpha, int T, int N, int K, void* comm_push, cudaStream_t st) {
  return gemm_tc_impl(wmode, a_f16, bn, x, x_stride, w, w_scale, alpha, nullptr, nullptr, nullptr, N, T, N, K, 1, nullptr,
                      nullptr, comm_push, st);
}
