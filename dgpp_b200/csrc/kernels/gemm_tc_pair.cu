// W4A16 prefill GEMM on CTA pairs: out[T, N] = alpha * x[T, K] . W[N, K]^T (+ residual), 4-bit weights (NVFP4 with
// e4m3 scales per 16, or MXFP4 with e8m0 scales per 32) expanded to bf16 in shared memory, bf16 activations, fp32
// accumulation in TMEM.  Same arithmetic as the single-CTA kernel of gemm_tc.cu (bit-identical results: same
// converted operands, same K order), different tiling:
//
//   two CTAs of a cluster (one TPC) own 256 weight rows x 256 tokens.  Each CTA streams and converts ITS 128 weight
//   rows and loads ITS 128 tokens of the activation tile; one `tcgen05.mma.cta_group::2` per K = 16 step, issued by
//   the first CTA, multiplies all 256 rows by all 256 tokens, each SM reading the other's half of the activation tile
//   out of its shared memory.  Per K = 64 block an SM therefore moves 16 KB of activations from L2 instead of 32 KB,
//   which is what bounds the single-CTA kernel at prefill sizes (a 128 x 256 tile reuses the bf16 activation tile too
//   little).  No TMA multicast: every CTA issues plain loads into its own shared memory onto its own barriers.
//
// Handshakes (all waits bounded, expiry -> status code, everything unwinds, TMEM freed):
//   local, per CTA:   raw_full / raw_empty (TMA -> converters), a_full (converters -> MMA side), b_full (TMA -> MMA
//                     side);
//   second -> first:  a relay thread of the second CTA waits for its own a_full / b_full of block i and arrives on
//                     peer_ready[i % SA] of the first CTA (release / acquire at cluster scope);
//   first -> both:    `tcgen05.commit` with a CTA mask arrives on a_empty / b_empty / acc_full at the same offset in
//                     both CTAs when the MMAs that read those stages have completed.
// Warp roles (320 threads): warp 0 TMA producer, warp 1 MMA issuer (first CTA) or relay (second CTA) + TMEM owner,
// warps 2..9 converters, warps 2..5 epilogue.
// (reference counterpart: src/kernels/fp4w_gemm.cu, the W4A16 prefill GEMM.)
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <string.h>

#include "common/common.h"
#include "common/dtypes.cuh"
#include "common/ptx.cuh"
#include "kernels/gemm_common.cuh"

namespace dgpp {

constexpr int kPrBM = 128;          // weight rows per CTA
constexpr int kPrTok = 128;         // tokens per CTA (half of the pair's 256-token tile)
constexpr int kPrBN = 256;          // tokens per pair tile = MMA N
constexpr int kPrBK = 64;
constexpr int kPrThreads = 320;
constexpr int kPrConvWarps = 8;
constexpr int kPrSB = 8, kPrSA = 3, kPrSR = 2;
constexpr int kPrStageB = kPrTok * 128;     // 16 KB
constexpr int kPrStageA = kPrBM * 128;      // 16 KB of bf16 (64 K per row)
constexpr int kPrStageRaw = kPrBM * 128;    // 16 KB of packed fp4 (256 K per row)
constexpr int kPrStageSf = kPrBM * 16;      // 2 KB of e4m3 scales (NVFP4)

struct PairParams {
  float alpha;
  bf16* out;
  const bf16* resid;
  const uint8_t* sf_plain;   // MXFP4: e8m0 scales [N, K / 32]
  DeviceStatus* status;
  int T, N, K, ldc;
};

constexpr size_t pair_smem_bytes() {
  return 1024 + static_cast<size_t>(kPrSB) * kPrStageB + static_cast<size_t>(kPrSA) * kPrStageA +
         static_cast<size_t>(kPrSR) * (kPrStageRaw + kPrStageSf) + (2 * kPrSB + 3 * kPrSA + 2 * kPrSR + 1) * 8 + 64;
}

__device__ __forceinline__ bool wait_bar_cluster(uint64_t* bar, uint32_t parity) {
  for (int i = 0; i < 4096; ++i)
    if (mbar_try_wait_cluster(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
    for (int i = 0; i < 2048; ++i)
      if (mbar_try_wait_cluster(bar, parity)) return true;
    if (clock64() - t0 > 4000000000ll) return false;
  }
}

template <int WMODE>   // 1 = NVFP4, 3 = MXFP4
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPrThreads, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap tmA,   // packed weights as bytes [N, K / 2], box 128 x 128
                    const __grid_constant__ CUtensorMap tmB,   // activations bf16 [T, K], box 64 x 128
                    const __grid_constant__ CUtensorMap tmSf,  // NVFP4 scales [N, K / 16], box 16 x 128
                    PairParams p) {
  extern __shared__ __align__(1024) unsigned char smem_dyn[];
  unsigned char* sp = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  unsigned char* sB = sp;    sp += kPrSB * kPrStageB;
  unsigned char* sA = sp;    sp += kPrSA * kPrStageA;
  unsigned char* sRaw = sp;  sp += kPrSR * kPrStageRaw;
  unsigned char* sSf = sp;   sp += kPrSR * kPrStageSf;
  uint64_t* b_full = reinterpret_cast<uint64_t*>(sp);
  uint64_t* b_empty = b_full + kPrSB;
  uint64_t* a_full = b_empty + kPrSB;
  uint64_t* a_empty = a_full + kPrSA;
  uint64_t* peer_ready = a_empty + kPrSA;      // used in the first CTA only
  uint64_t* raw_full = peer_ready + kPrSA;
  uint64_t* raw_empty = raw_full + kPrSR;
  uint64_t* acc_full = raw_empty + kPrSR;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int n0 = blockIdx.x * kPrBM;
  const int m0 = blockIdx.y * kPrBN;
  const int mh = m0 + static_cast<int>(rank) * kPrTok;
  const int nkb = p.K / kPrBK;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kPrSB; ++i) { mbar_init(&b_full[i], 1); mbar_init(&b_empty[i], 1); }
    for (int i = 0; i < kPrSA; ++i) { mbar_init(&a_full[i], kPrConvWarps); mbar_init(&a_empty[i], 1); mbar_init(&peer_ready[i], 1); }
    for (int i = 0; i < kPrSR; ++i) { mbar_init(&raw_full[i], 1); mbar_init(&raw_empty[i], kPrConvWarps); }
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    if (WMODE == 1) tma_prefetch_desc(&tmSf);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, kPrBN);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_barrier();      // the other CTA's barriers exist before anything arrives on them from here
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (own weights, own token half)
    if (elect_one()) {
      for (int i = 0; i < nkb; ++i) {
        if (i % 4 == 0) {
          const int r = i / 4, sr = r % kPrSR;
          if (!wait_bar(&raw_empty[sr], ((r / kPrSR) & 1) ^ 1)) { report(p.status, kTimeoutStageEmpty, 21); *abort_flag = 1; break; }
          mbar_expect_tx(&raw_full[sr], kPrStageRaw + (WMODE == 1 ? kPrStageSf : 0));
          tma_load_2d(sRaw + sr * kPrStageRaw, &tmA, i * 32, n0, &raw_full[sr]);
          if (WMODE == 1) tma_load_2d(sSf + sr * kPrStageSf, &tmSf, i * 4, n0, &raw_full[sr]);
        }
        const int sb = i % kPrSB;
        if (!wait_bar(&b_empty[sb], ((i / kPrSB) & 1) ^ 1)) { report(p.status, kTimeoutStageEmpty, 22); *abort_flag = 1; break; }
        mbar_expect_tx(&b_full[sb], kPrStageB);
        tma_load_2d(sB + sb * kPrStageB, &tmB, i * kPrBK, mh, &b_full[sb]);
        if (*abort_flag) break;
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      if (rank == 0) {
        // ---------------------------------------------------------------- MMA issuer of the pair
        constexpr uint32_t idesc = umma_idesc_f16(2 * kPrBM, kPrBN, 1u, 1u);
        for (int i = 0; i < nkb; ++i) {
          const int sb = i % kPrSB, sa = i % kPrSA;
          if (!wait_bar(&b_full[sb], (i / kPrSB) & 1)) { report(p.status, kTimeoutTmaFull, 23); *abort_flag = 1; break; }
          if (!wait_bar(&a_full[sa], (i / kPrSA) & 1)) { report(p.status, kTimeoutConvert, 24); *abort_flag = 1; break; }
          if (!wait_bar_cluster(&peer_ready[sa], (i / kPrSA) & 1)) { report(p.status, kTimeoutPeerFlag, 25); *abort_flag = 1; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(sA + sa * kPrStageA), b_addr = smem_u32(sB + sb * kPrStageB);
#pragma unroll
          for (int kk = 0; kk < kPrBK / 16; ++kk)
            umma_f16_pair(tmem_base, umma_desc_sw128(a_addr + kk * 32), umma_desc_sw128(b_addr + kk * 32), idesc,
                          (i > 0 || kk > 0) ? 1u : 0u);
          umma_commit_pair(&b_empty[sb], 3);
          umma_commit_pair(&a_empty[sa], 3);
          if (*abort_flag) break;
        }
        umma_commit_pair(acc_full, 3);
      } else {
        // ---------------------------------------------------------------- relay: this CTA's stages of block i are ready
        for (int i = 0; i < nkb; ++i) {
          const int sb = i % kPrSB, sa = i % kPrSA;
          if (!wait_bar(&b_full[sb], (i / kPrSB) & 1)) { report(p.status, kTimeoutTmaFull, 26); *abort_flag = 1; break; }
          if (!wait_bar(&a_full[sa], (i / kPrSA) & 1)) { report(p.status, kTimeoutConvert, 27); *abort_flag = 1; break; }
          mbar_arrive_remote(mapa_shared(smem_u32(&peer_ready[sa]), 0u));
          if (*abort_flag) break;
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ converters (warps 2..9): e2m1 -> bf16
    const int ct = threadIdx.x - 64;       // 0..255
    const int row = ct >> 1, half = ct & 1;
    for (int i = 0; i < nkb; ++i) {
      const int r = i / 4, sub = i % 4, sr = r % kPrSR, sa = i % kPrSA;
      bool ok = true;
      if (sub == 0) ok = wait_bar(&raw_full[sr], (r / kPrSR) & 1);
      if (ok) ok = wait_bar(&a_empty[sa], ((i / kPrSA) & 1) ^ 1);
      if (!ok) { report(p.status, kTimeoutTmaFull, 28); *abort_flag = 1; break; }
      const unsigned char* raw = sRaw + sr * kPrStageRaw + row * 128;
      unsigned char* dst = sA + sa * kPrStageA + row * 128;
      // 32 weights = 16 packed bytes at logical 16-byte chunk (sub * 2 + half) of the swizzled 128-byte row
      const int cl = sub * 2 + half;
      Pack16 w;
      w.u = *reinterpret_cast<const uint4*>(raw + ((cl ^ (row & 7)) << 4));
      float s0f, s1f;
      if (WMODE == 1) {
        const unsigned char* sf = sSf + sr * kPrStageSf + row * 16 + sub * 4 + half * 2;
        s0f = e4m3_to_f32(sf[0]);
        s1f = e4m3_to_f32(sf[1]);
      } else {
        const int nrow = min(n0 + row, p.N - 1);
        s0f = s1f = e8m0_to_f32(p.sf_plain[static_cast<size_t>(nrow) * (p.K / 32) + i * 2 + half]);
      }
      // f16 bits >> 3 read as bf16 equal value * 2^-112; 2^112 is folded into the (exact) bf16 scale
      const bf162 s0 = __float2bfloat162_rn(s0f * 5.192296858534828e33f);
      const bf162 s1 = __float2bfloat162_rn(s1f * 5.192296858534828e33f);
      Pack16 o[4];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        __half2 h = e2m1x2_to_h2(w.b[j]);
        const uint32_t hb = *reinterpret_cast<uint32_t*>(&h);
        uint32_t bb = ((hb & 0x7FFF7FFFu) >> 3) | (hb & 0x80008000u);
        bf162 v = __hmul2(*reinterpret_cast<bf162*>(&bb), j < 8 ? s0 : s1);
        o[j >> 2].w[j & 3] = *reinterpret_cast<uint32_t*>(&v);
      }
#pragma unroll
      for (int c = 0; c < 4; ++c)
        *reinterpret_cast<uint4*>(dst + (((half * 4 + c) ^ (row & 7)) << 4)) = o[c].u;
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&a_full[sa]);
        if (sub == 3 || i == nkb - 1) mbar_arrive(&raw_empty[sr]);
      }
      if (*abort_flag) break;
    }
  }

  // ------------------------------------------------------------------ epilogue (warps 2..5): own 128 rows x 256 tokens
  if (warp >= 2 && warp < 6) {
    const int q = warp & 3;
    const bool ok = nkb > 0 ? wait_bar_cluster(acc_full, 0) : true;
    if (!ok) { report(p.status, kTimeoutAccum, 29); *abort_flag = 1; }
    tc_fence_after();
    const int n = n0 + q * 32 + lane;
    const int cols = min(kPrBN, p.T - m0);
    if (ok && !*abort_flag) {
#pragma unroll 1
      for (int c0 = 0; c0 < kPrBN; c0 += 16) {
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
              const size_t o = static_cast<size_t>(m0 + m) * p.ldc + n;
              float y = __uint_as_float(r[j]) * p.alpha;
              if (p.resid) y = bf16_to_f32(p.resid[o]) + bf16_to_f32(f32_to_bf16(y));
              p.out[o] = f32_to_bf16(y);
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  cluster_barrier();      // neither CTA leaves (or frees TMEM) while the other may still read its shared memory
  if (warp == 1) tmem_dealloc_pair(tmem_base, kPrBN);
}

template <int WMODE>
static int launch_pair(const CUtensorMap& tA, const CUtensorMap& tB, const CUtensorMap& tSf, const PairParams& p, cudaStream_t st) {
  auto kern = gemm_tc_pair_kernel<WMODE>;
  static bool attr = false;
  constexpr size_t smem = pair_smem_bytes();
  static_assert(smem <= 227 * 1024, "shared memory budget exceeded");
  if (!attr) {
    DGPP_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    attr = true;
  }
  dim3 grid(p.N / kPrBM, dgpp_ceil_div(p.T, kPrBN), 1);
  kern<<<grid, kPrThreads, smem, st>>>(tA, tB, tSf, p);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

}  // namespace dgpp

using namespace dgpp;

// wmode: 1 nvfp4 (w_scale = e4m3 scales [N, K / 16]), 3 mxfp4 (w_scale = e8m0 scales [N, K / 32]).  N % 256 == 0,
// K % 256 == 0.  out bf16 [T, ldc]; resid optional (out = bf16(resid + bf16(alpha * acc))).
DGPP_API int dgpp_gemm_tc_pair(int wmode, const void* x, int64_t x_stride, const void* w, const void* w_scale, float alpha,
                               void* out, const void* resid, int ldc, int T, int N, int K, cudaStream_t st) {
  DGPP_REQUIRE(wmode == 1 || wmode == 3, "gemm_tc_pair: 4-bit weights only (wmode %d)", wmode);
  DGPP_REQUIRE(T >= 1 && N >= 256 && N % 256 == 0, "gemm_tc_pair: N %d must be a multiple of 256", N);
  DGPP_REQUIRE(K % 256 == 0, "gemm_tc_pair: K %d must be a multiple of 256", K);
  DGPP_REQUIRE(out != nullptr && w_scale != nullptr, "gemm_tc_pair: output and scales required");
  PairParams p;
  p.alpha = alpha;
  p.out = static_cast<bf16*>(out);
  p.resid = static_cast<const bf16*>(resid);
  p.sf_plain = wmode == 3 ? static_cast<const uint8_t*>(w_scale) : nullptr;
  p.status = device_status_ptr();
  p.T = T; p.N = N; p.K = K; p.ldc = ldc;
  CUtensorMap tA, tB, tSf;
  memset(&tSf, 0, sizeof(tSf));
  if (make_tmap_2d(&tB, x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, T, x_stride * 2, 64, kPrTok, CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
  if (make_tmap_2d(&tA, w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, K / 2, N, K / 2, 128, kPrBM, CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
  if (wmode == 1 &&
      make_tmap_2d(&tSf, w_scale, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, K / 16, N, K / 16, 16, kPrBM, CU_TENSOR_MAP_SWIZZLE_NONE))
    return -1;
  return wmode == 1 ? launch_pair<1>(tA, tB, tSf, p, st) : launch_pair<3>(tA, tB, tSf, p, st);
}
