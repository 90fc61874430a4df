// FP8 x FP8 linear on tcgen05 kind::f8f6f4 with block scales promoted in the loop.
//
//   weights      e4m3 [N, K] with one fp32 scale per 128 x 128 block (the "fp8" checkpoint format)
//   activations  quantised here: e4m3 [T, K] with one fp32 scale per token and 128 columns (fp8_act_quant_kernel)
//   out[t, n] = sum over K blocks kb of  ws[n / 128, kb] * xs[t, kb] * ( Wq[n, kb] . Xq[t, kb] )
//
// The weights are the A operand (a 128-row weight tile = the 128 TMEM lanes), the token tile is N of the MMA.  One K
// block (128 columns = four MMA k-steps) is accumulated in TMEM without scales; the epilogue warps then read it and add
// it, scaled by the block's two scales, to fp32 registers ("promotion") while the tensor core already works on the next
// block in the other TMEM buffer.  Nothing converts the e4m3 bytes: HBM -> TMA -> shared memory -> tensor core.
// Warps: 0 = TMA producer (tiles + the block's activation scales, which ride a ring twice as deep as the tile ring:
// an epilogue may still read them after the MMAs have released the tile stage), 1 = MMA issuer / TMEM owner, 2..5 and
// 6..9 = two promotion sets, each covering all 128 weight rows and half of the token columns (token tiles of 16 use
// one set).  Bounded waits throughout.
// Split K (grid z): fp32 partials [z][T][N], folded in ascending z by fp8_splitk_fold_kernel.
// (reference counterparts: src/kernels/fp8_gemm.cu:23-111 activation quantisers, :199 fp8_gemm_kernel with in-loop
//  promotion, src/kernels/scale_gemm.cu block-scaled FP8 weights.)
#include <cuda.h>
#include <math.h>
#include <string.h>

#include "common/common.h"
#include "common/dtypes.cuh"
#include "common/ptx.cuh"
#include "kernels/gemm_common.cuh"

namespace dgpp {

constexpr int kF8Threads = 320;   // TMA warp, MMA warp, two epilogue sets of four warps
constexpr int kF8BM = 128;      // weight rows per tile
constexpr int kF8BK = 128;      // K columns per scale block = bytes per tile row

// x [T, K] bf16 -> q [T_pad, K] e4m3, xs [K / 128, T_pad] fp32 (scale = amax / 448 per token and block; 1 for a zero
// block).  grid (T), 128 threads: warp w quantises blocks w, w + 4, ...
__global__ void __launch_bounds__(128) fp8_act_quant_kernel(const bf16* __restrict__ x, int64_t x_stride,
                                                            uint8_t* __restrict__ q, float* __restrict__ xs, int K, int T_pad) {
  pdl_wait();
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int kb = warp; kb < K / kF8BK; kb += 4) {
    const bf16* src = x + static_cast<size_t>(t) * x_stride + kb * kF8BK + lane * 4;
    float v[4];
    float am = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) { v[j] = bf16_to_f32(src[j]); am = fmaxf(am, fabsf(v[j])); }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
    const float sc = am > 0.f ? am / 448.f : 1.f;
    const float inv = 1.f / sc;
    uint32_t packed = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) packed |= static_cast<uint32_t>(f32_to_e4m3(v[j] * inv)) << (8 * j);
    *reinterpret_cast<uint32_t*>(q + static_cast<size_t>(t) * K + kb * kF8BK + lane * 4) = packed;
    if (lane == 0) xs[static_cast<size_t>(kb) * T_pad + t] = sc;
  }
}

struct F8Params {
  const float* ws;      // [ceil(N / 128), K / 128]
  const float* xs;      // [K / 128, T_pad]
  bf16* out;            // [T, ldc]
  float* partial;       // [splits, T, N] when splits > 1
  DeviceStatus* status;
  int T, T_pad, N, K, ldc, splits;
};

template <int BN, int STAGES>
__global__ void __launch_bounds__(kF8Threads, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, F8Params p) {
  constexpr int kABytes = kF8BM * kF8BK, kBBytes = BN * kF8BK;
  constexpr int kTmemCols = 2 * BN < 32 ? 32 : 2 * BN;
  constexpr int kSets = BN >= 32 ? 2 : 1;        // promotion sets in use
  constexpr int CH = BN / kSets;                 // token columns per set
  constexpr int kXsSlots = 2 * STAGES;
  extern __shared__ __align__(1024) unsigned char smem_dyn[];
  unsigned char* sp = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  unsigned char* sA = sp;  sp += STAGES * kABytes;
  unsigned char* sB = sp;  sp += STAGES * kBBytes;
  float* sXs = reinterpret_cast<float*>(sp);  sp += kXsSlots * BN * sizeof(float);
  uint64_t* full = reinterpret_cast<uint64_t*>(sp);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;   // [2]
  uint64_t* acc_empty = acc_full + 2;    // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * kF8BM, t0 = blockIdx.y * BN, z = blockIdx.z;
  const int KB = p.K / kF8BK;
  const int per = (KB + p.splits - 1) / p.splits;
  const int kb0 = z * per, kb1 = min(KB, kb0 + per);
  const int nkb = max(0, kb1 - kb0);

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], 4 * kSets); }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmW);
    tma_prefetch_desc(&tmX);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (elect_one()) {
      // the weights do not depend on the previous kernel: only the activation loads wait for it
      bool waited = false;
      for (int i = 0; i < nkb; ++i) {
        const int s = i % STAGES;
        if (!wait_bar(&empty[s], ((i / STAGES) & 1) ^ 1)) { report(p.status, kTimeoutStageEmpty, 61); *abort_flag = 1; break; }
        mbar_expect_tx(&full[s], kABytes + kBBytes + BN * sizeof(float));
        tma_load_2d(sA + s * kABytes, &tmW, (kb0 + i) * kF8BK, n0, &full[s]);
        if (!waited) { pdl_wait(); waited = true; }
        tma_load_2d(sB + s * kBBytes, &tmX, (kb0 + i) * kF8BK, t0, &full[s]);
        bulk_load_1d(sXs + (i % kXsSlots) * BN, p.xs + static_cast<size_t>(kb0 + i) * p.T_pad + t0, BN * sizeof(float), &full[s]);
        if (*abort_flag) break;
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc_f8(kF8BM, BN, 0u, 0u);
      for (int i = 0; i < nkb; ++i) {
        const int s = i % STAGES, b = i & 1;
        if (!wait_bar(&acc_empty[b], ((i >> 1) & 1) ^ 1)) { report(p.status, kTimeoutAccum, 62); *abort_flag = 1; break; }
        if (!wait_bar(&full[s], (i / STAGES) & 1)) { report(p.status, kTimeoutTmaFull, 63); *abort_flag = 1; break; }
        tc_fence_after();
        const uint32_t a_addr = smem_u32(sA + s * kABytes), b_addr = smem_u32(sB + s * kBBytes);
#pragma unroll
        for (int k = 0; k < kF8BK / 32; ++k)
          umma_f8f6f4(tmem_base + b * BN, umma_desc_sw128(a_addr + k * 32), umma_desc_sw128(b_addr + k * 32), idesc,
                      k > 0 ? 1u : 0u);
        umma_commit(&acc_full[b]);
        umma_commit(&empty[s]);
        if (*abort_flag) break;
      }
    }
  } else if ((warp - 2) / 4 < kSets) {
    pdl_wait();
    const int set = (warp - 2) / 4;
    const int quad = warp & 3;
    const int row = quad * 32 + lane;                    // weight row inside the tile = TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const int col0 = set * CH;
    float acc[CH];
#pragma unroll
    for (int c = 0; c < CH; ++c) acc[c] = 0.f;
    const float* wsr = p.ws + static_cast<size_t>(blockIdx.x) * KB;
    bool ok = true;
    for (int i = 0; i < nkb && ok; ++i) {
      const int b = i & 1, kb = kb0 + i;
      if (!wait_bar(&acc_full[b], (i >> 1) & 1)) { report(p.status, kTimeoutAccum, 64); *abort_flag = 1; ok = false; break; }
      tc_fence_after();
      const float wsc = wsr[kb];
      const float* xsr = sXs + (i % kXsSlots) * BN + col0;
#pragma unroll
      for (int c0 = 0; c0 < CH; c0 += 16) {
        uint32_t raw[16];
        tmem_ld_x16(tmem_base + b * BN + col0 + c0 + lane_addr, raw);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 16; ++c) acc[c0 + c] = fmaf(__uint_as_float(raw[c]), wsc * xsr[c0 + c], acc[c0 + c]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[b]);
    }
    const int n = n0 + row;
    if (ok && n < p.N) {
      if (p.splits == 1) {
#pragma unroll
        for (int c = 0; c < CH; ++c)
          if (t0 + col0 + c < p.T) p.out[static_cast<size_t>(t0 + col0 + c) * p.ldc + n] = f32_to_bf16(acc[c]);
      } else {
        float* dst = p.partial + static_cast<size_t>(z) * p.T * p.N;
#pragma unroll
        for (int c = 0; c < CH; ++c)
          if (t0 + col0 + c < p.T) dst[static_cast<size_t>(t0 + col0 + c) * p.N + n] = acc[c];
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
}

__global__ void fp8_splitk_fold_kernel(const float* __restrict__ partial, bf16* __restrict__ out, int T, int N, int ldc,
                                       int splits) {
  pdl_wait();
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= static_cast<int64_t>(T) * N) return;
  float s = 0.f;
  for (int z = 0; z < splits; ++z) s += partial[static_cast<int64_t>(z) * T * N + i];
  out[(i / N) * ldc + i % N] = f32_to_bf16(s);
}

template <int BN, int STAGES>
static int launch_f8(const CUtensorMap& tW, const CUtensorMap& tX, const F8Params& p, cudaStream_t st) {
  constexpr size_t smem = 1024 + STAGES * (kF8BM * kF8BK + BN * kF8BK) + 2 * STAGES * BN * 4 + (2 * STAGES + 4) * 8 + 64;
  static_assert(smem <= 227 * 1024, "gemm_fp8: shared memory over the per-CTA limit");
  static bool attr = false;
  if (!attr) {
    DGPP_CUDA_OK(cudaFuncSetAttribute(gemm_fp8_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      static_cast<int>(smem)));
    attr = true;
  }
  dim3 grid(dgpp_ceil_div(p.N, kF8BM), dgpp_ceil_div(p.T, BN), p.splits);
  gemm_fp8_kernel<BN, STAGES><<<grid, kF8Threads, smem, st>>>(tW, tX, p);
  DGPP_CUDA_OK(cudaGetLastError());
  if (p.splits > 1) {
    const int64_t n = static_cast<int64_t>(p.T) * p.N;
    fp8_splitk_fold_kernel<<<static_cast<unsigned>(dgpp_ceil_div64(n, 256)), 256, 0, st>>>(p.partial, p.out, p.T, p.N, p.ldc,
                                                                                         p.splits);
    DGPP_CUDA_OK(cudaGetLastError());
  }
  return 0;
}

}  // namespace dgpp

using namespace dgpp;

// x [T, K] bf16 -> q [T_pad, K] e4m3 + xs [K / 128, T_pad] fp32.  Rows T .. T_pad of q must be zero (they are never written).
DGPP_API int dgpp_fp8_act_quant(const void* x, int64_t x_stride, void* q, void* xs, int T, int T_pad, int K, cudaStream_t st) {
  DGPP_REQUIRE(K % 128 == 0 && T <= T_pad, "fp8_act_quant: K %d must be a multiple of 128 (T %d, T_pad %d)", K, T, T_pad);
  if (T == 0) return 0;
  fp8_act_quant_kernel<<<T, 128, 0, st>>>(static_cast<const bf16*>(x), x_stride, static_cast<uint8_t*>(q),
                                          static_cast<float*>(xs), K, T_pad);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

// out [T, N] bf16 = block-scaled FP8 weights x FP8 activations.  bn = token tile (16 / 32 / 64 / 128), T_pad a multiple
// of it; partial: fp32 [splits, T, N] when splits > 1.
DGPP_API int dgpp_gemm_fp8(const void* wq, const void* ws, const void* xq, const void* xs, void* out, void* partial, int ldc,
                           int T, int T_pad, int N, int K, int bn, int splits, cudaStream_t st) {
  DGPP_REQUIRE(K % 128 == 0 && T_pad % bn == 0 && T <= T_pad && splits >= 1, "gemm_fp8: bad sizes (K %d T %d / %d bn %d)", K, T,
               T_pad, bn);
  DGPP_REQUIRE(splits == 1 || partial != nullptr, "gemm_fp8: split K needs the partial buffer");
  if (T == 0) return 0;
  F8Params p;
  p.ws = static_cast<const float*>(ws); p.xs = static_cast<const float*>(xs);
  p.out = static_cast<bf16*>(out); p.partial = static_cast<float*>(partial);
  p.status = device_status_ptr();
  p.T = T; p.T_pad = T_pad; p.N = N; p.K = K; p.ldc = ldc; p.splits = splits;
  CUtensorMap tW, tX;
  if (make_tmap_2d(&tW, wq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, K, N, K, 128, 128, CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
  if (make_tmap_2d(&tX, xq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, K, T_pad, K, 128, bn, CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
  switch (bn) {
    case 16: return launch_f8<16, 8>(tW, tX, p, st);
    case 32: return launch_f8<32, 8>(tW, tX, p, st);
    case 64: return launch_f8<64, 6>(tW, tX, p, st);
    case 128: return launch_f8<128, 6>(tW, tX, p, st);
  }
  dgpp_set_error("gemm_fp8: token tile %d not instantiated", bn);
  return -1;
}
