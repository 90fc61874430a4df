// NVFP4 x NVFP4 linear layer on the block-scaled tensor-core path (tcgen05 kind::mxf4nvf4,
// scale_vec::4X: one ue4m3 scale per 16 elements for both operands, scale factors in TMEM):
//
//     C[T, N] = alpha_w * g[t] * sum_r  Wq[N, K] . Xq_r[T, K]^T
//
// The packed e2m1 weight bytes go from HBM through TMA into shared memory and straight into the
// tensor core: no thread ever touches a weight.  Activations arrive already quantised by
// `act_quant_nvfp4_kernel` as R "residual terms": x ~= g[t] * (x_1 + x_2 + ... + x_R), each term an
// NVFP4 tensor of what the previous terms left over.  All R terms accumulate into the same fp32
// TMEM accumulator, so R = 1 is plain W4A4 and R = 3 carries about 8 mantissa bits of the bf16
// activation (every term removes ~2.6 bits of the remaining error) at no extra weight traffic.
//
// Layout: weight tile = UMMA A (128 rows), token tile = UMMA B (BN = 16..256 rows).  One pipeline
// stage covers 256 K: 128 bytes of packed fp4 per row (one 128-byte swizzle row = four K=64 MMAs).
// Scale factors are read from their checkpoint layout [rows, K/16] by four helper warps that write
// them as the 512-byte "32 lanes x 16 bytes" atoms tcgen05.cp expects (row m, factor i of a K=64 step
// -> byte (m % 32) * 16 + (m / 32) * 4 + i); the MMA thread copies the atoms into TMEM.
//
// Warp roles (192 threads): warp 0 TMA producer, warp 1 MMA issuer / TMEM owner, warps 2..5 scale
// staging then epilogue.  Split-K as in gemm_tc.cu (deterministic ascending fold by the last CTA).
// (reference counterpart: src/kernels/moe_w4a4.cu:87,139,476 -- block-scaled mma.sync m16n8k64 there.)
#include <cuda.h>
#include <string.h>

#include "common/common.h"
#include "common/dtypes.cuh"
#include "common/ptx.cuh"
#include "kernels/gemm_common.cuh"

namespace dgpp {

constexpr int kF4Threads = 192;
constexpr int kF4BM = 128;
constexpr int kF4StageK = 256;            // K elements per stage
constexpr int kF4StageA = kF4BM * 128;    // 16 KB of packed fp4
constexpr int kF4Atom = 512;              // bytes of one scale-factor atom (128 rows x 4 factors)

struct Fp4Params {
  float alpha;                 // weight tensor scale
  const float* g;              // per-token activation scale [T]
  const uint8_t* sfa;          // weight scales [N, K/16] (e4m3 bytes, checkpoint layout)
  const uint8_t* sfb;          // activation scales [R, T_pad, K/16]
  bf16* out;
  float* out32;
  const bf16* resid;
  float* ws;
  uint32_t* counters;
  DeviceStatus* status;
  int T, T_pad, N, K, ldc, R;
  int stages_per_split;
};

template <int BN, int RMAX, int S>
__global__ void __launch_bounds__(kF4Threads, 1)
gemm_fp4_kernel(const __grid_constant__ CUtensorMap tmA,   // packed weights as bytes [N, K/2]
                const __grid_constant__ CUtensorMap tmB,   // packed activations as bytes [R*T_pad, K/2]
                Fp4Params p) {
  constexpr int kStageB = BN * 128;                  // one term
  constexpr int kAtomsB = BN > 128 ? 2 : 1;          // 128-row atoms per K=64 step
  constexpr int kSfaBytes = 4 * kF4Atom;             // 4 K-steps
  constexpr int kSfbBytes = 4 * kAtomsB * kF4Atom;   // per term
  extern __shared__ __align__(1024) unsigned char smem_dyn[];
  unsigned char* sp = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  unsigned char* sA = sp;    sp += S * kF4StageA;
  unsigned char* sB = sp;    sp += S * RMAX * kStageB;
  unsigned char* sSfa = sp;  sp += S * kSfaBytes;
  unsigned char* sSfb = sp;  sp += S * RMAX * kSfbBytes;
  uint64_t* full = reinterpret_cast<uint64_t*>(sp);
  uint64_t* empty = full + S;
  uint64_t* sf_ready = empty + S;
  uint64_t* acc_full = sf_ready + S;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* last_flag = const_cast<int*>(abort_flag) + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * kF4BM;
  const int m0 = blockIdx.y * BN;
  const int split = blockIdx.z, splits = gridDim.z;
  const int total_stages = p.K / kF4StageK;
  const int st_begin = split * p.stages_per_split;
  const int st_end = min(total_stages, st_begin + p.stages_per_split);
  const int nst = max(0, st_end - st_begin);
  const int R = p.R;
  // TMEM columns: accumulator, then double-buffered scale factors (4 columns per K=64 step and 128 rows)
  constexpr uint32_t kColD = BN < 32 ? 32 : BN;
  constexpr uint32_t kColSfa = 16;
  constexpr uint32_t kColSfb = 16 * kAtomsB;
  constexpr uint32_t kNeed = kColD + 2 * kColSfa + 2 * RMAX * kColSfb;
  constexpr uint32_t kTmemCols = kNeed <= 32 ? 32 : (kNeed <= 64 ? 64 : (kNeed <= 128 ? 128 : (kNeed <= 256 ? 256 : 512)));

  if (threadIdx.x == 0) {
    for (int i = 0; i < S; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
      mbar_init(&sf_ready[i], 4);
    }
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    *last_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_sfa = tmem_base + kColD;
  const uint32_t tmem_sfb = tmem_sfa + 2 * kColSfa;
  pdl_wait();

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      for (int i = 0; i < nst; ++i) {
        const int s = i % S;
        if (!wait_bar(&empty[s], ((i / S) & 1) ^ 1)) { report(p.status, kTimeoutStageEmpty, 11); *abort_flag = 1; break; }
        mbar_expect_tx(&full[s], kF4StageA + R * kStageB);
        const int xb = (st_begin + i) * 128;  // byte column of this stage
        tma_load_2d(sA + s * kF4StageA, &tmA, xb, n0, &full[s]);
        for (int r = 0; r < R; ++r)
          tma_load_2d(sB + (s * RMAX + r) * kStageB, &tmB, xb, r * p.T_pad + m0, &full[s]);
        if (*abort_flag) break;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc_fp4bs(kF4BM, BN, 0u);
      for (int i = 0; i < nst; ++i) {
        const int s = i % S;
        const uint32_t par = (i / S) & 1;
        if (!wait_bar(&full[s], par)) { report(p.status, kTimeoutTmaFull, 12); *abort_flag = 1; break; }
        if (!wait_bar(&sf_ready[s], par)) { report(p.status, kTimeoutConvert, 13); *abort_flag = 1; break; }
        tc_fence_after();
        const uint32_t buf = i & 1;
        const uint32_t t_sfa = tmem_sfa + buf * kColSfa;
        // scale factors: shared memory atoms -> TMEM (32 lanes x 16 bytes, replicated to the 4 lane quadrants)
        for (int j = 0; j < 4; ++j)
          tmem_cp_32x128b_warpx4(t_sfa + 4 * j, umma_desc_nosw(smem_u32(sSfa + s * kSfaBytes + j * kF4Atom), 0, 128));
        for (int r = 0; r < R; ++r) {
          const uint32_t t_sfb = tmem_sfb + (buf * RMAX + r) * kColSfb;
          for (int j = 0; j < 4 * kAtomsB; ++j)
            tmem_cp_32x128b_warpx4(t_sfb + 4 * j,
                                   umma_desc_nosw(smem_u32(sSfb + (s * RMAX + r) * kSfbBytes + j * kF4Atom), 0, 128));
        }
        const uint32_t a_addr = smem_u32(sA + s * kF4StageA);
        for (int r = 0; r < R; ++r) {
          const uint32_t b_addr = smem_u32(sB + (s * RMAX + r) * kStageB);
          const uint32_t t_sfb = tmem_sfb + (buf * RMAX + r) * kColSfb;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            umma_nvfp4(tmem_base, umma_desc_sw128(a_addr + j * 32), umma_desc_sw128(b_addr + j * 32), idesc,
                       t_sfa + 4 * j, t_sfb + 4 * kAtomsB * j, (i > 0 || r > 0 || j > 0) ? 1u : 0u);
          }
        }
        umma_commit(&empty[s]);
        if (*abort_flag) break;
      }
      umma_commit(acc_full);
    }
  } else {
    // ------------------------------------------------------------------ scale-factor staging (warps 2..5)
    const int t = threadIdx.x - 64;  // 0..127 = row inside a 128-row atom
    const int sf_pitch = p.K / 16;
    const int arow = min(n0 + t, p.N - 1);
    const uint8_t* a_src = p.sfa + static_cast<size_t>(arow) * sf_pitch + static_cast<size_t>(st_begin) * 16;
    const uint32_t atom_off = (t & 31) * 16 + (t >> 5) * 4;
    uint4 a_next = nst > 0 ? *reinterpret_cast<const uint4*>(a_src) : make_uint4(0, 0, 0, 0);
    for (int i = 0; i < nst; ++i) {
      const int s = i % S;
      const uint4 a_cur = a_next;
      if (i + 1 < nst) a_next = *reinterpret_cast<const uint4*>(a_src + static_cast<size_t>(i + 1) * 16);
      // activation scales of this stage (small: BN rows per term), loaded before the wait
      uint4 b_cur[RMAX * kAtomsB];
#pragma unroll
      for (int r = 0; r < RMAX; ++r) {
#pragma unroll
        for (int h = 0; h < kAtomsB; ++h) {
          const int row = m0 + h * 128 + t;
          b_cur[r * kAtomsB + h] = make_uint4(0, 0, 0, 0);
          if (r < R && h * 128 + t < BN && row < p.T)
            b_cur[r * kAtomsB + h] = *reinterpret_cast<const uint4*>(
                p.sfb + (static_cast<size_t>(r) * p.T_pad + row) * sf_pitch + static_cast<size_t>(st_begin + i) * 16);
        }
      }
      if (!wait_bar(&empty[s], ((i / S) & 1) ^ 1)) { report(p.status, kTimeoutStageEmpty, 14); *abort_flag = 1; break; }
      unsigned char* da = sSfa + s * kSfaBytes + atom_off;
      *reinterpret_cast<uint32_t*>(da + 0 * kF4Atom) = a_cur.x;
      *reinterpret_cast<uint32_t*>(da + 1 * kF4Atom) = a_cur.y;
      *reinterpret_cast<uint32_t*>(da + 2 * kF4Atom) = a_cur.z;
      *reinterpret_cast<uint32_t*>(da + 3 * kF4Atom) = a_cur.w;
#pragma unroll
      for (int r = 0; r < RMAX; ++r) {
        if (r < R) {
#pragma unroll
          for (int h = 0; h < kAtomsB; ++h) {
            // K-step j of atom-group h lives at atom index j * kAtomsB + h
            unsigned char* db = sSfb + (s * RMAX + r) * kSfbBytes + atom_off;
            const uint4 v = b_cur[r * kAtomsB + h];
            *reinterpret_cast<uint32_t*>(db + (0 * kAtomsB + h) * kF4Atom) = v.x;
            *reinterpret_cast<uint32_t*>(db + (1 * kAtomsB + h) * kF4Atom) = v.y;
            *reinterpret_cast<uint32_t*>(db + (2 * kAtomsB + h) * kF4Atom) = v.z;
            *reinterpret_cast<uint32_t*>(db + (3 * kAtomsB + h) * kF4Atom) = v.w;
          }
        }
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sf_ready[s]);
      if (*abort_flag) break;
    }

    // ------------------------------------------------------------------ epilogue (same warps)
    const int q = warp & 3;
    const bool ok = nst > 0 ? wait_bar(acc_full, 0) : true;
    if (!ok) { report(p.status, kTimeoutAccum, 15); *abort_flag = 1; }
    tc_fence_after();
    const int n = n0 + q * 32 + lane;
    const int cols = min(BN, p.T - m0);
    if (ok && !*abort_flag) {
      float* wsp = splits > 1 ? p.ws + (static_cast<size_t>(split) * p.T + m0) * p.N : nullptr;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 16) {
        if (c0 >= cols) break;
        uint32_t r[16];
        if (nst > 0) {
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
              } else {
                const size_t o = static_cast<size_t>(m0 + m) * p.ldc + n;
                float y = v * p.alpha * p.g[m0 + m];
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
    if (splits > 1) {
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
          for (int m = 0; m < cols; ++m) {
            float acc = 0.f;
            for (int s2 = 0; s2 < splits; ++s2)
              acc += __ldcg(p.ws + (static_cast<size_t>(s2) * p.T + m0 + m) * p.N + n);
            const size_t o = static_cast<size_t>(m0 + m) * p.ldc + n;
            float y = acc * p.alpha * p.g[m0 + m];
            if (p.out32) p.out32[o] = y;
            if (p.out) {
              if (p.resid) y = bf16_to_f32(p.resid[o]) + bf16_to_f32(f32_to_bf16(y));
              p.out[o] = f32_to_bf16(y);
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

// --------------------------------------------------------------------------------------------------
// Activation quantiser: bf16 rows -> R residual NVFP4 terms.
//   g[t]      = max|x[t, :]| / (6 * 256)      (fp32; the e4m3 block scales then stay <= 256)
//   term r    : block scale s = e4m3(amax_16(res) / (6 g)), codes = e2m1(res / (s g)), res -= codes * s * g
// q: [R, T_pad, K/2] bytes (low nibble = even k), sf: [R, T_pad, K/16] e4m3 bytes.  One warp per row.
// Optional fused input transforms: `gate_up` != null quantises swiglu(gate_up) instead of x.
__global__ void __launch_bounds__(256)
act_quant_nvfp4_kernel(const bf16* __restrict__ x, int64_t x_stride, uint8_t* __restrict__ q,
                       uint8_t* __restrict__ sf, float* __restrict__ g, int T, int T_pad, int K, int R) {
  pdl_wait();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= T) return;
  const bf16* row = x + static_cast<size_t>(warp) * x_stride;
  const int groups = K / 16;
  float amax = 0.f;
  for (int gi = lane; gi < groups; gi += 32) {
    Pack16 a, b;
    a.u = reinterpret_cast<const uint4*>(row + gi * 16)[0];
    b.u = reinterpret_cast<const uint4*>(row + gi * 16)[1];
#pragma unroll
    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fmaxf(fabsf(bf16_to_f32(a.h[j])), fabsf(bf16_to_f32(b.h[j]))));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float gs = amax > 0.f ? amax / (6.f * 256.f) : 1.f;
  if (lane == 0) g[warp] = gs;
  const float inv_g = 1.f / gs;
  for (int gi = lane; gi < groups; gi += 32) {
    Pack16 a, b;
    a.u = reinterpret_cast<const uint4*>(row + gi * 16)[0];
    b.u = reinterpret_cast<const uint4*>(row + gi * 16)[1];
    float res[16];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      res[j] = bf16_to_f32(a.h[j]) * inv_g;
      res[8 + j] = bf16_to_f32(b.h[j]) * inv_g;
    }
    for (int r = 0; r < R; ++r) {
      float bm = 0.f;
#pragma unroll
      for (int j = 0; j < 16; ++j) bm = fmaxf(bm, fabsf(res[j]));
      const uint8_t sb = f32_to_e4m3(bm * (1.f / 6.f));
      const float s = e4m3_to_f32(sb);
      const float inv_s = s > 0.f ? 1.f / s : 0.f;
      uint32_t lo = 0, hi = 0;
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const uint32_t c = f32_to_e2m1(res[j] * inv_s);
        res[j] -= e2m1_to_f32(c) * s;
        if (j < 8) lo |= c << (4 * j); else hi |= c << (4 * (j - 8));
      }
      const size_t ro = static_cast<size_t>(r) * T_pad + warp;
      *reinterpret_cast<uint2*>(q + ro * (K / 2) + gi * 8) = make_uint2(lo, hi);
      sf[ro * groups + gi] = sb;
    }
  }
}

template <int BN, int RMAX>
struct Fp4Cfg {
  static constexpr int kAtomsB = BN > 128 ? 2 : 1;
  static constexpr size_t stage_bytes() {
    return kF4StageA + static_cast<size_t>(RMAX) * BN * 128 + 4 * kF4Atom + static_cast<size_t>(RMAX) * 4 * kAtomsB * kF4Atom;
  }
  static constexpr int S = (200 * 1024) / stage_bytes() > 6 ? 6 : (200 * 1024) / stage_bytes();
  static constexpr size_t smem() { return 1024 + S * stage_bytes() + (3 * S + 1) * 8 + 64; }
};

template <int BN, int RMAX>
static int launch_fp4(const CUtensorMap& tA, const CUtensorMap& tB, const Fp4Params& p, int splits, cudaStream_t st) {
  using C = Fp4Cfg<BN, RMAX>;
  static_assert(C::S >= 2, "not enough shared memory for two stages");
  auto kern = gemm_fp4_kernel<BN, RMAX, C::S>;
  static bool attr = false;
  constexpr size_t smem = C::smem();
  static_assert(smem <= 227 * 1024, "shared memory budget exceeded");
  if (!attr) {
    DGPP_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    attr = true;
  }
  dim3 grid(dgpp_ceil_div(p.N, kF4BM), dgpp_ceil_div(p.T, BN), splits);
  kern<<<grid, kF4Threads, smem, st>>>(tA, tB, p);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

}  // namespace dgpp

using namespace dgpp;

// Quantise T rows of bf16 activations into R residual NVFP4 terms (see act_quant_nvfp4_kernel).
DGPP_API int dgpp_act_quant_nvfp4(const void* x, int64_t x_stride, void* q, void* sf, void* g, int T, int T_pad,
                                  int K, int R, cudaStream_t st) {
  DGPP_REQUIRE(K % 16 == 0, "act_quant: K %d must be a multiple of 16", K);
  DGPP_REQUIRE(R >= 1 && R <= 4, "act_quant: R %d outside 1..4", R);
  if (T == 0) return 0;
  act_quant_nvfp4_kernel<<<dgpp_ceil_div(T * 32, 256), 256, 0, st>>>(
      static_cast<const bf16*>(x), x_stride, static_cast<uint8_t*>(q), static_cast<uint8_t*>(sf),
      static_cast<float*>(g), T, T_pad, K, R);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

// out[T, N] = alpha * g[t] * sum_r Wq . Xq_r^T.   xq: [R, T_pad, K/2], xsf: [R, T_pad, K/16], g: [T].
DGPP_API int dgpp_gemm_fp4(int bn, const void* xq, const void* xsf, const void* g, int R, int T_pad, const void* wq,
                           const void* wsf, float alpha, void* out, void* out32, const void* resid, int ldc, int T,
                           int N, int K, int splits, void* ws, void* counters, cudaStream_t st) {
  DGPP_REQUIRE(K % 256 == 0, "gemm_fp4: K %d must be a multiple of 256", K);
  DGPP_REQUIRE(R >= 1 && R <= 4, "gemm_fp4: R %d outside 1..4", R);
  DGPP_REQUIRE(splits >= 1, "gemm_fp4: splits must be >= 1");
  DGPP_REQUIRE(splits == 1 || (ws && counters), "gemm_fp4: split-K needs workspace and counters");
  DGPP_REQUIRE(out || out32, "gemm_fp4: no output");
  DGPP_REQUIRE(T_pad >= T, "gemm_fp4: T_pad < T");
  Fp4Params p;
  p.alpha = alpha;
  p.g = static_cast<const float*>(g);
  p.sfa = static_cast<const uint8_t*>(wsf);
  p.sfb = static_cast<const uint8_t*>(xsf);
  p.out = static_cast<bf16*>(out);
  p.out32 = static_cast<float*>(out32);
  p.resid = static_cast<const bf16*>(resid);
  p.ws = static_cast<float*>(ws);
  p.counters = static_cast<uint32_t*>(counters);
  p.status = device_status_ptr();
  p.T = T; p.T_pad = T_pad; p.N = N; p.K = K; p.ldc = ldc; p.R = R;
  const int stages = K / 256;
  const int per = dgpp_ceil_div(stages, splits);
  p.stages_per_split = per;
  splits = dgpp_ceil_div(stages, per);
  CUtensorMap tA, tB;
  if (make_tmap_2d(&tA, wq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, K / 2, N, K / 2, 128, kF4BM, CU_TENSOR_MAP_SWIZZLE_128B))
    return -1;
  if (make_tmap_2d(&tB, xq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, K / 2, static_cast<uint64_t>(R) * T_pad, K / 2, 128,
                   bn, CU_TENSOR_MAP_SWIZZLE_128B))
    return -1;
  if (R > 1) {
    DGPP_REQUIRE(bn <= 64, "gemm_fp4: residual terms need bn <= 64 (bn=%d)", bn);
    if (bn == 16) return launch_fp4<16, 4>(tA, tB, p, splits, st);
    if (bn == 32) return launch_fp4<32, 4>(tA, tB, p, splits, st);
    if (bn == 64) return launch_fp4<64, 4>(tA, tB, p, splits, st);
  } else {
    if (bn == 16) return launch_fp4<16, 1>(tA, tB, p, splits, st);
    if (bn == 32) return launch_fp4<32, 1>(tA, tB, p, splits, st);
    if (bn == 64) return launch_fp4<64, 1>(tA, tB, p, splits, st);
    if (bn == 128) return launch_fp4<128, 1>(tA, tB, p, splits, st);
    if (bn == 256) return launch_fp4<256, 1>(tA, tB, p, splits, st);
  }
  dgpp_set_error("gemm_fp4: unsupported bn %d", bn);
  return -1;
}
