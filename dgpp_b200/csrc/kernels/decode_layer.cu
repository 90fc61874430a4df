// One persistent kernel per decoder-layer boundary of the decode step (rows <= 16, NVFP4 weights).
//
// A decode step of a dense layer is four weight-streaming GEMMs of a few microseconds each, separated by row-wide
// operators (attention-output fold, add + RMSNorm, SwiGLU, RoPE + KV append) that each need the complete output of
// the GEMM before them.  Launched one by one, every one of these ~10 kernels pays its own launch, prologue, first
// HBM round trip and tail, and HBM idles in between.  Here ONE grid of (number of SMs) CTAs walks a list of
// phases; a grid-wide barrier (a monotonic counter in device memory, bounded waits) separates the phases, and the
// weight stream never stops:
//
//   warp 0   weight producer: TMA loads of packed e2m1 tiles + their scale atoms into a deep shared-memory ring.  It
//            never waits for a phase barrier (weights do not depend on activations), so while the other warps sit in
//            a barrier or in a row-wide phase, the ring already fills with the NEXT GEMM's tiles.
//   warp 1   MMA issuer: tcgen05.cp scale atoms -> TMEM, tcgen05.mma kind::mxf4nvf4 (block scale, ue4m3 / 16) into one
//            of two TMEM accumulators, so the read-out of tile i overlaps the main loop of tile i + 1.
//   warp 2   activation producer: after the phase barrier, TMA loads of the quantised activation rows + scale atoms.
//   warps 4-7 workers: GEMM read-out (fp32 split-K partials, or SwiGLU of a gate / up tile pair), and the row-wide
//            phases between GEMMs:
//              ROW A / ROW C  one CTA per (row, column segment): A folds split-K partials (and, tensor parallel,
//                    exchanges the bf16 partial slice with every peer through the symmetric region and folds ranks
//                    in ascending order), adds the residual and publishes partial row statistics -- or folds the
//                    split-KV attention partials, or takes plain rows; after a grid barrier C finishes the row
//                    operator (RMSNorm) and quantises the slice to three NVFP4 residual terms
//              UNITQ every CTA quantises 16-element groups of the SwiGLU output
//              ROPE  one warp per (row, head): fold the qkv partials, per-head RMSNorm, RoPE, FP8 KV append
//
// Arithmetic (rounding points, reduction orders) is that of the stand-alone kernels gemm_fp4_kernel,
// act_quant_cluster_kernel and rope_kv_kernel, so a step through this kernel reproduces theirs bit for bit when
// the split-K partition is the same.
// (reference counterpart of the step structure: src/engine/graph_engine.hpp:2269-2337 capture of one decode pass,
//  per-layer fold sites src/models/qwen/model35.cpp:1952-1960,2108-2116.)
#include <cuda.h>
#include <string.h>

#include "common/common.h"
#include "common/dtypes.cuh"
#include "common/ptx.cuh"
#include "kernels/comm.cuh"
#include "kernels/decode_layer.h"
#include "kernels/gemm_common.cuh"

namespace dgpp {

constexpr int kDlThreads = 256;
constexpr int kDlBN = 48;                 // MMA N: 16 token rows x 3 residual terms
constexpr int kDlBnTok = 16;
constexpr int kDlTerms = 3;
constexpr int kDlSA = 8;                  // weight ring stages
constexpr int kDlSB = 8;                  // activation ring stages
constexpr int kDlStageA = 128 * 128;      // 16 KB packed fp4 (128 weight rows x 256 K)
constexpr int kDlStageB = kDlBN * 128;    // 6 KB
constexpr int kDlSf = 4 * 512;            // scale atoms of one stage (4 K=64 steps)
constexpr int kDlRowBuf = 8192;           // one unit's slice of a bf16 row (up to 4096 elements)
constexpr int kTimeoutGridBarrier = 7;
static_assert(kDlSA == 8 && kDlSB == 8, "the ring loops index slots with & 7 and take the phase bit from >> 3");

struct DlMaps {
  CUtensorMap a[kDlMaxGemm];
  CUtensorMap b[kDlMaxAct];
};

struct DlGemm {
  const uint8_t* sfa;
  float alpha;
  int N, K, tiles, splits, per, act, pair;
};
struct DlAct {
  uint8_t* q;
  uint8_t* sf;
  float* g;
  int K;
};
struct DlRowq {
  int mode, src_gemm, out_act, tp_fold, cl;
  const bf16* in;
  int64_t in_stride;
  const bf16* norm_w;
  bf16* x_out;
};

struct DlParams {
  int rows, nphase;
  int ph_type[kDlMaxPhase], ph_idx[kDlMaxPhase];
  DlGemm gemm[kDlMaxGemm];
  DlAct act[kDlMaxAct];
  DlRowq rowq[kDlMaxRowq];
  bf16* x;
  int H;
  float eps, limit;
  int one_plus_w;
  float* ws;
  bf16* hbuf;
  float* amax_part;
  float* stats;              // [16 rows][8 segments][2]: partial sum of squares, partial maximum of the row phases
  int unitq_act, inter;
  const float* part_ml;
  const float* part_acc;
  int att_splits, hq, d;
  // rope / KV append
  int rope_gemm;
  bf16* qkv;
  const int32_t* positions;
  const int32_t* row_req;
  const int32_t* block_table;
  const float* inv_freq;
  const bf16* q_norm_w;
  const bf16* k_norm_w;
  uint8_t* k_cache;
  uint8_t* v_cache;
  float* k_scale;
  float* v_scale;
  int hkv, rot_dim, page, max_blocks, kv_fp8;
  float mscale;
  int tp, tp_folds;
  CommState comm;
  unsigned long long* trace; // debug: %globaltimer stamps of CTA 0 and of the last CTA (see dgpp_decode_layer_set_trace)
  unsigned long long* ctl;   // [0] arrivals of the grid barrier (monotonic), [1] its value when this launch began
  DeviceStatus* status;
};

__device__ __forceinline__ unsigned long long ld_acquire_gpu_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void fence_proxy_async_global() {
  asm volatile("fence.proxy.async.global;" ::: "memory");
}
__device__ __forceinline__ void bar_workers() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// Wait until the barrier counter reaches `target`; gives up after ~2 s or as soon as another kernel instance
// reported a failure (then the whole grid unwinds within one poll interval instead of one time-out per phase).
__device__ __forceinline__ bool grid_wait(const unsigned long long* ctr, unsigned long long target,
                                          const DeviceStatus* st) {
  for (int i = 0; i < 2048; ++i)
    if (ld_acquire_gpu_u64(ctr) >= target) return true;
  const long long t0 = clock64();
  for (;;) {
    for (int i = 0; i < 256; ++i) {
      if (ld_acquire_gpu_u64(ctr) >= target) return true;
      __nanosleep(32);
    }
    if (*reinterpret_cast<const volatile int*>(&st->code) != 0) return false;
    if (clock64() - t0 > 4000000000ll) return false;
  }
}

__device__ __forceinline__ float dl_warp_red(float v, bool is_max) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float u = __shfl_xor_sync(0xffffffffu, v, o);
    v = is_max ? fmaxf(v, u) : v + u;
  }
  return v;
}

// Quantise one 16-element group (values already divided by the row scale) into the three residual terms of token
// row m and store codes + block scales in the layout the GEMM's activation loads expect (one token tile of 16).
__device__ __forceinline__ void dl_quant_group(float* res, const DlAct& a, int m, int gi) {
  const int st = gi >> 4, step = (gi >> 2) & 3, fi = gi & 3;
#pragma unroll
  for (int r = 0; r < kDlTerms; ++r) {
    float bm = 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) bm = fmaxf(bm, fabsf(res[j]));
    const uint8_t sb = f32_to_e4m3(bm * (1.f / 6.f));
    const float s = e4m3_value_f32(bm * (1.f / 6.f));
    const float inv_s = s > 0.f ? 1.f / s : 0.f;
    float sc[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) sc[j] = res[j] * inv_s;
    const uint32_t w0 = f32x8_to_e2m1x8(sc), w1 = f32x8_to_e2m1x8(sc + 8);
    e2m1x8_residual(w0, s, res);
    e2m1x8_residual(w1, s, res + 8);
    const int brow = r * kDlBnTok + m;
    *reinterpret_cast<uint2*>(a.q + static_cast<size_t>(brow) * (a.K / 2) + gi * 8) = make_uint2(w0, w1);
    a.sf[static_cast<size_t>(st * 4 + step) * 512 + (brow & 31) * 16 + (brow >> 5) * 4 + fi] = sb;
  }
}

// ---- the same mbarrier / TMA / commit operations on 32-bit shared-window addresses (no generic -> shared
// conversion per call; the single-thread producer and MMA loops are issue-bound)
__device__ __forceinline__ bool mbar_try_wait_a(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred P;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t}\n"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded (~2 s) wait; false on expiry.
__device__ __forceinline__ bool wait_bar_a(uint32_t bar, uint32_t parity) {
  if (mbar_try_wait_a(bar, parity)) return true;
  for (int i = 0; i < 4096; ++i)
    if (mbar_try_wait_a(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
    for (int i = 0; i < 2048; ++i)
      if (mbar_try_wait_a(bar, parity)) return true;
    if (clock64() - t0 > 4000000000ll) return false;
  }
}
__device__ __forceinline__ void mbar_expect_tx_a(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tma_load_2d_a(uint32_t dst, const CUtensorMap* m, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void bulk_load_1d_a(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void umma_commit_a(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__global__ void __launch_bounds__(kDlThreads, 1)
decode_layer_kernel(const __grid_constant__ DlMaps maps, const __grid_constant__ DlParams p) {
  extern __shared__ __align__(1024) unsigned char smem_dyn[];
  unsigned char* sp = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  unsigned char* sA = sp;    sp += kDlSA * kDlStageA;
  unsigned char* sB = sp;    sp += kDlSB * kDlStageB;
  unsigned char* sSfa = sp;  sp += kDlSA * kDlSf;
  unsigned char* sSfb = sp;  sp += kDlSB * kDlSf;
  bf16* row_s = reinterpret_cast<bf16*>(sp);  sp += kDlRowBuf;
  float* wred = reinterpret_cast<float*>(sp);  sp += 8 * 4 * sizeof(float);     // [segment][worker warp]
  float* rowv = reinterpret_cast<float*>(sp);  sp += 256 * sizeof(float);       // per-row scratch: [0..15] row scales, [16..31] 1 / rms, rest reductions
  uint64_t* fullA = reinterpret_cast<uint64_t*>(sp);
  uint64_t* emptyA = fullA + kDlSA;
  uint64_t* fullB = emptyA + kDlSA;
  uint64_t* emptyB = fullB + kDlSB;
  uint64_t* accF = emptyB + kDlSB;
  uint64_t* accE = accF + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accE + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* live_s = abort_flag + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr uint32_t kTmemCols = 256;   // 2 accumulators x 64 + 2 x 16 weight scales + 2 x 16 activation scales
  if (threadIdx.x == 0) {
    for (int i = 0; i < kDlSA; ++i) { mbar_init(&fullA[i], 1); mbar_init(&emptyA[i], 1); }
    for (int i = 0; i < kDlSB; ++i) { mbar_init(&fullB[i], 1); mbar_init(&emptyB[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&accF[i], 1); mbar_init(&accE[i], 4); }
    *abort_flag = 0;
    *live_s = 1;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_sfa = tmem_base + 128;
  const uint32_t tmem_sfb = tmem_sfa + 32;
  const int G = gridDim.x;

  // shared-memory addresses as 32-bit window offsets (the single-thread loops below are issue-bound: no generic ->
  // shared conversions, divisions or parameter-space indexing inside them)
  const uint32_t aA = smem_u32(sA), aB = smem_u32(sB), aSfa = smem_u32(sSfa), aSfb = smem_u32(sSfb);
  const uint32_t bFullA = smem_u32(fullA), bEmptyA = smem_u32(emptyA), bFullB = smem_u32(fullB), bEmptyB = smem_u32(emptyB);

  if (warp == 0) {
    // ---------------------------------------------------------------- weight producer (never waits for a phase)
    if (elect_one()) {
      for (int i = 0; i < kDlMaxGemm; ++i)
        if (p.gemm[i].N > 0) tma_prefetch_desc(&maps.a[i]);
      uint32_t ga = 0;
      bool ok = true;
      // one weight stage: ring slot ga % 8, tile rows y.. of the stage-tiled matrix + its 2 KB of scale atoms
      auto issue = [&](const CUtensorMap* tm, int y, const uint8_t* sf) {
        const uint32_t s = ga & (kDlSA - 1);
        if (!wait_bar_a(bEmptyA + s * 8, ((ga >> 3) & 1) ^ 1)) { ok = false; return; }
        const uint32_t bar = bFullA + s * 8;
        mbar_expect_tx_a(bar, kDlStageA + kDlSf);
        tma_load_2d_a(aA + s * kDlStageA, tm, 0, y, bar);
        bulk_load_1d_a(aSfa + s * kDlSf, sf, kDlSf, bar);
        ++ga;
      };
      for (int ph = 0; ph < p.nphase && ok; ++ph) {
        if (p.ph_type[ph] != kDlPhGemm) continue;
        const int gi = p.ph_idx[ph];
        const CUtensorMap* tm = &maps.a[gi];
        const uint8_t* sfa = p.gemm[gi].sfa;
        const int tiles = p.gemm[gi].tiles, per = p.gemm[gi].per, pair = p.gemm[gi].pair;
        const int total = p.gemm[gi].K >> 8, items = tiles * p.gemm[gi].splits;
        for (int item = blockIdx.x; item < items && ok; item += G) {
          const int tile = item % tiles, split = item / tiles;
          const int st0 = split * per, st1 = min(total, st0 + per);
          int t0 = tile * total + st0, t1 = (tile + tiles) * total + st0;      // stage index in the tiled matrix: gate / up
          for (int st = st0; st < st1 && ok; ++st, ++t0, ++t1) {
            issue(tm, t0 * 128, sfa + static_cast<size_t>(t0) * kDlSf);
            if (pair && ok) issue(tm, t1 * 128, sfa + static_cast<size_t>(t1) * kDlSf);
          }
        }
      }
      if (!ok) {
        if (!*abort_flag) { report(p.status, kTimeoutStageEmpty, 100); *abort_flag = 1; }
        // unwinding: let the copies still in flight land before the CTA's shared memory is given back
        for (uint32_t k = ga > static_cast<uint32_t>(kDlSA) ? ga - kDlSA : 0; k < ga; ++k)
          wait_bar(&fullA[k % kDlSA], (k / kDlSA) & 1);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc_fp4bs(128, kDlBN, 0u);
      // descriptors are linear in the shared-memory address (14-bit field of 16-byte units): base + offset >> 4
      const uint64_t dA0 = umma_desc_sw128(aA), dB0 = umma_desc_sw128(aB);
      const uint64_t dSfa0 = umma_desc_nosw(aSfa, 0, 128), dSfb0 = umma_desc_nosw(aSfb, 0, 128);
      uint32_t ga = 0, gb = 0, acc_i = 0;
      bool ok = true;
      // one weight stage: scale atoms -> TMEM, four K=64 MMAs into accumulator `d_tmem`; with_b: the activation stage's
      // scale atoms are copied too (the second tile of a gate / up pair reuses the ones already in TMEM)
      auto stage = [&](uint32_t d_tmem, uint32_t sa, uint32_t sb, bool with_b, bool first) {
        const uint32_t t_sfa = tmem_sfa + (ga & 1) * 16, t_sfb = tmem_sfb + (gb & 1) * 16;
        const uint64_t dsa = dSfa0 + sa * (kDlSf >> 4), dsb = dSfb0 + sb * (kDlSf >> 4);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          tmem_cp_32x128b_warpx4(t_sfa + 4 * j, dsa + j * (512 >> 4));
          if (with_b) tmem_cp_32x128b_warpx4(t_sfb + 4 * j, dsb + j * (512 >> 4));
        }
        const uint64_t da = dA0 + sa * (kDlStageA >> 4), db = dB0 + sb * (kDlStageB >> 4);
#pragma unroll
        for (int j = 0; j < 4; ++j)
          umma_nvfp4(d_tmem, da + j * 2, db + j * 2, idesc, t_sfa + 4 * j, t_sfb + 4 * j, (!first || j > 0) ? 1u : 0u);
      };
      for (int ph = 0; ph < p.nphase && ok; ++ph) {
        if (p.ph_type[ph] != kDlPhGemm) continue;
        const int gi = p.ph_idx[ph];
        const int tiles = p.gemm[gi].tiles, per = p.gemm[gi].per, pair = p.gemm[gi].pair;
        const int total = p.gemm[gi].K >> 8, items = tiles * p.gemm[gi].splits;
        for (int item = blockIdx.x; item < items && ok; item += G) {
          const int split = item / tiles;
          const int st0 = split * per, st1 = min(total, st0 + per);
          const int nacc = pair ? 2 : 1;
          for (int h = 0; h < nacc && ok; ++h) {
            const uint32_t ai = acc_i + h;
            ok = wait_bar(&accE[ai & 1], ((ai >> 1) & 1) ^ 1);
          }
          if (!ok) break;
          tc_fence_after();
          const uint32_t d0 = tmem_base + (acc_i & 1) * 64, d1 = tmem_base + ((acc_i + 1) & 1) * 64;
          for (int st = st0; st < st1; ++st) {
            const uint32_t sa = ga & (kDlSA - 1), sb = gb & (kDlSB - 1);
            if (!wait_bar_a(bFullA + sa * 8, (ga >> 3) & 1) || !wait_bar_a(bFullB + sb * 8, (gb >> 3) & 1)) { ok = false; break; }
            tc_fence_after();
            stage(d0, sa, sb, true, st == st0);
            umma_commit_a(bEmptyA + sa * 8);
            ++ga;
            if (pair) {
              const uint32_t sa2 = ga & (kDlSA - 1);
              if (!wait_bar_a(bFullA + sa2 * 8, (ga >> 3) & 1)) { ok = false; break; }
              tc_fence_after();
              stage(d1, sa2, sb, false, st == st0);
              umma_commit_a(bEmptyA + sa2 * 8);
              ++ga;
            }
            umma_commit_a(bEmptyB + sb * 8);
            ++gb;
          }
          if (ok) {
            umma_commit(&accF[acc_i & 1]);
            if (pair) umma_commit(&accF[(acc_i + 1) & 1]);
          }
          acc_i += nacc;
        }
      }
      if (!ok && !*abort_flag) { report(p.status, kTimeoutTmaFull, 300); *abort_flag = 1; }
    }
    __syncwarp();
  } else if (warp == 2) {
    // ---------------------------------------------------------------- activation producer
    if (elect_one()) {
      pdl_wait();
      for (int i = 0; i < kDlMaxAct; ++i)
        if (p.act[i].K > 0) tma_prefetch_desc(&maps.b[i]);
      const unsigned long long base = __ldcg(p.ctl + 1);
      uint32_t gb = 0;
      bool ok = true;
      for (int ph = 0; ph < p.nphase && ok; ++ph) {
        if (p.ph_type[ph] != kDlPhGemm) continue;
        const int gi = p.ph_idx[ph];
        const int ai = p.gemm[gi].act;
        const CUtensorMap* tm = &maps.b[ai];
        const uint8_t* sfb = p.act[ai].sf;
        const int tiles = p.gemm[gi].tiles, per = p.gemm[gi].per;
        const int total = p.gemm[gi].K >> 8, items = tiles * p.gemm[gi].splits;
        if (ph > 0 && !grid_wait(p.ctl, base + static_cast<unsigned long long>(ph) * G, p.status)) {
          if (!*abort_flag) { report(p.status, kTimeoutGridBarrier, 400 + ph); *abort_flag = 1; }
          ok = false;
          break;
        }
        fence_proxy_async_global();   // the rows were written with ordinary stores by other CTAs; TMA reads them
        for (int item = blockIdx.x; item < items && ok; item += G) {
          const int split = item / tiles;
          const int st0 = split * per, st1 = min(total, st0 + per);
          for (int st = st0; st < st1; ++st, ++gb) {     // (a gate / up pair shares each activation stage)
            const uint32_t s = gb & (kDlSB - 1);
            if (!wait_bar_a(bEmptyB + s * 8, ((gb >> 3) & 1) ^ 1)) { ok = false; break; }
            const uint32_t bar = bFullB + s * 8;
            mbar_expect_tx_a(bar, kDlStageB + kDlSf);
            tma_load_2d_a(aB + s * kDlStageB, tm, st * 128, 0, bar);
            bulk_load_1d_a(aSfb + s * kDlSf, sfb + static_cast<size_t>(st) * kDlSf, kDlSf, bar);
          }
        }
      }
      if (!ok) {
        if (!*abort_flag) { report(p.status, kTimeoutStageEmpty, 500); *abort_flag = 1; }
        for (uint32_t k = gb > static_cast<uint32_t>(kDlSB) ? gb - kDlSB : 0; k < gb; ++k)
          wait_bar(&fullB[k % kDlSB], (k / kDlSB) & 1);
      }
    }
    __syncwarp();
  } else if (warp >= 4) {
    // ---------------------------------------------------------------- workers
    const int wtid = threadIdx.x - 128, q = warp & 3;
    const int tr_sel = blockIdx.x == 0 ? 0 : (static_cast<int>(blockIdx.x) == G - 1 ? 1 : -1);
    auto stamp = [&](int slot) {
      if (p.trace != nullptr && tr_sel >= 0 && wtid == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t) :: "memory");
        p.trace[tr_sel * 32 + slot] = t;
      }
    };
    stamp(30);
    pdl_wait();
    stamp(31);
    const unsigned long long base = __ldcg(p.ctl + 1);
    const uint32_t epoch0 = p.tp ? __ldcg(p.comm.epoch) : 0u;
    uint32_t acc_i = 0;
    int tp_seq = 0;
    const int rows = p.rows;
    for (int ph = 0; ph < p.nphase; ++ph) {
      // every CTA passes barrier ph - 1 before it arrives for phase ph (keeps the monotonic counter unambiguous)
      if (wtid == 0) {
        if (ph > 0 && !*abort_flag && !grid_wait(p.ctl, base + static_cast<unsigned long long>(ph) * G, p.status)) {
          if (!*abort_flag) { report(p.status, kTimeoutGridBarrier, 600 + ph); *abort_flag = 1; }
        }
        *live_s = *abort_flag ? 0 : 1;
      }
      bar_workers();
      stamp(2 * ph);
      const bool live = *live_s != 0;
      const int type = p.ph_type[ph], idx = p.ph_idx[ph];
      bool wrote_act = false;
      if (type == kDlPhGemm) {
        const DlGemm& g = p.gemm[idx];
        const int items = g.tiles * g.splits;
        const float* gvec = p.act[g.act].g;
        for (int item = blockIdx.x; item < items; item += G) {
          const int tile = item % g.tiles, split = item / g.tiles;
          bool good = live;
          // ---- read-out
          float v[2][16];
          for (int half = 0; half < (g.pair ? 2 : 1); ++half, ++acc_i) {
            const uint32_t buf = acc_i & 1;
            bool ok = good && !*abort_flag && wait_bar(&accF[buf], (acc_i >> 1) & 1);
            ok = __all_sync(0xffffffffu, ok);
            if (good && !ok && lane == 0 && !*abort_flag) { report(p.status, kTimeoutAccum, 700 + ph); *abort_flag = 1; }
            good = good && ok;
#pragma unroll
            for (int j = 0; j < 16; ++j) v[half][j] = 0.f;
            if (good) {
              tc_fence_after();
#pragma unroll
              for (int r = 0; r < kDlTerms; ++r) {
                uint32_t rr[16];
                tmem_ld_x16(tmem_base + buf * 64 + (static_cast<uint32_t>(q * 32) << 16) + r * kDlBnTok, rr);
#pragma unroll
                for (int j = 0; j < 16; ++j) v[half][j] += __uint_as_float(rr[j]);
              }
              tc_fence_before();
              __syncwarp();
              if (lane == 0) mbar_arrive(&accE[buf]);
            }
          }
          if (!g.pair) {
            const int n = tile * 128 + q * 32 + lane;
            if (good && n < g.N) {
#pragma unroll
              for (int m = 0; m < 16; ++m)
                if (m < rows) __stcg(p.ws + (static_cast<size_t>(split) * 16 + m) * g.N + n, v[0][m]);
            }
          } else {
            // gate tile in v[0], up tile in v[1]: h = bf16(bf16(silu(gate)) * up), per-row max |h| of this tile pair
            const int n = tile * 128 + q * 32 + lane;
            const int I = g.N / 2;
#pragma unroll
            for (int m = 0; m < 16; ++m) {
              float am = 0.f;
              if (m < rows) {
                if (good && n < I) {
                  const float gsc = __ldcg(gvec + m);
                  float gv = bf16_to_f32(f32_to_bf16(v[0][m] * g.alpha * gsc));
                  float uv = bf16_to_f32(f32_to_bf16(v[1][m] * g.alpha * gsc));
                  if (p.limit > 0.f) { gv = fminf(gv, p.limit); uv = fminf(fmaxf(uv, -p.limit), p.limit); }
                  const float sl = bf16_to_f32(f32_to_bf16(gv / (1.f + __expf(-gv))));
                  const bf16 h = f32_to_bf16(sl * uv);
                  p.hbuf[static_cast<size_t>(m) * I + n] = h;
                  am = fabsf(bf16_to_f32(h));
                }
                am = dl_warp_red(am, true);
                if (lane == 0) rowv[32 + q * 8 + (m & 7)] = am;
              }
              if ((m & 7) == 7 || m == 15) {
                // rows m - 7 .. m of the four warps are in rowv[32..63]: publish them, then reuse the slots
                bar_workers();
                const int mb = m & ~7;
                if (wtid < 8 && mb + wtid < rows)
                  p.amax_part[static_cast<size_t>(tile) * 16 + mb + wtid] =
                      fmaxf(fmaxf(rowv[32 + wtid], rowv[40 + wtid]), fmaxf(rowv[48 + wtid], rowv[56 + wtid]));
                bar_workers();
              }
            }
          }
        }
      } else if (type == kDlPhRowA || type == kDlPhRowC) {
        // Row-wide operators run as (row, column segment) units, one per CTA (taken from the end of the grid: those
        // CTAs have the fewest GEMM items).  Step A produces the unit's slice of the bf16 row in shared memory and
        // publishes its partial row statistics; step C (after a grid barrier, same CTA, slice still in shared
        // memory) reads the row's statistics, finishes the row operator and quantises the slice.
        const DlRowq& R = p.rowq[idx];
        const DlAct* oa = R.out_act >= 0 ? &p.act[R.out_act] : nullptr;
        const int K = R.mode == 3 ? p.hq * p.d : (R.mode == 2 ? p.H : oa->K);
        const int cl = R.cl, kseg = K / cl, nvec = kseg / 8;
        const int u = G - 1 - static_cast<int>(blockIdx.x);
        const bool mine = live && u >= 0 && u < rows * cl;
        const int m = mine ? u / cl : 0, c = mine ? u % cl : 0;
        const int col0 = c * kseg;
        if (type == kDlPhRowA) {
          float ss = 0.f, pm = 0.f;
          if (R.mode == 2) {
            const DlGemm* sg = R.src_gemm >= 0 ? &p.gemm[R.src_gemm] : nullptr;
            const float sc_g = (mine && sg) ? __ldcg(p.act[sg->act].g + m) : 0.f;
            const bool tpf = R.tp_fold && p.tp;
            const uint32_t epoch = epoch0 + 1 + tp_seq;
            const int parity = epoch & 1;
            if (tpf) ++tp_seq;
            bool flags_ok = true;
            if (tpf) {
              // push this rank's bf16 partial slice into slot `rank` of every rank, then raise the unit's flag everywhere
              if (mine) {
                for (int i = wtid; i < nvec; i += 128) {
                  const int col = col0 + i * 8;
                  float acc[8];
#pragma unroll
                  for (int j = 0; j < 8; ++j) acc[j] = 0.f;
                  for (int sp2 = 0; sp2 < sg->splits; ++sp2) {
                    const float4* w4 = reinterpret_cast<const float4*>(p.ws + (static_cast<size_t>(sp2) * 16 + m) * sg->N + col);
                    const float4 a0 = __ldcg(w4), a1 = __ldcg(w4 + 1);
                    acc[0] += a0.x; acc[1] += a0.y; acc[2] += a0.z; acc[3] += a0.w;
                    acc[4] += a1.x; acc[5] += a1.y; acc[6] += a1.z; acc[7] += a1.w;
                  }
                  Pack16 d;
#pragma unroll
                  for (int j = 0; j < 8; ++j) d.h[j] = f32_to_bf16(acc[j] * sg->alpha * sc_g);
                  for (int r = 0; r < p.comm.world; ++r) {
                    const int dst = (p.comm.rank + r) % p.comm.world;
                    st_v4_global(payload(p.comm, dst, parity, p.comm.rank) + (static_cast<size_t>(m) * K + col) * 2, d.u);
                  }
                }
                __threadfence_system();
              }
              bar_workers();
              if (mine && wtid < p.comm.world) {
                st_release_sys(flag(p.comm, wtid, parity, p.comm.rank, u), epoch);
                if (!wait_flag(flag(p.comm, p.comm.rank, parity, wtid, u), epoch)) {
                  if (atomicCAS(&p.status->code, 0, kTimeoutPeerFlag) == 0) p.status->detail = wtid;
                  atomicAdd(&p.status->count, 1);
                  *abort_flag = 1;
                }
              }
              bar_workers();
              flags_ok = !*abort_flag;
            }
            if (mine && flags_ok) {
              const bf16* xr = p.x + static_cast<size_t>(m) * K;
              for (int i = wtid; i < nvec; i += 128) {
                const int col = col0 + i * 8;
                Pack16 x, wv;
                x.u = __ldcg(reinterpret_cast<const uint4*>(xr + col));
                wv.u = *reinterpret_cast<const uint4*>(R.norm_w + col);
                if (tpf) {
                  float acc[8];
#pragma unroll
                  for (int j = 0; j < 8; ++j) acc[j] = 0.f;
                  for (int r = 0; r < p.comm.world; ++r) {
                    Pack16 d;
                    d.u = ld_v4_global_volatile(payload(p.comm, p.comm.rank, parity, r) + (static_cast<size_t>(m) * K + col) * 2);
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[j] += bf16_to_f32(d.h[j]);
                  }
#pragma unroll
                  for (int j = 0; j < 8; ++j) x.h[j] = f32_to_bf16(bf16_to_f32(x.h[j]) + bf16_to_f32(f32_to_bf16(acc[j])));
                  *reinterpret_cast<uint4*>(p.x + static_cast<size_t>(m) * K + col) = x.u;
                } else if (sg) {
                  float acc[8];
#pragma unroll
                  for (int j = 0; j < 8; ++j) acc[j] = 0.f;
                  for (int sp2 = 0; sp2 < sg->splits; ++sp2) {
                    const float4* w4 = reinterpret_cast<const float4*>(p.ws + (static_cast<size_t>(sp2) * 16 + m) * sg->N + col);
                    const float4 a0 = __ldcg(w4), a1 = __ldcg(w4 + 1);
                    acc[0] += a0.x; acc[1] += a0.y; acc[2] += a0.z; acc[3] += a0.w;
                    acc[4] += a1.x; acc[5] += a1.y; acc[6] += a1.z; acc[7] += a1.w;
                  }
#pragma unroll
                  for (int j = 0; j < 8; ++j)
                    x.h[j] = f32_to_bf16(bf16_to_f32(x.h[j]) + bf16_to_f32(f32_to_bf16(acc[j] * sg->alpha * sc_g)));
                  *reinterpret_cast<uint4*>(p.x + static_cast<size_t>(m) * K + col) = x.u;
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  const float f = bf16_to_f32(x.h[j]);
                  ss += f * f;
                  float gw = bf16_to_f32(wv.h[j]);
                  if (p.one_plus_w) gw += 1.f;
                  pm = fmaxf(pm, fabsf(f * gw));
                }
                *reinterpret_cast<uint4*>(row_s + i * 8) = x.u;
              }
            }
          } else if (R.mode == 3) {
            if (mine) {
              const int D = p.d, S = p.att_splits;
              for (int i = wtid; i < nvec; i += 128) {
                const int col = col0 + i * 8, h = col / D, d0 = col % D;
                const size_t rh = static_cast<size_t>(m) * p.hq + h;
                // all (max, sum) pairs and accumulator slices of the splits are requested before any is used
                const float2* mlp = reinterpret_cast<const float2*>(p.part_ml) + rh * S;
                const float* accp = p.part_acc + rh * S * D + d0;
                float mm = -INFINITY, ll = 0.f, acc[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[j] = 0.f;
                for (int s0 = 0; s0 < S; s0 += 4) {
                  float2 ml[4];
                  float4 pv[4][2];
#pragma unroll
                  for (int t = 0; t < 4; ++t) {
                    const bool on = s0 + t < S;
                    ml[t] = on ? __ldcg(mlp + s0 + t) : make_float2(-INFINITY, 0.f);
                    const float4* pa = reinterpret_cast<const float4*>(accp + static_cast<size_t>(s0 + t) * D);
                    pv[t][0] = on ? __ldcg(pa) : make_float4(0.f, 0.f, 0.f, 0.f);
                    pv[t][1] = on ? __ldcg(pa + 1) : make_float4(0.f, 0.f, 0.f, 0.f);
                  }
                  if (s0 == 0) {
                    // the row maximum over ALL splits comes first (same arithmetic as the stand-alone combine)
                    for (int s2 = 0; s2 < S; ++s2) mm = fmaxf(mm, s2 < 4 ? ml[s2 & 3].x : __ldcg(mlp + s2).x);
                  }
#pragma unroll
                  for (int t = 0; t < 4; ++t) {
                    if (s0 + t >= S) break;
                    const float ms = ml[t].x;
                    const float cw = ms == -INFINITY ? 0.f : __expf(ms - mm);
                    ll += ml[t].y * cw;
                    acc[0] += pv[t][0].x * cw; acc[1] += pv[t][0].y * cw; acc[2] += pv[t][0].z * cw; acc[3] += pv[t][0].w * cw;
                    acc[4] += pv[t][1].x * cw; acc[5] += pv[t][1].y * cw; acc[6] += pv[t][1].z * cw; acc[7] += pv[t][1].w * cw;
                  }
                }
                Pack16 x;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  x.h[j] = f32_to_bf16(ll > 0.f ? acc[j] / ll : 0.f);
                  pm = fmaxf(pm, fabsf(bf16_to_f32(x.h[j])));
                }
                *reinterpret_cast<uint4*>(row_s + i * 8) = x.u;
                if (R.x_out) *reinterpret_cast<uint4*>(R.x_out + static_cast<size_t>(m) * K + col) = x.u;
              }
            }
          } else {
            if (mine) {
              const bf16* rr = R.in + static_cast<size_t>(m) * R.in_stride + col0;
              for (int i = wtid; i < nvec; i += 128) {
                Pack16 x;
                x.u = __ldcg(reinterpret_cast<const uint4*>(rr + i * 8));
#pragma unroll
                for (int j = 0; j < 8; ++j) pm = fmaxf(pm, fabsf(bf16_to_f32(x.h[j])));
                *reinterpret_cast<uint4*>(row_s + i * 8) = x.u;
                if (R.x_out) *reinterpret_cast<uint4*>(R.x_out + static_cast<size_t>(m) * K + col0 + i * 8) = x.u;
              }
            }
          }
          // the unit's partial statistics (same warp / CTA reduction order as the cluster quantiser)
          ss = dl_warp_red(ss, false);
          pm = dl_warp_red(pm, true);
          if (lane == 0) { wred[q] = ss; wred[4 + q] = pm; }
          bar_workers();
          if (mine && wtid == 0) {
            float r = wred[0];
            for (int i = 1; i < 4; ++i) r += wred[i];
            p.stats[(m * 8 + c) * 2] = r;
            p.stats[(m * 8 + c) * 2 + 1] = fmaxf(fmaxf(wred[4], wred[5]), fmaxf(wred[6], wred[7]));
          }
        } else {
          float amax = 0.f;
          if (mine) {
            float tot = 0.f, pmx = 0.f;
            for (int i = 0; i < cl; ++i) {
              tot += __ldcg(p.stats + (m * 8 + i) * 2);
              pmx = fmaxf(pmx, __ldcg(p.stats + (m * 8 + i) * 2 + 1));
            }
            amax = pmx;
            if (R.mode == 2) {
              const float rstd = rsqrtf(tot / static_cast<float>(K) + p.eps);
              amax = pmx * rstd * 1.0079f;      // bound on the normalised row's maximum (see act_quant_cluster_kernel)
              for (int i = wtid; i < nvec; i += 128) {
                Pack16 x, ww;
                x.u = *reinterpret_cast<const uint4*>(row_s + i * 8);
                ww.u = *reinterpret_cast<const uint4*>(R.norm_w + col0 + i * 8);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  const float nrm = bf16_to_f32(f32_to_bf16(bf16_to_f32(x.h[j]) * rstd));
                  float gw = bf16_to_f32(ww.h[j]);
                  if (p.one_plus_w) gw += 1.f;
                  x.h[j] = f32_to_bf16(nrm * gw);
                }
                *reinterpret_cast<uint4*>(row_s + i * 8) = x.u;
                if (R.x_out) *reinterpret_cast<uint4*>(R.x_out + static_cast<size_t>(m) * K + col0 + i * 8) = x.u;
              }
            }
          }
          bar_workers();      // the finished slice is complete in shared memory
          if (mine && oa) {
            const float gs = amax > 0.f ? amax / (6.f * 256.f) : 1.f;
            if (c == 0 && wtid == 0) oa->g[m] = gs;
            const float inv_g = 1.f / gs;
            for (int gl = wtid; gl < kseg / 16; gl += 128) {
              Pack16 lo, hi;
              lo.u = *reinterpret_cast<const uint4*>(row_s + gl * 16);
              hi.u = *reinterpret_cast<const uint4*>(row_s + gl * 16 + 8);
              float res[16];
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                res[j] = bf16_to_f32(lo.h[j]) * inv_g;
                res[8 + j] = bf16_to_f32(hi.h[j]) * inv_g;
              }
              dl_quant_group(res, *oa, m, col0 / 16 + gl);
            }
            wrote_act = true;
          }
        }
      } else if (type == kDlPhUnitq) {
        const DlAct& oa = p.act[p.unitq_act];
        const int I = p.inter, pairs = I / 128, groups = I / 16;
        // row scales: max over the tile pairs' partial maxima (thread t owns row t % 16 of parts t, t + 128, ...)
        float am = 0.f;
        if (live && (wtid & 15) < rows) {
#pragma unroll 8
          for (int e = wtid; e < pairs * 16; e += 128) am = fmaxf(am, __ldcg(p.amax_part + e));
        }
        rowv[64 + wtid] = am;
        bar_workers();
        if (wtid < 16) {
          float a = 0.f;
          for (int j = 0; j < 8; ++j) a = fmaxf(a, rowv[64 + wtid + 16 * j]);
          rowv[wtid] = a > 0.f ? a / (6.f * 256.f) : 1.f;
        }
        bar_workers();
        if (live) {
          if (blockIdx.x == 0 && wtid < rows) oa.g[wtid] = rowv[wtid];
          const int total = rows * groups;
          for (int u = blockIdx.x * 128 + wtid; u < total; u += G * 128) {
            const int m = u / groups, gi = u % groups;
            Pack16 lo, hi;
            const uint4* src = reinterpret_cast<const uint4*>(p.hbuf + static_cast<size_t>(m) * I + gi * 16);
            lo.u = __ldcg(src);
            hi.u = __ldcg(src + 1);
            const float inv_g = 1.f / rowv[m];
            float res[16];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              res[j] = bf16_to_f32(lo.h[j]) * inv_g;
              res[8 + j] = bf16_to_f32(hi.h[j]) * inv_g;
            }
            dl_quant_group(res, oa, m, gi);
          }
          wrote_act = true;
        }
        bar_workers();
      } else if (type == kDlPhRope) {
        const DlGemm& sg = p.gemm[p.rope_gemm];
        const int heads = p.hq + 2 * p.hkv;
        constexpr int D = 128, PER = 4;
        if (live) {
          for (int u = blockIdx.x * 4 + q; u < rows * heads; u += G * 4) {
            const int row = u / heads, head = u % heads;
            // the cache slot's address chain (position -> request -> block) is in flight while the head is computed
            const int pos = p.positions[row];
            const int req = p.row_req[row];
            const int blk = p.block_table[static_cast<size_t>(req) * p.max_blocks + pos / p.page];
            const float sc_g = __ldcg(p.act[sg.act].g + row);
            float v[PER];
#pragma unroll
            for (int j = 0; j < PER; ++j) {
              const int n = head * D + lane + 32 * j;
              float acc = 0.f;
              for (int s = 0; s < sg.splits; ++s) acc += __ldcg(p.ws + (static_cast<size_t>(s) * 16 + row) * sg.N + n);
              v[j] = bf16_to_f32(f32_to_bf16(acc * sg.alpha * sc_g));
            }
            bf16* dstq = p.qkv + static_cast<size_t>(row) * heads * D + static_cast<size_t>(head) * D;
            const bool is_q = head < p.hq;
            const bool is_k = !is_q && head < p.hq + p.hkv;
            const bf16* nw = is_q ? p.q_norm_w : (is_k ? p.k_norm_w : nullptr);
            if (nw) {
              float ss = 0.f;
#pragma unroll
              for (int j = 0; j < PER; ++j) ss += v[j] * v[j];
#pragma unroll
              for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
              const float rstd = rsqrtf(ss / D + p.eps);
#pragma unroll
              for (int j = 0; j < PER; ++j) {
                float gw = bf16_to_f32(nw[lane + 32 * j]);
                if (p.one_plus_w) gw += 1.f;
                v[j] = bf16_to_f32(f32_to_bf16(bf16_to_f32(f32_to_bf16(v[j] * rstd)) * gw));
              }
            }
            if (is_q || is_k) {
              const int half = p.rot_dim / 2;
              float r[PER];
              if (p.rot_dim == D) {
#pragma unroll
                for (int j = 0; j < PER / 2; ++j) {
                  float sn, cs;
                  sincosf(static_cast<float>(pos) * p.inv_freq[lane + 32 * j], &sn, &cs);
                  sn *= p.mscale;
                  cs *= p.mscale;
                  const float x0 = v[j], x1 = v[j + PER / 2];
                  r[j] = x0 * cs - x1 * sn;
                  r[j + PER / 2] = x1 * cs + x0 * sn;
                }
              } else {
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
                  if (a < p.rot_dim) {
                    float sn, cs;
                    sincosf(static_cast<float>(pos) * p.inv_freq[a < half ? a : a - half], &sn, &cs);
                    sn *= p.mscale;
                    cs *= p.mscale;
                    r[j] = a < half ? v[j] * cs - partner * sn : v[j] * cs + partner * sn;
                  } else {
                    r[j] = v[j];
                  }
                }
              }
#pragma unroll
              for (int j = 0; j < PER; ++j) v[j] = bf16_to_f32(f32_to_bf16(r[j]));
            }
#pragma unroll
            for (int j = 0; j < PER; ++j) dstq[lane + 32 * j] = f32_to_bf16(v[j]);
            if (is_q) continue;
            const int off = pos % p.page;
            const int kvh = is_k ? head - p.hq : head - p.hq - p.hkv;
            const size_t tok = (static_cast<size_t>(blk) * p.hkv + kvh) * p.page + off;
            if (p.kv_fp8) {
              float am = 0.f;
#pragma unroll
              for (int j = 0; j < PER; ++j) am = fmaxf(am, fabsf(v[j]));
#pragma unroll
              for (int o = 16; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
              const float scale = am > 0.f ? am / 448.f : 1.f;
              const float inv = 1.f / scale;
              uint8_t* dst = (is_k ? p.k_cache : p.v_cache) + tok * D;
#pragma unroll
              for (int j = 0; j < PER; ++j) dst[lane + 32 * j] = f32_to_e4m3(v[j] * inv);
              if (lane == 0) (is_k ? p.k_scale : p.v_scale)[tok] = scale;
            } else {
              bf16* dst = reinterpret_cast<bf16*>(is_k ? p.k_cache : p.v_cache) + tok * D;
#pragma unroll
              for (int j = 0; j < PER; ++j) dst[lane + 32 * j] = f32_to_bf16(v[j]);
            }
          }
        }
      }
      // ---- end of phase: publish this CTA's writes, then arrive at the grid barrier
      if (wrote_act) fence_proxy_async_global();
      __threadfence();
      bar_workers();
      stamp(2 * ph + 1);
      if (wtid == 0) {
        const unsigned long long old = atomicAdd(p.ctl, 1ull);
        if (ph == p.nphase - 1 && old + 1 == base + static_cast<unsigned long long>(p.nphase) * G) {
          // last CTA of the launch: the next launch starts counting from here; collective epochs move on
          p.ctl[1] = old + 1;
          if (p.tp && p.tp_folds) *p.comm.epoch = epoch0 + p.tp_folds;
          __threadfence();
        }
      }
    }
  } else {
    pdl_wait();
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
}

}  // namespace dgpp

using namespace dgpp;

namespace dgpp {
__device__ unsigned long long g_dl_ctl[2];
static unsigned long long* dl_ctl_ptr() {
  static thread_local int cached_dev = -1;
  static thread_local unsigned long long* cached = nullptr;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
  if (dev != cached_dev) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_dl_ctl) != cudaSuccess) return nullptr;
    cached = static_cast<unsigned long long*>(p);
    cached_dev = dev;
  }
  return cached;
}
}  // namespace dgpp

static unsigned long long* g_dl_trace = nullptr;
// Debug aid: while a device buffer of 64 uint64 is set, worker thread 0 of CTA 0 (slots 0..31) and of the last CTA
// (slots 32..63) store %globaltimer (ns): slot 2*ph when phase ph starts (its barrier wait is over), 2*ph + 1 when
// the CTA has finished the phase; slot 30 at kernel entry, 31 when the preceding grid has completed.
DGPP_API int dgpp_decode_layer_set_trace(void* dev_u64x64) {
  g_dl_trace = static_cast<unsigned long long*>(dev_u64x64);
  return 0;
}

// Zero the grid-barrier words of the current device (after a launch that reported a failure, or in tests).
DGPP_API int dgpp_decode_layer_reset(cudaStream_t st) {
  unsigned long long* c = dl_ctl_ptr();
  DGPP_REQUIRE(c != nullptr, "decode_layer: no control block on the current device");
  DGPP_CUDA_OK(cudaMemsetAsync(c, 0, 2 * sizeof(unsigned long long), st));
  return 0;
}

DGPP_API int dgpp_decode_layer_grid() {
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
  return sms;
}

DGPP_API int dgpp_decode_layer(const DgppDecodeLayerArgs* a, cudaStream_t st) {
  DGPP_REQUIRE(a != nullptr, "decode_layer: null arguments");
  DGPP_REQUIRE(a->rows >= 1 && a->rows <= kDlBnTok, "decode_layer: %d rows (1..16 supported)", a->rows);
  DGPP_REQUIRE(a->nphase >= 1 && a->nphase <= kDlMaxPhase, "decode_layer: bad phase count %d", a->nphase);
  const int grid = a->grid > 0 ? a->grid : dgpp_decode_layer_grid();
  DGPP_REQUIRE(grid >= a->rows, "decode_layer: grid %d smaller than the row count", grid);
  DlParams p;
  memset(&p, 0, sizeof(p));
  DlMaps maps;
  memset(&maps, 0, sizeof(maps));
  p.rows = a->rows;
  p.nphase = a->nphase;
  bool act_used[kDlMaxAct] = {false, false, false};
  bool gemm_used[kDlMaxGemm] = {false, false, false, false};
  int tp_folds = 0;
  for (int i = 0; i < a->nphase; ++i) {
    const int t = a->ph_type[i], ix = a->ph_idx[i];
    p.ph_type[i] = t;
    p.ph_idx[i] = ix;
    if (t == kDlPhGemm) {
      DGPP_REQUIRE(ix >= 0 && ix < kDlMaxGemm, "decode_layer: phase %d names GEMM %d", i, ix);
      gemm_used[ix] = true;
    } else if (t == kDlPhRowA || t == kDlPhRowC) {
      DGPP_REQUIRE(ix >= 0 && ix < kDlMaxRowq, "decode_layer: phase %d names row phase %d", i, ix);
      if (t == kDlPhRowA && a->rowq[ix].tp_fold && a->comm) ++tp_folds;
    } else {
      DGPP_REQUIRE(t == kDlPhUnitq || t == kDlPhRope, "decode_layer: phase %d has unknown type %d", i, t);
    }
  }
  for (int i = 0; i < kDlMaxAct; ++i) {
    const DgppDlAct& s = a->act[i];
    if (!s.q) continue;
    DGPP_REQUIRE(s.K % 256 == 0 && s.K > 0, "decode_layer: activation width %d must be a multiple of 256", s.K);
    p.act[i].q = static_cast<uint8_t*>(s.q);
    p.act[i].sf = static_cast<uint8_t*>(s.sf);
    p.act[i].g = static_cast<float*>(s.g);
    p.act[i].K = s.K;
    if (make_tmap_2d(&maps.b[i], s.q, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, s.K / 2, kDlBN, s.K / 2, 128, kDlBN,
                     CU_TENSOR_MAP_SWIZZLE_128B))
      return -1;
    act_used[i] = true;
  }
  for (int i = 0; i < kDlMaxGemm; ++i) {
    if (!gemm_used[i]) continue;
    const DgppDlGemm& s = a->gemm[i];
    DGPP_REQUIRE(s.wq && s.wsf && s.K % 256 == 0 && s.N % 128 == 0, "decode_layer: GEMM %d: N %d %% 128, K %d %% 256", i, s.N, s.K);
    DGPP_REQUIRE(s.act >= 0 && s.act < kDlMaxAct && act_used[s.act] && a->act[s.act].K == s.K,
                 "decode_layer: GEMM %d reads activation %d of another width", i, s.act);
    DlGemm& g = p.gemm[i];
    g.sfa = static_cast<const uint8_t*>(s.wsf);
    g.alpha = s.alpha;
    g.N = s.N; g.K = s.K; g.act = s.act; g.pair = s.pair;
    if (s.pair) DGPP_REQUIRE(s.N % 256 == 0, "decode_layer: gate/up GEMM needs N %% 256 == 0, got %d", s.N);
    g.tiles = s.pair ? s.N / 256 : s.N / 128;
    const int stages = s.K / 256;
    int splits = s.pair ? 1 : (s.splits > 0 ? s.splits : grid / g.tiles);
    if (splits < 1) splits = 1;
    if (s.splits <= 0 && splits > stages / 4) splits = stages / 4 > 0 ? stages / 4 : 1;
    if (splits > stages) splits = stages;
    g.per = dgpp_ceil_div(stages, splits);
    g.splits = dgpp_ceil_div(stages, g.per);
    if (!s.pair)
      DGPP_REQUIRE(static_cast<int64_t>(g.splits) * 16 * s.N <= a->ws_floats, "decode_layer: workspace too small for GEMM %d", i);
    // stage-tiled weights: [N / 128 tiles][K / 256 stages][128 rows][128 bytes], so one stage is 16 KB of contiguous
    // memory (a row-major matrix would scatter it over 128 rows K / 2 bytes apart)
    if (make_tmap_2d(&maps.a[i], s.wq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, 128,
                     static_cast<uint64_t>(s.N / 128) * stages * 128, 128, 128, 128, CU_TENSOR_MAP_SWIZZLE_128B))
      return -1;
  }
  for (int i = 0; i < kDlMaxRowq; ++i) {
    const DgppDlRowq& s = a->rowq[i];
    DlRowq& r = p.rowq[i];
    r.mode = s.mode; r.src_gemm = s.src_gemm; r.out_act = s.out_act; r.tp_fold = s.tp_fold;
    r.in = static_cast<const bf16*>(s.in);
    r.in_stride = s.in_stride;
    r.norm_w = static_cast<const bf16*>(s.norm_w);
    r.x_out = static_cast<bf16*>(s.x_out);
    r.cl = 1;
  }
  for (int i = 0; i < a->nphase; ++i) {
    if (a->ph_type[i] != kDlPhRowA) continue;
    DGPP_REQUIRE(i + 1 < a->nphase && a->ph_type[i + 1] == kDlPhRowC && a->ph_idx[i + 1] == a->ph_idx[i],
                 "decode_layer: row phase %d is not followed by its finishing step", i);
    DlRowq& r = p.rowq[a->ph_idx[i]];
    DGPP_REQUIRE(r.mode == 0 || r.mode == 2 || r.mode == 3, "decode_layer: row phase mode %d", r.mode);
    DGPP_REQUIRE(r.out_act < kDlMaxAct && (r.out_act < 0 || act_used[r.out_act]), "decode_layer: row phase output %d", r.out_act);
    const int K = r.mode == 3 ? a->hq * a->d : (r.mode == 2 ? a->H : (r.out_act >= 0 ? a->act[r.out_act].K : 0));
    DGPP_REQUIRE(K > 0 && K % 256 == 0, "decode_layer: row width %d must be a multiple of 256", K);
    DGPP_REQUIRE(r.out_act < 0 || a->act[r.out_act].K == K, "decode_layer: row phase writes an activation of another width");
    DGPP_REQUIRE(a->stats != nullptr, "decode_layer: row phases need the statistics buffer");
    // column segments per row: the cluster quantiser's split (act_quant_cluster_kernel), so the sum of squares folds
    // in the same order; fewer when the units would outnumber the CTAs or the peer flags
    r.cl = 8;
    while (r.cl > 1 && (a->rows * r.cl > grid || (a->comm && r.tp_fold && a->rows * r.cl > kCommMaxCtas))) r.cl /= 2;
    DGPP_REQUIRE(a->rows * r.cl <= grid && (K / r.cl) * 2 <= kDlRowBuf, "decode_layer: %d rows of %d columns do not fit the grid", a->rows, K);
    if (r.mode == 2) {
      DGPP_REQUIRE(a->x && r.norm_w, "decode_layer: add + RMSNorm phase without residual / weight");
      DGPP_REQUIRE(r.src_gemm < kDlMaxGemm && (r.src_gemm < 0 || (gemm_used[r.src_gemm] && a->gemm[r.src_gemm].N == K)),
                   "decode_layer: add + RMSNorm phase reads GEMM %d of another width", r.src_gemm);
      DGPP_REQUIRE(!r.tp_fold || r.src_gemm >= 0, "decode_layer: a cross-rank fold needs a GEMM to fold");
    }
    if (r.mode == 3) DGPP_REQUIRE(a->part_ml && a->part_acc && a->att_splits >= 1 && a->d % 8 == 0, "decode_layer: attention partials missing");
    if (r.mode == 0) DGPP_REQUIRE(r.in != nullptr && r.out_act >= 0, "decode_layer: plain row phase without input");
  }
  p.x = static_cast<bf16*>(a->x);
  p.H = a->H; p.eps = a->eps; p.limit = a->limit; p.one_plus_w = a->one_plus_w;
  p.ws = static_cast<float*>(a->ws);
  p.hbuf = static_cast<bf16*>(a->hbuf);
  p.amax_part = static_cast<float*>(a->amax_part);
  p.stats = static_cast<float*>(a->stats);
  p.unitq_act = a->unitq_act;
  p.inter = a->inter;
  p.part_ml = static_cast<const float*>(a->part_ml);
  p.part_acc = static_cast<const float*>(a->part_acc);
  p.att_splits = a->att_splits; p.hq = a->hq; p.d = a->d;
  p.rope_gemm = a->rope_gemm;
  p.qkv = static_cast<bf16*>(a->qkv);
  p.positions = static_cast<const int32_t*>(a->positions);
  p.row_req = static_cast<const int32_t*>(a->row_req);
  p.block_table = static_cast<const int32_t*>(a->block_table);
  p.inv_freq = static_cast<const float*>(a->inv_freq);
  p.q_norm_w = static_cast<const bf16*>(a->q_norm_w);
  p.k_norm_w = static_cast<const bf16*>(a->k_norm_w);
  p.k_cache = static_cast<uint8_t*>(a->k_cache);
  p.v_cache = static_cast<uint8_t*>(a->v_cache);
  p.k_scale = static_cast<float*>(a->k_scale);
  p.v_scale = static_cast<float*>(a->v_scale);
  p.hkv = a->hkv; p.rot_dim = a->rot_dim; p.page = a->page; p.max_blocks = a->max_blocks; p.kv_fp8 = a->kv_fp8;
  p.mscale = a->mscale;
  for (int i = 0; i < a->nphase; ++i) {
    if (a->ph_type[i] == kDlPhUnitq) {
      DGPP_REQUIRE(a->unitq_act >= 0 && a->unitq_act < kDlMaxAct && act_used[a->unitq_act] && a->inter == a->act[a->unitq_act].K &&
                   a->hbuf && a->amax_part, "decode_layer: SwiGLU quantise phase is not fully described");
    }
    if (a->ph_type[i] == kDlPhRope) {
      DGPP_REQUIRE(a->rope_gemm >= 0 && a->rope_gemm < kDlMaxGemm && gemm_used[a->rope_gemm], "decode_layer: RoPE phase without its GEMM");
      DGPP_REQUIRE(a->d == 128 && a->gemm[a->rope_gemm].N == (a->hq + 2 * a->hkv) * 128, "decode_layer: RoPE phase needs head_dim 128");
      DGPP_REQUIRE(a->qkv && a->positions && a->row_req && a->block_table && a->inv_freq && a->k_cache && a->v_cache,
                   "decode_layer: RoPE phase arguments missing");
      DGPP_REQUIRE(a->rot_dim % 2 == 0 && a->rot_dim <= 128 && a->rot_dim > 0, "decode_layer: bad rot_dim %d", a->rot_dim);
    }
    if (a->ph_type[i] == kDlPhGemm && a->gemm[a->ph_idx[i]].pair)
      DGPP_REQUIRE(a->hbuf && a->amax_part && a->inter * 2 == a->gemm[a->ph_idx[i]].N, "decode_layer: gate/up GEMM without SwiGLU buffers");
  }
  p.tp = 0;
  p.tp_folds = tp_folds;
  if (a->comm) {
    const DgppComm* c = static_cast<const DgppComm*>(a->comm);
    p.tp = 1;
    p.comm = c->st;
    DGPP_REQUIRE(static_cast<size_t>(a->rows) * a->H * 2 <= c->st.slot_bytes, "decode_layer: rows do not fit the symmetric slot");
  }
  p.trace = g_dl_trace;
  p.ctl = dl_ctl_ptr();
  DGPP_REQUIRE(p.ctl != nullptr, "decode_layer: no control block on the current device");
  p.status = device_status_ptr();
  constexpr size_t smem = 1024 + static_cast<size_t>(kDlSA) * (kDlStageA + kDlSf) + static_cast<size_t>(kDlSB) * (kDlStageB + kDlSf) +
                          kDlRowBuf + 8 * 4 * 4 + 256 * 4 + (2 * kDlSA + 2 * kDlSB + 4) * 8 + 64;
  static_assert(smem <= 227 * 1024, "decode_layer: shared memory budget exceeded");
  static bool attr = false;
  if (!attr) {
    DGPP_CUDA_OK(cudaFuncSetAttribute(decode_layer_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    attr = true;
  }
  decode_layer_kernel<<<grid, kDlThreads, smem, st>>>(maps, p);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}
