// NVFP4 x NVFP4 linear layer on the block-scaled tensor-core path (tcgen05 kind::mxf4nvf4,
// scale_vec::4X: one ue4m3 scale per 16 elements for both operands, scale factors in TMEM):
//
//     C[T, N] = alpha_w * g[t] * sum_r  Wq[N, K] . Xq_r[T, K]^T
//
// The packed e2m1 weight bytes go from HBM through TMA into shared memory and straight into the
// tensor core: no thread ever touches a weight or a scale.  Activations arrive already quantised by
// `fused_act_quant_kernel` as R "residual terms": x ~= g[t] * (x_1 + x_2 + ... + x_R), each term an
// NVFP4 tensor of what the previous terms left over.  All R terms accumulate into the same fp32
// TMEM accumulator, so R = 1 is plain W4A4 and R = 3 carries about 8 mantissa bits of the bf16
// activation (every term removes ~2.6 bits of the remaining error) at no extra weight traffic.
//
// Layout: weight tile = UMMA A (128 rows), token tile = UMMA B (BN = 16..256 rows).  One pipeline
// stage covers 256 K: 128 bytes of packed fp4 per row (one 128-byte swizzle row = four K=64 MMAs).
//
// Scale factors travel in the layout tcgen05.cp consumes, so a stage's factors are one contiguous bulk
// copy: for a tile of 128 rows and a K=64 step the 512-byte "atom" holds factor i of row m at byte
// (m % 32) * 16 + (m / 32) * 4 + i.  Weight scales are permuted into [n_tile][stage][4 steps][atom] once at
// bind time (an index permutation of the checkpoint bytes); the activation quantiser writes its scales in
// [term][token_tile][stage][4 steps][atoms of the tile] directly.
//
// Warp roles (192 threads): warp 0 TMA / bulk-copy producer, warp 1 MMA issuer + TMEM owner (copies the
// atoms into TMEM with tcgen05.cp, then issues the MMAs), warps 2..5 epilogue.  Split-K as in gemm_tc.cu
// (deterministic ascending fold by the last CTA of a tile).
// (reference counterpart: src/kernels/moe_w4a4.cu:87,139,476 -- block-scaled mma.sync m16n8k64 there.)
#include <cuda.h>
#include <string.h>

#include "common/common.h"
#include "common/dtypes.cuh"
#include "common/ptx.cuh"
#include "kernels/comm.cuh"
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
  const uint8_t* sfa;          // weight scales, tiled [n_tiles][stages][4][512]
  const uint8_t* sfb;          // activation scales, tiled [R][token_tiles][stages][4 * atoms][512]
  bf16* out;
  float* out32;
  const bf16* resid;
  float* ws;
  uint32_t* counters;
  DeviceStatus* status;
  int T, T_pad, N, K, ldc, R;
  int stages_per_split;
  // Fused all-reduce push (tensor-parallel o_proj / down_proj at decode sizes): instead of writing `out`, the CTA
  // that finishes an output tile stores it as bf16 into slot `rank` of EVERY rank's symmetric region and raises
  // flag[parity][rank][n tile] = epoch there.  The consumer (fold + add + RMSNorm + quantise) waits on the flags.
  int push;
  CommState comm;
  // Grouped mode (mixture-of-experts): the weight matrix is the experts' matrices stacked along N
  // ([experts * N, K]); blockIdx.x = slot * group_tiles + n tile, group_list[slot] = expert id of the slot or -1
  // (inactive slot: the CTA does nothing).  Outputs of slot s start at out + s * group_out_stride (elements);
  // with group_b the activations / their scales / g are per slot as well (down projection), otherwise every
  // slot multiplies the same token tile (gate / up projection).
  const int32_t* group_list;
  const float* group_alpha;    // per-expert tensor scale, replaces alpha
  int group_tiles, group_b, grid_x;
  int64_t group_out_stride;
  // L2 prefetch of what the NEXT weight-streaming kernel will read (decode): once this CTA's own loads are issued,
  // its producer warp asks L2 for a slice of [pf_ptr, pf_ptr + pf_bytes).  The small kernels between two projections
  // (quantiser, RoPE, attention over a short context) leave HBM idle; the prefetch fills that time.  A hint only.
  const unsigned char* pf_ptr;
  int64_t pf_bytes;
  unsigned long long* trace;  // debug: CTA (0,0,0) stores %globaltimer at 7 points of its life (see dgpp_gemm_fp4_set_trace)
  int preload;             // dense mode: issue the weight half of the first ring stages before waiting on the preceding grid
  // Split-K inside a thread-block cluster (decode projections with few output tiles): the gridDim.z CTAs of one output
  // tile form a cluster (1, 1, splits); each runs its share of the K stages, then the partial accumulators of ranks
  // 1.. travel through distributed shared memory into rank 0's (by then idle) operand ring and rank 0 adds them in
  // ascending rank order.  No workspace, no global counters; two cluster barriers.
  int cluster_split;
};

// One bf16 of the finished output tile -> slot `rank` of every rank (destinations staggered by rank).
__device__ __forceinline__ void push_value(const Fp4Params& p, int parity, size_t idx, bf16 v) {
  for (int r = 0; r < p.comm.world; ++r) {
    const int dst = (p.comm.rank + r) % p.comm.world;
    reinterpret_cast<bf16*>(payload(p.comm, dst, parity, p.comm.rank))[idx] = v;
  }
}
// Called by the 128 epilogue threads of the CTA that wrote the tile: make the stores visible at system scope, then
// raise this tile's flag on every rank.
__device__ __forceinline__ void push_flags(const Fp4Params& p, int parity, uint32_t epoch, int warp, int lane) {
  __threadfence_system();
  asm volatile("bar.sync 1, 128;" ::: "memory");
  if (warp == 2 && lane < p.comm.world) st_release_sys(flag(p.comm, lane, parity, p.comm.rank, blockIdx.x), epoch);
}

// BN = MMA N = (token tile) x (residual terms): with R > 1 the terms of one token tile are stacked along N
// (rows r * bn_tok + m of the B operand) so a K=64 step is ONE tcgen05.mma whatever R is; the epilogue adds the
// R column groups.  Stacking needs the whole batch in one token tile (decode); R = 1 tiles freely.
template <int BN, int S>
__global__ void __launch_bounds__(kF4Threads, BN <= 96 ? 2 : 1)
gemm_fp4_kernel(const __grid_constant__ CUtensorMap tmA,   // packed weights as bytes [N, K/2]
                const __grid_constant__ CUtensorMap tmB,   // packed activations as bytes [R*T_pad, K/2]
                Fp4Params p) {
  constexpr int kStageB = BN * 128;
  constexpr int RMAX = 1;
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
  uint64_t* acc_full = empty + S;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* last_flag = const_cast<int*>(abort_flag) + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool tracing = p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
  auto stamp = [&](int slot) {
    if (tracing) {
      unsigned long long t;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t) :: "memory");
      p.trace[slot] = t;
    }
  };
  if (threadIdx.x == 0) stamp(0);
  const int bn_tok = BN / p.R;             // tokens per tile
  const int m0 = blockIdx.y * bn_tok;
  const int split = blockIdx.z, splits = gridDim.z;
  const int total_stages = p.K / kF4StageK;
  const int st_begin = split * p.stages_per_split;
  const int st_end = min(total_stages, st_begin + p.stages_per_split);
  const int R = 1;  // terms are stacked inside the single B tile
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
  if (threadIdx.x == 0) stamp(1);
  // Weights never depend on the preceding grid.  In dense mode the producer therefore fills the first ring stages
  // with weight tiles and their scales BEFORE it waits for that grid: under programmatic dependent launch this CTA
  // is already resident while the small kernel in front of it (the activation quantiser) still runs, so the weight
  // stream of up to S stages per CTA overlaps with it and the first MMA no longer pays an HBM round trip.  The
  // activation half of each of those stages is issued after the wait, onto the same barrier.  (Grouped mode picks
  // its weight tile from the routing result and cannot start early.)
  const int pre = (p.group_list || !p.preload) ? 0 : min(max(0, st_end - st_begin), S);
  if (warp == 0 && pre > 0) {
    if (elect_one()) {
      const uint8_t* sfa_pre = p.sfa + static_cast<size_t>(blockIdx.x) * total_stages * kSfaBytes;
      for (int i = 0; i < pre; ++i) {
        mbar_expect_tx(&full[i], kF4StageA + kSfaBytes + R * (kStageB + kSfbBytes));
        tma_load_2d(sA + i * kF4StageA, &tmA, (st_begin + i) * 128, blockIdx.x * kF4BM, &full[i]);
        bulk_load_1d(sSfa + i * kSfaBytes, sfa_pre + static_cast<size_t>(st_begin + i) * kSfaBytes, kSfaBytes, &full[i]);
      }
    }
    __syncwarp();
  }
  pdl_wait();
  if (threadIdx.x == 0) stamp(2);
  // tile of the (stacked) weight matrix, output / activation group
  int tile_x = blockIdx.x, grp = 0;
  bool active = true;
  float alpha = p.alpha;
  if (p.group_list) {
    grp = blockIdx.x / p.group_tiles;
    const int e = p.group_list[grp];
    active = e >= 0;
    tile_x = (active ? e : 0) * p.group_tiles + blockIdx.x % p.group_tiles;
    if (active && p.group_alpha) alpha = p.group_alpha[e];
  }
  const int n0 = tile_x * kF4BM;
  const int nst = active ? max(0, st_end - st_begin) : 0;
  const int b_row0 = (p.group_b ? grp * p.R * p.T_pad : 0) + blockIdx.y * BN;
  const size_t sfb_grp = p.group_b ? static_cast<size_t>(grp) * (p.T_pad / bn_tok) * total_stages * kSfbBytes : 0;
  const float* gvec = p.g + (p.group_b ? grp * p.T_pad : 0);

  bool acc_ok = true;      // epilogue warps: the accumulator completed within the wait bound
  if (warp == 0) {
    // ------------------------------------------------------------------ producer: weights, activations, scales
    if (elect_one()) {
      const int token_tiles = p.T_pad / bn_tok;
      const uint8_t* sfa_tile = p.sfa + static_cast<size_t>(tile_x) * total_stages * kSfaBytes;
      for (int i = 0; i < nst; ++i) {
        const int s = i % S;
        const int st = st_begin + i;
        const int xb = st * 128;  // byte column of this stage
        if (i >= pre) {           // (the weight half of the first `pre` stages is already in flight)
          if (!wait_bar(&empty[s], ((i / S) & 1) ^ 1)) { report(p.status, kTimeoutStageEmpty, 11); *abort_flag = 1; break; }
          mbar_expect_tx(&full[s], kF4StageA + kSfaBytes + R * (kStageB + kSfbBytes));
          tma_load_2d(sA + s * kF4StageA, &tmA, xb, n0, &full[s]);
          bulk_load_1d(sSfa + s * kSfaBytes, sfa_tile + static_cast<size_t>(st) * kSfaBytes, kSfaBytes, &full[s]);
        }
        for (int r = 0; r < R; ++r) {
          tma_load_2d(sB + (s * RMAX + r) * kStageB, &tmB, xb, b_row0, &full[s]);
          const uint8_t* sfb = p.sfb + sfb_grp + ((static_cast<size_t>(r) * token_tiles + blockIdx.y) * total_stages + st) * kSfbBytes;
          bulk_load_1d(sSfb + (s * RMAX + r) * kSfbBytes, sfb, kSfbBytes, &full[s]);
        }
        if (*abort_flag) break;
      }
    }
    __syncwarp();
    if (p.pf_bytes > 0) {
      constexpr int64_t kChunk = 16384;
      const int64_t ctas = static_cast<int64_t>(gridDim.x) * gridDim.y * gridDim.z;
      const int64_t cta = (static_cast<int64_t>(blockIdx.z) * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
      for (int64_t off = (cta * 32 + lane) * kChunk; off < p.pf_bytes; off += ctas * 32 * kChunk) {
        const uint32_t n = static_cast<uint32_t>(min(kChunk, p.pf_bytes - off)) & ~15u;
        if (n) l2_prefetch_bulk(p.pf_ptr + off, n);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc_fp4bs(kF4BM, BN, 0u);
      for (int i = 0; i < nst; ++i) {
        const int s = i % S;
        if (!wait_bar(&full[s], (i / S) & 1)) { report(p.status, kTimeoutTmaFull, 12); *abort_flag = 1; break; }
        if (i == 0) stamp(3);
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
      stamp(4);
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5): wait for the accumulator
    acc_ok = nst > 0 ? wait_bar(acc_full, 0) : true;
    if (!acc_ok) { report(p.status, kTimeoutAccum, 15); *abort_flag = 1; }
    acc_ok = __all_sync(0xffffffffu, acc_ok);            // the TMEM loads below stay warp-uniform
    if (warp == 2 && lane == 0) stamp(5);
    tc_fence_after();
  }
  if (p.cluster_split) {
    // Every thread of every CTA of the cluster passes the same two barriers, whatever happened before (a CTA that
    // gave up on a wait still arrives), so the cluster cannot block on a peer.
    const int q = warp & 3;
    const int cols = min(bn_tok, p.T - m0);
    float* red = reinterpret_cast<float*>(sA);          // rank 0: [splits - 1][bn_tok][128] partials of the peers
    cluster_barrier();                                   // every CTA's mainloop is over: rank 0's operand ring is idle
    if (warp >= 2 && split > 0 && acc_ok && !*abort_flag) {
      for (int c0 = 0; c0 < bn_tok; c0 += 16) {
        if (c0 >= cols) break;
        float v[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = 0.f;
        if (nst > 0) {
          for (int r = 0; r < p.R; ++r) {
            uint32_t rr[16];
            tmem_ld_x16(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + r * bn_tok + c0, rr);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] += __uint_as_float(rr[j]);
          }
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int m = c0 + j;
          if (m < cols)
            st_shared_cluster_f32(mapa_shared(smem_u32(red + (static_cast<size_t>(split - 1) * bn_tok + m) * kF4BM + q * 32 + lane), 0u),
                                  v[j]);
        }
      }
    }
    cluster_barrier();                                   // the partials have landed in rank 0
    if (warp >= 2 && split == 0) {
      const int n = n0 + q * 32 + lane;
      const uint32_t push_epoch = p.push ? *p.comm.epoch + 1 : 0u;
      const int push_parity = push_epoch & 1;
      if (acc_ok && !*abort_flag) {
        for (int c0 = 0; c0 < bn_tok; c0 += 16) {
          if (c0 >= cols) break;
          float v[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = 0.f;
          if (nst > 0) {
            for (int r = 0; r < p.R; ++r) {
              uint32_t rr[16];
              tmem_ld_x16(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + r * bn_tok + c0, rr);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 16; ++j) v[j] += __uint_as_float(rr[j]);
            }
          }
          if (n < p.N) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int m = c0 + j;
              if (m < cols) {
                float acc = v[j];
                for (int s2 = 1; s2 < splits; ++s2) acc += red[(static_cast<size_t>(s2 - 1) * bn_tok + m) * kF4BM + q * 32 + lane];
                const size_t o = static_cast<size_t>(m0 + m) * p.ldc + n;
                float y = acc * alpha * gvec[m0 + m];
                if (p.push) {
                  push_value(p, push_parity, static_cast<size_t>(m0 + m) * p.N + n, f32_to_bf16(y));
                  continue;
                }
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
      if (p.push) push_flags(p, push_parity, push_epoch, warp, lane);
    }
  } else if (warp >= 2) {
    const int q = warp & 3;
    const bool ok = acc_ok;
    // n: output column (within the expert in grouped mode); n_ws: column in the split-K workspace
    const int n = (p.group_list ? (blockIdx.x % p.group_tiles) * kF4BM : n0) + q * 32 + lane;
    const int n_ws = blockIdx.x * kF4BM + q * 32 + lane, N_ws = p.group_list ? gridDim.x * kF4BM : p.N;
    const size_t out_grp = p.group_list ? static_cast<size_t>(grp) * p.group_out_stride : 0;
    const int cols = min(bn_tok, p.T - m0);
    const uint32_t push_epoch = p.push ? *p.comm.epoch + 1 : 0u;
    const int push_parity = push_epoch & 1;
    if (ok && !*abort_flag && active) {
      float* wsp = splits > 1 ? p.ws + (static_cast<size_t>(split) * p.T + m0) * N_ws : nullptr;
#pragma unroll 1
      for (int c0 = 0; c0 < bn_tok; c0 += 16) {
        if (c0 >= cols) break;
        float v[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = 0.f;
        if (nst > 0) {
          for (int r = 0; r < p.R; ++r) {  // add the residual-term column groups
            uint32_t rr[16];
            tmem_ld_x16(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + r * bn_tok + c0, rr);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] += __uint_as_float(rr[j]);
          }
        }
        if (n < p.N) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int m = c0 + j;
            if (m < cols) {
              if (splits > 1) {
                wsp[static_cast<size_t>(m) * N_ws + n_ws] = v[j];
              } else {
                const size_t o = out_grp + static_cast<size_t>(m0 + m) * p.ldc + n;
                float y = v[j] * alpha * gvec[m0 + m];
                if (p.push) {
                  push_value(p, push_parity, static_cast<size_t>(m0 + m) * p.N + n, f32_to_bf16(y));
                  continue;
                }
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
    if (p.push && splits == 1) push_flags(p, push_parity, push_epoch, warp, lane);
    if (splits > 1 && active) {
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
          // The partials of 4 rows x 4 splits are requested together (16 independent L2 loads in flight per thread)
          // and then added in ascending split order: the sum is the one a plain loop gives, without one L2 round
          // trip per (row, split).
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
                  t[mm][ss] = live ? __ldcg(p.ws + (static_cast<size_t>(s0 + ss) * p.T + m0 + mb + mm) * N_ws + n_ws) : 0.f;
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
              const size_t o = out_grp + static_cast<size_t>(m0 + m) * p.ldc + n;
              float y = acc[mm] * alpha * gvec[m0 + m];
              if (p.push) {
                push_value(p, push_parity, static_cast<size_t>(m0 + m) * p.N + n, f32_to_bf16(y));
                continue;
              }
              if (p.out32) p.out32[o] = y;
              if (p.out) {
                if (p.resid) y = bf16_to_f32(p.resid[o]) + bf16_to_f32(f32_to_bf16(y));
                p.out[o] = f32_to_bf16(y);
              }
            }
          }
        }
        if (warp == 2 && lane == 0) p.counters[blockIdx.y * gridDim.x + blockIdx.x] = 0;
        if (p.push) push_flags(p, push_parity, push_epoch, warp, lane);
      }
    }
  
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) stamp(6);
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
}

// --------------------------------------------------------------------------------------------------
// Activation producer + quantiser: one CTA per row computes the row's bf16 activation (optionally with the
// operator that precedes the linear layer fused in), then splits it into R residual NVFP4 terms:
//   g[t]   = max|x[t, :]| / (6 * 256)            (fp32; the e4m3 block scales then stay <= 256)
//   term r : block scale s = e4m3(amax_16(res) / 6), codes = e2m1(res / s), res -= codes * s   (res in units of g)
// MODE 0: x = in                                    (plain rows)
// MODE 1: x = swiglu(in = [gate | up])               bf16( bf16(silu(gate)) * up )
// MODE 2: x = rmsnorm(resid + delta) * w             resid_out = bf16(resid + delta); x = bf16(w * bf16(r * rstd))
// q  rows are ordered [token tile][term][token in tile]; sf : [T_pad / bn][K / 256][4 steps][atoms][512] e4m3 bytes in
//      tcgen05.cp atom order, where the B-operand row of (term r, token m) is r * bn + m and atoms = (R * bn > 128 ? 2 : 1)
// The bf16 activation itself is also written when `x_out` is given (the prefill path and tests read it).
struct QuantArgs {
  const bf16* in;        // MODE 0: [T, K]; MODE 1: [T, 2K]; MODE 2: residual [T, K]
  int64_t in_stride;
  const bf16* delta;     // MODE 2 (optional)
  const bf16* w;         // MODE 2 norm weight
  bf16* resid_out;       // MODE 2
  bf16* x_out;           // optional bf16 copy of the activation
  uint8_t* q;
  uint8_t* sf;
  float* g;
  int T, T_pad, K, R, bn;
  float eps, limit, alpha;     // alpha > 0: gate * sigmoid(alpha * gate) * (up + 1) in the swiglu mode
  int one_plus_w;
};

template <int MODE>
__global__ void __launch_bounds__(256) fused_act_quant_kernel(QuantArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* row_s = reinterpret_cast<bf16*>(smem_raw);  // [K]
  __shared__ float red[8];
  pdl_wait();
  const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  const int K = a.K, nvec = K / 8;
  auto block_reduce = [&](float v, bool is_max) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float u = __shfl_xor_sync(0xffffffffu, v, o);
      v = is_max ? fmaxf(v, u) : v + u;
    }
    if (lane == 0) red[wid] = v;
    __syncthreads();
    float r = red[0];
    for (int i = 1; i < 8; ++i) r = is_max ? fmaxf(r, red[i]) : r + red[i];
    __syncthreads();
    return r;
  };
  float amax = 0.f, bound = 0.f;
  if (MODE == 2) {
    const bf16* rr = a.in + static_cast<size_t>(t) * a.in_stride;
    float ss = 0.f, pm = 0.f;
    for (int i = tid; i < nvec; i += 256) {
      Pack16 x;
      x.u = reinterpret_cast<const uint4*>(rr)[i];
      if (a.delta) {
        Pack16 d;
        d.u = reinterpret_cast<const uint4*>(a.delta + static_cast<size_t>(t) * K)[i];
#pragma unroll
        for (int j = 0; j < 8; ++j) x.h[j] = f32_to_bf16(bf16_to_f32(x.h[j]) + bf16_to_f32(d.h[j]));
        reinterpret_cast<uint4*>(a.resid_out + static_cast<size_t>(t) * K)[i] = x.u;
      }
      Pack16 wv;
      wv.u = reinterpret_cast<const uint4*>(a.w)[i];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float f = bf16_to_f32(x.h[j]);
        ss += f * f;
        float gw = bf16_to_f32(wv.h[j]);
        if (a.one_plus_w) gw += 1.f;
        pm = fmaxf(pm, fabsf(f * gw));
      }
      reinterpret_cast<uint4*>(row_s)[i] = x.u;
    }
    const float rstd = rsqrtf(block_reduce(ss, false) / static_cast<float>(K) + a.eps);
    // row scale from the bound max |x w| * rstd * 1.0079 (see act_quant_cluster_kernel): no second reduction pass
    bound = block_reduce(pm, true) * rstd * 1.0079f;
    for (int i = tid; i < nvec; i += 256) {
      Pack16 x, ww;
      x.u = reinterpret_cast<const uint4*>(row_s)[i];
      ww.u = reinterpret_cast<const uint4*>(a.w)[i];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float nrm = bf16_to_f32(f32_to_bf16(bf16_to_f32(x.h[j]) * rstd));
        float gw = bf16_to_f32(ww.h[j]);
        if (a.one_plus_w) gw += 1.f;
        x.h[j] = f32_to_bf16(nrm * gw);
      }
      reinterpret_cast<uint4*>(row_s)[i] = x.u;
      if (a.x_out) reinterpret_cast<uint4*>(a.x_out + static_cast<size_t>(t) * K)[i] = x.u;
    }
  } else {
    const bf16* rr = a.in + static_cast<size_t>(t) * a.in_stride;
    for (int i = tid; i < nvec; i += 256) {
      Pack16 x;
      x.u = reinterpret_cast<const uint4*>(rr)[i];
      if (MODE == 1) {
        Pack16 u;
        u.u = reinterpret_cast<const uint4*>(rr + K)[i];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float gv = bf16_to_f32(x.h[j]), uv = bf16_to_f32(u.h[j]);
          if (a.limit > 0.f) { gv = fminf(gv, a.limit); uv = fminf(fmaxf(uv, -a.limit), a.limit); }
          float sl;
          if (a.alpha > 0.f) {
            sl = bf16_to_f32(f32_to_bf16(gv / (1.f + __expf(-a.alpha * gv))));
            uv += 1.f;
          } else {
            sl = bf16_to_f32(f32_to_bf16(gv / (1.f + __expf(-gv))));
          }
          x.h[j] = f32_to_bf16(sl * uv);
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(bf16_to_f32(x.h[j])));
      reinterpret_cast<uint4*>(row_s)[i] = x.u;
      if (a.x_out) reinterpret_cast<uint4*>(a.x_out + static_cast<size_t>(t) * K)[i] = x.u;
    }
  }
  __syncthreads();
  amax = MODE == 2 ? bound : block_reduce(amax, true);
  const float gs = amax > 0.f ? amax / (6.f * 256.f) : 1.f;
  if (tid == 0) a.g[t] = gs;
  const float inv_g = 1.f / gs;
  const int groups = K / 16, stages = K / 256;
  // B-operand rows of a token tile: term r of token m sits at row r * bn + m (terms stacked along the MMA N axis)
  const int atoms = a.R * a.bn > 128 ? 2 : 1;
  const int tile = t / a.bn, m = t % a.bn;
  const size_t tiles = static_cast<size_t>(a.T_pad / a.bn);
  for (int gi = tid; gi < groups; gi += 256) {
    Pack16 lo, hi;
    lo.u = reinterpret_cast<const uint4*>(row_s + gi * 16)[0];
    hi.u = reinterpret_cast<const uint4*>(row_s + gi * 16)[1];
    float res[16];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      res[j] = bf16_to_f32(lo.h[j]) * inv_g;
      res[8 + j] = bf16_to_f32(hi.h[j]) * inv_g;
    }
    const int st = gi >> 4, step = (gi >> 2) & 3, fi = gi & 3;
    for (int r = 0; r < a.R; ++r) {
      float bm = 0.f;
#pragma unroll
      for (int j = 0; j < 16; ++j) bm = fmaxf(bm, fabsf(res[j]));
      const uint8_t sb = f32_to_e4m3(bm * (1.f / 6.f));
      const float s = e4m3_value_f32(bm * (1.f / 6.f));   // value of the code sb, without an fp8 decode of it
      const float inv_s = s > 0.f ? 1.f / s : 0.f;
      float sc[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) sc[j] = res[j] * inv_s;
      const uint32_t w0 = f32x8_to_e2m1x8(sc), w1 = f32x8_to_e2m1x8(sc + 8);
      e2m1x8_residual(w0, s, res);
      e2m1x8_residual(w1, s, res + 8);
      const size_t ro = static_cast<size_t>(tile) * a.R * a.bn + static_cast<size_t>(r) * a.bn + m;
      *reinterpret_cast<uint2*>(a.q + ro * (K / 2) + gi * 8) = make_uint2(w0, w1);
      const int brow = r * a.bn + m, h = brow >> 7, mm = brow & 127;
      const size_t atom_idx = ((static_cast<size_t>(tile) * stages + st) * 4 + step) * atoms + h;
      a.sf[atom_idx * kF4Atom + (mm & 31) * 16 + (mm >> 5) * 4 + fi] = sb;
    }
  }
}

template <int BN>
struct Fp4Cfg {
  static constexpr int kAtomsB = BN > 128 ? 2 : 1;
  static constexpr size_t stage_bytes() {
    return kF4StageA + static_cast<size_t>(BN) * 128 + 4 * kF4Atom + static_cast<size_t>(4) * kAtomsB * kF4Atom;
  }
  // small token tiles (decode): two CTAs per SM, each <= ~110 KB; large tiles: one CTA with a deep ring
  static constexpr size_t kBudget = BN <= 96 ? 108 * 1024 : 200 * 1024;
  static constexpr int S = kBudget / stage_bytes() > 6 ? 6 : static_cast<int>(kBudget / stage_bytes());
  static constexpr size_t smem() { return 1024 + S * stage_bytes() + (2 * S + 1) * 8 + 64; }
};

template <int BN>
static int launch_fp4(const CUtensorMap& tA, const CUtensorMap& tB, const Fp4Params& p, int splits, cudaStream_t st) {
  using C = Fp4Cfg<BN>;
  static_assert(C::S >= 2, "not enough shared memory for two stages");
  auto kern = gemm_fp4_kernel<BN, C::S>;
  static bool attr = false;
  constexpr size_t smem = C::smem();
  static_assert(smem <= 227 * 1024, "shared memory budget exceeded");
  if (!attr) {
    DGPP_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    attr = true;
  }
  const int bn_tok = BN / p.R;
  dim3 grid(p.grid_x > 0 ? p.grid_x : dgpp_ceil_div(p.N, kF4BM), dgpp_ceil_div(p.T, bn_tok), splits);
  if (p.cluster_split) {
    DGPP_REQUIRE(splits >= 2 && splits <= 8, "gemm_fp4: cluster split-K takes 2..8 splits, got %d", splits);
    DGPP_REQUIRE(static_cast<size_t>(splits - 1) * bn_tok * kF4BM * 4 <= static_cast<size_t>(C::S) * kF4StageA,
                 "gemm_fp4: %d splits x %d tokens do not fit the operand ring for the cluster fold", splits, bn_tok);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kF4Threads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 1;
    at[0].val.clusterDim.y = 1;
    at[0].val.clusterDim.z = static_cast<unsigned>(splits);
    cfg.attrs = at;
    cfg.numAttrs = 1;
    DGPP_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, tA, tB, p));
    return 0;
  }
  kern<<<grid, kF4Threads, smem, st>>>(tA, tB, p);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

}  // namespace dgpp

using namespace dgpp;

// Fused activation producer + NVFP4 quantiser (see fused_act_quant_kernel).  mode: 0 plain, 1 swiglu, 2 add+rmsnorm.
// sf must be zero-initialised once (rows that are never written keep scale 0); its size is
// R * (T_pad / bn) * (K / 256) * 4 * atoms * 512 bytes with atoms = (bn > 128 ? 2 : 1).
DGPP_API int dgpp_act_quant_nvfp4(int mode, const void* in, int64_t in_stride, const void* delta, const void* w,
                                  void* resid_out, void* x_out, void* q, void* sf, void* g, int T, int T_pad, int K,
                                  int R, int bn, float eps, float limit, float alpha, int one_plus_w, cudaStream_t st) {
  DGPP_REQUIRE(K % 256 == 0, "act_quant: K %d must be a multiple of 256", K);
  DGPP_REQUIRE(R >= 1 && R <= 4, "act_quant: R %d outside 1..4", R);
  DGPP_REQUIRE(bn == 16 || bn == 32 || bn == 64 || bn == 128 || bn == 256, "act_quant: bad token tile %d", bn);
  DGPP_REQUIRE(T_pad % bn == 0 && T_pad >= T, "act_quant: T_pad %d must be a multiple of bn %d and >= T", T_pad, bn);
  DGPP_REQUIRE(static_cast<size_t>(K) * 2 <= 96 * 1024, "act_quant: K %d too large", K);
  if (T == 0) return 0;
  QuantArgs a;
  a.in = static_cast<const bf16*>(in);
  a.in_stride = in_stride;
  a.delta = static_cast<const bf16*>(delta);
  a.w = static_cast<const bf16*>(w);
  a.resid_out = static_cast<bf16*>(resid_out);
  a.x_out = static_cast<bf16*>(x_out);
  a.q = static_cast<uint8_t*>(q);
  a.sf = static_cast<uint8_t*>(sf);
  a.g = static_cast<float*>(g);
  a.T = T; a.T_pad = T_pad; a.K = K; a.R = R; a.bn = bn; a.eps = eps; a.limit = limit; a.alpha = alpha; a.one_plus_w = one_plus_w;
  const size_t smem = static_cast<size_t>(K) * 2;
  static bool attr = false;
  if (!attr) {
    cudaFuncSetAttribute(fused_act_quant_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
    cudaFuncSetAttribute(fused_act_quant_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
    cudaFuncSetAttribute(fused_act_quant_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
    attr = true;
  }
  if (mode == 0) fused_act_quant_kernel<0><<<T, 256, smem, st>>>(a);
  else if (mode == 1) fused_act_quant_kernel<1><<<T, 256, smem, st>>>(a);
  else if (mode == 2) fused_act_quant_kernel<2><<<T, 256, smem, st>>>(a);
  else { dgpp_set_error("act_quant: unknown mode %d", mode); return -1; }
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

// out[T, N] = alpha * g[t] * sum_r Wq . Xq_r^T.   xq: [R, T_pad, K/2]; xsf / wsf_tiled: tiled scale factors; g: [T].
// One-shot hint for the NEXT dgpp_gemm_fp4 / dgpp_gemm_fp4_grouped call of this thread: the bytes its CTAs ask L2
// to fetch once their own loads are issued (normally the packed weights of the projection that runs next).
static unsigned long long* g_trace = nullptr;
// Debug aid: while a device buffer of 8 uint64 is set, CTA (0,0,0) of every dgpp_gemm_fp4 launch stores %globaltimer
// (ns) at: 0 entry, 1 prologue done, 2 preceding grid complete, 3 first stage landed, 4 last MMA issued,
// 5 accumulator complete, 6 epilogue done.  Pass null to switch it off.
DGPP_API int dgpp_gemm_fp4_set_trace(void* dev_u64x8) {
  g_trace = static_cast<unsigned long long*>(dev_u64x8);
  return 0;
}
static int g_preload = 1;
// Process-wide switch of the pre-wait weight preload (on by default; off for A/B measurements).
DGPP_API int dgpp_gemm_fp4_set_preload(int on) {
  g_preload = on ? 1 : 0;
  return 0;
}
static thread_local const unsigned char* g_pf_ptr = nullptr;
static thread_local int64_t g_pf_bytes = 0;
DGPP_API int dgpp_gemm_fp4_set_prefetch(const void* ptr, int64_t bytes) {
  DGPP_REQUIRE(bytes >= 0 && (reinterpret_cast<uintptr_t>(ptr) & 15) == 0, "gemm_fp4 prefetch: unaligned range");
  g_pf_ptr = static_cast<const unsigned char*>(ptr);
  g_pf_bytes = ptr ? bytes : 0;
  return 0;
}

DGPP_API int dgpp_gemm_fp4(int bn, const void* xq, const void* xsf, const void* g, int R, int T_pad, const void* wq,
                           const void* wsf_tiled, float alpha, void* out, void* out32, const void* resid, int ldc,
                           int T, int N, int K, int splits, void* ws, void* counters, void* comm_push,
                           cudaStream_t st) {
  DGPP_REQUIRE(K % 256 == 0, "gemm_fp4: K %d must be a multiple of 256", K);
  DGPP_REQUIRE(R >= 1 && R <= 4, "gemm_fp4: R %d outside 1..4", R);
  DGPP_REQUIRE(splits >= 1, "gemm_fp4: splits must be >= 1");
  DGPP_REQUIRE(splits == 1 || (ws && counters) || (!ws && !counters), "gemm_fp4: split-K takes a workspace with counters, or neither (cluster form)");
  DGPP_REQUIRE(out || out32 || comm_push, "gemm_fp4: no output");
  DGPP_REQUIRE(T_pad >= T && T_pad % bn == 0, "gemm_fp4: T_pad %d must cover T and be a multiple of bn %d", T_pad, bn);
  Fp4Params p;
  p.alpha = alpha;
  p.g = static_cast<const float*>(g);
  p.sfa = static_cast<const uint8_t*>(wsf_tiled);
  p.sfb = static_cast<const uint8_t*>(xsf);
  p.out = static_cast<bf16*>(out);
  p.out32 = static_cast<float*>(out32);
  p.resid = static_cast<const bf16*>(resid);
  p.ws = static_cast<float*>(ws);
  p.counters = static_cast<uint32_t*>(counters);
  p.status = device_status_ptr();
  p.T = T; p.T_pad = T_pad; p.N = N; p.K = K; p.ldc = ldc; p.R = R;
  p.push = 0;
  p.pf_ptr = g_pf_ptr; p.pf_bytes = g_pf_bytes;
  p.preload = g_preload;
  p.trace = g_trace;
  g_pf_ptr = nullptr; g_pf_bytes = 0;
  p.group_list = nullptr; p.group_alpha = nullptr; p.group_tiles = 0; p.group_b = 0; p.grid_x = 0; p.group_out_stride = 0;
  memset(&p.comm, 0, sizeof(p.comm));
  if (comm_push) {
    const DgppComm* c = static_cast<const DgppComm*>(comm_push);
    DGPP_REQUIRE(T <= bn, "gemm_fp4 push: %d rows do not fit one token tile of %d", T, bn);
    DGPP_REQUIRE(N % 128 == 0 && N / 128 <= kCommMaxCtas, "gemm_fp4 push: N %d needs N %% 128 == 0 and <= %d tiles", N,
                 kCommMaxCtas);
    DGPP_REQUIRE(static_cast<size_t>(T) * N * 2 <= c->st.slot_bytes, "gemm_fp4 push: %d x %d exceeds the slot", T, N);
    p.push = 1;
    p.comm = c->st;
  }
  const int stages = K / 256;
  const int per = dgpp_ceil_div(stages, splits);
  p.stages_per_split = per;
  splits = dgpp_ceil_div(stages, per);
  // split-K without a workspace = the cluster form (partials through distributed shared memory)
  p.cluster_split = (splits > 1 && ws == nullptr) ? 1 : 0;
  DGPP_REQUIRE(splits == 1 || p.cluster_split || counters != nullptr, "gemm_fp4: split-K needs workspace and counters");
  CUtensorMap tA, tB;
  if (make_tmap_2d(&tA, wq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, K / 2, N, K / 2, 128, kF4BM, CU_TENSOR_MAP_SWIZZLE_128B))
    return -1;
  const int bnn = bn * R;  // MMA N: the R terms of a token tile are stacked
  if (make_tmap_2d(&tB, xq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, K / 2, static_cast<uint64_t>(R) * T_pad, K / 2, 128,
                   bnn, CU_TENSOR_MAP_SWIZZLE_128B))
    return -1;
  DGPP_REQUIRE(bnn <= 256 && bnn % 16 == 0, "gemm_fp4: token tile %d x %d terms does not fit one MMA", bn, R);
  switch (bnn) {
    case 16: return launch_fp4<16>(tA, tB, p, splits, st);
    case 32: return launch_fp4<32>(tA, tB, p, splits, st);
    case 48: return launch_fp4<48>(tA, tB, p, splits, st);
    case 64: return launch_fp4<64>(tA, tB, p, splits, st);
    case 96: return launch_fp4<96>(tA, tB, p, splits, st);
    case 128: return launch_fp4<128>(tA, tB, p, splits, st);
    case 192: return launch_fp4<192>(tA, tB, p, splits, st);
    case 256: return launch_fp4<256>(tA, tB, p, splits, st);
  }
  dgpp_set_error("gemm_fp4: unsupported bn %d", bn);
  return -1;
}

// Grouped (mixture-of-experts) form: wq / wsf_tiled hold `experts` matrices of [N, K] stacked along N; slot s of
// group_list (device, int32, `slots` entries, -1 = unused) names the expert whose matrix multiplies
//   group_b = 0: the one shared token tile xq (gate / up projection of every active expert)
//   group_b = 1: the slot's own token tile, xq rows [s * R * T_pad, (s + 1) * R * T_pad) (down projection)
// and writes out + s * group_out_stride + t * ldc + n.  T <= bn (one token tile per group); T_pad = bn.
DGPP_API int dgpp_gemm_fp4_grouped(int bn, const void* xq, const void* xsf, const void* g, int R, const void* wq,
                                   const void* wsf_tiled, const void* group_alpha, void* out, int ldc,
                                   int64_t group_out_stride, int T, int N, int K, int experts, int slots,
                                   const void* group_list, int group_b, int splits, void* ws, void* counters,
                                   cudaStream_t st) {
  DGPP_REQUIRE(K % 256 == 0 && N % 128 == 0, "gemm_fp4_grouped: K %d %% 256 and N %d %% 128 must be 0", K, N);
  DGPP_REQUIRE(R >= 1 && R <= 4 && T >= 1 && T <= bn, "gemm_fp4_grouped: %d rows / %d terms do not fit one token tile of %d", T, R, bn);
  DGPP_REQUIRE(experts >= 1 && slots >= 1 && group_list && out, "gemm_fp4_grouped: bad group arguments");
  DGPP_REQUIRE(splits >= 1 && (splits == 1 || (ws && counters)), "gemm_fp4_grouped: split-K needs workspace and counters");
  const int bnn = bn * R;
  DGPP_REQUIRE(bnn <= 256 && bnn % 16 == 0, "gemm_fp4_grouped: token tile %d x %d terms does not fit one MMA", bn, R);
  Fp4Params p;
  p.alpha = 1.f;
  p.g = static_cast<const float*>(g);
  p.sfa = static_cast<const uint8_t*>(wsf_tiled);
  p.sfb = static_cast<const uint8_t*>(xsf);
  p.out = static_cast<bf16*>(out);
  p.out32 = nullptr;
  p.resid = nullptr;
  p.ws = static_cast<float*>(ws);
  p.counters = static_cast<uint32_t*>(counters);
  p.status = device_status_ptr();
  p.T = T; p.T_pad = bn; p.N = N; p.K = K; p.ldc = ldc; p.R = R;
  p.push = 0;
  p.pf_ptr = g_pf_ptr; p.pf_bytes = g_pf_bytes;
  p.preload = g_preload;
  p.trace = g_trace;
  g_pf_ptr = nullptr; g_pf_bytes = 0;
  memset(&p.comm, 0, sizeof(p.comm));
  p.group_list = static_cast<const int32_t*>(group_list);
  p.group_alpha = static_cast<const float*>(group_alpha);
  p.group_tiles = N / 128;
  p.group_b = group_b;
  p.grid_x = slots * p.group_tiles;
  p.cluster_split = 0;
  p.group_out_stride = group_out_stride;
  const int stages = K / 256;
  const int per = dgpp_ceil_div(stages, splits);
  p.stages_per_split = per;
  splits = dgpp_ceil_div(stages, per);
  CUtensorMap tA, tB;
  if (make_tmap_2d(&tA, wq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, K / 2, static_cast<uint64_t>(experts) * N, K / 2, 128,
                   kF4BM, CU_TENSOR_MAP_SWIZZLE_128B))
    return -1;
  const uint64_t b_rows = static_cast<uint64_t>(R) * bn * (group_b ? slots : 1);
  if (make_tmap_2d(&tB, xq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, K / 2, b_rows, K / 2, 128, bnn, CU_TENSOR_MAP_SWIZZLE_128B))
    return -1;
  switch (bnn) {
    case 16: return launch_fp4<16>(tA, tB, p, splits, st);
    case 32: return launch_fp4<32>(tA, tB, p, splits, st);
    case 48: return launch_fp4<48>(tA, tB, p, splits, st);
    case 64: return launch_fp4<64>(tA, tB, p, splits, st);
    case 96: return launch_fp4<96>(tA, tB, p, splits, st);
    case 128: return launch_fp4<128>(tA, tB, p, splits, st);
    case 192: return launch_fp4<192>(tA, tB, p, splits, st);
    case 256: return launch_fp4<256>(tA, tB, p, splits, st);
  }
  dgpp_set_error("gemm_fp4_grouped: unsupported bn %d", bn);
  return -1;
}
