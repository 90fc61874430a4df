// Activation producer + NVFP4 residual-term quantiser, one thread-block CLUSTER per row.
//
// A decode batch has only a handful of rows, so one CTA per row leaves the GPU idle; here the K columns of a row
// are split over the CTAs of a cluster (up to 8), and the two row-wide reductions (sum of squares for RMSNorm,
// max |x| for the activation scale) go through distributed shared memory: every CTA stores its partial into the
// shared memory of every CTA of the cluster, the cluster synchronises, and every CTA folds its own copy of the
// partials in ascending CTA order (so all CTAs compute bit-identical row statistics, and nobody reads a peer's
// shared memory after the barrier).
//
// Modes, output layout and arithmetic are those of fused_act_quant_kernel in gemm_fp4.cu:
//   0 plain rows, 1 swiglu([gate | up]), 2 rmsnorm(resid + delta) * w
//   q rows [token tile][term][token], scale factors in tcgen05.cp atom order per token tile.
#include <cooperative_groups.h>
#include <string.h>

#include "common/common.h"
#include "common/dtypes.cuh"
#include "common/ptx.cuh"
#include "kernels/comm.cuh"

namespace cg = cooperative_groups;

namespace dgpp {

constexpr int kAqThreads = 128;
constexpr int kAqAtom = 512;

struct ClusterQuantArgs {
  const bf16* in;
  int64_t in_stride;
  const bf16* delta;
  const bf16* w;
  bf16* resid_out;
  bf16* x_out;
  uint8_t* q;
  uint8_t* sf;
  float* g;
  int T, T_pad, K, R, bn, cl;
  DeviceStatus* status;
  float eps, limit, alpha;     // alpha > 0: gate * sigmoid(alpha * gate) * (up + 1) in the swiglu mode
  int one_plus_w;
  // MODE 2 with fold = 1: `delta` is not read from memory but folded from the W partial tiles that the
  // tensor-parallel GEMMs pushed into this rank's symmetric region (ascending rank order, fp32, one bf16
  // rounding: the bits an all-reduce would have produced).  The kernel waits for the tile flags it needs and its
  // last CTA advances the collective epoch.
  int fold;
  CommState comm;
  // Grouped rows (mixture-of-experts): row t belongs to slot t / bn; rows of inactive slots (group_list[slot] < 0)
  // and rows t % bn >= group_rows are skipped.
  const int32_t* group_list;
  int group_rows;
  // MODE 3: the row is the decode-attention output, folded here from the split-KV partials (max / sum pairs and
  // unnormalised accumulators per (row, head, split)) in the arithmetic of the stand-alone combine kernel, so the
  // combine launch and one round trip of the attention output disappear.
  const float* part_ml;
  const float* part_acc;
  int splits, hq, D;
};

__device__ __forceinline__ float warp_red(float v, bool is_max) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float u = __shfl_xor_sync(0xffffffffu, v, o);
    v = is_max ? fmaxf(v, u) : v + u;
  }
  return v;
}

template <int MODE>
__global__ void __launch_bounds__(kAqThreads) act_quant_cluster_kernel(ClusterQuantArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* seg = reinterpret_cast<bf16*>(smem_raw);  // this CTA's K / cl columns
  __shared__ float wred[kAqThreads / 32];
  // partials of every CTA of the cluster, PUSHED here by their owners before the cluster barrier: [0][i] sum of
  // squares, [1][i] max |x| of CTA i's segment.  After the barrier a CTA reads only its own copy, so no CTA's shared
  // memory is touched by a peer once the barrier has passed and no closing barrier is needed.
  __shared__ float part[2][8];
  cg::cluster_group cluster = cg::this_cluster();
  pdl_wait();
  const int c = blockIdx.x, t = blockIdx.y, tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  if (a.group_list && (a.group_list[t / a.bn] < 0 || t % a.bn >= a.group_rows)) return;   // whole cluster leaves together
  const int cl = a.cl, K = a.K, kseg = K / cl, k0 = c * kseg, nvec = kseg / 8;
  auto cta_reduce = [&](float v, bool is_max) {
    v = warp_red(v, is_max);
    if (lane == 0) wred[wid] = v;
    __syncthreads();
    float r = wred[0];
    for (int i = 1; i < kAqThreads / 32; ++i) r = is_max ? fmaxf(r, wred[i]) : r + wred[i];
    __syncthreads();
    return r;
  };
  auto cluster_push = [&](int slot, float v) {
    if (tid < cl) *cluster.map_shared_rank(&part[slot][c], tid) = v;
  };
  auto cluster_fold = [&](int slot, bool is_max) {
    float r = 0.f;
    for (int i = 0; i < cl; ++i) r = is_max ? fmaxf(r, part[slot][i]) : r + part[slot][i];
    return r;
  };
  float amax = 0.f;
  uint32_t fold_epoch = 0;
  int fold_parity = 0;
  if (MODE == 2 && a.fold) {
    fold_epoch = *a.comm.epoch + 1;
    fold_parity = fold_epoch & 1;
    const int tile0 = k0 / 128, ntile = (k0 + kseg - 1) / 128 - tile0 + 1;
    for (int i = tid; i < ntile * a.comm.world; i += kAqThreads) {
      const int src = i / ntile, tl = tile0 + i % ntile;
      if (!wait_flag(flag(a.comm, a.comm.rank, fold_parity, src, tl), fold_epoch)) {
        if (atomicCAS(&a.status->code, 0, kTimeoutPeerFlag) == 0) a.status->detail = src;
        atomicAdd(&a.status->count, 1);
      }
    }
    __syncthreads();
  }
  if (MODE == 2) {
    const bf16* rr = a.in + static_cast<size_t>(t) * a.in_stride + k0;
    float ss = 0.f, pm = 0.f;
    for (int i = tid; i < nvec; i += kAqThreads) {
      Pack16 x;
      x.u = reinterpret_cast<const uint4*>(rr)[i];
      if (a.fold) {
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
        for (int r = 0; r < a.comm.world; ++r) {
          Pack16 d;
          d.u = ld_v4_global_volatile(payload(a.comm, a.comm.rank, fold_parity, r) +
                                      (static_cast<size_t>(t) * K + k0) * 2 + static_cast<size_t>(i) * 16);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] += bf16_to_f32(d.h[j]);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) x.h[j] = f32_to_bf16(bf16_to_f32(x.h[j]) + bf16_to_f32(f32_to_bf16(acc[j])));
        reinterpret_cast<uint4*>(a.resid_out + static_cast<size_t>(t) * K + k0)[i] = x.u;
      } else if (a.delta) {
        Pack16 d;
        d.u = reinterpret_cast<const uint4*>(a.delta + static_cast<size_t>(t) * K + k0)[i];
#pragma unroll
        for (int j = 0; j < 8; ++j) x.h[j] = f32_to_bf16(bf16_to_f32(x.h[j]) + bf16_to_f32(d.h[j]));
        reinterpret_cast<uint4*>(a.resid_out + static_cast<size_t>(t) * K + k0)[i] = x.u;
      }
      Pack16 wv;
      wv.u = reinterpret_cast<const uint4*>(a.w + k0)[i];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float f = bf16_to_f32(x.h[j]);
        ss += f * f;
        float gw = bf16_to_f32(wv.h[j]);
        if (a.one_plus_w) gw += 1.f;
        pm = fmaxf(pm, fabsf(f * gw));
      }
      reinterpret_cast<uint4*>(seg)[i] = x.u;
    }
    ss = cta_reduce(ss, false);
    pm = cta_reduce(pm, true);
    cluster_push(0, ss);
    cluster_push(1, pm);
    cluster.sync();
    const float rstd = rsqrtf(cluster_fold(0, false) / static_cast<float>(K) + a.eps);
    // Row scale from a bound instead of the exact maximum of the normalised row: |bf16(bf16(x rstd) w)| <=
    // |x w| rstd (1 + 2^-8)^2, so max |x w| * rstd * 1.0079 covers every element (at most 0.8 % above the true
    // maximum) and is known from this single pass: no second row-wide reduction.
    amax = cluster_fold(1, true) * rstd * 1.0079f;
    for (int i = tid; i < nvec; i += kAqThreads) {
      Pack16 x, ww;
      x.u = reinterpret_cast<const uint4*>(seg)[i];
      ww.u = reinterpret_cast<const uint4*>(a.w + k0)[i];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float nrm = bf16_to_f32(f32_to_bf16(bf16_to_f32(x.h[j]) * rstd));
        float gw = bf16_to_f32(ww.h[j]);
        if (a.one_plus_w) gw += 1.f;
        x.h[j] = f32_to_bf16(nrm * gw);
      }
      reinterpret_cast<uint4*>(seg)[i] = x.u;
      if (a.x_out) reinterpret_cast<uint4*>(a.x_out + static_cast<size_t>(t) * K + k0)[i] = x.u;
    }
  } else if (MODE == 3) {
    for (int i = tid; i < nvec; i += kAqThreads) {
      const int col = k0 + i * 8, h = col / a.D, d0 = col % a.D;
      const size_t rh = static_cast<size_t>(t) * a.hq + h;
      float mm = -INFINITY;
      for (int sp = 0; sp < a.splits; ++sp) mm = fmaxf(mm, a.part_ml[(rh * a.splits + sp) * 2]);
      float ll = 0.f, acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
      for (int sp = 0; sp < a.splits; ++sp) {
        const float ms = a.part_ml[(rh * a.splits + sp) * 2];
        const float cw = ms == -INFINITY ? 0.f : __expf(ms - mm);
        ll += a.part_ml[(rh * a.splits + sp) * 2 + 1] * cw;
        const float4* pa = reinterpret_cast<const float4*>(a.part_acc + (rh * a.splits + sp) * a.D + d0);
        const float4 p0 = pa[0], p1 = pa[1];
        acc[0] += p0.x * cw; acc[1] += p0.y * cw; acc[2] += p0.z * cw; acc[3] += p0.w * cw;
        acc[4] += p1.x * cw; acc[5] += p1.y * cw; acc[6] += p1.z * cw; acc[7] += p1.w * cw;
      }
      Pack16 x;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        x.h[j] = f32_to_bf16(ll > 0.f ? acc[j] / ll : 0.f);
        amax = fmaxf(amax, fabsf(bf16_to_f32(x.h[j])));
      }
      reinterpret_cast<uint4*>(seg)[i] = x.u;
      if (a.x_out) reinterpret_cast<uint4*>(a.x_out + static_cast<size_t>(t) * K + k0)[i] = x.u;
    }
  } else {
    const bf16* rr = a.in + static_cast<size_t>(t) * a.in_stride + k0;
    for (int i = tid; i < nvec; i += kAqThreads) {
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
      reinterpret_cast<uint4*>(seg)[i] = x.u;
      if (a.x_out) reinterpret_cast<uint4*>(a.x_out + static_cast<size_t>(t) * K + k0)[i] = x.u;
    }
  }
  if (MODE != 2) {
    amax = cta_reduce(amax, true);
    cluster_push(1, amax);
    cluster.sync();
    amax = cluster_fold(1, true);
  } else {
    __syncthreads();      // the normalised segment is complete in shared memory
  }
  const float gs = amax > 0.f ? amax / (6.f * 256.f) : 1.f;
  if (c == 0 && tid == 0) a.g[t] = gs;
  const float inv_g = 1.f / gs;
  const int stages = K / 256;
  const int atoms = a.R * a.bn > 128 ? 2 : 1;
  const int tile = t / a.bn, m = t % a.bn;
  for (int gl = tid; gl < kseg / 16; gl += kAqThreads) {
    const int gi = k0 / 16 + gl;
    Pack16 lo, hi;
    lo.u = reinterpret_cast<const uint4*>(seg + gl * 16)[0];
    hi.u = reinterpret_cast<const uint4*>(seg + gl * 16)[1];
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
      a.sf[atom_idx * kAqAtom + (mm & 31) * 16 + (mm >> 5) * 4 + fi] = sb;
    }
  }
  if (MODE == 2 && a.fold && tid == 0) {
    __threadfence();
    if (atomicAdd(a.comm.done_ctas, 1u) == gridDim.x * gridDim.y - 1) {
      *a.comm.done_ctas = 0;
      *a.comm.epoch = fold_epoch;
      __threadfence();
    }
  }
}

template <int MODE>
static int launch_cluster(const ClusterQuantArgs& a, cudaStream_t st) {
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(a.cl, a.T, 1);
  cfg.blockDim = dim3(kAqThreads, 1, 1);
  cfg.dynamicSmemBytes = static_cast<size_t>(a.K / a.cl) * 2;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = a.cl;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  DGPP_CUDA_OK(cudaLaunchKernelEx(&cfg, act_quant_cluster_kernel<MODE>, a));
  return 0;
}

}  // namespace dgpp

using namespace dgpp;

// Same contract as dgpp_act_quant_nvfp4, row split over a cluster of `cl` CTAs (1, 2, 4 or 8; K / cl % 16 == 0).
DGPP_API int dgpp_act_quant_nvfp4_cluster(int mode, const void* in, int64_t in_stride, const void* delta,
                                          const void* w, void* resid_out, void* x_out, void* q, void* sf, void* g,
                                          int T, int T_pad, int K, int R, int bn, int cl, float eps, float limit,
                                          float alpha, int one_plus_w, void* comm_fold, const void* group_list, int group_rows,
                                          cudaStream_t st) {
  DGPP_REQUIRE(K % 256 == 0, "act_quant: K %d must be a multiple of 256", K);
  DGPP_REQUIRE(cl == 1 || cl == 2 || cl == 4 || cl == 8, "act_quant: cluster size %d not in {1,2,4,8}", cl);
  DGPP_REQUIRE((K / cl) % 16 == 0 && K % cl == 0, "act_quant: K %d does not split over %d CTAs", K, cl);
  DGPP_REQUIRE(R >= 1 && R <= 4 && R * bn <= 256, "act_quant: bad terms %d / tile %d", R, bn);
  DGPP_REQUIRE(T_pad % bn == 0 && T_pad >= T, "act_quant: T_pad %d must be a multiple of bn %d and >= T", T_pad, bn);
  DGPP_REQUIRE(static_cast<size_t>(K / cl) * 2 <= 48 * 1024, "act_quant: segment too large");
  if (T == 0) return 0;
  ClusterQuantArgs a;
  a.in = static_cast<const bf16*>(in);
  a.in_stride = in_stride;
  a.delta = static_cast<const bf16*>(delta);
  a.w = static_cast<const bf16*>(w);
  a.resid_out = static_cast<bf16*>(resid_out);
  a.x_out = static_cast<bf16*>(x_out);
  a.q = static_cast<uint8_t*>(q);
  a.sf = static_cast<uint8_t*>(sf);
  a.g = static_cast<float*>(g);
  a.T = T; a.T_pad = T_pad; a.K = K; a.R = R; a.bn = bn; a.cl = cl; a.eps = eps; a.limit = limit; a.alpha = alpha;
  a.one_plus_w = one_plus_w;
  a.status = device_status_ptr();
  a.group_list = static_cast<const int32_t*>(group_list);
  a.group_rows = group_rows;
  a.fold = 0;
  memset(&a.comm, 0, sizeof(a.comm));
  if (comm_fold) {
    const DgppComm* c = static_cast<const DgppComm*>(comm_fold);
    DGPP_REQUIRE(mode == 2, "act_quant: the all-reduce fold exists for the add + RMSNorm mode only");
    DGPP_REQUIRE(resid_out != nullptr, "act_quant fold: resid_out required");
    DGPP_REQUIRE(K % 128 == 0 && K / 128 <= kCommMaxCtas && static_cast<size_t>(T) * K * 2 <= c->st.slot_bytes,
                 "act_quant fold: %d x %d does not fit the symmetric slot / flag table", T, K);
    a.fold = 1;
    a.comm = c->st;
  }
  if (mode == 0) return launch_cluster<0>(a, st);
  if (mode == 1) return launch_cluster<1>(a, st);
  if (mode == 2) return launch_cluster<2>(a, st);
  dgpp_set_error("act_quant: unknown mode %d", mode);
  return -1;
}

// Decode attention epilogue: fold the split-KV partials of dgpp_attn_decode_tc / dgpp_attn_decode (called with a null
// output) and quantise the rows for the o projection in one launch.  K = hq * d; x_out (optional) receives the bf16
// attention output [T, K].
DGPP_API int dgpp_attn_combine_quant(const void* part_ml, const void* part_acc, int splits, int hq, int d, void* x_out,
                                     void* q, void* sf, void* g, int T, int T_pad, int R, int bn, int cl,
                                     cudaStream_t st) {
  const int K = hq * d;
  DGPP_REQUIRE(part_ml && part_acc && splits >= 1, "attn_combine_quant: partials required");
  DGPP_REQUIRE(K % 256 == 0 && d % 8 == 0, "attn_combine_quant: hq %d x d %d must give K %% 256 == 0", hq, d);
  DGPP_REQUIRE(cl == 1 || cl == 2 || cl == 4 || cl == 8, "attn_combine_quant: cluster size %d not in {1,2,4,8}", cl);
  DGPP_REQUIRE((K / cl) % 16 == 0 && K % cl == 0, "attn_combine_quant: K %d does not split over %d CTAs", K, cl);
  DGPP_REQUIRE(R >= 1 && R <= 4 && R * bn <= 256, "attn_combine_quant: bad terms %d / tile %d", R, bn);
  DGPP_REQUIRE(T_pad % bn == 0 && T_pad >= T, "attn_combine_quant: T_pad %d must be a multiple of bn %d and >= T", T_pad, bn);
  DGPP_REQUIRE(static_cast<size_t>(K / cl) * 2 <= 48 * 1024, "attn_combine_quant: segment too large");
  if (T == 0) return 0;
  ClusterQuantArgs a;
  memset(&a, 0, sizeof(a));
  a.x_out = static_cast<bf16*>(x_out);
  a.q = static_cast<uint8_t*>(q);
  a.sf = static_cast<uint8_t*>(sf);
  a.g = static_cast<float*>(g);
  a.T = T; a.T_pad = T_pad; a.K = K; a.R = R; a.bn = bn; a.cl = cl; a.eps = 0.f; a.limit = 0.f; a.alpha = 0.f;
  a.status = device_status_ptr();
  a.part_ml = static_cast<const float*>(part_ml);
  a.part_acc = static_cast<const float*>(part_acc);
  a.splits = splits; a.hq = hq; a.D = d;
  return launch_cluster<3>(a, st);
}
