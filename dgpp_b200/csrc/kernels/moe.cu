// Mixture-of-experts control kernels: router, active-expert list, ordered combine.
//
//   moe_router_logits_kernel / moe_router_select_kernel
//                       fp32 logits = hidden . gate^T (bf16 operands, fp32 accumulation, warp per expert and 8 tokens,
//                       fixed shuffle tree); then one CTA per token: scores = sigmoid (or softmax) of the logits, selection on
//                       score + correction bias (group-limited when n_group > 1: a group's rank is the sum of its
//                       two best selection values, the best topk_group groups stay), weights from the UNCORRECTED
//                       scores, optional normalisation by (sum + 1e-20), times the routed scaling factor.  Ties go
//                       to the lower expert id; ids are emitted in ascending order = accumulation order.
//   moe_active_kernel   one CTA: experts used by any token -> ascending list padded with -1 (the grouped GEMM's
//                       slot list) and the inverse map expert -> slot
//   moe_combine_kernel  out[t] = bf16( sum_j w[t, j] * y[slot(id[t, j])][t] (+ shared[t]) ), fp32, ascending j
// The expert matrices themselves run through the grouped block-scaled GEMM (gemm_fp4.cu).
// (reference counterparts: src/kernels/glm_moe.cu:86-331 router, :1447 moe_accum_ordered_kernel.)
#include <math.h>

#include "common/common.h"
#include "common/dtypes.cuh"
#include "common/ptx.cuh"
#include "kernels/comm.cuh"

namespace dgpp {

constexpr int kMoeMaxExperts = 512;
constexpr int kMoeMaxTopK = 16;
constexpr int kRouterThreads = 256;

struct RouterArgs {
  const bf16* x;         // [T, H] (normed hidden)
  int64_t x_stride;
  const bf16* gate;      // [E, H]
  const float* bias;     // [E] selection correction, may be null
  int32_t* ids;          // [T, k] ascending
  float* weights;        // [T, k]
  float* logits_out;     // [T, E] optional (tests, auditing)
  int T, H, E, k, n_group, topk_group;
  int softmax, norm_topk;
  float scaling;
};

constexpr int kRouterRowsPerCta = 8;

// Router logits: grid (ceil(E / 8), ceil(T / 8)), 8 warps.  A warp owns one expert and up to 8 token rows: it walks the
// expert's gate row once (lane-strided 16-byte loads) and keeps one fp32 accumulator per row, so the gate matrix is
// read T / 8 times instead of T times and the work of a decode step spreads over E / 8 CTAs instead of T.  The
// accumulation order of every (token, expert) dot product (lane-strided fmaf chain, xor-shuffle tree) does not depend on
// the grid, so logits are identical for every batch composition.
__global__ void __launch_bounds__(kRouterThreads) moe_router_logits_kernel(RouterArgs a) {
  pdl_wait();
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const int e = blockIdx.x * (kRouterThreads / 32) + wid;
  const int t0 = blockIdx.y * kRouterRowsPerCta;
  if (e >= a.E) return;
  const int nt = min(kRouterRowsPerCta, a.T - t0);
  const bf16* gr = a.gate + static_cast<size_t>(e) * a.H;
  float acc[kRouterRowsPerCta];
#pragma unroll
  for (int r = 0; r < kRouterRowsPerCta; ++r) acc[r] = 0.f;
  for (int i = lane * 8; i < a.H; i += 32 * 8) {
    Pack16 gv;
    gv.u = *reinterpret_cast<const uint4*>(gr + i);
    float g[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) g[j] = bf16_to_f32(gv.h[j]);
#pragma unroll
    for (int r = 0; r < kRouterRowsPerCta; ++r) {
      if (r < nt) {
        Pack16 xv;
        xv.u = *reinterpret_cast<const uint4*>(a.x + static_cast<size_t>(t0 + r) * a.x_stride + i);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[r] = fmaf(bf16_to_f32(xv.h[j]), g[j], acc[r]);
      }
    }
  }
#pragma unroll
  for (int r = 0; r < kRouterRowsPerCta; ++r) {
    float v = acc[r];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0 && r < nt) a.logits_out[static_cast<size_t>(t0 + r) * a.E + e] = v;
  }
}

// Selection: one CTA per token over its row of logits.
__global__ void __launch_bounds__(kRouterThreads) moe_router_select_kernel(RouterArgs a) {
  __shared__ float score[kMoeMaxExperts];   // uncorrected
  __shared__ float sel[kMoeMaxExperts];     // selection value
  __shared__ float grp[64];
  __shared__ float wred[kRouterThreads / 32];
  __shared__ int pick_id[kMoeMaxTopK];
  pdl_wait();
  const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  for (int e = tid; e < a.E; e += kRouterThreads) score[e] = a.logits_out[static_cast<size_t>(t) * a.E + e];
  __syncthreads();
  if (a.softmax) {
    // softmax over all experts: max, then the sum of exp, each by a fixed tree (thread-strided partials, xor-shuffle
    // within the warp, the 8 warp results in warp order), so the value does not depend on timing
    __shared__ float mx_s, sum_s;
    float m = -INFINITY;
    for (int e = tid; e < a.E; e += kRouterThreads) m = fmaxf(m, score[e]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) wred[wid] = m;
    __syncthreads();
    if (tid == 0) {
      float mm = wred[0];
      for (int w = 1; w < kRouterThreads / 32; ++w) mm = fmaxf(mm, wred[w]);
      mx_s = mm;
    }
    __syncthreads();
    float sp = 0.f;
    for (int e = tid; e < a.E; e += kRouterThreads) sp += expf(score[e] - mx_s);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sp += __shfl_xor_sync(0xffffffffu, sp, o);
    if (lane == 0) wred[wid] = sp;
    __syncthreads();
    if (tid == 0) {
      float ss = 0.f;
      for (int w = 0; w < kRouterThreads / 32; ++w) ss += wred[w];
      sum_s = ss;
    }
    __syncthreads();
    for (int e = tid; e < a.E; e += kRouterThreads) score[e] = expf(score[e] - mx_s) / sum_s;
  } else {
    for (int e = tid; e < a.E; e += kRouterThreads) score[e] = 1.f / (1.f + expf(-score[e]));
  }
  __syncthreads();
  for (int e = tid; e < a.E; e += kRouterThreads) sel[e] = score[e] + (a.bias ? a.bias[e] : 0.f);
  __syncthreads();
  if (a.n_group > 1) {
    const int per = a.E / a.n_group;
    if (tid < a.n_group) {
      float b1 = -INFINITY, b2 = -INFINITY;
      for (int e = tid * per; e < (tid + 1) * per; ++e) {
        const float v = sel[e];
        if (v > b1) { b2 = b1; b1 = v; } else if (v > b2) { b2 = v; }
      }
      grp[tid] = b1 + (per > 1 ? b2 : 0.f);
    }
    __syncthreads();
    if (tid == 0) {
      // keep the topk_group best groups (ties to the lower group id); the others can no longer be selected
      bool keep[64];
      for (int g = 0; g < a.n_group; ++g) keep[g] = false;
      for (int r = 0; r < a.topk_group; ++r) {
        int best = -1;
        for (int g = 0; g < a.n_group; ++g)
          if (!keep[g] && (best < 0 || grp[g] > grp[best])) best = g;
        if (best >= 0) keep[best] = true;
      }
      for (int g = 0; g < a.n_group; ++g)
        if (!keep[g])
          for (int e = g * per; e < (g + 1) * per; ++e) sel[e] = -INFINITY;
    }
    __syncthreads();
  }
  // k rounds of arg-max by warp 0 (ties to the lower expert id)
  if (wid == 0) {
    for (int r = 0; r < a.k; ++r) {
      float bv = -INFINITY;
      int bi = 0x7fffffff;
      for (int e = lane; e < a.E; e += 32) {
        const float v = sel[e];
        if (v > bv || (v == bv && e < bi)) { bv = v; bi = e; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
      }
      if (lane == 0) {
        pick_id[r] = bi < a.E ? bi : 0;
        if (bi < a.E) sel[bi] = -INFINITY;
      }
      __syncwarp();
    }
    if (lane == 0) {
      // ascending ids (insertion sort, k <= 16), weights from the uncorrected scores
      for (int i = 1; i < a.k; ++i) {
        const int v = pick_id[i];
        int j = i - 1;
        while (j >= 0 && pick_id[j] > v) { pick_id[j + 1] = pick_id[j]; --j; }
        pick_id[j + 1] = v;
      }
      float sum = 0.f;
      for (int i = 0; i < a.k; ++i) sum += score[pick_id[i]];
      for (int i = 0; i < a.k; ++i) {
        float w = score[pick_id[i]];
        if (a.norm_topk) w = w / (sum + 1e-20f);
        a.ids[t * a.k + i] = pick_id[i];
        a.weights[t * a.k + i] = w * a.scaling;
      }
    }
  }
}

// ids: [T, k].  list: [slots] ascending active experts then -1; slot_of: [E]; n_active: [1].
__global__ void __launch_bounds__(512) moe_active_kernel(const int32_t* ids, int T, int k, int E, int slots,
                                                         int32_t* list, int32_t* slot_of, int32_t* n_active, int e_begin,
                                                         int e_end) {
  __shared__ int flag[kMoeMaxExperts];
  pdl_wait();
  const int tid = threadIdx.x;
  for (int e = tid; e < E; e += blockDim.x) flag[e] = 0;
  __syncthreads();
  for (int i = tid; i < T * k; i += blockDim.x) {
    const int e = ids[i];
    if (e >= 0 && e < E) flag[e] = 1;
  }
  __syncthreads();
  // expert parallelism: only experts [e_begin, e_end) live here; the list holds LOCAL indices (e - e_begin).
  // Ascending positions by a block-wide exclusive scan of the flags (thread e <-> expert e; E <= 512 = blockDim).
  __shared__ int warp_cnt[16];
  const int lane = tid & 31, wid = tid >> 5;
  const bool on = tid < E && flag[tid] && tid >= e_begin && tid < e_end;
  const unsigned bal = __ballot_sync(0xffffffffu, on);
  if (lane == 0) warp_cnt[wid] = __popc(bal);
  __syncthreads();
  int before = __popc(bal & ((1u << lane) - 1u)), total = 0;
  for (int w = 0; w < 16; ++w) {
    if (w < wid) before += warp_cnt[w];
    total += warp_cnt[w];
  }
  if (tid < E) {
    const bool listed = on && before < slots;
    slot_of[tid] = listed ? before : -1;
    if (listed) list[before] = tid - e_begin;
  }
  const int n = min(total, slots);
  if (tid == 0) *n_active = n;
  for (int sidx = n + tid; sidx < slots; sidx += blockDim.x) list[sidx] = -1;
}

// y: [slots, rows_per_slot, H] bf16; shared (optional): [T, H] bf16; out: [T, H] bf16.
__global__ void __launch_bounds__(256) moe_combine_kernel(const bf16* __restrict__ y, const bf16* __restrict__ shared,
                                                          const int32_t* __restrict__ ids, const float* __restrict__ w,
                                                          const int32_t* __restrict__ slot_of, bf16* __restrict__ out,
                                                          int T, int H, int k, int rows_per_slot) {
  pdl_wait();
  const int t = blockIdx.y;
  const int v = blockIdx.x * blockDim.x + threadIdx.x;   // 8-wide vector index
  if (v * 8 >= H) return;
  float acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.f;
  for (int i = 0; i < k; ++i) {
    const int e = ids[t * k + i];
    const int s = slot_of[e];
    if (s < 0) continue;
    const float wi = w[t * k + i];
    Pack16 p;
    p.u = *reinterpret_cast<const uint4*>(y + (static_cast<size_t>(s) * rows_per_slot + t) * H + v * 8);
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = fmaf(wi, bf16_to_f32(p.h[j]), acc[j]);
  }
  if (shared) {
    Pack16 p;
    p.u = *reinterpret_cast<const uint4*>(shared + static_cast<size_t>(t) * H + v * 8);
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] += bf16_to_f32(p.h[j]);
  }
  Pack16 o;
#pragma unroll
  for (int j = 0; j < 8; ++j) o.h[j] = f32_to_bf16(acc[j]);
  *reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * H + v * 8) = o.u;
}

// Expert-parallel combine fused with the all-reduce push: every rank holds a slice of the experts and computes, for
// ALL tokens, the weighted sum over ITS experts; instead of writing that partial locally, the CTA owning a 128-column
// tile stores it into slot `rank` of every rank's symmetric region and raises the tile flag there (the protocol of
// the tensor-parallel GEMM push).  The consumer is the fold + add + RMSNorm + quantise kernel of the next layer, so
// the combine, the cross-rank sum and the next norm need no separate collective launch.
// Experts that live on other ranks have slot_of[e] < 0 here and are skipped; `shared` is added by the rank that owns it.
// grid (H / 128), 128 threads; rows <= 16.
__global__ void __launch_bounds__(128) moe_combine_push_kernel(const bf16* __restrict__ y, const bf16* __restrict__ shared,
                                                               const int32_t* __restrict__ ids, const float* __restrict__ w,
                                                               const int32_t* __restrict__ slot_of, CommState comm, int T,
                                                               int H, int k, int rows_per_slot) {
  pdl_wait();
  const uint32_t epoch = *comm.epoch + 1;
  const int parity = epoch & 1;
  const int col0 = blockIdx.x * 128;
  for (int idx = threadIdx.x; idx < T * 16; idx += blockDim.x) {
    const int t = idx / 16, c = col0 + (idx % 16) * 8;
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int i = 0; i < k; ++i) {
      const int s = slot_of[ids[t * k + i]];
      if (s < 0) continue;
      const float wi = w[t * k + i];
      Pack16 p;
      p.u = *reinterpret_cast<const uint4*>(y + (static_cast<size_t>(s) * rows_per_slot + t) * H + c);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = fmaf(wi, bf16_to_f32(p.h[j]), acc[j]);
    }
    if (shared) {
      Pack16 p;
      p.u = *reinterpret_cast<const uint4*>(shared + static_cast<size_t>(t) * H + c);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += bf16_to_f32(p.h[j]);
    }
    Pack16 o;
#pragma unroll
    for (int j = 0; j < 8; ++j) o.h[j] = f32_to_bf16(acc[j]);
    for (int r = 0; r < comm.world; ++r) {
      const int dst = (comm.rank + r) % comm.world;
      st_v4_global(payload(comm, dst, parity, comm.rank) + (static_cast<size_t>(t) * H + c) * 2, o.u);
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < comm.world) st_release_sys(flag(comm, threadIdx.x, parity, comm.rank, blockIdx.x), epoch);
}

}  // namespace dgpp

using namespace dgpp;

DGPP_API int dgpp_moe_route(const void* x, int64_t x_stride, const void* gate, const void* bias, void* ids, void* weights,
                            void* logits_out, int T, int H, int E, int k, int n_group, int topk_group, int softmax,
                            int norm_topk, float scaling, cudaStream_t st) {
  DGPP_REQUIRE(E >= 1 && E <= kMoeMaxExperts && k >= 1 && k <= kMoeMaxTopK && k <= E, "moe_route: E %d / k %d unsupported", E, k);
  DGPP_REQUIRE(H % 8 == 0, "moe_route: hidden %d must be a multiple of 8", H);
  DGPP_REQUIRE(n_group <= 1 || (n_group <= 64 && E % n_group == 0 && topk_group >= 1 && topk_group <= n_group),
               "moe_route: bad grouping %d / %d", n_group, topk_group);
  if (T == 0) return 0;
  RouterArgs a;
  a.x = static_cast<const bf16*>(x); a.x_stride = x_stride;
  a.gate = static_cast<const bf16*>(gate);
  a.bias = static_cast<const float*>(bias);
  a.ids = static_cast<int32_t*>(ids);
  a.weights = static_cast<float*>(weights);
  a.logits_out = static_cast<float*>(logits_out);
  a.T = T; a.H = H; a.E = E; a.k = k; a.n_group = n_group; a.topk_group = topk_group;
  a.softmax = softmax; a.norm_topk = norm_topk; a.scaling = scaling;
  DGPP_REQUIRE(logits_out != nullptr, "moe_route: a [T, E] fp32 logits buffer is required");
  dim3 grid(dgpp_ceil_div(E, kRouterThreads / 32), dgpp_ceil_div(T, kRouterRowsPerCta));
  moe_router_logits_kernel<<<grid, kRouterThreads, 0, st>>>(a);
  DGPP_CUDA_OK(cudaGetLastError());
  moe_router_select_kernel<<<T, kRouterThreads, 0, st>>>(a);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

DGPP_API int dgpp_moe_active(const void* ids, int T, int k, int E, int slots, void* list, void* slot_of, void* n_active,
                             int e_begin, int e_end, cudaStream_t st) {
  DGPP_REQUIRE(E >= 1 && E <= kMoeMaxExperts && slots >= 1, "moe_active: bad sizes");
  moe_active_kernel<<<1, 512, 0, st>>>(static_cast<const int32_t*>(ids), T, k, E, slots, static_cast<int32_t*>(list),
                                       static_cast<int32_t*>(slot_of), static_cast<int32_t*>(n_active), e_begin,
                                       e_end > 0 ? e_end : E);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

DGPP_API int dgpp_moe_combine(const void* y, const void* shared, const void* ids, const void* w, const void* slot_of,
                              void* out, int T, int H, int k, int rows_per_slot, cudaStream_t st) {
  DGPP_REQUIRE(H % 8 == 0, "moe_combine: hidden %d must be a multiple of 8", H);
  if (T == 0) return 0;
  dim3 grid(dgpp_ceil_div(H / 8, 256), T);
  moe_combine_kernel<<<grid, 256, 0, st>>>(static_cast<const bf16*>(y), static_cast<const bf16*>(shared),
                                           static_cast<const int32_t*>(ids), static_cast<const float*>(w),
                                           static_cast<const int32_t*>(slot_of), static_cast<bf16*>(out), T, H, k,
                                           rows_per_slot);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

// Expert-parallel form of dgpp_moe_combine: pushes this rank's partial to every rank (see moe_combine_push_kernel).
DGPP_API int dgpp_moe_combine_push(const void* y, const void* shared, const void* ids, const void* w, const void* slot_of,
                                   void* comm, int T, int H, int k, int rows_per_slot, cudaStream_t st) {
  DGPP_REQUIRE(comm != nullptr, "moe_combine_push: communicator required");
  const DgppComm* c = static_cast<const DgppComm*>(comm);
  DGPP_REQUIRE(T >= 1 && T <= 16, "moe_combine_push: %d rows outside 1..16", T);
  DGPP_REQUIRE(H % 128 == 0 && H / 128 <= kCommMaxCtas && static_cast<size_t>(T) * H * 2 <= c->st.slot_bytes,
               "moe_combine_push: %d x %d does not fit the symmetric slot / flag table", T, H);
  moe_combine_push_kernel<<<H / 128, 128, 0, st>>>(static_cast<const bf16*>(y), static_cast<const bf16*>(shared),
                                                   static_cast<const int32_t*>(ids), static_cast<const float*>(w),
                                                   static_cast<const int32_t*>(slot_of), c->st, T, H, k, rows_per_slot);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}
