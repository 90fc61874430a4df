// Gated DeltaNet linear attention: causal depthwise convolution, gated delta-rule recurrence, gated RMSNorm.
//
// Per head the state S is [dk, dv] fp32.  For token t with decay a_t = exp(g_t), write strength b_t, unit-norm
// q_t, k_t (q also scaled by dk^-1/2) and value v_t:
//     S   <- a_t * S
//     u   =  b_t * (v_t - S^T k_t)          (what the memory does not already return for k_t)
//     S   <- S + k_t u^T
//     o_t =  S^T q_t
// Every column S[:, j] evolves on its own, so a (request, head) is split over dv / 32 CTAs; a thread keeps
// 16 rows of one column in registers for the whole token loop, 8 threads share a column (shuffle reductions in a
// fixed order).  The same kernel serves decode (one token per request) and chunked prefill (a run of tokens of one
// request, state carried in and out), so prefill and decode agree bit for bit.
//     g_t = -exp(A_log[h]) * softplus(alpha_t + dt_bias[h]),  b_t = sigmoid(beta_t)
// (reference counterparts: src/kernels/gdn_chunk.cu chunked scan, src/kernels/kda.cu recurrent step.)
#include <math.h>
#include <string.h>

#include "common/common.h"
#include "common/dtypes.cuh"
#include "common/ptx.cuh"

namespace dgpp {

constexpr int kGdnCols = 32;      // state columns per CTA
constexpr int kGdnParts = 8;      // threads per column
constexpr int kGdnThreads = kGdnCols * kGdnParts;
constexpr int kGdnChunk = 16;     // tokens staged in shared memory at a time

struct GdnArgs {
  const bf16* q;          // [T, hk * dk]   (after conv + SiLU)
  const bf16* k;          // [T, hk * dk]
  const bf16* v;          // [T, hv * dv]
  int64_t q_stride, k_stride, v_stride;
  const bf16* alpha;      // [T, hv] raw decay input
  const bf16* beta;       // [T, hv] raw write-strength input
  int64_t ab_stride;
  const float* A_log;     // [hv]
  const float* dt_bias;   // [hv]
  float* state;           // [slots, hv, dk, dv] fp32
  const int32_t* row_slot;   // [T] state slot of each row (decode) or null: all rows belong to `slot`
  int slot;
  bf16* out;              // [T, hv * dv]
  float* prep;            // scratch: qn [T, hk, dk] | kn [T, hk, dk] | decay [T, hv] | beta [T, hv]
  int T, hk, hv, dk, dv;
  int sequential;         // 1: rows are consecutive tokens of ONE request (prefill); 0: one token per request
  // speculative verify rows: seg > 0 = the rows come in runs of `seg` consecutive tokens, run r belonging to state slot
  // row_slot[r * seg]; snap (optional): [T, hv, dk, dv] receives the state after every row, so a partial accept can
  // roll the slot back to any row of its run without replaying it
  int seg;
  float* snap;
  // KDA form (per-channel decay): gate_k [T, hv * dk] raw gate rows, dt_bias then has hv * dk entries and the decay of key
  // channel c of head h is exp(lower_bound / (1 + exp(-exp(A_log[h]) * (gate_k[t, h, c] + dt_bias[h, c])))); alpha unused
  const bf16* gate_k;
  int64_t gate_stride;
  float lower_bound;
};

// Token-parallel part: unit-norm q (scaled by dk^-1/2) and k per key head, decay and write strength per value head.
// grid (T, hk + 1): blocks y < hk normalise one key head (dk threads), block y == hk does the per-head scalars.
template <int DK>
__global__ void __launch_bounds__(DK) gdn_prep_kernel(GdnArgs a) {
  __shared__ float red[2][DK / 32];
  pdl_wait();
  const int t = blockIdx.x, tid = threadIdx.x;
  float* qn = a.prep;
  float* kn = qn + static_cast<size_t>(a.T) * a.hk * DK;
  float* dec = kn + static_cast<size_t>(a.T) * a.hk * DK;
  float* bet = dec + static_cast<size_t>(a.T) * a.hv;
  if (static_cast<int>(blockIdx.y) > a.hk) {
    // KDA: per-channel decay of value head (blockIdx.y - hk - 1), one thread per key channel
    const int h = static_cast<int>(blockIdx.y) - a.hk - 1;
    float* deck = bet + static_cast<size_t>(a.T) * a.hv;
    const float x = bf16_to_f32(a.gate_k[static_cast<size_t>(t) * a.gate_stride + h * DK + tid]) + a.dt_bias[h * DK + tid];
    const float g = a.lower_bound / (1.f + expf(-expf(a.A_log[h]) * x));
    deck[(static_cast<size_t>(t) * a.hv + h) * DK + tid] = expf(g);
    return;
  }
  if (blockIdx.y == static_cast<unsigned>(a.hk) && a.gate_k) {
    for (int h = tid; h < a.hv; h += DK) {
      dec[static_cast<size_t>(t) * a.hv + h] = 1.f;
      bet[static_cast<size_t>(t) * a.hv + h] = 1.f / (1.f + expf(-bf16_to_f32(a.beta[static_cast<size_t>(t) * a.ab_stride + h])));
    }
    return;
  }
  if (blockIdx.y == static_cast<unsigned>(a.hk)) {
    for (int h = tid; h < a.hv; h += DK) {
      const float al = bf16_to_f32(a.alpha[static_cast<size_t>(t) * a.ab_stride + h]) + a.dt_bias[h];
      const float softplus = al > 20.f ? al : log1pf(expf(al));
      dec[static_cast<size_t>(t) * a.hv + h] = expf(-expf(a.A_log[h]) * softplus);
      bet[static_cast<size_t>(t) * a.hv + h] = 1.f / (1.f + expf(-bf16_to_f32(a.beta[static_cast<size_t>(t) * a.ab_stride + h])));
    }
    return;
  }
  const int h = blockIdx.y;
  const float qv = bf16_to_f32(a.q[static_cast<size_t>(t) * a.q_stride + h * DK + tid]);
  const float kv = bf16_to_f32(a.k[static_cast<size_t>(t) * a.k_stride + h * DK + tid]);
  float q2 = qv * qv, k2 = kv * kv;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    q2 += __shfl_xor_sync(0xffffffffu, q2, o);
    k2 += __shfl_xor_sync(0xffffffffu, k2, o);
  }
  if ((tid & 31) == 0) { red[0][tid >> 5] = q2; red[1][tid >> 5] = k2; }
  __syncthreads();
  float qs = 0.f, ks = 0.f;
#pragma unroll
  for (int w = 0; w < DK / 32; ++w) { qs += red[0][w]; ks += red[1][w]; }
  const size_t o = (static_cast<size_t>(t) * a.hk + h) * DK + tid;
  qn[o] = qv * rsqrtf(qs + 1e-6f) * rsqrtf(static_cast<float>(DK));
  kn[o] = kv * rsqrtf(ks + 1e-6f);
}

// Sequential part.  Thread (column j, part p) keeps state rows p, p + 8, p + 16, ... of column j in registers; the
// normalised keys / queries of kGdnChunk tokens are staged in shared memory (one block-wide sync pair per chunk).
template <int DK, bool KDA = false>
__global__ void __launch_bounds__(kGdnThreads) gdn_recurrent_kernel(GdnArgs a) {
  constexpr int PER = DK / kGdnParts;          // state rows per thread
  __shared__ float ks[kGdnChunk][DK], qs[kGdnChunk][DK];
  __shared__ float dks[KDA ? kGdnChunk : 1][KDA ? DK : 1];     // KDA: per-channel decays of the staged tokens
  __shared__ float vs[kGdnChunk][kGdnCols], ds[kGdnChunk], bs[kGdnChunk];
  pdl_wait();
  const int tid = threadIdx.x;
  const int col = tid / kGdnParts, part = tid % kGdnParts;
  const int h = blockIdx.y, j = blockIdx.x * kGdnCols + col;
  const int hk_idx = h / (a.hv / a.hk);        // value heads share key heads in groups
  const int first = a.seg > 0 ? blockIdx.z * a.seg : (a.sequential ? 0 : blockIdx.z);
  const int last = a.seg > 0 ? first + a.seg : (a.sequential ? a.T : blockIdx.z + 1);
  const int slot0 = a.row_slot ? a.row_slot[first] : a.slot;
  const float* qn = a.prep;
  const float* kn = qn + static_cast<size_t>(a.T) * a.hk * DK;
  const float* dec = kn + static_cast<size_t>(a.T) * a.hk * DK;
  const float* bet = dec + static_cast<size_t>(a.T) * a.hv;
  const float* deck = bet + static_cast<size_t>(a.T) * a.hv;
  float* sp = a.state + ((static_cast<size_t>(slot0) * a.hv + h) * DK) * a.dv + j;
  float s[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) s[i] = sp[static_cast<size_t>(part + kGdnParts * i) * a.dv];
  for (int t0 = first; t0 < last; t0 += kGdnChunk) {
    const int n = min(kGdnChunk, last - t0);
    __syncthreads();                            // the previous chunk's readers are done
    for (int i = tid; i < n * DK; i += kGdnThreads) {
      const int tt = i / DK, d = i % DK;
      const size_t o = (static_cast<size_t>(t0 + tt) * a.hk + hk_idx) * DK + d;
      ks[tt][d] = kn[o];
      qs[tt][d] = qn[o];
      if (KDA) dks[tt][d] = deck[(static_cast<size_t>(t0 + tt) * a.hv + h) * DK + d];
    }
    for (int i = tid; i < n * kGdnCols; i += kGdnThreads) {
      const int tt = i / kGdnCols, c = i % kGdnCols;
      vs[tt][c] = bf16_to_f32(a.v[static_cast<size_t>(t0 + tt) * a.v_stride + h * a.dv + blockIdx.x * kGdnCols + c]);
    }
    if (tid < n) {
      ds[tid] = dec[static_cast<size_t>(t0 + tid) * a.hv + h];
      bs[tid] = bet[static_cast<size_t>(t0 + tid) * a.hv + h];
    }
    __syncthreads();
    for (int tt = 0; tt < n; ++tt) {
      const float decay = ds[tt];
      float m = 0.f;
#pragma unroll
      for (int i = 0; i < PER; ++i) {
        s[i] *= KDA ? dks[tt][part + kGdnParts * i] : decay;
        m = fmaf(s[i], ks[tt][part + kGdnParts * i], m);
      }
#pragma unroll
      for (int o = kGdnParts / 2; o > 0; o >>= 1) m += __shfl_xor_sync(0xffffffffu, m, o);
      const float u = bs[tt] * (vs[tt][col] - m);
      float ov = 0.f;
#pragma unroll
      for (int i = 0; i < PER; ++i) {
        s[i] = fmaf(ks[tt][part + kGdnParts * i], u, s[i]);
        ov = fmaf(s[i], qs[tt][part + kGdnParts * i], ov);
      }
#pragma unroll
      for (int o = kGdnParts / 2; o > 0; o >>= 1) ov += __shfl_xor_sync(0xffffffffu, ov, o);
      if (part == 0) a.out[static_cast<size_t>(t0 + tt) * a.hv * a.dv + h * a.dv + j] = f32_to_bf16(ov);
      if (a.snap) {
        float* np = a.snap + ((static_cast<size_t>(t0 + tt) * a.hv + h) * DK) * a.dv + j;
#pragma unroll
        for (int i = 0; i < PER; ++i) np[static_cast<size_t>(part + kGdnParts * i) * a.dv] = s[i];
      }
    }
  }
#pragma unroll
  for (int i = 0; i < PER; ++i) sp[static_cast<size_t>(part + kGdnParts * i) * a.dv] = s[i];
}

// Causal depthwise convolution (kernel width W <= 4) + SiLU over channels, with the last W - 1 inputs of every
// channel carried per state slot (two passes: outputs in parallel over tokens, then the tail update).  x: [T, C] bf16 rows; sequential = 1: consecutive tokens of one request.
struct ConvArgs {
  const bf16* x;
  int64_t x_stride;
  const bf16* w;        // [C, W]
  const bf16* bias;     // [C] or null
  float* state;         // [slots, W - 1, C] fp32 (oldest first)
  const int32_t* row_slot;
  int slot;
  bf16* out;            // [T, C]
  int T, C, W, sequential;
  int seg;              // > 0: runs of `seg` consecutive tokens per request (see GdnArgs::seg)
  float* snap;          // optional [T, W - 1, C]: the tail after every row of a run
};

// Output pass, parallel over tokens and channels: out[t, c] = silu(b + sum_i w[i] * X(t - (W - 1) + i)), where X(u)
// is row u of the chunk for u >= 0 and the carried tail (state) for u < 0.  grid (C / 256, rows).
__global__ void __launch_bounds__(256) gdn_conv_kernel(ConvArgs a) {
  pdl_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= a.C) return;
  const int t = blockIdx.y;
  const int run0 = a.seg > 0 ? t - t % a.seg : (a.sequential ? 0 : t);     // first row of this row's run
  const int slot = a.row_slot ? a.row_slot[run0] : a.slot;
  const float* st = a.state + static_cast<size_t>(slot) * (a.W - 1) * a.C + c;
  float acc = a.bias ? bf16_to_f32(a.bias[c]) : 0.f;
  for (int i = 0; i < a.W; ++i) {
    const int u = (t - run0) - (a.W - 1) + i;                   // index inside the run; batched single tokens: only the row itself is new
    float xv;
    if (u >= 0) xv = bf16_to_f32(a.x[static_cast<size_t>(run0 + u) * a.x_stride + c]);
    else xv = st[static_cast<size_t>(a.W - 1 + u) * a.C];
    acc = fmaf(bf16_to_f32(a.w[c * a.W + i]), xv, acc);
  }
  a.out[static_cast<size_t>(t) * a.C + c] = f32_to_bf16(acc / (1.f + expf(-acc)));
}

// State pass (after the output pass): the tail becomes the last W - 1 inputs.  One thread per (channel, request):
// it reads everything it needs before it writes, so the in-place shift is safe.  grid (C / 256, sequential ? 1 : rows).
__global__ void __launch_bounds__(256) gdn_conv_state_kernel(ConvArgs a) {
  pdl_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= a.C) return;
  const int r = blockIdx.y;                                     // run (segment / batched mode) or 0
  const int n = a.seg > 0 ? a.seg : (a.sequential ? a.T : 1);   // new inputs of this request
  const int run0 = a.seg > 0 ? r * a.seg : (a.sequential ? 0 : r);
  const int slot = a.row_slot ? a.row_slot[run0] : a.slot;
  float* st = a.state + static_cast<size_t>(slot) * (a.W - 1) * a.C + c;
  float nv[3] = {0.f, 0.f, 0.f};
  if (a.snap) {
    // the tail after the first j inputs of the run, j = 1..n (a rollback target for every row)
    for (int j = 1; j <= n; ++j)
      for (int i = 0; i < a.W - 1; ++i) {
        const int u = j - (a.W - 1) + i;
        const float v = u >= 0 ? bf16_to_f32(a.x[static_cast<size_t>(run0 + u) * a.x_stride + c])
                               : st[static_cast<size_t>(a.W - 1 + u) * a.C];
        a.snap[(static_cast<size_t>(run0 + j - 1) * (a.W - 1) + i) * a.C + c] = v;
      }
  }
  for (int i = 0; i < a.W - 1; ++i) {
    const int u = n - (a.W - 1) + i;                            // input index that lands in tail position i
    nv[i] = u >= 0 ? bf16_to_f32(a.x[static_cast<size_t>(run0 + u) * a.x_stride + c])
                   : st[static_cast<size_t>(a.W - 1 + u) * a.C];
  }
  for (int i = 0; i < a.W - 1; ++i) st[static_cast<size_t>(i) * a.C] = nv[i];
}

// Decode form (one new token per request, no snapshots): output and tail shift in one pass.  A thread owns one
// (request, channel): it reads the tail and the new input, writes the output, then the shifted tail.  grid (C / 256, rows).
__global__ void __launch_bounds__(256) gdn_conv_decode_kernel(ConvArgs a) {
  pdl_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= a.C) return;
  const int t = blockIdx.y;
  float* st = a.state + static_cast<size_t>(a.row_slot[t]) * (a.W - 1) * a.C + c;
  float v[4];
  for (int i = 0; i < a.W - 1; ++i) v[i] = st[static_cast<size_t>(i) * a.C];
  v[a.W - 1] = bf16_to_f32(a.x[static_cast<size_t>(t) * a.x_stride + c]);
  float acc = a.bias ? bf16_to_f32(a.bias[c]) : 0.f;
  for (int i = 0; i < a.W; ++i) acc = fmaf(bf16_to_f32(a.w[c * a.W + i]), v[i], acc);
  a.out[static_cast<size_t>(t) * a.C + c] = f32_to_bf16(acc / (1.f + expf(-acc)));
  for (int i = 0; i < a.W - 1; ++i) st[static_cast<size_t>(i) * a.C] = v[i + 1];
}

// out[t, h, :] = rmsnorm(o[t, h, :]) * w * silu(z[t, h, :]); one warp per (row, head).
__global__ void __launch_bounds__(256) gated_rmsnorm_kernel(const bf16* __restrict__ o, const bf16* __restrict__ z,
                                                            int64_t z_stride, const bf16* __restrict__ w,
                                                            bf16* __restrict__ out, int rows, int heads, int d, float eps) {
  pdl_wait();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= rows * heads) return;
  const int t = warp / heads, h = warp % heads;
  const bf16* op = o + (static_cast<size_t>(t) * heads + h) * d;
  const bf16* zp = z + static_cast<size_t>(t) * z_stride + h * d;
  float ss = 0.f;
  for (int i = lane; i < d; i += 32) { const float f = bf16_to_f32(op[i]); ss += f * f; }
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, s);
  const float rstd = rsqrtf(ss / static_cast<float>(d) + eps);
  for (int i = lane; i < d; i += 32) {
    const float n = bf16_to_f32(f32_to_bf16(bf16_to_f32(op[i]) * rstd)) * bf16_to_f32(w[i]);
    const float zv = bf16_to_f32(zp[i]);
    out[(static_cast<size_t>(t) * heads + h) * d + i] = f32_to_bf16(n * (zv / (1.f + expf(-zv))));
  }
}

}  // namespace dgpp

using namespace dgpp;

static int gdn_recurrent_launch(const void* q, int64_t q_stride, const void* k, int64_t k_stride, const void* v,
                                int64_t v_stride, const void* alpha, const void* beta, int64_t ab_stride,
                                const void* A_log, const void* dt_bias, void* state, const void* row_slot, int slot,
                                void* out, void* prep, int T, int hk, int hv, int dk, int dv, int sequential, int seg,
                                void* snap, cudaStream_t st, const void* gate_k = nullptr, int64_t gate_stride = 0,
                                float lower_bound = 0.f) {
  DGPP_REQUIRE(gate_k == nullptr || dk == 64 || dk == 128, "kda: key dim %d unsupported (64 or 128)", dk);
  DGPP_REQUIRE(seg == 0 || (row_slot && T % seg == 0 && !sequential), "gdn: runs of %d rows need row_slot and T %% seg == 0", seg);
  DGPP_REQUIRE(dk == 64 || dk == 128 || dk == 256, "gdn: key dim %d unsupported", dk);
  DGPP_REQUIRE(dv % kGdnCols == 0 && hk > 0 && hv % hk == 0, "gdn: bad head geometry hk %d hv %d dv %d", hk, hv, dv);
  DGPP_REQUIRE(sequential || row_slot, "gdn: batched single-token rows need row_slot");
  DGPP_REQUIRE(prep != nullptr, "gdn: scratch of T * (2 * hk * dk + 2 * hv) floats required");
  if (T == 0) return 0;
  GdnArgs a;
  a.q = static_cast<const bf16*>(q); a.k = static_cast<const bf16*>(k); a.v = static_cast<const bf16*>(v);
  a.q_stride = q_stride; a.k_stride = k_stride; a.v_stride = v_stride;
  a.alpha = static_cast<const bf16*>(alpha); a.beta = static_cast<const bf16*>(beta); a.ab_stride = ab_stride;
  a.A_log = static_cast<const float*>(A_log); a.dt_bias = static_cast<const float*>(dt_bias);
  a.state = static_cast<float*>(state);
  a.row_slot = static_cast<const int32_t*>(row_slot);
  a.slot = slot;
  a.out = static_cast<bf16*>(out);
  a.prep = static_cast<float*>(prep);
  a.T = T; a.hk = hk; a.hv = hv; a.dk = dk; a.dv = dv; a.sequential = sequential;
  a.seg = seg; a.snap = static_cast<float*>(snap);
  a.gate_k = static_cast<const bf16*>(gate_k); a.gate_stride = gate_stride; a.lower_bound = lower_bound;
  dim3 pgrid(T, hk + 1 + (gate_k ? hv : 0));
  if (dk == 64) gdn_prep_kernel<64><<<pgrid, 64, 0, st>>>(a);
  else if (dk == 128) gdn_prep_kernel<128><<<pgrid, 128, 0, st>>>(a);
  else gdn_prep_kernel<256><<<pgrid, 256, 0, st>>>(a);
  DGPP_CUDA_OK(cudaGetLastError());
  dim3 grid(dv / kGdnCols, hv, seg > 0 ? T / seg : (sequential ? 1 : T));
  if (gate_k) {
    if (dk == 64) gdn_recurrent_kernel<64, true><<<grid, kGdnThreads, 0, st>>>(a);
    else gdn_recurrent_kernel<128, true><<<grid, kGdnThreads, 0, st>>>(a);
    DGPP_CUDA_OK(cudaGetLastError());
    return 0;
  }
  if (dk == 64) gdn_recurrent_kernel<64><<<grid, kGdnThreads, 0, st>>>(a);
  else if (dk == 128) gdn_recurrent_kernel<128><<<grid, kGdnThreads, 0, st>>>(a);
  else gdn_recurrent_kernel<256><<<grid, kGdnThreads, 0, st>>>(a);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

DGPP_API int dgpp_gdn_recurrent(const void* q, int64_t q_stride, const void* k, int64_t k_stride, const void* v,
                                int64_t v_stride, const void* alpha, const void* beta, int64_t ab_stride,
                                const void* A_log, const void* dt_bias, void* state, const void* row_slot, int slot,
                                void* out, void* prep, int T, int hk, int hv, int dk, int dv, int sequential,
                                cudaStream_t st) {
  return gdn_recurrent_launch(q, q_stride, k, k_stride, v, v_stride, alpha, beta, ab_stride, A_log, dt_bias, state, row_slot,
                              slot, out, prep, T, hk, hv, dk, dv, sequential, 0, nullptr, st);
}

// Runs of `seg` consecutive rows per request (speculative verify), with per-row state snapshots in `snap` (may be null).
DGPP_API int dgpp_gdn_recurrent_runs(const void* q, int64_t q_stride, const void* k, int64_t k_stride, const void* v,
                                     int64_t v_stride, const void* alpha, const void* beta, int64_t ab_stride,
                                     const void* A_log, const void* dt_bias, void* state, const void* row_slot, void* out,
                                     void* prep, int T, int hk, int hv, int dk, int dv, int seg, void* snap,
                                     cudaStream_t st) {
  DGPP_REQUIRE(seg >= 1, "gdn_recurrent_runs: run length %d", seg);
  return gdn_recurrent_launch(q, q_stride, k, k_stride, v, v_stride, alpha, beta, ab_stride, A_log, dt_bias, state, row_slot,
                              0, out, prep, T, hk, hv, dk, dv, 0, seg, snap, st);
}

// KDA (per-channel decay) recurrence: gate [T, hv * dk] raw gate rows, dt_bias [hv * dk], beta [T, hv] raw write strengths,
// lower_bound < 0; prep: T * (2 hk dk + 2 hv + hv dk) floats.  seg / snap as in dgpp_gdn_recurrent_runs (seg 0: `sequential`
// decides between one request's consecutive tokens and one token per request).
DGPP_API int dgpp_kda_recurrent(const void* q, int64_t q_stride, const void* k, int64_t k_stride, const void* v,
                                int64_t v_stride, const void* gate, int64_t gate_stride, const void* beta, int64_t beta_stride,
                                const void* A_log, const void* dt_bias, float lower_bound, void* state, const void* row_slot,
                                int slot, void* out, void* prep, int T, int hk, int hv, int dk, int dv, int sequential, int seg,
                                void* snap, cudaStream_t st) {
  DGPP_REQUIRE(gate != nullptr && lower_bound < 0.f, "kda: gate rows and a negative lower bound required");
  return gdn_recurrent_launch(q, q_stride, k, k_stride, v, v_stride, beta, beta, beta_stride, A_log, dt_bias, state, row_slot,
                              slot, out, prep, T, hk, hv, dk, dv, seg > 0 ? 0 : sequential, seg, snap, st, gate, gate_stride,
                              lower_bound);
}

// Token-parallel preparation alone (unit-norm q / k, decay, write strength into `prep`); the chunked scan
// (gdn_chunk.cu) consumes the same scratch layout.
DGPP_API int dgpp_gdn_prep(const void* q, int64_t q_stride, const void* k, int64_t k_stride, const void* alpha,
                           const void* beta, int64_t ab_stride, const void* A_log, const void* dt_bias, void* prep, int T,
                           int hk, int hv, int dk, cudaStream_t st) {
  DGPP_REQUIRE(dk == 64 || dk == 128 || dk == 256, "gdn: key dim %d unsupported", dk);
  DGPP_REQUIRE(prep != nullptr, "gdn: scratch of T * (2 * hk * dk + 2 * hv) floats required");
  if (T == 0) return 0;
  GdnArgs a;
  memset(&a, 0, sizeof(a));
  a.q = static_cast<const bf16*>(q); a.k = static_cast<const bf16*>(k);
  a.q_stride = q_stride; a.k_stride = k_stride;
  a.alpha = static_cast<const bf16*>(alpha); a.beta = static_cast<const bf16*>(beta); a.ab_stride = ab_stride;
  a.A_log = static_cast<const float*>(A_log); a.dt_bias = static_cast<const float*>(dt_bias);
  a.prep = static_cast<float*>(prep);
  a.T = T; a.hk = hk; a.hv = hv; a.dk = dk;
  dim3 pgrid(T, hk + 1);
  if (dk == 64) gdn_prep_kernel<64><<<pgrid, 64, 0, st>>>(a);
  else if (dk == 128) gdn_prep_kernel<128><<<pgrid, 128, 0, st>>>(a);
  else gdn_prep_kernel<256><<<pgrid, 256, 0, st>>>(a);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

static int gdn_conv_launch(const void* x, int64_t x_stride, const void* w, const void* bias, void* state,
                           const void* row_slot, int slot, void* out, int T, int C, int W, int sequential, int seg,
                           void* snap, cudaStream_t st) {
  DGPP_REQUIRE(seg == 0 || (row_slot && T % seg == 0 && !sequential), "gdn_conv: runs of %d rows need row_slot and T %% seg == 0", seg);
  DGPP_REQUIRE(W >= 1 && W <= 4, "gdn_conv: kernel width %d outside 1..4", W);
  DGPP_REQUIRE(sequential || row_slot, "gdn_conv: batched single-token rows need row_slot");
  if (T == 0) return 0;
  ConvArgs a;
  a.x = static_cast<const bf16*>(x); a.x_stride = x_stride;
  a.w = static_cast<const bf16*>(w); a.bias = static_cast<const bf16*>(bias);
  a.state = static_cast<float*>(state);
  a.row_slot = static_cast<const int32_t*>(row_slot);
  a.slot = slot;
  a.out = static_cast<bf16*>(out);
  a.T = T; a.C = C; a.W = W; a.sequential = sequential;
  a.seg = seg; a.snap = static_cast<float*>(snap);
  if (!sequential && seg == 0 && !snap) {       // batched decode rows: one kernel
    gdn_conv_decode_kernel<<<dim3(dgpp_ceil_div(C, 256), T), 256, 0, st>>>(a);
    DGPP_CUDA_OK(cudaGetLastError());
    return 0;
  }
  gdn_conv_kernel<<<dim3(dgpp_ceil_div(C, 256), T), 256, 0, st>>>(a);
  DGPP_CUDA_OK(cudaGetLastError());
  if (W > 1) {
    gdn_conv_state_kernel<<<dim3(dgpp_ceil_div(C, 256), seg > 0 ? T / seg : (sequential ? 1 : T)), 256, 0, st>>>(a);
    DGPP_CUDA_OK(cudaGetLastError());
  }
  return 0;
}

DGPP_API int dgpp_gdn_conv(const void* x, int64_t x_stride, const void* w, const void* bias, void* state,
                           const void* row_slot, int slot, void* out, int T, int C, int W, int sequential,
                           cudaStream_t st) {
  return gdn_conv_launch(x, x_stride, w, bias, state, row_slot, slot, out, T, C, W, sequential, 0, nullptr, st);
}

DGPP_API int dgpp_gdn_conv_runs(const void* x, int64_t x_stride, const void* w, const void* bias, void* state,
                                const void* row_slot, void* out, int T, int C, int W, int seg, void* snap, cudaStream_t st) {
  DGPP_REQUIRE(seg >= 1, "gdn_conv_runs: run length %d", seg);
  return gdn_conv_launch(x, x_stride, w, bias, state, row_slot, 0, out, T, C, W, 0, seg, snap, st);
}

DGPP_API int dgpp_gated_rmsnorm(const void* o, const void* z, int64_t z_stride, const void* w, void* out, int rows,
                                int heads, int d, float eps, cudaStream_t st) {
  if (rows == 0) return 0;
  const int warps = rows * heads;
  gated_rmsnorm_kernel<<<dgpp_ceil_div(warps * 32, 256), 256, 0, st>>>(
      static_cast<const bf16*>(o), static_cast<const bf16*>(z), z_stride, static_cast<const bf16*>(w),
      static_cast<bf16*>(out), rows, heads, d, eps);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}
