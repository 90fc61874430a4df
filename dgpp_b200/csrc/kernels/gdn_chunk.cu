// Gated DeltaNet, chunked form of the delta-rule recurrence for prefill (a run of consecutive tokens of one request).
//
// Same recurrence as gdn_recurrent_kernel (gdn.cu), per head with state S [dk, dv], decay a_t, write strength b_t:
//     S_t = a_t S_{t-1} + k_t u_t^T,   u_t = b_t (v_t - (a_t S_{t-1})^T k_t),   o_t = S_t^T q_t
// Over a chunk of C = 64 tokens with G_i = sum_{j<=i} log a_j (so gamma_i / gamma_j = exp(G_i - G_j) <= 1 for j <= i)
// and S_0 the state at the chunk start, the u_t solve a unit lower-triangular system:
//     (I + L) U = B (V - diag(gamma) K S_0),        L_ij = b_i exp(G_i - G_j) (k_i . k_j)   (j < i)
//     U  = U0 - W S_0,   U0 = T B V,   W = T B diag(gamma) K,   T = (I + L)^-1
//     O  = diag(gamma) Q S_0 + P U,                 P_ij = exp(G_i - G_j) (q_i . k_j)        (j <= i)
//     S_C = gamma_C S_0 + (diag(gamma_C / gamma) K)^T U
// Kernel 1 (gdn_chunk_prep_kernel) is parallel over (chunk, head): it builds L and P from K K^T and Q K^T, inverts
// I + L by forward substitution in shared memory and leaves W, U0, P and G in scratch.  Kernel 2
// (gdn_chunk_state_kernel) walks the chunks of a head in order, one CTA per (head, 32 state columns), with the state
// slice resident in shared memory: three small GEMMs per chunk instead of 64 dependent token steps.
// All arithmetic is fp32 on the CUDA cores with fixed summation orders (deterministic); against the token-sequential
// kernel the results differ by fp32 re-association only.
// (reference counterparts: src/kernels/gdn_chunk.cu:70 gdn_chunk_prep_kernel, :316 gdn_chunk_state_kernel.)
#include <math.h>

#include "common/common.h"
#include "common/dtypes.cuh"
#include "common/ptx.cuh"

namespace dgpp {

constexpr int kGcC = 64;          // tokens per chunk
constexpr int kGcCols = 32;       // state columns per CTA of the sequential kernel
constexpr int kGcThreads = 256;

struct GdnChunkArgs {
  const float* qn;        // [T, hk, dk] unit-norm queries (scaled by dk^-1/2)
  const float* kn;        // [T, hk, dk] unit-norm keys
  const float* dec;       // [T, hv] decay a_t
  const float* bet;       // [T, hv] write strength b_t
  const bf16* v;          // [T, hv * dv]
  int64_t v_stride;
  float* W;               // scratch [chunks, hv, C, dk]
  float* U0;              // scratch [chunks, hv, C, dv]
  float* P;               // scratch [chunks, hv, C, C]
  float* G;               // scratch [chunks, hv, C] cumulative log decay within the chunk
  float* state;           // [hv, dk, dv] of the request's slot
  bf16* out;              // [T, hv * dv]
  int T, hk, hv, dk, dv, chunks;
};

// ------------------------------------------------------------------------------------------------ kernel 1
// grid (chunks, hv), 256 threads.  Shared memory: Ks [C][DK + 4], Xs [C][DK + 4] (queries, later values), Ls [C][C + 1],
// Ts [C][C + 1], g[C], b[C].
template <int DK>
__global__ void __launch_bounds__(kGcThreads) gdn_chunk_prep_kernel(GdnChunkArgs a) {
  constexpr int LD = DK + 4, LC = kGcC + 1;
  extern __shared__ __align__(16) float gsm[];
  float* Ks = gsm;
  float* Xs = Ks + kGcC * LD;
  float* Ls = Xs + kGcC * LD;
  float* Ts = Ls + kGcC * LC;
  float* gs = Ts + kGcC * LC;
  float* bs = gs + kGcC;
  pdl_wait();
  const int c = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int hk_idx = h / (a.hv / a.hk);
  const int t0 = c * kGcC, n = min(kGcC, a.T - t0);
  // keys, queries (rows beyond the run are zero: they neither read nor write the memory)
  for (int i = tid; i < kGcC * (DK / 4); i += kGcThreads) {
    const int r = i / (DK / 4), q4 = i % (DK / 4);
    float4 kv = make_float4(0.f, 0.f, 0.f, 0.f), qv = kv;
    if (r < n) {
      const size_t o = (static_cast<size_t>(t0 + r) * a.hk + hk_idx) * DK + q4 * 4;
      kv = *reinterpret_cast<const float4*>(a.kn + o);
      qv = *reinterpret_cast<const float4*>(a.qn + o);
    }
    *reinterpret_cast<float4*>(Ks + r * LD + q4 * 4) = kv;
    *reinterpret_cast<float4*>(Xs + r * LD + q4 * 4) = qv;
  }
  if (tid < kGcC) {
    // cumulative log decay of the chunk: two warps load 32 tokens each and scan them, the second adds the first's total
    const int r = tid;
    float g = r < n ? logf(a.dec[static_cast<size_t>(t0 + r) * a.hv + h]) : 0.f;
    bs[r] = r < n ? a.bet[static_cast<size_t>(t0 + r) * a.hv + h] : 0.f;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float u = __shfl_up_sync(0xffffffffu, g, o);
      if ((r & 31) >= o) g += u;
    }
    gs[r] = g;
  }
  __syncthreads();
  if (tid >= 32 && tid < kGcC) gs[tid] += gs[31];
  __syncthreads();
  float* Gout = a.G + (static_cast<size_t>(c) * a.hv + h) * kGcC;
  if (tid < kGcC) Gout[tid] = gs[tid];
  // A = K K^T and Q K^T on a 16 x 16 thread grid, 4 x 4 outputs per thread
  {
    const int ty = tid / 16, tx = tid % 16;
    float kk[4][4], qk[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) kk[i][j] = qk[i][j] = 0.f;
    for (int d = 0; d < DK; d += 4) {
      float4 kr[4], qr[4], kc[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        kr[i] = *reinterpret_cast<const float4*>(Ks + (ty + 16 * i) * LD + d);
        qr[i] = *reinterpret_cast<const float4*>(Xs + (ty + 16 * i) * LD + d);
        kc[i] = *reinterpret_cast<const float4*>(Ks + (tx + 16 * i) * LD + d);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          kk[i][j] += kr[i].x * kc[j].x + kr[i].y * kc[j].y + kr[i].z * kc[j].z + kr[i].w * kc[j].w;
          qk[i][j] += qr[i].x * kc[j].x + qr[i].y * kc[j].y + qr[i].z * kc[j].z + qr[i].w * kc[j].w;
        }
    }
    float* Pout = a.P + (static_cast<size_t>(c) * a.hv + h) * kGcC * kGcC;
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int r = ty + 16 * i, cc = tx + 16 * j;
        const float e = cc <= r ? expf(gs[r] - gs[cc]) : 0.f;
        Ls[r * LC + cc] = cc < r ? bs[r] * e * kk[i][j] : 0.f;
        Pout[r * kGcC + cc] = e * qk[i][j];
      }
  }
  __syncthreads();
  // T = (I + L)^-1 by forward substitution: row i = e_i - sum_{j < i} L[i][j] * row j.  Thread c owns column c.
  if (tid < kGcC) {
    for (int i = 0; i < kGcC; ++i) {
      float acc = i == tid ? 1.f : 0.f;
      for (int j = tid; j < i; ++j) acc -= Ls[i * LC + j] * Ts[j * LC + tid];    // (rows j < column index are zero)
      Ts[i * LC + tid] = i >= tid ? acc : 0.f;
      __syncwarp();
    }
  }
  __syncthreads();
  // values into Xs (scaled by b), keys scaled by b * gamma in place
  for (int i = tid; i < kGcC * DK; i += kGcThreads) {
    const int r = i / DK, d = i % DK;
    Ks[r * LD + d] *= bs[r] * expf(gs[r]);
  }
  const int DV = a.dv;
  float* Wout = a.W + (static_cast<size_t>(c) * a.hv + h) * kGcC * DK;
  float* Uout = a.U0 + (static_cast<size_t>(c) * a.hv + h) * kGcC * DV;
  // W = T K' : [C, DK], 256 threads -> thread (ty = tid / 32: 8 rows, tx = tid % 32: DK / 32 columns)
  __syncthreads();
  {
    const int ty = tid / 32, tx = tid % 32;
    constexpr int CW = DK / 32;
    float acc[8][CW];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int j = 0; j < CW; ++j) acc[i][j] = 0.f;
    for (int j = 0; j < kGcC; ++j) {
      float kv[CW];
#pragma unroll
      for (int q = 0; q < CW; ++q) kv[q] = Ks[j * LD + tx + 32 * q];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float t = Ts[(ty * 8 + i) * LC + j];
#pragma unroll
        for (int q = 0; q < CW; ++q) acc[i][q] += t * kv[q];
      }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int q = 0; q < CW; ++q) Wout[(ty * 8 + i) * DK + tx + 32 * q] = acc[i][q];
  }
  // U0 = T (B V) : [C, DV] in column panels of DK columns (Xs holds one panel)
  for (int p0 = 0; p0 < DV; p0 += DK) {
    const int pw = min(DK, DV - p0);
    __syncthreads();
    for (int i = tid; i < kGcC * pw; i += kGcThreads) {
      const int r = i / pw, d = i % pw;
      Xs[r * LD + d] = r < n ? bs[r] * bf16_to_f32(a.v[static_cast<size_t>(t0 + r) * a.v_stride + h * DV + p0 + d]) : 0.f;
    }
    __syncthreads();
    const int ty = tid / 32, tx = tid % 32;
    constexpr int CW = DK / 32;
    float acc[8][CW];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int j = 0; j < CW; ++j) acc[i][j] = 0.f;
    for (int j = 0; j < kGcC; ++j) {
      float vv[CW];
#pragma unroll
      for (int q = 0; q < CW; ++q) vv[q] = (tx + 32 * q) < pw ? Xs[j * LD + tx + 32 * q] : 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float t = Ts[(ty * 8 + i) * LC + j];
#pragma unroll
        for (int q = 0; q < CW; ++q) acc[i][q] += t * vv[q];
      }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int q = 0; q < CW; ++q)
        if (tx + 32 * q < pw) Uout[(ty * 8 + i) * DV + p0 + tx + 32 * q] = acc[i][q];
  }
}

// ------------------------------------------------------------------------------------------------ kernel 2
// grid (dv / 32, hv), 256 threads; the CTA owns state columns [32 * blockIdx.x, +32) of head blockIdx.y for the whole
// run.  Shared memory: S [DK][32], two operand buffers A[2][C][DK + 4] (W, Q, K of a chunk pass through them in turn:
// while one is multiplied the next is copied in with cp.async), Ps [C][C + 4], U [C][32], g[2][C].
// Output tiles are [C, 32]: thread (ty = tid / 8 -> rows 2 ty, 2 ty + 1; tx = tid % 8 -> columns 4 tx .. 4 tx + 3).
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const uint32_t d = smem_u32(dst);
  const int n = valid ? 16 : 0;           // 0 source bytes: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

template <int DK>
__global__ void __launch_bounds__(kGcThreads) gdn_chunk_state_kernel(GdnChunkArgs a) {
  constexpr int LD = DK + 4, LP = kGcC + 4;
  extern __shared__ __align__(16) float gsm[];
  float* Ss = gsm;                          // [DK][32]
  float* Ab = Ss + DK * kGcCols;            // [2][C][LD]
  float* Ps = Ab + 2 * kGcC * LD;           // [C][LP]
  float* Us = Ps + kGcC * LP;               // [C][32]
  float* gb = Us + kGcC * kGcCols;          // [2][C]
  pdl_wait();
  const int tid = threadIdx.x, h = blockIdx.y, j0 = blockIdx.x * kGcCols;
  const int hk_idx = h / (a.hv / a.hk);
  const int ty = tid / 8, tx = tid % 8;
  float* sp = a.state + (static_cast<size_t>(h) * DK) * a.dv + j0;
  for (int i = tid; i < DK * kGcCols; i += kGcThreads) Ss[i] = sp[static_cast<size_t>(i / kGcCols) * a.dv + i % kGcCols];
  // asynchronous copy of C rows of DK floats (rows >= n are zero-filled) into operand buffer `buf`
  auto load_rows = [&](int buf, const float* src, int64_t row_stride, int n) {
    float* dst = Ab + buf * kGcC * LD;
    for (int i = tid; i < kGcC * (DK / 4); i += kGcThreads) {
      const int r = i / (DK / 4), q4 = i % (DK / 4);
      cp_async16(dst + r * LD + q4 * 4, src + static_cast<size_t>(r < n ? r : 0) * row_stride + q4 * 4, r < n);
    }
  };
  auto load_w = [&](int buf, int c) {      // W of chunk c and the chunk's cumulative log decay
    const size_t ch = static_cast<size_t>(c) * a.hv + h;
    load_rows(buf, a.W + ch * kGcC * DK, DK, kGcC);
    if (tid < kGcC / 4) cp_async16(gb + (c & 1) * kGcC + tid * 4, a.G + ch * kGcC + tid * 4, true);
    cp_async_commit();
  };
  auto load_qp = [&](int buf, int c, int t0, int n) {
    const size_t ch = static_cast<size_t>(c) * a.hv + h;
    load_rows(buf, a.qn + (static_cast<size_t>(t0) * a.hk + hk_idx) * DK, static_cast<int64_t>(a.hk) * DK, n);
    for (int i = tid; i < kGcC * (kGcC / 4); i += kGcThreads) {
      const int r = i / (kGcC / 4), q4 = i % (kGcC / 4);
      cp_async16(Ps + r * LP + q4 * 4, a.P + ch * kGcC * kGcC + r * kGcC + q4 * 4, true);
    }
    cp_async_commit();
  };
  // acc[2][4] += A[rows 2 ty, 2 ty + 1][0..DK) . Ss[0..DK)[4 tx ..]
  auto rows_times_state = [&](const float* As, float (&acc)[2][4]) {
#pragma unroll 4
    for (int d = 0; d < DK; d += 4) {
      const float4 a0 = *reinterpret_cast<const float4*>(As + (2 * ty) * LD + d);
      const float4 a1 = *reinterpret_cast<const float4*>(As + (2 * ty + 1) * LD + d);
      const float av0[4] = {a0.x, a0.y, a0.z, a0.w}, av1[4] = {a1.x, a1.y, a1.z, a1.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float4 s4 = *reinterpret_cast<const float4*>(Ss + (d + e) * kGcCols + 4 * tx);
        acc[0][0] += av0[e] * s4.x; acc[0][1] += av0[e] * s4.y; acc[0][2] += av0[e] * s4.z; acc[0][3] += av0[e] * s4.w;
        acc[1][0] += av1[e] * s4.x; acc[1][1] += av1[e] * s4.y; acc[1][2] += av1[e] * s4.z; acc[1][3] += av1[e] * s4.w;
      }
    }
  };
  int buf = 0;
  load_w(buf, 0);
  for (int c = 0; c < a.chunks; ++c) {
    const int t0 = c * kGcC, n = min(kGcC, a.T - t0);
    const size_t ch = static_cast<size_t>(c) * a.hv + h;
    const float* gs = gb + (c & 1) * kGcC;
    // ---- U = U0 - W S          (W in Ab[buf]; meanwhile Q and P stream into the other buffer)
    float4 u0[2];
#pragma unroll
    for (int i = 0; i < 2; ++i)
      u0[i] = *reinterpret_cast<const float4*>(a.U0 + ch * kGcC * a.dv + static_cast<size_t>(2 * ty + i) * a.dv + j0 + 4 * tx);
    cp_async_wait_all();
    __syncthreads();                                   // W landed; the previous chunk's readers of Ps / Us / Ab[buf ^ 1] are done
    load_qp(buf ^ 1, c, t0, n);
    {
      float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
      rows_times_state(Ab + buf * kGcC * LD, acc);
#pragma unroll
      for (int i = 0; i < 2; ++i)
        *reinterpret_cast<float4*>(Us + (2 * ty + i) * kGcCols + 4 * tx) =
            make_float4(u0[i].x - acc[i][0], u0[i].y - acc[i][1], u0[i].z - acc[i][2], u0[i].w - acc[i][3]);
    }
    buf ^= 1;
    cp_async_wait_all();
    __syncthreads();                                   // Q, P landed; U complete; W's readers are done
    // ---- O = diag(gamma) Q S + P U          (meanwhile K streams into the buffer W left)
    load_rows(buf ^ 1, a.kn + (static_cast<size_t>(t0) * a.hk + hk_idx) * DK, static_cast<int64_t>(a.hk) * DK, n);
    cp_async_commit();
    {
      float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
      rows_times_state(Ab + buf * kGcC * LD, acc);
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const float gm = expf(gs[2 * ty + i]);
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[i][e] *= gm;
      }
#pragma unroll 4
      for (int j = 0; j < kGcC; j += 4) {
        const float4 p0 = *reinterpret_cast<const float4*>(Ps + (2 * ty) * LP + j);
        const float4 p1 = *reinterpret_cast<const float4*>(Ps + (2 * ty + 1) * LP + j);
        const float pv0[4] = {p0.x, p0.y, p0.z, p0.w}, pv1[4] = {p1.x, p1.y, p1.z, p1.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float4 u4 = *reinterpret_cast<const float4*>(Us + (j + e) * kGcCols + 4 * tx);
          acc[0][0] += pv0[e] * u4.x; acc[0][1] += pv0[e] * u4.y; acc[0][2] += pv0[e] * u4.z; acc[0][3] += pv0[e] * u4.w;
          acc[1][0] += pv1[e] * u4.x; acc[1][1] += pv1[e] * u4.y; acc[1][2] += pv1[e] * u4.z; acc[1][3] += pv1[e] * u4.w;
        }
      }
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int r = 2 * ty + i;
        if (r < n) {
          Pack16 o;
          o.h[0] = f32_to_bf16(acc[i][0]); o.h[1] = f32_to_bf16(acc[i][1]);
          o.h[2] = f32_to_bf16(acc[i][2]); o.h[3] = f32_to_bf16(acc[i][3]);
          *reinterpret_cast<uint2*>(a.out + static_cast<size_t>(t0 + r) * a.hv * a.dv + h * a.dv + j0 + 4 * tx) =
              make_uint2(o.w[0], o.w[1]);
        }
      }
    }
    __syncthreads();                                   // every reader of U (P U) is done before U is rescaled
    // ---- U' = diag(gamma_C / gamma) U   (each thread scales the 8 values it wrote; rows beyond n have u = 0)
    {
      const float gl = gs[kGcC - 1];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int r = 2 * ty + i;
        const float f = expf(gl - gs[r]);
        float4* u = reinterpret_cast<float4*>(Us + r * kGcCols + 4 * tx);
        float4 v = *u;
        v.x *= f; v.y *= f; v.z *= f; v.w *= f;
        *u = v;
      }
    }
    buf ^= 1;
    cp_async_wait_all();
    __syncthreads();                                   // K landed; U' complete; Q's readers are done
    // ---- S = gamma_C S + K^T U'          (meanwhile the next chunk's W streams into the buffer Q left)
    if (c + 1 < a.chunks) load_w(buf ^ 1, c + 1);
    {
      const float* Ks = Ab + buf * kGcC * LD;
      const float gC = expf(gs[kGcC - 1]);
      for (int rg = ty * 4; rg < DK; rg += 128) {
        float acc[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float4 s4 = *reinterpret_cast<const float4*>(Ss + (rg + i) * kGcCols + 4 * tx);
          acc[i][0] = gC * s4.x; acc[i][1] = gC * s4.y; acc[i][2] = gC * s4.z; acc[i][3] = gC * s4.w;
        }
#pragma unroll 4
        for (int j = 0; j < kGcC; ++j) {
          const float4 k4 = *reinterpret_cast<const float4*>(Ks + j * LD + rg);
          const float4 u4 = *reinterpret_cast<const float4*>(Us + j * kGcCols + 4 * tx);
          const float kv[4] = {k4.x, k4.y, k4.z, k4.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            acc[i][0] += kv[i] * u4.x; acc[i][1] += kv[i] * u4.y; acc[i][2] += kv[i] * u4.z; acc[i][3] += kv[i] * u4.w;
          }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i)
          *reinterpret_cast<float4*>(Ss + (rg + i) * kGcCols + 4 * tx) = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
      }
    }
    buf ^= 1;                                          // the next chunk's W is (being) copied into Ab[buf]
  }
  __syncthreads();
  for (int i = tid; i < DK * kGcCols; i += kGcThreads) sp[static_cast<size_t>(i / kGcCols) * a.dv + i % kGcCols] = Ss[i];
}

}  // namespace dgpp

using namespace dgpp;

// Chunked prefill form of dgpp_gdn_recurrent (sequential rows of ONE request).  qn / kn / dec / bet are the outputs of
// the token-parallel preparation (gdn_prep_kernel's scratch layout); scratch holds chunks * hv * 64 * (dk + dv + 65)
// floats.  state points at the slot's [hv, dk, dv] block and is updated in place.
DGPP_API int dgpp_gdn_chunk_scan(const void* qn, const void* kn, const void* dec, const void* bet, const void* v,
                                 int64_t v_stride, void* state, void* out, void* scratch, int64_t scratch_floats, int T,
                                 int hk, int hv, int dk, int dv, cudaStream_t st) {
  DGPP_REQUIRE(dk == 64 || dk == 128, "gdn_chunk: key dim %d (64 or 128)", dk);
  DGPP_REQUIRE(dv % kGcCols == 0 && hk > 0 && hv % hk == 0, "gdn_chunk: bad head geometry hk %d hv %d dv %d", hk, hv, dv);
  if (T == 0) return 0;
  const int chunks = dgpp_ceil_div(T, kGcC);
  const int64_t per = static_cast<int64_t>(chunks) * hv * kGcC;
  DGPP_REQUIRE(scratch && scratch_floats >= per * (dk + dv + kGcC + 1), "gdn_chunk: scratch of %lld floats required",
               static_cast<long long>(per * (dk + dv + kGcC + 1)));
  GdnChunkArgs a;
  a.qn = static_cast<const float*>(qn); a.kn = static_cast<const float*>(kn);
  a.dec = static_cast<const float*>(dec); a.bet = static_cast<const float*>(bet);
  a.v = static_cast<const bf16*>(v); a.v_stride = v_stride;
  float* s = static_cast<float*>(scratch);
  a.W = s; s += per * dk;
  a.U0 = s; s += per * dv;
  a.P = s; s += per * kGcC;
  a.G = s;
  a.state = static_cast<float*>(state);
  a.out = static_cast<bf16*>(out);
  a.T = T; a.hk = hk; a.hv = hv; a.dk = dk; a.dv = dv; a.chunks = chunks;
  const size_t smem1 = (2 * kGcC * (dk + 4) + 2 * kGcC * (kGcC + 1) + 2 * kGcC) * sizeof(float);
  const size_t smem2 = (static_cast<size_t>(dk) * kGcCols + 2 * kGcC * (dk + 4) + kGcC * (kGcC + 4) + kGcC * kGcCols + 2 * kGcC) * sizeof(float);
  static bool attr = false;
  if (!attr) {
    DGPP_CUDA_OK(cudaFuncSetAttribute(gdn_chunk_prep_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
    DGPP_CUDA_OK(cudaFuncSetAttribute(gdn_chunk_prep_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
    DGPP_CUDA_OK(cudaFuncSetAttribute(gdn_chunk_state_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
    DGPP_CUDA_OK(cudaFuncSetAttribute(gdn_chunk_state_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
    attr = true;
  }
  dim3 g1(chunks, hv), g2(dv / kGcCols, hv);
  if (dk == 64) {
    gdn_chunk_prep_kernel<64><<<g1, kGcThreads, smem1, st>>>(a);
    gdn_chunk_state_kernel<64><<<g2, kGcThreads, smem2, st>>>(a);
  } else {
    gdn_chunk_prep_kernel<128><<<g1, kGcThreads, smem1, st>>>(a);
    gdn_chunk_state_kernel<128><<<g2, kGcThreads, smem2, st>>>(a);
  }
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}
