// Elementwise / row operators of two model families.
//
// nGPT-style normalisations (hypersphere residuals):
//   justnorm(x)                 = bf16(fp32(x) * rstd),  rstd = 1 / sqrt(sum fp32(x)^2 + eps); the row sum is taken in fp64
//                                 (every bf16 square is exact there), rounded once to fp32 before eps is added
//   slerp_alpha(a, b, alpha, s) = justnorm(bf16(a ra) + lr (bf16(b rb) - bf16(a ra))),  lr = |fp32(alpha[col]) s|;
//                                 the operands are normalised to bf16, the interpolation and its normalisation stay fp32
//                                 until the final conversion
// Gated residual over hc parallel residual branches R [rows, hc, H] with normed copy Rn:
//   gate_act     t = bf16(silu(bf16(t / hc)))                                   (between the two gate projections)
//   mix_finish   x = bf16((sum_i fp32(bf16(bf16(sigmoid(logit_i)) Rn_i))) / hc)  (branches in ascending order)
//   combine      s_i = 2 bf16(sigmoid(bf16(dot_i / hc))),  R_i = bf16(R_i + bf16(y s_i)),  dot_i = <W_inj[i], Rn[row]> over hc H
// One CTA per row, fixed reduction order (xor-shuffle tree, warps ascending): deterministic and capturable.
// (reference counterparts: src/kernels/dory_norm.cu, src/kernels/qwen_gr.cu.)
#include <math.h>

#include "common/common.h"
#include "common/dtypes.cuh"
#include "common/ptx.cuh"

namespace dgpp {

constexpr int kFamThreads = 256;

__device__ __forceinline__ double block_sum_f64(double v, double* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  __syncthreads();
  double t = 0.0;
  for (int i = 0; i < kFamThreads / 32; ++i) t += scratch[i];
  __syncthreads();
  return t;
}
__device__ __forceinline__ float block_sum_f32(float v, float* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
  for (int i = 0; i < kFamThreads / 32; ++i) t += scratch[i];
  __syncthreads();
  return t;
}
__device__ __forceinline__ float rstd_of(const bf16* row, int dim, float eps, double* scratch) {
  double ss = 0.0;
  for (int i = threadIdx.x; i < dim; i += kFamThreads) {
    const double f = static_cast<double>(bf16_to_f32(row[i]));
    ss += f * f;
  }
  const double total = block_sum_f64(ss, scratch);
  return 1.f / sqrtf(static_cast<float>(total) + eps);
}

__global__ void __launch_bounds__(kFamThreads) justnorm_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, int dim, float eps) {
  __shared__ double scratch[kFamThreads / 32];
  pdl_wait();
  const bf16* row = x + static_cast<size_t>(blockIdx.x) * dim;
  const float r = rstd_of(row, dim, eps, scratch);
  for (int i = threadIdx.x; i < dim; i += kFamThreads) y[static_cast<size_t>(blockIdx.x) * dim + i] = f32_to_bf16(bf16_to_f32(row[i]) * r);
}

__global__ void __launch_bounds__(kFamThreads) slerp_alpha_kernel(const bf16* __restrict__ a, const bf16* __restrict__ b,
                                                                  const bf16* __restrict__ alpha, float s, bf16* __restrict__ out,
                                                                  int dim, float eps) {
  extern __shared__ float mix[];                      // [dim] the interpolated row, fp32
  __shared__ double scratch[kFamThreads / 32];
  pdl_wait();
  const bf16* ar = a + static_cast<size_t>(blockIdx.x) * dim;
  const bf16* br = b + static_cast<size_t>(blockIdx.x) * dim;
  const float ra = rstd_of(ar, dim, eps, scratch), rb = rstd_of(br, dim, eps, scratch);
  double ss = 0.0;
  for (int i = threadIdx.x; i < dim; i += kFamThreads) {
    const float an = bf16_to_f32(f32_to_bf16(bf16_to_f32(ar[i]) * ra));
    const float bn = bf16_to_f32(f32_to_bf16(bf16_to_f32(br[i]) * rb));
    const float lr = fabsf(bf16_to_f32(alpha[i]) * s);
    const float m = an + lr * (bn - an);
    mix[i] = m;
    ss += static_cast<double>(m) * static_cast<double>(m);
  }
  const double total = block_sum_f64(ss, scratch);
  const float r = 1.f / sqrtf(static_cast<float>(total) + eps);
  for (int i = threadIdx.x; i < dim; i += kFamThreads) out[static_cast<size_t>(blockIdx.x) * dim + i] = f32_to_bf16(mix[i] * r);
}

__global__ void gr_gate_act_kernel(bf16* __restrict__ t, int64_t n, int hc) {
  pdl_wait();
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float v = bf16_to_f32(f32_to_bf16(bf16_to_f32(t[i]) / static_cast<float>(hc)));
  t[i] = f32_to_bf16(v / (1.f + expf(-v)));
}

// logits, rn: [rows, hc, H]; x: [rows, H].  grid (ceil(H / 256), rows).
__global__ void __launch_bounds__(256) gr_mix_finish_kernel(const bf16* __restrict__ logits, const bf16* __restrict__ rn,
                                                            bf16* __restrict__ x, int hc, int H) {
  pdl_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= H) return;
  const size_t base = static_cast<size_t>(blockIdx.y) * hc * H;
  float acc = 0.f;
  for (int i = 0; i < hc; ++i) {
    const float l = bf16_to_f32(logits[base + static_cast<size_t>(i) * H + c]);
    const float g = bf16_to_f32(f32_to_bf16(1.f / (1.f + expf(-l))));
    acc += bf16_to_f32(f32_to_bf16(g * bf16_to_f32(rn[base + static_cast<size_t>(i) * H + c])));
  }
  x[static_cast<size_t>(blockIdx.y) * H + c] = f32_to_bf16(acc / static_cast<float>(hc));
}

// One CTA per row: hc dots of length hc * H against Rn[row], then the row-wide update of the hc branches.
__global__ void __launch_bounds__(kFamThreads) gr_combine_kernel(bf16* __restrict__ r_state, const bf16* __restrict__ rn,
                                                                 const bf16* __restrict__ w_inject, const bf16* __restrict__ y,
                                                                 float* __restrict__ gates, int hc, int H) {
  __shared__ float scratch[kFamThreads / 32];
  __shared__ float s_gate[16];
  pdl_wait();
  const size_t row = blockIdx.x;
  const int W = hc * H;
  const bf16* rr = rn + row * W;
  for (int i = 0; i < hc; ++i) {
    float d = 0.f;
    for (int k = threadIdx.x; k < W; k += kFamThreads) d = fmaf(bf16_to_f32(w_inject[static_cast<size_t>(i) * W + k]), bf16_to_f32(rr[k]), d);
    const float dot = block_sum_f32(d, scratch);
    if (threadIdx.x == 0) {
      const float q = bf16_to_f32(f32_to_bf16(dot / static_cast<float>(hc)));
      s_gate[i] = 2.f * bf16_to_f32(f32_to_bf16(1.f / (1.f + expf(-q))));
      if (gates) gates[row * hc + i] = s_gate[i];
    }
  }
  __syncthreads();
  for (int k = threadIdx.x; k < W; k += kFamThreads) {
    const int i = k / H, c = k % H;
    const float add = bf16_to_f32(f32_to_bf16(bf16_to_f32(y[row * H + c]) * s_gate[i]));
    r_state[row * W + k] = f32_to_bf16(bf16_to_f32(r_state[row * W + k]) + add);
  }
}

}  // namespace dgpp

using namespace dgpp;

DGPP_API int dgpp_justnorm(const void* x, void* y, int rows, int dim, float eps, cudaStream_t st) {
  DGPP_REQUIRE(dim >= 1 && dim <= 65536, "justnorm: dim %d", dim);
  if (rows == 0) return 0;
  justnorm_kernel<<<rows, kFamThreads, 0, st>>>(static_cast<const bf16*>(x), static_cast<bf16*>(y), dim, eps);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

DGPP_API int dgpp_slerp_alpha(const void* a, const void* b, const void* alpha, float s, void* out, int rows, int dim, float eps,
                              cudaStream_t st) {
  DGPP_REQUIRE(dim >= 1 && dim <= 11 * 1024, "slerp_alpha: dim %d outside 1..11264", dim);
  if (rows == 0) return 0;
  slerp_alpha_kernel<<<rows, kFamThreads, static_cast<size_t>(dim) * sizeof(float), st>>>(
      static_cast<const bf16*>(a), static_cast<const bf16*>(b), static_cast<const bf16*>(alpha), s, static_cast<bf16*>(out), dim, eps);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

DGPP_API int dgpp_gr_gate_act(void* t, int64_t rows, int r, int hc, cudaStream_t st) {
  const int64_t n = rows * r;
  if (n == 0) return 0;
  gr_gate_act_kernel<<<static_cast<unsigned>(dgpp_ceil_div64(n, 256)), 256, 0, st>>>(static_cast<bf16*>(t), n, hc);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

DGPP_API int dgpp_gr_mix_finish(const void* logits, const void* rn, void* x, int rows, int hc, int H, cudaStream_t st) {
  if (rows == 0) return 0;
  gr_mix_finish_kernel<<<dim3(dgpp_ceil_div(H, 256), rows), 256, 0, st>>>(static_cast<const bf16*>(logits), static_cast<const bf16*>(rn),
                                                                        static_cast<bf16*>(x), hc, H);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

DGPP_API int dgpp_gr_combine(void* r_state, const void* rn, const void* w_inject, const void* y, void* gates, int rows, int hc, int H,
                             cudaStream_t st) {
  DGPP_REQUIRE(hc >= 1 && hc <= 16, "gr_combine: %d branches (1..16)", hc);
  if (rows == 0) return 0;
  gr_combine_kernel<<<rows, kFamThreads, 0, st>>>(static_cast<bf16*>(r_state), static_cast<const bf16*>(rn),
                                                  static_cast<const bf16*>(w_inject), static_cast<const bf16*>(y),
                                                  static_cast<float*>(gates), hc, H);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

// ---------------------------------------------------------------------------------------------------------------------
// Manifold-constrained hyper-connections over n residual streams [tokens, n, D] (n <= 8):
//   flat    = unweighted RMSNorm of the flattened streams (fp32, eps = norm_eps)
//   logits  = flat . fn^T                       fn: bf16 [(2 + n) n, n D]
//   pre     = sigmoid(logits[0:n] scale[0] + base[0:n]) + hc_eps                 stream-collapse weights
//   post    = 2 sigmoid(logits[n:2n] scale[1] + base[n:2n])                      placement of the block output
//   comb    = softmax over the last axis of (logits[2n:] scale[2] + base[2n:]) viewed [n, n], + hc_eps, then
//             Sinkhorn-Knopp: one column normalisation, then (iters - 1) times (row, column); every division adds
//             hc_eps to its denominator
//   collapsed = bf16(sum_j pre[j] streams[j])   (fp32 accumulation)
// and the fold of a block output h:  streams'[i] = bf16(bf16(post_i h) + bf16(sum_j comb[j, i] streams[j])) with post and
// comb rounded to bf16 before the products.
// One CTA per token; the (2 + n) n dots share one pass over the row (inv_rms applied to the finished sums).
// (reference counterparts: src/kernels/glm_mhc.cu, semantics in src/models/glm/mhc.hpp.)
namespace dgpp {

constexpr int kMhcMaxN = 8;

template <int N>
__global__ void __launch_bounds__(kFamThreads) mhc_compute_kernel(const bf16* __restrict__ streams, const bf16* __restrict__ fn,
                                                                  const float* __restrict__ base, const float* __restrict__ scale,
                                                                  bf16* __restrict__ collapsed, bf16* __restrict__ post_out,
                                                                  bf16* __restrict__ comb_out, int D, int iters, float hc_eps,
                                                                  float norm_eps) {
  constexpr int n = N, C = (2 + N) * N;
  __shared__ float part[C + 1][kFamThreads / 32];
  __shared__ float pre_s[N];
  pdl_wait();
  const size_t tok = blockIdx.x;
  const int W = n * D;
  const bf16* row = streams + tok * W;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // one pass: sum of squares and the C dots (each thread keeps C + 1 partials; C <= 80)
  float ss = 0.f;
  float dots[C];
#pragma unroll
  for (int c = 0; c < C; ++c) dots[c] = 0.f;
  for (int k = threadIdx.x; k < W; k += kFamThreads) {
    const float x = bf16_to_f32(row[k]);
    ss = fmaf(x, x, ss);
#pragma unroll
    for (int c = 0; c < C; ++c) dots[c] = fmaf(x, bf16_to_f32(fn[static_cast<size_t>(c) * W + k]), dots[c]);
  }
#pragma unroll
  for (int c = 0; c <= C; ++c) {
    float v = c < C ? dots[c] : ss;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0) part[c][warp] = v;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float tot[C + 1];
    for (int c = 0; c <= C; ++c) {
      float t = 0.f;
      for (int w = 0; w < kFamThreads / 32; ++w) t += part[c][w];
      tot[c] = t;
    }
    const float inv_rms = rsqrtf(tot[C] / static_cast<float>(W) + norm_eps);
    float comb[N][N];
    for (int j = 0; j < n; ++j) {
      pre_s[j] = 1.f / (1.f + expf(-(tot[j] * inv_rms * scale[0] + base[j]))) + hc_eps;
      const float po = 2.f / (1.f + expf(-(tot[n + j] * inv_rms * scale[1] + base[n + j])));
      post_out[tok * n + j] = f32_to_bf16(po);
    }
    for (int j = 0; j < n; ++j) {
      float m = -INFINITY;
      for (int i = 0; i < n; ++i) {
        comb[j][i] = tot[2 * n + j * n + i] * inv_rms * scale[2] + base[2 * n + j * n + i];
        m = fmaxf(m, comb[j][i]);
      }
      float s = 0.f;
      for (int i = 0; i < n; ++i) { comb[j][i] = expf(comb[j][i] - m); s += comb[j][i]; }
      for (int i = 0; i < n; ++i) comb[j][i] = comb[j][i] / s + hc_eps;
    }
    auto col_pass = [&]() {
      for (int i = 0; i < n; ++i) {
        float s = 0.f;
        for (int j = 0; j < n; ++j) s += comb[j][i];
        for (int j = 0; j < n; ++j) comb[j][i] = comb[j][i] / (s + hc_eps);
      }
    };
    auto row_pass = [&]() {
      for (int j = 0; j < n; ++j) {
        float s = 0.f;
        for (int i = 0; i < n; ++i) s += comb[j][i];
        for (int i = 0; i < n; ++i) comb[j][i] = comb[j][i] / (s + hc_eps);
      }
    };
    col_pass();
    for (int it = 1; it < iters; ++it) { row_pass(); col_pass(); }
    for (int j = 0; j < n; ++j)
      for (int i = 0; i < n; ++i) comb_out[(tok * n + j) * n + i] = f32_to_bf16(comb[j][i]);
  }
  __syncthreads();
  for (int d = threadIdx.x; d < D; d += kFamThreads) {
    float acc = 0.f;
    for (int j = 0; j < n; ++j) acc = fmaf(pre_s[j], bf16_to_f32(row[static_cast<size_t>(j) * D + d]), acc);
    collapsed[tok * D + d] = f32_to_bf16(acc);
  }
}

// streams' [tokens, n, D] (may alias streams): grid (ceil(D / 256), tokens).
__global__ void __launch_bounds__(256) mhc_fold_kernel(const bf16* __restrict__ streams, const bf16* __restrict__ h,
                                                       const bf16* __restrict__ post, const bf16* __restrict__ comb,
                                                       bf16* __restrict__ out, int n, int D) {
  pdl_wait();
  const int d = blockIdx.x * blockDim.x + threadIdx.x;
  if (d >= D) return;
  const size_t tok = blockIdx.y;
  float s[kMhcMaxN];
  for (int j = 0; j < n; ++j) s[j] = bf16_to_f32(streams[(tok * n + j) * D + d]);
  const float hv = bf16_to_f32(h[tok * D + d]);
  for (int i = 0; i < n; ++i) {
    float mix = 0.f;
    for (int j = 0; j < n; ++j) mix = fmaf(bf16_to_f32(comb[(tok * n + j) * n + i]), s[j], mix);
    const float placed = bf16_to_f32(f32_to_bf16(bf16_to_f32(post[tok * n + i]) * hv));
    out[(tok * n + i) * D + d] = f32_to_bf16(placed + bf16_to_f32(f32_to_bf16(mix)));
  }
}

}  // namespace dgpp

DGPP_API int dgpp_mhc_compute(const void* streams, const void* fn, const void* base, const void* scale, void* collapsed, void* post,
                              void* comb, int tokens, int n, int D, int iters, float hc_eps, float norm_eps, cudaStream_t st) {
  DGPP_REQUIRE((n == 2 || n == 4 || n == 8) && D >= 1 && iters >= 1, "mhc_compute: %d streams (2, 4 or 8), D %d, iters %d", n, D, iters);
  if (tokens == 0) return 0;
#define DGPP_MHC(NV)                                                                                                              \
  dgpp::mhc_compute_kernel<NV><<<tokens, dgpp::kFamThreads, 0, st>>>(                                                            \
      static_cast<const bf16*>(streams), static_cast<const bf16*>(fn), static_cast<const float*>(base), static_cast<const float*>(scale), \
      static_cast<bf16*>(collapsed), static_cast<bf16*>(post), static_cast<bf16*>(comb), D, iters, hc_eps, norm_eps)
  if (n == 2) DGPP_MHC(2); else if (n == 4) DGPP_MHC(4); else DGPP_MHC(8);
#undef DGPP_MHC
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

DGPP_API int dgpp_mhc_fold(const void* streams, const void* h, const void* post, const void* comb, void* out, int tokens, int n, int D,
                           cudaStream_t st) {
  DGPP_REQUIRE(n >= 1 && n <= dgpp::kMhcMaxN, "mhc_fold: %d streams (1..8)", n);
  if (tokens == 0) return 0;
  dgpp::mhc_fold_kernel<<<dim3(dgpp_ceil_div(D, 256), tokens), 256, 0, st>>>(static_cast<const bf16*>(streams), static_cast<const bf16*>(h),
                                                                           static_cast<const bf16*>(post), static_cast<const bf16*>(comb),
                                                                           static_cast<bf16*>(out), n, D);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}
