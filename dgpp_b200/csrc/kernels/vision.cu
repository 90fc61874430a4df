// Vision-tower kernels: everything of a ViT encoder that is not a GEMM.  The linears and both attention products
// (Q.K^T and P.V, per head) run on the tcgen05 GEMM (gemm_tc.cu, bf16 operands); these kernels prepare their operands:
//   patchify        uint8 canvas [H, W, 3] -> normalised bf16 patch rows [patches, 3*p*p], merge groups contiguous
//   layernorm       bf16 rows, bf16 weight / bias, fp32 statistics
//   bias_act        x = resid + act(x + bias), act in {none, gelu(erf), gelu(tanh)}
//   qkv_split_rope  [T, 3*hidden] -> head-major q, k (2-D RoPE: first half of a head by row, second half by column)
//                   and V transposed [heads, d, T_pad] (the K-major "weight" operand of the P.V product)
//   softmax_rows    in-place row softmax of the scaled scores, padding columns forced to zero
// (reference counterparts: src/kernels/glm_vision.cu, qwen_vision.cu -- patchify, pos-embed, LayerNorm, GELU, QKV split
//  + 2-D RoPE, softmax, un-head, spatial merge; the GEMMs are cuBLASLt there.)
#include <math.h>

#include "common/common.h"
#include "common/dtypes.cuh"
#include "common/ptx.cuh"

namespace dgpp {

__global__ void vis_patchify_kernel(const uint8_t* __restrict__ img, bf16* __restrict__ out, int H, int W, int p, int m,
                                    float m0, float m1, float m2, float s0, float s1, float s2) {
  pdl_wait();
  const int gw = W / p / m;                       // merge groups per row
  const int patch = blockIdx.x;                   // output row
  const int grp = patch / (m * m), in = patch % (m * m);
  const int py = (grp / gw) * m + in / m, px = (grp % gw) * m + in % m;
  const int feat = 3 * p * p;
  for (int f = threadIdx.x; f < feat; f += blockDim.x) {
    const int c = f / (p * p), y = (f / p) % p, x = f % p;
    const float v = static_cast<float>(img[(static_cast<size_t>(py * p + y) * W + px * p + x) * 3 + c]) * (1.f / 255.f);
    const float mean = c == 0 ? m0 : (c == 1 ? m1 : m2), sd = c == 0 ? s0 : (c == 1 ? s1 : s2);
    out[static_cast<size_t>(patch) * feat + f] = f32_to_bf16((v - mean) / sd);
  }
}

__device__ __forceinline__ float block_sum(float v, float* sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) sh[w] = v;
  __syncthreads();
  float r = 0.f;
  for (int i = 0; i < (blockDim.x >> 5); ++i) r += sh[i];
  __syncthreads();
  return r;
}

__global__ void __launch_bounds__(256)
layernorm_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, const bf16* __restrict__ b,
                 bf16* __restrict__ out, int H, float eps) {
  __shared__ float sh[8];
  pdl_wait();
  const bf16* row = x + static_cast<size_t>(blockIdx.x) * H;
  float s = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) s += bf16_to_f32(row[i]);
  const float mean = block_sum(s, sh) / H;
  float q = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float d = bf16_to_f32(row[i]) - mean;
    q += d * d;
  }
  const float rstd = rsqrtf(block_sum(q, sh) / H + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float y = (bf16_to_f32(row[i]) - mean) * rstd * bf16_to_f32(w[i]) + (b ? bf16_to_f32(b[i]) : 0.f);
    out[static_cast<size_t>(blockIdx.x) * H + i] = f32_to_bf16(y);
  }
}

__global__ void bias_act_kernel(bf16* __restrict__ x, const bf16* __restrict__ bias, const bf16* __restrict__ resid,
                                int64_t total, int N, int act) {
  pdl_wait();
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  float v = bf16_to_f32(x[i]) + (bias ? bf16_to_f32(bias[i % N]) : 0.f);
  if (act == 1) v = 0.5f * v * (1.f + erff(v * 0.70710678118654752f));
  else if (act == 2) v = 0.5f * v * (1.f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
  if (resid) v += bf16_to_f32(resid[i]);
  x[i] = f32_to_bf16(v);
}

// One block per token.  bias (optional): the qkv projection's bias, added before the rotation.
__global__ void __launch_bounds__(256)
vis_qkv_split_rope_kernel(const bf16* __restrict__ qkv, const bf16* __restrict__ bias, const int32_t* __restrict__ pos_y,
                          const int32_t* __restrict__ pos_x, bf16* __restrict__ q_h, bf16* __restrict__ k_h,
                          bf16* __restrict__ vt_h, int T, int T_pad, int heads, int d, float theta) {
  pdl_wait();
  const int t = blockIdx.x, hid = heads * d;
  const bf16* row = qkv + static_cast<size_t>(t) * 3 * hid;
  const int half = d / 2, quarter = d / 4;          // a head's halves rotate by row / column, pairs (i, i + quarter)
  auto val = [&](int col) { return bf16_to_f32(row[col]) + (bias ? bf16_to_f32(bias[col]) : 0.f); };
  // q and k: thread per rotation pair
  for (int i = threadIdx.x; i < 2 * heads * half; i += blockDim.x) {
    const int which = i / (heads * half), r = i % (heads * half);
    const int h = r / half, j = r % half;            // j: pair index inside the head (0 .. d/2)
    const int seg = j / quarter, jj = j % quarter;   // seg 0: row half, 1: column half
    const int c0 = h * d + seg * half + jj, c1 = c0 + quarter;
    const float pos = static_cast<float>(seg == 0 ? pos_y[t] : pos_x[t]);
    const float ang = pos * powf(theta, -static_cast<float>(jj) / static_cast<float>(quarter));
    float sn, cs;
    sincosf(ang, &sn, &cs);
    const float a = val(which * hid + c0), b = val(which * hid + c1);
    bf16* dst = (which == 0 ? q_h : k_h) + (static_cast<size_t>(h) * T + t) * d;
    dst[seg * half + jj] = f32_to_bf16(a * cs - b * sn);
    dst[seg * half + jj + quarter] = f32_to_bf16(b * cs + a * sn);
  }
  for (int i = threadIdx.x; i < hid; i += blockDim.x) {
    const int h = i / d, j = i % d;
    vt_h[(static_cast<size_t>(h) * d + j) * T_pad + t] = f32_to_bf16(val(2 * hid + i));
  }
}

__global__ void __launch_bounds__(256)
softmax_rows_kernel(bf16* __restrict__ s, int cols, int ld) {
  __shared__ float sh[8];
  pdl_wait();
  bf16* row = s + static_cast<size_t>(blockIdx.x) * ld;
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < cols; i += blockDim.x) mx = fmaxf(mx, bf16_to_f32(row[i]));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = mx;
  __syncthreads();
  mx = sh[0];
  for (int i = 1; i < (blockDim.x >> 5); ++i) mx = fmaxf(mx, sh[i]);
  __syncthreads();
  float sum = 0.f;
  for (int i = threadIdx.x; i < cols; i += blockDim.x) sum += __expf(bf16_to_f32(row[i]) - mx);
  const float inv = 1.f / block_sum(sum, sh);
  for (int i = threadIdx.x; i < ld; i += blockDim.x)
    row[i] = f32_to_bf16(i < cols ? __expf(bf16_to_f32(row[i]) - mx) * inv : 0.f);
}

}  // namespace dgpp

using namespace dgpp;

DGPP_API int dgpp_vis_patchify(const void* img, void* out, int H, int W, int p, int m, const float* mean,
                               const float* std_, cudaStream_t st) {
  DGPP_REQUIRE(p >= 1 && m >= 1 && H % (p * m) == 0 && W % (p * m) == 0, "vis_patchify: %d x %d is not a multiple of %d", H, W, p * m);
  const int patches = (H / p) * (W / p);
  vis_patchify_kernel<<<patches, 128, 0, st>>>(static_cast<const uint8_t*>(img), static_cast<bf16*>(out), H, W, p, m,
                                              mean[0], mean[1], mean[2], std_[0], std_[1], std_[2]);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

DGPP_API int dgpp_layernorm(const void* x, const void* w, const void* b, void* out, int rows, int H, float eps,
                            cudaStream_t st) {
  if (rows == 0) return 0;
  layernorm_kernel<<<rows, 256, 0, st>>>(static_cast<const bf16*>(x), static_cast<const bf16*>(w),
                                         static_cast<const bf16*>(b), static_cast<bf16*>(out), H, eps);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

// act: 0 none, 1 GELU (erf), 2 GELU (tanh).  x [rows, N] in place; bias [N] and resid [rows, N] optional.
DGPP_API int dgpp_bias_act(void* x, const void* bias, const void* resid, int rows, int N, int act, cudaStream_t st) {
  const int64_t total = static_cast<int64_t>(rows) * N;
  if (total == 0) return 0;
  bias_act_kernel<<<static_cast<int>(dgpp_ceil_div64(total, 256)), 256, 0, st>>>(
      static_cast<bf16*>(x), static_cast<const bf16*>(bias), static_cast<const bf16*>(resid), total, N, act);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

DGPP_API int dgpp_vis_qkv_split_rope(const void* qkv, const void* bias, const void* pos_y, const void* pos_x, void* q_h,
                                     void* k_h, void* vt_h, int T, int T_pad, int heads, int d, float theta,
                                     cudaStream_t st) {
  DGPP_REQUIRE(d % 4 == 0 && T_pad >= T, "vis_qkv_split_rope: head_dim %d must be a multiple of 4", d);
  if (T == 0) return 0;
  vis_qkv_split_rope_kernel<<<T, 256, 0, st>>>(static_cast<const bf16*>(qkv), static_cast<const bf16*>(bias),
                                              static_cast<const int32_t*>(pos_y), static_cast<const int32_t*>(pos_x),
                                              static_cast<bf16*>(q_h), static_cast<bf16*>(k_h), static_cast<bf16*>(vt_h),
                                              T, T_pad, heads, d, theta);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

DGPP_API int dgpp_softmax_rows(void* s, int rows, int cols, int ld, cudaStream_t st) {
  DGPP_REQUIRE(cols >= 1 && ld >= cols, "softmax_rows: bad shape %d / %d", cols, ld);
  if (rows == 0) return 0;
  softmax_rows_kernel<<<rows, 256, 0, st>>>(static_cast<bf16*>(s), cols, ld);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}
