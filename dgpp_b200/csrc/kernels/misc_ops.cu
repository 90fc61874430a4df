// Small operators of the MoE / quantised-checkpoint families.
//
//   moe_hash_routes_kernel     table routing: a token's experts are tid2eid[token id] (top_k ascending ids) instead of the
//                              top-k of its scores; weights = the token's scores at those ids, normalised by
//                              (ascending-order sum + 1e-20) when asked, times the routed scaling factor
//   hadamard32_rows_kernel     block-diagonal normalised Walsh-Hadamard rotation of bf16 rows in blocks of 32 (one warp
//                              lane per element, five xor-shuffle butterfly stages at strides 1, 2, 4, 8, 16: lane j
//                              takes v_j + v_{j^s} when bit s of j is clear, v_{j^s} - v_j when set), one multiply by
//                              fp32(1 / sqrt(32)), one bf16 rounding; rows with index == period - 1 (mod period) are left
//                              untouched (period 0: every row is rotated)
//   hadamard32_quant_int8_kernel   the same rotation followed by int8 codes per group of 128 rotated bf16 values:
//                              scale = max(amax / 127, 1e-30), code = clamp(rint(x / scale), -128, 127)
//   ple_embed_add_kernel       hashed bigram embeddings: row r of x gets table[(prev[r] * 1000003 + token[r] * 7919 + 12345)
//                              mod table rows] added (fp32 sum, one bf16 rounding); the ids never visit the host
// (reference counterparts: src/kernels/glm_moe.cu:923 moe_hash_routes_kernel, src/kernels/hadamard32.cu,
//  src/kernels/qwen_ple.cu hash ids + gather.)
#include <math.h>

#include "common/common.h"
#include "common/dtypes.cuh"
#include "common/ptx.cuh"

namespace dgpp {

constexpr float kH32Scale = 0.17677669529663687f;

__global__ void moe_hash_routes_kernel(const int32_t* __restrict__ tokens, const int32_t* __restrict__ tid2eid,
                                       const float* __restrict__ scores, int32_t* __restrict__ ids, float* __restrict__ weights,
                                       int T, int vocab, int E, int k, float scaling, int norm_topk) {
  pdl_wait();
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T) return;
  int tok = tokens[t];
  if (tok < 0 || tok >= vocab) tok = 0;          // padding row: any table row (its output is never read)
  const int32_t* row = tid2eid + static_cast<size_t>(tok) * k;
  float sum = 0.f;
  for (int i = 0; i < k; ++i) sum = __fadd_rn(sum, scores[static_cast<size_t>(t) * E + row[i]]);
  sum = __fadd_rn(sum, 1e-20f);
  for (int i = 0; i < k; ++i) {
    const float s = scores[static_cast<size_t>(t) * E + row[i]];
    ids[static_cast<size_t>(t) * k + i] = row[i];
    weights[static_cast<size_t>(t) * k + i] = (norm_topk ? __fdiv_rn(s, sum) : s) * scaling;
  }
}

// grid (rows), 128 threads
__global__ void __launch_bounds__(128) ple_embed_add_kernel(const int32_t* __restrict__ tokens, const int32_t* __restrict__ prev,
                                                            const bf16* __restrict__ table, bf16* __restrict__ x, int hidden,
                                                            int table_rows) {
  pdl_wait();
  const int r = blockIdx.x;
  const long long id = (static_cast<long long>(prev[r]) * 1000003ll + static_cast<long long>(tokens[r]) * 7919ll + 12345ll) %
                       static_cast<long long>(table_rows);
  const bf16* src = table + static_cast<size_t>(id < 0 ? id + table_rows : id) * hidden;
  bf16* dst = x + static_cast<size_t>(r) * hidden;
  for (int i = threadIdx.x; i < hidden; i += 128) dst[i] = f32_to_bf16(__fadd_rn(bf16_to_f32(dst[i]), bf16_to_f32(src[i])));
}

__device__ __forceinline__ float h32_lane(float v, int lane) {
#pragma unroll
  for (int s = 1; s < 32; s <<= 1) {
    const float o = __shfl_xor_sync(0xffffffffu, v, s);
    v = (lane & s) ? __fsub_rn(o, v) : __fadd_rn(v, o);
  }
  return __fmul_rn(v, kH32Scale);
}

// grid (rows), 256 threads: warp w rotates blocks w, w + 8, ...
__global__ void __launch_bounds__(256) hadamard32_rows_kernel(const bf16* __restrict__ in, int64_t in_stride, bf16* __restrict__ out,
                                                              int64_t out_stride, int K, int period) {
  pdl_wait();
  const int r = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (period > 0 && r % period == period - 1) return;
  for (int b = warp; b < K / 32; b += 8) {
    const float v = bf16_to_f32(in[static_cast<size_t>(r) * in_stride + b * 32 + lane]);
    out[static_cast<size_t>(r) * out_stride + b * 32 + lane] = f32_to_bf16(h32_lane(v, lane));
  }
}

// grid (rows), 128 threads: warp w handles groups w, w + 4, ... of 128 values (four blocks of 32).
__global__ void __launch_bounds__(128) hadamard32_quant_int8_kernel(const bf16* __restrict__ in, int64_t in_stride,
                                                                    int8_t* __restrict__ codes, int64_t code_stride,
                                                                    float* __restrict__ scales, int64_t scale_stride, int K,
                                                                    int period) {
  pdl_wait();
  const int r = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (period > 0 && r % period == period - 1) return;
  for (int g = warp; g < K / 128; g += 4) {
    float v[4];
    float am = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float x = bf16_to_f32(in[static_cast<size_t>(r) * in_stride + g * 128 + j * 32 + lane]);
      v[j] = bf16_to_f32(f32_to_bf16(h32_lane(x, lane)));      // the codes are taken from the rotated bf16 values
      am = fmaxf(am, fabsf(v[j]));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
    const float sc = fmaxf(__fdiv_rn(am, 127.f), 1e-30f);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float q = fminf(fmaxf(rintf(__fdiv_rn(v[j], sc)), -128.f), 127.f);
      codes[static_cast<size_t>(r) * code_stride + g * 128 + j * 32 + lane] = static_cast<int8_t>(q);
    }
    if (lane == 0) scales[static_cast<size_t>(r) * scale_stride + g] = sc;
  }
}

}  // namespace dgpp

using namespace dgpp;

DGPP_API int dgpp_moe_hash_routes(const void* tokens, const void* tid2eid, const void* scores, void* ids, void* weights, int T,
                                  int vocab, int E, int k, float scaling, int norm_topk, cudaStream_t st) {
  DGPP_REQUIRE(k >= 1 && k <= 16 && E >= k && vocab >= 1, "moe_hash_routes: bad sizes (k %d E %d vocab %d)", k, E, vocab);
  if (T == 0) return 0;
  moe_hash_routes_kernel<<<dgpp_ceil_div(T, 64), 64, 0, st>>>(static_cast<const int32_t*>(tokens), static_cast<const int32_t*>(tid2eid),
                                                              static_cast<const float*>(scores), static_cast<int32_t*>(ids),
                                                              static_cast<float*>(weights), T, vocab, E, k, scaling, norm_topk);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

DGPP_API int dgpp_ple_embed_add(const void* tokens, const void* prev, const void* table, void* x, int rows, int hidden,
                                int table_rows, cudaStream_t st) {
  DGPP_REQUIRE(hidden >= 1 && table_rows >= 1, "ple_embed_add: bad sizes");
  if (rows == 0) return 0;
  ple_embed_add_kernel<<<rows, 128, 0, st>>>(static_cast<const int32_t*>(tokens), static_cast<const int32_t*>(prev),
                                             static_cast<const bf16*>(table), static_cast<bf16*>(x), hidden, table_rows);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

DGPP_API int dgpp_hadamard32_rows(const void* in, int64_t in_stride, void* out, int64_t out_stride, int rows, int K, int period,
                                  cudaStream_t st) {
  DGPP_REQUIRE(K % 32 == 0 && period >= 0, "hadamard32: K %d must be a multiple of 32", K);
  if (rows == 0) return 0;
  hadamard32_rows_kernel<<<rows, 256, 0, st>>>(static_cast<const bf16*>(in), in_stride, static_cast<bf16*>(out), out_stride, K, period);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

DGPP_API int dgpp_hadamard32_quant_int8(const void* in, int64_t in_stride, void* codes, int64_t code_stride, void* scales,
                                        int64_t scale_stride, int rows, int K, int period, cudaStream_t st) {
  DGPP_REQUIRE(K % 128 == 0 && period >= 0, "hadamard32_quant_int8: K %d must be a multiple of 128", K);
  if (rows == 0) return 0;
  hadamard32_quant_int8_kernel<<<rows, 128, 0, st>>>(static_cast<const bf16*>(in), in_stride, static_cast<int8_t*>(codes), code_stride,
                                                     static_cast<float*>(scales), scale_stride, K, period);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}
