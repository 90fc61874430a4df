// Weight-streaming GEMV on CUDA cores for very small row counts (1..4 activation rows):
//   y[m, n] = alpha * sum_k x[m, k] * dequant(W)[n, k]
// for weights stored exactly as the checkpoint has them:
//   * NVFP4: e2m1 pairs [N, K/2] + one e4m3 scale per 16 along K [N, K/16] + fp32 tensor scale
//   * MXFP4: e2m1 pairs [N, K/2] + one e8m0 scale per 32 along K [N, K/32]
//   * BF16 : [N, K]
// fp32 accumulation in a fixed order (lane-local over k, then an xor-tree over lanes), so the result
// for a row is independent of how many rows share the launch.  Larger row counts go through the
// tcgen05 GEMM in gemm_tc.cu.
// (operator family described by src/kernels/fp4_gemv.cu:17 and src/kernels/bf16_gemv.cu:16 of the reference)
#include "common/common.h"
#include "common/dtypes.cuh"
#include "common/ptx.cuh"

namespace dgpp {

constexpr int kGemvThreads = 256;
constexpr int kGemvWarps = kGemvThreads / 32;
constexpr int kGemvRowsPerWarp = 2;

__device__ __forceinline__ float warp_sum_g(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// GROUP = 16 -> e4m3 scales (NVFP4); GROUP = 32 -> e8m0 scales (MXFP4).
template <int MR, int GROUP>
__global__ void __launch_bounds__(kGemvThreads)
gemv_fp4_kernel(const bf16* __restrict__ x, const uint8_t* __restrict__ wq, const uint8_t* __restrict__ wscale,
                float alpha, bf16* __restrict__ y, float* __restrict__ y32, int N, int K, int64_t x_stride,
                int64_t y_stride) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* xs = reinterpret_cast<bf16*>(smem_raw);  // [MR][K]
  pdl_wait();
  for (int m = 0; m < MR; ++m)
    for (int i = threadIdx.x; i < K / 8; i += blockDim.x)
      reinterpret_cast<uint4*>(xs + static_cast<size_t>(m) * K)[i] =
          reinterpret_cast<const uint4*>(x + m * x_stride)[i];
  __syncthreads();

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int groups = K / GROUP;
  constexpr int R = kGemvRowsPerWarp;
  constexpr int WBYTES = GROUP / 2;  // packed bytes per scale group
  for (int n0 = (blockIdx.x * kGemvWarps + warp) * R; n0 < N; n0 += gridDim.x * kGemvWarps * R) {
    float acc[R][MR];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int m = 0; m < MR; ++m) acc[r][m] = 0.f;

    for (int g = lane; g < groups; g += 32) {
      // activations of this group, converted once and reused by every weight row
      float xf[MR][GROUP];
#pragma unroll
      for (int m = 0; m < MR; ++m) {
#pragma unroll
        for (int v = 0; v < GROUP / 8; ++v) {
          Pack16 p;
          p.u = reinterpret_cast<const uint4*>(xs + static_cast<size_t>(m) * K + static_cast<size_t>(g) * GROUP)[v];
#pragma unroll
          for (int j = 0; j < 8; ++j) xf[m][v * 8 + j] = bf16_to_f32(p.h[j]);
        }
      }
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const int n = n0 + r < N ? n0 + r : N - 1;
        const uint8_t* wrow = wq + static_cast<size_t>(n) * (K / 2) + static_cast<size_t>(g) * WBYTES;
        uint8_t wb[WBYTES];
        if (GROUP == 16) {
          uint2 t = *reinterpret_cast<const uint2*>(wrow);
          *reinterpret_cast<uint2*>(wb) = t;
        } else {
          uint4 t = *reinterpret_cast<const uint4*>(wrow);
          *reinterpret_cast<uint4*>(wb) = t;
        }
        const uint8_t sb = wscale[static_cast<size_t>(n) * groups + g];
        const float sc = GROUP == 16 ? e4m3_to_f32(sb) : e8m0_to_f32(sb);
        float part[MR];
#pragma unroll
        for (int m = 0; m < MR; ++m) part[m] = 0.f;
#pragma unroll
        for (int j = 0; j < WBYTES; ++j) {
          const float2 wf = __half22float2(e2m1x2_to_h2(wb[j]));
#pragma unroll
          for (int m = 0; m < MR; ++m) {
            part[m] = fmaf(wf.x, xf[m][2 * j], part[m]);
            part[m] = fmaf(wf.y, xf[m][2 * j + 1], part[m]);
          }
        }
#pragma unroll
        for (int m = 0; m < MR; ++m) acc[r][m] = fmaf(part[m], sc, acc[r][m]);
      }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
#pragma unroll
      for (int m = 0; m < MR; ++m) {
        const float t = warp_sum_g(acc[r][m]) * alpha;
        if (lane == 0 && n0 + r < N) {
          if (y) y[m * y_stride + n0 + r] = f32_to_bf16(t);
          if (y32) y32[m * y_stride + n0 + r] = t;
        }
      }
    }
  }
}

template <int MR>
__global__ void __launch_bounds__(kGemvThreads)
gemv_bf16_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, float alpha, bf16* __restrict__ y,
                 float* __restrict__ y32, int N, int K, int64_t x_stride, int64_t y_stride) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* xs = reinterpret_cast<bf16*>(smem_raw);
  pdl_wait();
  for (int m = 0; m < MR; ++m)
    for (int i = threadIdx.x; i < K / 8; i += blockDim.x)
      reinterpret_cast<uint4*>(xs + static_cast<size_t>(m) * K)[i] =
          reinterpret_cast<const uint4*>(x + m * x_stride)[i];
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int R = kGemvRowsPerWarp;
  const int nvec = K / 8;
  for (int n0 = (blockIdx.x * kGemvWarps + warp) * R; n0 < N; n0 += gridDim.x * kGemvWarps * R) {
    float acc[R][MR];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int m = 0; m < MR; ++m) acc[r][m] = 0.f;
    for (int v = lane; v < nvec; v += 32) {
      float xf[MR][8];
#pragma unroll
      for (int m = 0; m < MR; ++m) {
        Pack16 p;
        p.u = reinterpret_cast<const uint4*>(xs + static_cast<size_t>(m) * K)[v];
#pragma unroll
        for (int j = 0; j < 8; ++j) xf[m][j] = bf16_to_f32(p.h[j]);
      }
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const int n = n0 + r < N ? n0 + r : N - 1;
        Pack16 p;
        p.u = reinterpret_cast<const uint4*>(w + static_cast<size_t>(n) * K)[v];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float wf = bf16_to_f32(p.h[j]);
#pragma unroll
          for (int m = 0; m < MR; ++m) acc[r][m] = fmaf(wf, xf[m][j], acc[r][m]);
        }
      }
    }
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int m = 0; m < MR; ++m) {
        const float t = warp_sum_g(acc[r][m]) * alpha;
        if (lane == 0 && n0 + r < N) {
          if (y) y[m * y_stride + n0 + r] = f32_to_bf16(t);
          if (y32) y32[m * y_stride + n0 + r] = t;
        }
      }
  }
}

template <int MR, int GROUP>
static int launch_fp4(const void* x, const void* wq, const void* ws, float alpha, void* y, void* y32, int N, int K,
                      int64_t xs, int64_t ys, cudaStream_t st) {
  const size_t smem = static_cast<size_t>(MR) * K * 2;
  static bool attr = false;
  if (!attr) {
    cudaFuncSetAttribute(gemv_fp4_kernel<MR, GROUP>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
    attr = true;
  }
  int blocks = dgpp_ceil_div(N, kGemvWarps * kGemvRowsPerWarp);
  if (blocks > 148 * 4) blocks = 148 * 4;
  gemv_fp4_kernel<MR, GROUP><<<blocks, kGemvThreads, smem, st>>>(
      static_cast<const bf16*>(x), static_cast<const uint8_t*>(wq), static_cast<const uint8_t*>(ws), alpha,
      static_cast<bf16*>(y), static_cast<float*>(y32), N, K, xs, ys);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

template <int MR>
static int launch_bf16(const void* x, const void* w, float alpha, void* y, void* y32, int N, int K, int64_t xs,
                       int64_t ys, cudaStream_t st) {
  const size_t smem = static_cast<size_t>(MR) * K * 2;
  static bool attr = false;
  if (!attr) {
    cudaFuncSetAttribute(gemv_bf16_kernel<MR>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
    attr = true;
  }
  int blocks = dgpp_ceil_div(N, kGemvWarps * kGemvRowsPerWarp);
  if (blocks > 148 * 4) blocks = 148 * 4;
  gemv_bf16_kernel<MR><<<blocks, kGemvThreads, smem, st>>>(static_cast<const bf16*>(x), static_cast<const bf16*>(w),
                                                          alpha, static_cast<bf16*>(y), static_cast<float*>(y32), N,
                                                          K, xs, ys);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

}  // namespace dgpp

using namespace dgpp;

// fmt: 0 = NVFP4 (e4m3 scale per 16), 1 = MXFP4 (e8m0 scale per 32), 2 = BF16 (wscale unused).
// rows must be 1..4; x: [rows, K] bf16 with row stride x_stride; y (bf16) and/or y32 (fp32): row stride y_stride.
DGPP_API int dgpp_gemv_quant(int fmt, const void* x, const void* wq, const void* wscale, float alpha, void* y,
                             void* y32, int rows, int N, int K, int64_t x_stride, int64_t y_stride,
                             cudaStream_t st) {
  DGPP_REQUIRE(rows >= 1 && rows <= 4, "gemv: rows %d outside 1..4", rows);
  DGPP_REQUIRE(K % 32 == 0 && K % 8 == 0, "gemv: K %d must be a multiple of 32", K);
  DGPP_REQUIRE(static_cast<size_t>(rows) * K * 2 <= 160 * 1024, "gemv: rows*K too large for shared memory");
  DGPP_REQUIRE(y || y32, "gemv: no output");
#define DGPP_GEMV_CASE(MR)                                                                              \
  case MR:                                                                                              \
    if (fmt == 0) return launch_fp4<MR, 16>(x, wq, wscale, alpha, y, y32, N, K, x_stride, y_stride, st); \
    if (fmt == 1) return launch_fp4<MR, 32>(x, wq, wscale, alpha, y, y32, N, K, x_stride, y_stride, st); \
    if (fmt == 2) return launch_bf16<MR>(x, wq, alpha, y, y32, N, K, x_stride, y_stride, st);            \
    break;
  switch (rows) {
    DGPP_GEMV_CASE(1)
    DGPP_GEMV_CASE(2)
    DGPP_GEMV_CASE(3)
    DGPP_GEMV_CASE(4)
  }
#undef DGPP_GEMV_CASE
  dgpp_set_error("gemv: unknown weight format %d", fmt);
  return -1;
}
