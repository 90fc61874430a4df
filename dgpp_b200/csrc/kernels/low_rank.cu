// Low-rank adapter projection: out += scale * (x A^T) B^T with A [r, K], B [N, r] in bf16 and the rank-r
// intermediate kept in fp32.  Two launches: `down` (one CTA per token: the row of x is staged in shared memory, each
// warp owns adapter rows j = warp, warp + W, ... and reduces lane-strided partial sums with a fixed shuffle tree) and
// `up_add` (one thread per output element, y row in shared memory, j ascending).  Both orders are fixed, so the
// result does not depend on the launch geometry.
// Tensor parallel use needs no collective of its own: for a row-split projection every rank adds the update computed
// from ITS slice of x and A into its partial output, and the projection's all-reduce sums the updates with the
// partials; for a column-split projection B is sliced with the weight.
// (reference counterparts: src/kernels/low_rank.cu project / add kernels, src/adapters/runtime.hpp Runtime::project,
//  Runtime::add; the reference sums the fp32 intermediate across ranks through a digit-packed bf16 all-reduce,
//  src/adapters/bus_sum.hpp:35-48.)
#include "common/common.h"
#include "common/dtypes.cuh"
#include "common/ptx.cuh"

namespace dgpp {

constexpr int kLrThreads = 256;

__global__ void __launch_bounds__(kLrThreads)
lora_down_kernel(const bf16* __restrict__ x, int64_t ldx, const bf16* __restrict__ A, float* __restrict__ y, int K, int r) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* xs = reinterpret_cast<bf16*>(smem_raw);
  pdl_wait();
  const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const bf16* xr = x + static_cast<size_t>(t) * ldx;
  for (int i = tid; i < K / 8; i += kLrThreads) reinterpret_cast<uint4*>(xs)[i] = reinterpret_cast<const uint4*>(xr)[i];
  __syncthreads();
  for (int j = warp; j < r; j += kLrThreads / 32) {
    const bf16* ar = A + static_cast<size_t>(j) * K;
    float acc = 0.f;
    for (int i = lane; i < K / 8; i += 32) {
      Pack16 a, b;
      a.u = reinterpret_cast<const uint4*>(ar)[i];
      b.u = reinterpret_cast<const uint4*>(xs)[i];
#pragma unroll
      for (int e = 0; e < 8; ++e) acc = fmaf(bf16_to_f32(a.h[e]), bf16_to_f32(b.h[e]), acc);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) y[static_cast<size_t>(t) * r + j] = acc;
  }
}

__global__ void __launch_bounds__(kLrThreads)
lora_up_add_kernel(const float* __restrict__ y, const bf16* __restrict__ B, bf16* __restrict__ out, int64_t ldc, float scale,
                   int N, int r) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* ys = reinterpret_cast<float*>(smem_raw);
  pdl_wait();
  const int t = blockIdx.y, n = blockIdx.x * kLrThreads + threadIdx.x;
  for (int j = threadIdx.x; j < r; j += kLrThreads) ys[j] = y[static_cast<size_t>(t) * r + j];
  __syncthreads();
  if (n >= N) return;
  const bf16* br = B + static_cast<size_t>(n) * r;
  float acc = 0.f;
  for (int j = 0; j < r; ++j) acc = fmaf(ys[j], bf16_to_f32(br[j]), acc);
  bf16* o = out + static_cast<size_t>(t) * ldc + n;
  *o = f32_to_bf16(bf16_to_f32(*o) + scale * acc);
}

}  // namespace dgpp

using namespace dgpp;

// x [T, K] bf16 (row stride ldx), A [r, K] bf16, B [N, r] bf16, y [T, r] fp32 scratch, out [T, N] bf16 (row stride
// ldc), updated in place.
extern "C" int dgpp_lora_apply(const void* x, int64_t ldx, const void* A, const void* B, void* y, void* out, int64_t ldc,
                               float scale, int T, int N, int K, int r, void* stream) {
  DGPP_REQUIRE(T > 0 && N > 0 && r > 0 && K % 8 == 0 && ldx % 8 == 0, "lora: bad shape T=%d N=%d K=%d r=%d", T, N, K, r);
  DGPP_REQUIRE(static_cast<size_t>(K) * 2 <= 200 * 1024, "lora: K %d does not fit shared memory", K);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t smem = static_cast<size_t>(K) * 2;
  if (smem > 48 * 1024)
    DGPP_CUDA_OK(cudaFuncSetAttribute(lora_down_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
  lora_down_kernel<<<T, kLrThreads, smem, st>>>(static_cast<const bf16*>(x), ldx, static_cast<const bf16*>(A),
                                               static_cast<float*>(y), K, r);
  DGPP_CUDA_OK(cudaGetLastError());
  lora_up_add_kernel<<<dim3((N + kLrThreads - 1) / kLrThreads, T), kLrThreads, static_cast<size_t>(r) * 4, st>>>(
      static_cast<const float*>(y), static_cast<const bf16*>(B), static_cast<bf16*>(out), ldc, scale, N, r);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}
