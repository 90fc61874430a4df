// Row-wise memory-bound ops: embedding gather, RMSNorm (+ fused residual add), SwiGLU,
// greedy argmax with lowest-index tie-break.  One CTA per row, 16-byte vector accesses,
// fixed-order reductions so results do not depend on launch geometry.
//
// Rounding points follow the bf16 PyTorch modules they replace:
//   rmsnorm:  y = bf16( w * bf16(x * rstd) ),   rstd = rsqrt(mean(x^2) + eps) in fp32
//   residual: r = bf16(r + d) before the norm
//   swiglu:   a = bf16( bf16(silu(g)) * u )
// (reference behaviour: src/kernels/add_rmsnorm.cu:28, src/kernels/kernels.cu:19,58,98,142 of the
// reference tree describe the same operator set.)
#include <cooperative_groups.h>
#include <string.h>

#include "common/common.h"
#include "common/dtypes.cuh"
#include "common/ptx.cuh"

namespace dgpp {

constexpr int kRowThreads = 256;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Sum over the CTA in a fixed order: lanes by xor-tree, then warps ascending.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) scratch[w] = v;
  __syncthreads();
  float t = 0.f;
  const int nw = blockDim.x >> 5;
  for (int i = 0; i < nw; ++i) t += scratch[i];
  __syncthreads();
  return t;
}

__global__ void __launch_bounds__(kRowThreads)
embed_gather_kernel(const int32_t* __restrict__ ids, const bf16* __restrict__ table, bf16* __restrict__ out,
                    int hidden, int vocab) {
  pdl_wait();
  const int row = blockIdx.x;
  int id = ids[row];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  const uint4* src = reinterpret_cast<const uint4*>(table + static_cast<size_t>(id) * hidden);
  uint4* dst = reinterpret_cast<uint4*>(out + static_cast<size_t>(row) * hidden);
  for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x) dst[i] = src[i];
}

// out = rmsnorm(resid (+ delta)); when delta != nullptr the sum is also written back to resid_out.
// gemma_style: weight is applied as (1 + w).
template <bool kAdd>
__global__ void __launch_bounds__(kRowThreads)
rmsnorm_kernel(const bf16* __restrict__ resid, const bf16* __restrict__ delta, const bf16* __restrict__ w,
               bf16* __restrict__ resid_out, bf16* __restrict__ out, int hidden, float eps, int one_plus_w) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* row_s = reinterpret_cast<bf16*>(smem_raw);
  __shared__ float scratch[32];
  pdl_wait();
  const size_t base = static_cast<size_t>(blockIdx.x) * hidden;
  const int nvec = hidden / 8;
  float ss = 0.f;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    Pack16 a;
    a.u = reinterpret_cast<const uint4*>(resid + base)[i];
    if (kAdd) {
      Pack16 d;
      d.u = reinterpret_cast<const uint4*>(delta + base)[i];
#pragma unroll
      for (int j = 0; j < 8; ++j) a.h[j] = f32_to_bf16(bf16_to_f32(a.h[j]) + bf16_to_f32(d.h[j]));
      reinterpret_cast<uint4*>(resid_out + base)[i] = a.u;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float f = bf16_to_f32(a.h[j]);
      ss += f * f;
    }
    reinterpret_cast<uint4*>(row_s)[i] = a.u;
  }
  const float total = block_sum(ss, scratch);
  const float rstd = rsqrtf(total / static_cast<float>(hidden) + eps);
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    Pack16 a, ww, o;
    a.u = reinterpret_cast<const uint4*>(row_s)[i];
    ww.u = reinterpret_cast<const uint4*>(w)[i];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float n = bf16_to_f32(f32_to_bf16(bf16_to_f32(a.h[j]) * rstd));
      float g = bf16_to_f32(ww.h[j]);
      if (one_plus_w) g += 1.f;
      o.h[j] = f32_to_bf16(n * g);
    }
    reinterpret_cast<uint4*>(out + base)[i] = o.u;
  }
}

// gate_up: [rows, 2*inter] (gate then up); out: [rows, inter].  limit > 0 clamps gate above and up both sides.
// alpha > 0 selects the scaled-sigmoid form  gate * sigmoid(alpha * gate) * (up + 1)  (alpha = 0: silu(gate) * up).
__global__ void __launch_bounds__(kRowThreads)
swiglu_kernel(const bf16* __restrict__ gate_up, bf16* __restrict__ out, int inter, float limit, float alpha) {
  pdl_wait();
  const size_t row = blockIdx.y;
  const bf16* g = gate_up + row * 2 * inter;
  const bf16* u = g + inter;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= inter / 8) return;
  Pack16 a, b, o;
  a.u = reinterpret_cast<const uint4*>(g)[i];
  b.u = reinterpret_cast<const uint4*>(u)[i];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    float gv = bf16_to_f32(a.h[j]);
    float uv = bf16_to_f32(b.h[j]);
    if (limit > 0.f) {
      gv = fminf(gv, limit);
      uv = fminf(fmaxf(uv, -limit), limit);
    }
    float s;
    if (alpha > 0.f) {
      s = bf16_to_f32(f32_to_bf16(gv / (1.f + __expf(-alpha * gv))));
      uv += 1.f;
    } else {
      s = bf16_to_f32(f32_to_bf16(gv / (1.f + __expf(-gv))));
    }
    o.h[j] = f32_to_bf16(s * uv);
  }
  reinterpret_cast<uint4*>(out + row * inter)[i] = o.u;
}

// Greedy pick: argmax over `vocab` logits per row, ties -> lowest index.  Writes the token id
// (offset by id_base, for vocab-sharded heads) and the winning value.
template <typename T>
__global__ void __launch_bounds__(1024)
argmax_kernel(const T* __restrict__ logits, int64_t row_stride, int vocab, int id_base,
              int32_t* __restrict__ out_id, float* __restrict__ out_val) {
  __shared__ float sv[32];
  __shared__ int si[32];
  pdl_wait();
  const T* row = logits + static_cast<size_t>(blockIdx.x) * row_stride;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    float v = static_cast<float>(row[i]);
    if (v > best || (v == best && i < bi)) {
      best = v;
      bi = i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float ov = __shfl_xor_sync(0xffffffffu, best, o);
    int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) {
      best = ov;
      bi = oi;
    }
  }
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) {
    sv[w] = best;
    si[w] = bi;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < (blockDim.x >> 5); ++i) {
      if (sv[i] > best || (sv[i] == best && si[i] < bi)) {
        best = sv[i];
        bi = si[i];
      }
    }
    out_id[blockIdx.x] = bi + id_base;
    if (out_val) out_val[blockIdx.x] = best;
  }
}

// The same pick with one row spread over a thread-block cluster (decode: a handful of rows of a 150K vocabulary would
// otherwise keep a handful of SMs busy): CTA c scans slice c of the row, pushes its (value, index) into CTA 0's
// shared memory, and after the cluster barrier CTA 0 picks among the slices in the same order rule (largest value,
// lowest index), so the result is the single-CTA kernel's.
template <typename T>
__global__ void __launch_bounds__(1024)
argmax_cluster_kernel(const T* __restrict__ logits, int64_t row_stride, int vocab, int id_base,
                      int32_t* __restrict__ out_id, float* __restrict__ out_val) {
  namespace cg = cooperative_groups;
  __shared__ float sv[32];
  __shared__ int si[32];
  __shared__ float cv[8];
  __shared__ int ci[8];
  cg::cluster_group cluster = cg::this_cluster();
  pdl_wait();
  const int c = blockIdx.x, ncl = gridDim.x;
  const T* row = logits + static_cast<size_t>(blockIdx.y) * row_stride;
  const int chunk = ((vocab + ncl - 1) / ncl + 3) & ~3;
  const int lo = c * chunk, hi = min(vocab, lo + chunk);
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    float v = static_cast<float>(row[i]);
    if (v > best || (v == best && i < bi)) {
      best = v;
      bi = i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float ov = __shfl_xor_sync(0xffffffffu, best, o);
    int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) {
      best = ov;
      bi = oi;
    }
  }
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) {
    sv[w] = best;
    si[w] = bi;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < (blockDim.x >> 5); ++i) {
      if (sv[i] > best || (sv[i] == best && si[i] < bi)) {
        best = sv[i];
        bi = si[i];
      }
    }
    *cluster.map_shared_rank(&cv[c], 0) = best;
    *cluster.map_shared_rank(&ci[c], 0) = bi;
  }
  cluster.sync();
  if (c == 0 && threadIdx.x == 0) {
    best = cv[0];
    bi = ci[0];
    for (int i = 1; i < ncl; ++i) {
      if (cv[i] > best || (cv[i] == best && ci[i] < bi)) {
        best = cv[i];
        bi = ci[i];
      }
    }
    out_id[blockIdx.y] = bi + id_base;
    if (out_val) out_val[blockIdx.y] = best;
  }
}

template <typename T>
static int launch_argmax_cluster(const T* logits, int64_t row_stride, int rows, int vocab, int id_base, int32_t* out_id,
                                 float* out_val, cudaStream_t st) {
  constexpr int kCl = 8;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(kCl, rows, 1);
  cfg.blockDim = dim3(1024, 1, 1);
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = kCl;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  DGPP_CUDA_OK(cudaLaunchKernelEx(&cfg, argmax_cluster_kernel<T>, logits, row_stride, vocab, id_base, out_id, out_val));
  return 0;
}

// dst[i] = src[i] (bf16 rows), used for snapshots and gathers inside graphs (no memcpy nodes).
__global__ void copy_rows_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, int64_t nvec) {
  pdl_wait();
  int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t step = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (; i < nvec; i += step) dst[i] = src[i];
}

// y = a + b (bf16, one rounding).
__global__ void add_kernel(const bf16* __restrict__ a, const bf16* __restrict__ b, bf16* __restrict__ y, int64_t n8) {
  pdl_wait();
  int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  Pack16 x, z;
  x.u = reinterpret_cast<const uint4*>(a)[i];
  z.u = reinterpret_cast<const uint4*>(b)[i];
#pragma unroll
  for (int j = 0; j < 8; ++j) x.h[j] = f32_to_bf16(bf16_to_f32(x.h[j]) + bf16_to_f32(z.h[j]));
  reinterpret_cast<uint4*>(y)[i] = x.u;
}

}  // namespace dgpp

using namespace dgpp;

DGPP_API int dgpp_embed_gather(const void* ids, const void* table, void* out, int rows, int hidden, int vocab,
                               cudaStream_t st) {
  DGPP_REQUIRE(hidden % 8 == 0, "embed_gather: hidden %d must be a multiple of 8", hidden);
  if (rows == 0) return 0;
  embed_gather_kernel<<<rows, kRowThreads, 0, st>>>(static_cast<const int32_t*>(ids),
                                                   static_cast<const bf16*>(table), static_cast<bf16*>(out), hidden,
                                                   vocab);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

DGPP_API int dgpp_rmsnorm(const void* resid, const void* delta, const void* w, void* resid_out, void* out, int rows,
                          int hidden, float eps, int one_plus_w, cudaStream_t st) {
  DGPP_REQUIRE(hidden % 8 == 0, "rmsnorm: hidden %d must be a multiple of 8", hidden);
  DGPP_REQUIRE(hidden * 2 <= 96 * 1024, "rmsnorm: hidden %d too large for the row buffer", hidden);
  if (rows == 0) return 0;
  const size_t smem = static_cast<size_t>(hidden) * 2;
  if (delta) {
    static bool attr_set = false;
    if (!attr_set) {
      cudaFuncSetAttribute(rmsnorm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
      cudaFuncSetAttribute(rmsnorm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
      attr_set = true;
    }
    rmsnorm_kernel<true><<<rows, kRowThreads, smem, st>>>(
        static_cast<const bf16*>(resid), static_cast<const bf16*>(delta), static_cast<const bf16*>(w),
        static_cast<bf16*>(resid_out), static_cast<bf16*>(out), hidden, eps, one_plus_w);
  } else {
    static bool attr_set2 = false;
    if (!attr_set2) {
      cudaFuncSetAttribute(rmsnorm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
      attr_set2 = true;
    }
    rmsnorm_kernel<false><<<rows, kRowThreads, smem, st>>>(static_cast<const bf16*>(resid), nullptr,
                                                          static_cast<const bf16*>(w), nullptr,
                                                          static_cast<bf16*>(out), hidden, eps, one_plus_w);
  }
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

DGPP_API int dgpp_swiglu(const void* gate_up, void* out, int rows, int inter, float limit, float alpha,
                         cudaStream_t st) {
  DGPP_REQUIRE(inter % 8 == 0, "swiglu: inter %d must be a multiple of 8", inter);
  if (rows == 0) return 0;
  dim3 grid(dgpp_ceil_div(inter / 8, kRowThreads), rows);
  swiglu_kernel<<<grid, kRowThreads, 0, st>>>(static_cast<const bf16*>(gate_up), static_cast<bf16*>(out), inter,
                                             limit, alpha);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

// dtype: 0 = bf16 logits, 1 = fp32 logits.
DGPP_API int dgpp_argmax(const void* logits, int dtype, int64_t row_stride, int rows, int vocab, int id_base,
                         void* out_id, void* out_val, cudaStream_t st) {
  if (rows == 0) return 0;
  if (rows <= 64 && vocab >= 16384) {   // few long rows: one cluster of 8 CTAs per row
    if (dtype == 0)
      return launch_argmax_cluster<bf16>(static_cast<const bf16*>(logits), row_stride, rows, vocab, id_base,
                                         static_cast<int32_t*>(out_id), static_cast<float*>(out_val), st);
    return launch_argmax_cluster<float>(static_cast<const float*>(logits), row_stride, rows, vocab, id_base,
                                        static_cast<int32_t*>(out_id), static_cast<float*>(out_val), st);
  }
  if (dtype == 0)
    argmax_kernel<bf16><<<rows, 1024, 0, st>>>(static_cast<const bf16*>(logits), row_stride, vocab, id_base,
                                              static_cast<int32_t*>(out_id), static_cast<float*>(out_val));
  else
    argmax_kernel<float><<<rows, 1024, 0, st>>>(static_cast<const float*>(logits), row_stride, vocab, id_base,
                                               static_cast<int32_t*>(out_id), static_cast<float*>(out_val));
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

DGPP_API int dgpp_copy_bytes(const void* src, void* dst, int64_t bytes, cudaStream_t st) {
  DGPP_REQUIRE(bytes % 16 == 0, "copy_bytes: size %lld must be a multiple of 16", (long long)bytes);
  if (bytes == 0) return 0;
  const int64_t nvec = bytes / 16;
  int blocks = static_cast<int>(nvec / 256 < 1 ? 1 : (nvec / 256 > 1184 ? 1184 : nvec / 256));
  copy_rows_kernel<<<blocks, 256, 0, st>>>(static_cast<const uint4*>(src), static_cast<uint4*>(dst), nvec);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

DGPP_API int dgpp_add_bf16(const void* a, const void* b, void* y, int64_t n, cudaStream_t st) {
  DGPP_REQUIRE(n % 8 == 0, "add: n must be a multiple of 8");
  if (n == 0) return 0;
  const int64_t n8 = n / 8;
  add_kernel<<<static_cast<int>(dgpp_ceil_div64(n8, 256)), 256, 0, st>>>(
      static_cast<const bf16*>(a), static_cast<const bf16*>(b), static_cast<bf16*>(y), n8);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

namespace dgpp {
// End-of-step bookkeeping for a host-free decode loop: the picked ids become the next input tokens,
// positions advance by one, and the ids are appended to a device ring [ring_steps, rows].
__global__ void decode_advance_kernel(const int32_t* __restrict__ picked, int32_t* __restrict__ tokens,
                                      int32_t* __restrict__ positions, int32_t* __restrict__ ring,
                                      int32_t* __restrict__ step_counter, int rows, int ring_steps) {
  pdl_wait();
  const int i = threadIdx.x;
  const int step = *step_counter;
  if (i < rows) {
    const int id = picked[i];
    tokens[i] = id;
    positions[i] += 1;
    if (ring) ring[static_cast<size_t>(step % ring_steps) * rows + i] = id;
  }
  __syncthreads();
  if (i == 0) *step_counter = step + 1;
}
}  // namespace dgpp

DGPP_API int dgpp_decode_advance(const void* picked, void* tokens, void* positions, void* ring, void* step_counter,
                                 int rows, int ring_steps, cudaStream_t st) {
  DGPP_REQUIRE(rows >= 1 && rows <= 1024, "decode_advance: rows %d outside 1..1024", rows);
  dgpp::decode_advance_kernel<<<1, 1024, 0, st>>>(static_cast<const int32_t*>(picked), static_cast<int32_t*>(tokens),
                                                 static_cast<int32_t*>(positions), static_cast<int32_t*>(ring),
                                                 static_cast<int32_t*>(step_counter), rows, ring_steps);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

// Batched segment copy: n independent (source, destination, bytes) copies described by a DEVICE table, one launch.
// Used for state snapshots / restores (many small per-layer tensors) inside captured graphs, where the segments are
// chosen by earlier kernels.  Addresses and sizes are multiples of 16 bytes.  grid (chunks, n).
// (reference counterpart: src/kernels/segment_copy.cu.)
namespace dgpp {
struct Segment {
  const void* src;
  void* dst;
  int64_t bytes;
};
__global__ void __launch_bounds__(256) segment_copy_kernel(const Segment* __restrict__ segs) {
  pdl_wait();
  const Segment s = segs[blockIdx.y];
  const int64_t vecs = s.bytes / 16;
  const uint4* src = static_cast<const uint4*>(s.src);
  uint4* dst = static_cast<uint4*>(s.dst);
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < vecs; i += static_cast<int64_t>(gridDim.x) * blockDim.x)
    dst[i] = src[i];
}
}  // namespace dgpp

// segs: device array of n {src, dst, bytes} records (24 bytes each); max_bytes: the largest segment (sizes the grid).
DGPP_API int dgpp_segment_copy(const void* segs, int n, int64_t max_bytes, cudaStream_t st) {
  DGPP_REQUIRE(n >= 0 && max_bytes >= 0 && max_bytes % 16 == 0, "segment_copy: sizes must be multiples of 16 bytes");
  if (n == 0 || max_bytes == 0) return 0;
  int64_t chunks = (max_bytes / 16 + 256 * 8 - 1) / (256 * 8);
  if (chunks > 64) chunks = 64;
  if (chunks < 1) chunks = 1;
  dgpp::segment_copy_kernel<<<dim3(static_cast<unsigned>(chunks), n), 256, 0, st>>>(static_cast<const dgpp::Segment*>(segs));
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}
