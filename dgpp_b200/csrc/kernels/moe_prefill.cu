// Mixture-of-experts at prefill sizes: counting sort of the (token, k-slot) pairs by expert, tile list, row gather and
// ordered combine around the grouped block-scaled expert GEMM (gemm_fp4.cu, grouped mode with one token tile per slot).
//
//   moe_segment_sort_kernel   one CTA.  Histogram of the pairs per local expert, tiles per expert = ceil(n_e / bn),
//                             exclusive scan -> first tile of every expert; then a STABLE rank of every pair inside its
//                             expert (pairs keep their (token, k) order), so row = tile * bn + rank % bn is a pure function
//                             of the routing result.  Outputs pair_row [T * k] (-1: expert lives on another rank),
//                             tile_expert [max_tiles] (local expert of every tile, -1 beyond the last one), n_tiles.
//   moe_gather_rows_kernel    xs[pair_row[p]] = x[p / k]   (bf16 rows; the quantiser and the grouped GEMM then see
//                             every tile as one "slot" of bn token rows)
//   moe_combine_rows_kernel   out[t] = sum_j w[t, j] * y[pair_row[t, j]] (+ shared[t]) in ascending j, fp32, one rounding
//
// (reference counterparts: src/kernels/glm_moe.cu:1382 moe_segment_count_kernel, :1553 moe_tile_list_kernel, gather /
//  ordered accumulate kernels of the same file.)
#include "common/common.h"
#include "common/dtypes.cuh"
#include "common/ptx.cuh"

namespace dgpp {

constexpr int kSortThreads = 1024;
constexpr int kSortWarps = kSortThreads / 32;
constexpr int kSortMaxExperts = 512;

struct SortArgs {
  const int32_t* ids;      // [T, k] global expert ids
  int32_t* pair_row;       // [T * k]
  int32_t* tile_expert;    // [max_tiles]
  int32_t* n_tiles;        // [1]
  int T, k, E, e_begin, e_end, bn, max_tiles;
};

__global__ void __launch_bounds__(kSortThreads) moe_segment_sort_kernel(SortArgs a) {
  // per-warp histograms (later: per-warp running offsets), the experts' totals / first tiles
  extern __shared__ int ssm[];
  int* hist = ssm;                                  // [warps][E]
  int* first_tile = hist + kSortWarps * a.E;        // [E]
  int* total = first_tile + a.E;                    // [E]
  pdl_wait();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int P = a.T * a.k;
  const int seg = (P + kSortWarps - 1) / kSortWarps;           // pairs per warp, contiguous and in order
  const int p0 = warp * seg, p1 = min(P, p0 + seg);
  for (int i = tid; i < kSortWarps * a.E; i += kSortThreads) hist[i] = 0;
  __syncthreads();
  // pass 1: histogram of this warp's segment (shared-memory atomics: counts are order-independent)
  for (int p = p0 + lane; p < p1; p += 32) {
    const int e = a.ids[p];
    if (e >= a.e_begin && e < a.e_end) atomicAdd(&hist[warp * a.E + (e - a.e_begin)], 1);
  }
  __syncthreads();
  // per expert: exclusive scan over the warps (a warp's pairs come before the next warp's) and the total
  for (int e = tid; e < a.E; e += kSortThreads) {
    int run = 0;
    for (int w = 0; w < kSortWarps; ++w) {
      const int c = hist[w * a.E + e];
      hist[w * a.E + e] = run;
      run += c;
    }
    total[e] = run;
  }
  __syncthreads();
  if (tid == 0) {
    int t = 0;
    for (int e = 0; e < a.E; ++e) {
      first_tile[e] = t;
      const int nt = (total[e] + a.bn - 1) / a.bn;
      for (int i = 0; i < nt && t + i < a.max_tiles; ++i) a.tile_expert[t + i] = e;
      t += nt;
    }
    *a.n_tiles = min(t, a.max_tiles);
    for (int i = t; i < a.max_tiles; ++i) a.tile_expert[i] = -1;
  }
  __syncthreads();
  // pass 2: stable rank.  A warp walks its segment 32 pairs at a time; lanes with the same expert form a group whose
  // members are ranked by lane order, the group's lowest lane advances the warp's running offset of that expert.
  for (int base = p0; base < p1; base += 32) {
    const int p = base + lane;
    int e = -1;
    if (p < p1) {
      const int g = a.ids[p];
      if (g >= a.e_begin && g < a.e_end) e = g - a.e_begin;
    }
    const unsigned same = __match_any_sync(0xffffffffu, e);
    const int rank_in_group = __popc(same & ((1u << lane) - 1u));
    const int leader = __ffs(same) - 1;
    int start = 0;
    if (e >= 0 && lane == leader) {
      start = hist[warp * a.E + e];
      hist[warp * a.E + e] = start + __popc(same);
    }
    start = __shfl_sync(0xffffffffu, start, leader);
    if (p < p1) {
      int row = -1;
      if (e >= 0) {
        const int r = start + rank_in_group;
        const int tile = first_tile[e] + r / a.bn;
        row = tile < a.max_tiles ? tile * a.bn + r % a.bn : -1;
      }
      a.pair_row[p] = row;
    }
    __syncwarp();
  }
}

// grid (T * k), 128 threads: one pair per CTA.
__global__ void __launch_bounds__(128) moe_gather_rows_kernel(const bf16* __restrict__ x, int64_t x_stride,
                                                              const int32_t* __restrict__ pair_row, bf16* __restrict__ xs,
                                                              int H, int k) {
  pdl_wait();
  const int p = blockIdx.x;
  const int row = pair_row[p];
  if (row < 0) return;
  const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(p / k) * x_stride);
  uint4* dst = reinterpret_cast<uint4*>(xs + static_cast<size_t>(row) * H);
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) dst[i] = src[i];
}

// grid (ceil(H / 8 / 256), T)
__global__ void __launch_bounds__(256) moe_combine_rows_kernel(const bf16* __restrict__ y, const bf16* __restrict__ shared,
                                                               const int32_t* __restrict__ pair_row, const float* __restrict__ w,
                                                               bf16* __restrict__ out, int H, int k) {
  pdl_wait();
  const int t = blockIdx.y;
  const int v = blockIdx.x * blockDim.x + threadIdx.x;
  if (v * 8 >= H) return;
  float acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.f;
  for (int i = 0; i < k; ++i) {
    const int row = pair_row[t * k + i];
    if (row < 0) continue;
    const float wi = w[t * k + i];
    Pack16 p;
    p.u = *reinterpret_cast<const uint4*>(y + static_cast<size_t>(row) * H + v * 8);
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

}  // namespace dgpp

using namespace dgpp;

// Sort the pairs of `ids` [T, k] by local expert (experts [e_begin, e_end) of E_global live here) into tiles of bn rows.
DGPP_API int dgpp_moe_segment_sort(const void* ids, void* pair_row, void* tile_expert, void* n_tiles, int T, int k,
                                   int e_begin, int e_end, int bn, int max_tiles, cudaStream_t st) {
  const int E = e_end - e_begin;
  DGPP_REQUIRE(E >= 1 && E <= kSortMaxExperts, "moe_segment_sort: %d local experts (1..%d)", E, kSortMaxExperts);
  DGPP_REQUIRE(bn >= 16 && max_tiles >= 1 && T >= 0 && k >= 1, "moe_segment_sort: bad sizes");
  if (T == 0) return 0;
  SortArgs a;
  a.ids = static_cast<const int32_t*>(ids);
  a.pair_row = static_cast<int32_t*>(pair_row);
  a.tile_expert = static_cast<int32_t*>(tile_expert);
  a.n_tiles = static_cast<int32_t*>(n_tiles);
  a.T = T; a.k = k; a.E = E; a.e_begin = e_begin; a.e_end = e_end; a.bn = bn; a.max_tiles = max_tiles;
  const size_t smem = (static_cast<size_t>(kSortWarps) * E + 2 * E) * sizeof(int);
  static bool attr = false;
  if (!attr) {
    DGPP_CUDA_OK(cudaFuncSetAttribute(moe_segment_sort_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
    attr = true;
  }
  moe_segment_sort_kernel<<<1, kSortThreads, smem, st>>>(a);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

DGPP_API int dgpp_moe_gather_rows(const void* x, int64_t x_stride, const void* pair_row, void* xs, int T, int H, int k,
                                  cudaStream_t st) {
  DGPP_REQUIRE(H % 8 == 0 && x_stride % 8 == 0, "moe_gather_rows: hidden %d / stride must be multiples of 8", H);
  if (T == 0) return 0;
  moe_gather_rows_kernel<<<T * k, 128, 0, st>>>(static_cast<const bf16*>(x), x_stride, static_cast<const int32_t*>(pair_row),
                                                static_cast<bf16*>(xs), H, k);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

DGPP_API int dgpp_moe_combine_rows(const void* y, const void* shared, const void* pair_row, const void* w, void* out, int T,
                                   int H, int k, cudaStream_t st) {
  DGPP_REQUIRE(H % 8 == 0, "moe_combine_rows: hidden %d must be a multiple of 8", H);
  if (T == 0) return 0;
  dim3 grid(dgpp_ceil_div(H / 8, 256), T);
  moe_combine_rows_kernel<<<grid, 256, 0, st>>>(static_cast<const bf16*>(y), static_cast<const bf16*>(shared),
                                                static_cast<const int32_t*>(pair_row), static_cast<const float*>(w),
                                                static_cast<bf16*>(out), H, k);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}
