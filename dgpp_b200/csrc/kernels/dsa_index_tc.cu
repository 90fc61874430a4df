// Lightning-indexer scores on the tensor cores (tcgen05 kind::f16 over bf16 keys, or kind::f8f6f4 over e4m3 keys):
//     scores[row, t] = sum_h w[row, h] * relu(q[row, h, :] . k[t, :])   for t <= position[row];  -inf beyond.
// One CTA serves one query row and a run of 128-token tiles of its context.  A tile of index keys [128 tokens, di = 128]
// arrives by TMA from the paged key cache (two 64-element column blocks, 128-byte swizzle) and is the A operand; the
// row's hi <= 64 query heads are the B operand (N = 64), written once per CTA.  D[token, head] lands in TMEM (tokens =
// lanes); an epilogue thread owns one token: it reads its 64 head dots, applies relu and the head weights in ascending
// head order and stores one fp32 score.  Key tiles run through a TMA ring, TMEM is double buffered, so loads, the
// 8 MMAs of a tile and the epilogue of the previous tile overlap.
// Warps: 0 = TMA producer, 1 = MMA issuer / TMEM owner, 2..5 = epilogue.  Bounded waits throughout.
// (reference counterparts: src/kernels/dsa.cu:1671 prefill_fused_score_keys_kernel, indexer decode scores.)
#include <cuda.h>
#include <math.h>
#include <string.h>

#include "common/common.h"
#include "common/dtypes.cuh"
#include "common/ptx.cuh"
#include "kernels/gemm_common.cuh"

namespace dgpp {

constexpr int kIxThreads = 192;
constexpr int kIxTile = 128;
constexpr int kIxHeads = 64;
constexpr int kIxStages = 3;
constexpr int kIxBlk = kIxTile * 128;   // 16 KB: one 64-element column block of a key tile

struct IndexTcParams {
  const bf16* q;        // [rows, hi, 128]
  const float* w;       // [rows, hi]
  const int32_t* block_table;
  const int32_t* row_req;
  const int32_t* positions;
  float* scores;        // [rows, ld]
  DeviceStatus* status;
  int rows, hi, page, max_blocks, ld, tiles_per_cta;
};

__global__ void __launch_bounds__(kIxThreads, 1)
dsa_index_tc_kernel(const __grid_constant__ CUtensorMap tmK, IndexTcParams p) {
  constexpr int kTileBytes = 2 * kIxBlk;
  constexpr int kQBlk = kIxHeads * 128;   // 8 KB
  extern __shared__ __align__(1024) unsigned char smem_dyn[];
  unsigned char* sp = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  unsigned char* sK = sp;  sp += kIxStages * kTileBytes;
  unsigned char* sQ = sp;  sp += 2 * kQBlk;
  float* sW = reinterpret_cast<float*>(sp);  sp += kIxHeads * sizeof(float);
  uint64_t* full = reinterpret_cast<uint64_t*>(sp);
  uint64_t* empty = full + kIxStages;
  uint64_t* acc_full = empty + kIxStages;   // [2]
  uint64_t* acc_empty = acc_full + 2;       // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.y;
  const int pos = p.positions[row];
  const int total_tiles = pos / kIxTile + 1;                 // tiles that hold a token <= pos
  const int tile0 = blockIdx.x * p.tiles_per_cta;
  const int ntiles = max(0, min(total_tiles, tile0 + p.tiles_per_cta) - tile0);
  const int32_t* bt = p.block_table + static_cast<size_t>(p.row_req[row]) * p.max_blocks;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kIxStages; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], 4); }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmK);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 128);
    tmem_relinquish();
  }
  pdl_wait();
  if (warp >= 2) {
    // query heads as the B operand: two column blocks of [64 heads, 64 elements]; heads beyond hi are zero
    const int t = threadIdx.x - 64;
    for (int i = t; i < kIxHeads * 16; i += 128) {
      const int h = i / 16, c = i % 16;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (h < p.hi) v = *reinterpret_cast<const uint4*>(p.q + (static_cast<size_t>(row) * p.hi + h) * 128 + c * 8);
      *reinterpret_cast<uint4*>(sQ + (c >> 3) * kQBlk + h * 128 + (((c & 7) ^ (h & 7)) << 4)) = v;
    }
    if (t < kIxHeads) sW[t] = t < p.hi ? p.w[static_cast<size_t>(row) * p.hi + t] : 0.f;
    fence_proxy_async_smem();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (elect_one()) {
      const int ppt = kIxTile / p.page;
      for (int i = 0; i < ntiles; ++i) {
        const int s = i % kIxStages;
        if (!wait_bar(&empty[s], ((i / kIxStages) & 1) ^ 1)) { report(p.status, kTimeoutStageEmpty, 71); *abort_flag = 1; break; }
        mbar_expect_tx(&full[s], kTileBytes);
        const int page0 = (tile0 + i) * kIxTile / p.page;
        for (int pg = 0; pg < ppt; ++pg) {
          const int pi = min(page0 + pg, p.max_blocks - 1);
          const int r0 = bt[pi] * p.page;
          tma_load_2d(sK + s * kTileBytes + pg * p.page * 128, &tmK, 0, r0, &full[s]);
          tma_load_2d(sK + s * kTileBytes + kIxBlk + pg * p.page * 128, &tmK, 64, r0, &full[s]);
        }
        if (*abort_flag) break;
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc_f16(128, kIxHeads, 1u, 1u);
      const uint32_t q_addr = smem_u32(sQ);
      for (int i = 0; i < ntiles; ++i) {
        const int s = i % kIxStages, b = i & 1;
        if (!wait_bar(&acc_empty[b], ((i >> 1) & 1) ^ 1)) { report(p.status, kTimeoutAccum, 72); *abort_flag = 1; break; }
        if (!wait_bar(&full[s], (i / kIxStages) & 1)) { report(p.status, kTimeoutTmaFull, 73); *abort_flag = 1; break; }
        tc_fence_after();
        const uint32_t k_addr = smem_u32(sK + s * kTileBytes);
#pragma unroll
        for (int kb = 0; kb < 2; ++kb)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_f16(tmem_base + b * kIxHeads, umma_desc_sw128(k_addr + kb * kIxBlk + k * 32),
                     umma_desc_sw128(q_addr + kb * kQBlk + k * 32), idesc, (kb > 0 || k > 0) ? 1u : 0u);
        umma_commit(&acc_full[b]);
        umma_commit(&empty[s]);
        if (*abort_flag) break;
      }
    }
  } else {
    const int quad = warp & 3;
    const int idx = quad * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    for (int i = 0; i < ntiles; ++i) {
      const int b = i & 1;
      if (!wait_bar(&acc_full[b], (i >> 1) & 1)) { report(p.status, kTimeoutAccum, 74); *abort_flag = 1; break; }
      tc_fence_after();
      float out = 0.f;
#pragma unroll
      for (int c0 = 0; c0 < kIxHeads; c0 += 16) {
        uint32_t raw[16];
        tmem_ld_x16(tmem_base + b * kIxHeads + c0 + lane_addr, raw);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 16; ++c) out = fmaf(sW[c0 + c], fmaxf(__uint_as_float(raw[c]), 0.f), out);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[b]);
      const int t = (tile0 + i) * kIxTile + idx;
      if (t < p.ld) p.scores[static_cast<size_t>(row) * p.ld + t] = t <= pos ? out : -INFINITY;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, 128);
}

// ---------------------------------------------------------------------------------------------- FP8 index keys
// Keys cached as e4m3 bytes [tokens, 128] with one fp32 scale per token (amax / 448); kind::f8f6f4.  A key tile is ONE
// 128-byte-swizzled block (128 tokens x 128 bytes, half the bytes of the bf16 form).  The query heads are split in the
// prologue into two e4m3 terms per head scale (value + 16 x residual, bf16-grade together) and stacked along N:
// columns 0..63 = first terms, 64..127 = second terms; the epilogue adds the pair, applies relu, the head weight times
// the head's query scale, and the token's key scale.
struct IndexTcFp8Params {
  const bf16* q;        // [rows, hi, 128]
  const float* w;       // [rows, hi]
  const float* kscale;  // [num_blocks * page]
  const int32_t* block_table;
  const int32_t* row_req;
  const int32_t* positions;
  float* scores;
  DeviceStatus* status;
  int rows, hi, page, max_blocks, ld, tiles_per_cta;
};

__global__ void __launch_bounds__(kIxThreads, 1)
dsa_index_tc_fp8_kernel(const __grid_constant__ CUtensorMap tmK, IndexTcFp8Params p) {
  constexpr int kTileBytes = kIxTile * 128;     // 16 KB
  constexpr int kQBytes = 2 * kIxHeads * 128;   // 16 KB: 128 B-operand rows of 128 e4m3 bytes
  extern __shared__ __align__(1024) unsigned char smem_dyn[];
  unsigned char* sp = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  unsigned char* sK = sp;  sp += kIxStages * kTileBytes;
  unsigned char* sQ = sp;  sp += kQBytes;
  float* sW = reinterpret_cast<float*>(sp);  sp += kIxHeads * sizeof(float);
  uint64_t* full = reinterpret_cast<uint64_t*>(sp);
  uint64_t* empty = full + kIxStages;
  uint64_t* acc_full = empty + kIxStages;   // [2]
  uint64_t* acc_empty = acc_full + 2;       // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.y;
  const int pos = p.positions[row];
  const int total_tiles = pos / kIxTile + 1;
  const int tile0 = blockIdx.x * p.tiles_per_cta;
  const int ntiles = max(0, min(total_tiles, tile0 + p.tiles_per_cta) - tile0);
  const int32_t* bt = p.block_table + static_cast<size_t>(p.row_req[row]) * p.max_blocks;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kIxStages; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], 4); }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmK);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  pdl_wait();
  if (warp >= 2) {
    // two threads per head: amax over the head, then the two e4m3 terms of the thread's 64 elements
    const int t = threadIdx.x - 64;
    const int h = t >> 1, half = t & 1;
    float v[64];
    float am = 0.f;
    if (h < p.hi) {
      const bf16* src = p.q + (static_cast<size_t>(row) * p.hi + h) * 128 + half * 64;
#pragma unroll
      for (int i = 0; i < 64; ++i) {
        v[i] = bf16_to_f32(src[i]);
        am = fmaxf(am, fabsf(v[i]));
      }
    } else {
#pragma unroll
      for (int i = 0; i < 64; ++i) v[i] = 0.f;
    }
    am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 1));
    const float sc = am > 0.f ? am / 448.f : 1.f;
    if (half == 0) sW[h] = h < p.hi ? p.w[static_cast<size_t>(row) * p.hi + h] * sc : 0.f;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      Pack16 b1, b2;
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const float x = v[c * 16 + j] / sc;
        b1.b[j] = f32_to_e4m3(x);
        b2.b[j] = f32_to_e4m3((x - e4m3_value_f32(x)) * 16.f);
      }
      const int chunk = half * 4 + c;
      *reinterpret_cast<uint4*>(sQ + h * 128 + ((chunk ^ (h & 7)) << 4)) = b1.u;
      *reinterpret_cast<uint4*>(sQ + (kIxHeads + h) * 128 + ((chunk ^ (h & 7)) << 4)) = b2.u;
    }
    fence_proxy_async_smem();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (elect_one()) {
      const int ppt = kIxTile / p.page;
      for (int i = 0; i < ntiles; ++i) {
        const int s = i % kIxStages;
        if (!wait_bar(&empty[s], ((i / kIxStages) & 1) ^ 1)) { report(p.status, kTimeoutStageEmpty, 75); *abort_flag = 1; break; }
        mbar_expect_tx(&full[s], kTileBytes);
        const int page0 = (tile0 + i) * kIxTile / p.page;
        for (int pg = 0; pg < ppt; ++pg) {
          const int pi = min(page0 + pg, p.max_blocks - 1);
          tma_load_2d(sK + s * kTileBytes + pg * p.page * 128, &tmK, 0, bt[pi] * p.page, &full[s]);
        }
        if (*abort_flag) break;
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc_f8(128, 2 * kIxHeads, 0u, 0u);
      const uint32_t q_addr = smem_u32(sQ);
      for (int i = 0; i < ntiles; ++i) {
        const int s = i % kIxStages, b = i & 1;
        if (!wait_bar(&acc_empty[b], ((i >> 1) & 1) ^ 1)) { report(p.status, kTimeoutAccum, 76); *abort_flag = 1; break; }
        if (!wait_bar(&full[s], (i / kIxStages) & 1)) { report(p.status, kTimeoutTmaFull, 77); *abort_flag = 1; break; }
        tc_fence_after();
        const uint32_t k_addr = smem_u32(sK + s * kTileBytes);
#pragma unroll
        for (int k = 0; k < 4; ++k)      // K = 32 bytes per instruction
          umma_f8f6f4(tmem_base + b * 2 * kIxHeads, umma_desc_sw128(k_addr + k * 32), umma_desc_sw128(q_addr + k * 32), idesc,
                      k > 0 ? 1u : 0u);
        umma_commit(&acc_full[b]);
        umma_commit(&empty[s]);
        if (*abort_flag) break;
      }
    }
  } else {
    const int quad = warp & 3;
    const int idx = quad * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    for (int i = 0; i < ntiles; ++i) {
      const int b = i & 1;
      if (!wait_bar(&acc_full[b], (i >> 1) & 1)) { report(p.status, kTimeoutAccum, 78); *abort_flag = 1; break; }
      tc_fence_after();
      float out = 0.f;
#pragma unroll
      for (int c0 = 0; c0 < kIxHeads; c0 += 16) {
        uint32_t r1[16], r2[16];
        tmem_ld_x16(tmem_base + b * 2 * kIxHeads + c0 + lane_addr, r1);
        tmem_ld_x16(tmem_base + b * 2 * kIxHeads + kIxHeads + c0 + lane_addr, r2);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 16; ++c)
          out = fmaf(sW[c0 + c], fmaxf(fmaf(__uint_as_float(r2[c]), 0.0625f, __uint_as_float(r1[c])), 0.f), out);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[b]);
      const int t = (tile0 + i) * kIxTile + idx;
      if (t < p.ld) {
        float y = -INFINITY;
        if (t <= pos) y = out * p.kscale[static_cast<size_t>(bt[t / p.page]) * p.page + t % p.page];
        p.scores[static_cast<size_t>(row) * p.ld + t] = y;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, 256);
}

// Index keys of new tokens into the FP8 cache: row r -> slot of (row_req[r], positions[r]); e4m3(k / scale), scale =
// amax / 448 (1 for an all-zero row).  One warp per row (128 elements, four per lane).
__global__ void __launch_bounds__(128) dsa_key_append_fp8_kernel(const bf16* __restrict__ k, int64_t k_stride,
                                                                 const int32_t* __restrict__ positions,
                                                                 const int32_t* __restrict__ row_req,
                                                                 const int32_t* __restrict__ block_table, int max_blocks,
                                                                 int page, uint8_t* __restrict__ cache,
                                                                 float* __restrict__ kscale, int rows) {
  pdl_wait();
  const int r = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (r >= rows) return;
  const int pos = positions[r];
  const size_t slot = static_cast<size_t>(block_table[static_cast<size_t>(row_req[r]) * max_blocks + pos / page]) * page + pos % page;
  float v[4];
  float am = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    v[j] = bf16_to_f32(k[static_cast<size_t>(r) * k_stride + lane * 4 + j]);
    am = fmaxf(am, fabsf(v[j]));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
  const float sc = am > 0.f ? am / 448.f : 1.f;
  uint32_t packed = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) packed |= static_cast<uint32_t>(f32_to_e4m3(v[j] / sc)) << (8 * j);
  reinterpret_cast<uint32_t*>(cache + slot * 128)[lane] = packed;
  if (lane == 0) kscale[slot] = sc;
}

// -inf for the positions of tiles no CTA visits (beyond the row's last tile).
__global__ void dsa_index_fill_kernel(float* __restrict__ scores, const int32_t* __restrict__ positions, int ld) {
  pdl_wait();
  const int row = blockIdx.y;
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  const int first = (positions[row] / kIxTile + 1) * kIxTile;
  if (t >= first && t < ld) scores[static_cast<size_t>(row) * ld + t] = -INFINITY;
}

}  // namespace dgpp

using namespace dgpp;

// q [rows, hi, 128] bf16, w [rows, hi] fp32, k paged [num_blocks, page, 128] bf16 -> scores [rows, ld] fp32.
DGPP_API int dgpp_dsa_index_tc(const void* q, const void* w, const void* k, const void* block_table, const void* row_req,
                               const void* positions, void* scores, int rows, int hi, int di, int page, int max_blocks,
                               int num_blocks, int ld, cudaStream_t st) {
  DGPP_REQUIRE(di == 128 && hi >= 1 && hi <= kIxHeads, "dsa_index_tc: geometry %d heads x %d (<= 64 x 128)", hi, di);
  DGPP_REQUIRE(page == 16 || page == 32 || page == 64 || page == 128, "dsa_index_tc: page %d unsupported", page);
  if (rows == 0) return 0;
  IndexTcParams p;
  p.q = static_cast<const bf16*>(q); p.w = static_cast<const float*>(w);
  p.block_table = static_cast<const int32_t*>(block_table);
  p.row_req = static_cast<const int32_t*>(row_req);
  p.positions = static_cast<const int32_t*>(positions);
  p.scores = static_cast<float*>(scores);
  p.status = device_status_ptr();
  p.rows = rows; p.hi = hi; p.page = page; p.max_blocks = max_blocks; p.ld = ld;
  const int max_tiles = dgpp_ceil_div(ld, kIxTile);
  // enough CTAs to cover the SMs, at most 8 tiles each
  int per = dgpp_ceil_div(max_tiles * rows, 296);
  per = per < 1 ? 1 : (per > 8 ? 8 : per);
  p.tiles_per_cta = per;
  CUtensorMap tK;
  if (make_tmap_2d(&tK, k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, 128, static_cast<uint64_t>(num_blocks) * page, 256, 64, page,
                   CU_TENSOR_MAP_SWIZZLE_128B))
    return -1;
  constexpr size_t smem = 1024 + kIxStages * 2 * kIxBlk + 2 * kIxHeads * 128 + kIxHeads * 4 + (2 * kIxStages + 4) * 8 + 64;
  static bool attr = false;
  if (!attr) {
    DGPP_CUDA_OK(cudaFuncSetAttribute(dsa_index_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    attr = true;
  }
  dim3 fgrid(dgpp_ceil_div(ld, 256), rows);
  dsa_index_fill_kernel<<<fgrid, 256, 0, st>>>(p.scores, p.positions, ld);
  DGPP_CUDA_OK(cudaGetLastError());
  dim3 grid(dgpp_ceil_div(max_tiles, per), rows);
  dsa_index_tc_kernel<<<grid, kIxThreads, smem, st>>>(tK, p);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

// FP8 form: k paged [num_blocks, page, 128] e4m3 bytes, kscale [num_blocks * page] fp32.
DGPP_API int dgpp_dsa_index_tc_fp8(const void* q, const void* w, const void* k, const void* kscale, const void* block_table,
                                   const void* row_req, const void* positions, void* scores, int rows, int hi, int di, int page,
                                   int max_blocks, int num_blocks, int ld, cudaStream_t st) {
  DGPP_REQUIRE(di == 128 && hi >= 1 && hi <= kIxHeads, "dsa_index_tc_fp8: geometry %d heads x %d (<= 64 x 128)", hi, di);
  DGPP_REQUIRE(page == 16 || page == 32 || page == 64 || page == 128, "dsa_index_tc_fp8: page %d unsupported", page);
  if (rows == 0) return 0;
  IndexTcFp8Params p;
  p.q = static_cast<const bf16*>(q); p.w = static_cast<const float*>(w); p.kscale = static_cast<const float*>(kscale);
  p.block_table = static_cast<const int32_t*>(block_table);
  p.row_req = static_cast<const int32_t*>(row_req);
  p.positions = static_cast<const int32_t*>(positions);
  p.scores = static_cast<float*>(scores);
  p.status = device_status_ptr();
  p.rows = rows; p.hi = hi; p.page = page; p.max_blocks = max_blocks; p.ld = ld;
  const int max_tiles = dgpp_ceil_div(ld, kIxTile);
  // about two CTAs per SM over all rows; up to 32 tiles each (the query split in a CTA's prologue costs about as much as
  // ten tiles of its main loop, so long contexts take longer runs instead of more CTAs)
  int per = dgpp_ceil_div(max_tiles * rows, 296);
  per = per < 1 ? 1 : (per > 32 ? 32 : per);
  p.tiles_per_cta = per;
  CUtensorMap tK;
  if (make_tmap_2d(&tK, k, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, 128, static_cast<uint64_t>(num_blocks) * page, 128, 128, page,
                   CU_TENSOR_MAP_SWIZZLE_128B))
    return -1;
  constexpr size_t smem = 1024 + kIxStages * kIxTile * 128 + 2 * kIxHeads * 128 + kIxHeads * 4 + (2 * kIxStages + 4) * 8 + 64;
  static bool attr = false;
  if (!attr) {
    DGPP_CUDA_OK(cudaFuncSetAttribute(dsa_index_tc_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    attr = true;
  }
  dim3 fgrid(dgpp_ceil_div(ld, 256), rows);
  dsa_index_fill_kernel<<<fgrid, 256, 0, st>>>(p.scores, p.positions, ld);
  DGPP_CUDA_OK(cudaGetLastError());
  dim3 grid(dgpp_ceil_div(max_tiles, per), rows);
  dsa_index_tc_fp8_kernel<<<grid, kIxThreads, smem, st>>>(tK, p);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

DGPP_API int dgpp_dsa_key_append_fp8(const void* k, int64_t k_stride, const void* positions, const void* row_req,
                                     const void* block_table, int max_blocks, int page, void* cache, void* kscale, int rows,
                                     cudaStream_t st) {
  if (rows == 0) return 0;
  dsa_key_append_fp8_kernel<<<dgpp_ceil_div(rows, 4), 128, 0, st>>>(static_cast<const bf16*>(k), k_stride,
                                                                   static_cast<const int32_t*>(positions),
                                                                   static_cast<const int32_t*>(row_req),
                                                                   static_cast<const int32_t*>(block_table), max_blocks, page,
                                                                   static_cast<uint8_t*>(cache), static_cast<float*>(kscale), rows);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}
