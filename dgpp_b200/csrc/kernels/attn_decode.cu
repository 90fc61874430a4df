// Paged GQA decode attention (one query position per row) over an FP8-e4m3 or bf16 KV cache,
// flash-decoding style: the KV range of every (row, kv head) is cut into `splits` contiguous
// chunks, each CTA keeps running (max, sum, weighted V) for the G = hq / hkv query heads that
// share its kv head, and a second kernel merges the chunk partials in ascending chunk order.
// Partials live in caller-provided scratch: ml [rows, hq, splits, 2] and acc [rows, hq, splits, D] fp32.
//
// Cache layout: k/v [blocks, hkv, page, D]; fp8 caches carry one fp32 scale per (token, kv head).
// A row attends to cache positions 0 .. positions[row] inclusive (its own K/V were just appended).
// Block-sparse form: with a selection list sel [rows, hkv, sel_k] (ascending block ids of sel_block tokens, -1 padded
// at the end, the block that holds the row's own position last) every (row, kv head) attends only to the tokens of
// its listed blocks; the kernel walks the concatenation of those blocks as one virtual sequence.
// (operator family: src/kernels/full_attn.cu:163,370 row kernel + combine, src/kernels/glm4_attn.cu:150,278)
#include <math.h>

#include "common/common.h"
#include "common/dtypes.cuh"
#include "common/ptx.cuh"

namespace dgpp {

struct AttnDecodeParams {
  const bf16* q;          // [rows, q_stride] query heads at column h * D
  int64_t q_stride;
  const uint8_t* k_cache;
  const uint8_t* v_cache;
  const float* k_scale;
  const float* v_scale;
  const int32_t* block_table;
  const int32_t* row_req;
  const int32_t* positions;
  float* part_ml;         // scratch
  float* part_acc;        // scratch
  bf16* out;              // [rows, hq * D]
  int rows, hq, hkv, page, max_blocks, splits, kv_fp8;
  float scale;            // softmax scale (1/sqrt(D) times any rope mscale^2)
  int window;             // > 0: attend only to the last `window` positions (sliding window); 0 = full
  const float* sink;      // optional [hq]: one more softmax column per head with this logit and no value
  const int32_t* sel;     // optional [rows, hkv, sel_k] block selection (see the header); null = dense
  int sel_k, sel_block;
};

// Normalisation with the optional sink column: out = acc / (l + exp(sink - m)), computed against max(m, sink).
__device__ __forceinline__ float finish_softmax(float a, float l, float m, const float* sink, int h) {
  if (sink != nullptr) {
    const float sk = sink[h];
    const float mx = fmaxf(m, sk);
    const float c = m == -INFINITY ? 0.f : __expf(m - mx);
    a *= c;
    l = l * c + __expf(sk - mx);
  }
  return l > 0.f ? a / l : 0.f;
}

constexpr int kDecWarps = 4;

template <int D, int G>
__global__ void __launch_bounds__(kDecWarps * 32) attn_decode_kernel(AttnDecodeParams p) {
  constexpr int PER = D / 32;
  __shared__ float q_s[G][D];
  __shared__ float red_m[kDecWarps][G];
  __shared__ float red_l[kDecWarps][G];
  __shared__ float red_acc[kDecWarps][G][D];
  pdl_wait();
  const int kvh = blockIdx.x, split = blockIdx.y, row = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int req = p.row_req[row];
  const int pos = p.positions[row];
  int len = pos + 1;
  const int32_t* sl = nullptr;
  if (p.sel != nullptr) {
    sl = p.sel + (static_cast<size_t>(row) * p.hkv + kvh) * p.sel_k;
    int n = 0;
    for (int j = 0; j < p.sel_k; ++j) n += sl[j] >= 0 ? 1 : 0;
    len = n > 0 ? (n - 1) * p.sel_block + pos % p.sel_block + 1 : 0;      // every listed block is full but the last
  }
  const int first = (p.window > 0 && len > p.window) ? len - p.window : 0;
  const int span = len - first;
  int per = (span + p.splits - 1) / p.splits;
  per = (per + 31) & ~31;
  const int t_begin = first + split * per;
  const int t_end = min(len, t_begin + per);

  for (int i = threadIdx.x; i < G * D; i += blockDim.x) {
    const int g = i / D, d = i % D;
    q_s[g][d] = bf16_to_f32(p.q[static_cast<size_t>(row) * p.q_stride + (kvh * G + g) * D + d]) * p.scale;
  }
  __syncthreads();

  float m[G], l[G], acc[G][PER];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int j = 0; j < PER; ++j) acc[g][j] = 0.f;
  }
  const int32_t* bt = p.block_table + static_cast<size_t>(req) * p.max_blocks;

  for (int t0 = t_begin + warp * 32; t0 < t_end; t0 += kDecWarps * 32) {
    const int t = t0 + lane;
    const bool valid = t < t_end;
    int tc = valid ? t : t_end - 1;
    if (sl != nullptr) tc = min(sl[tc / p.sel_block] * p.sel_block + tc % p.sel_block, pos);   // virtual -> cache position
    const size_t tok = (static_cast<size_t>(bt[tc / p.page]) * p.hkv + kvh) * p.page + tc % p.page;
    float s[G];
#pragma unroll
    for (int g = 0; g < G; ++g) s[g] = 0.f;
    if (p.kv_fp8) {
      const uint4* kr = reinterpret_cast<const uint4*>(p.k_cache + tok * D);
#pragma unroll 2
      for (int c = 0; c < D / 16; ++c) {
        Pack16 kb;
        kb.u = kr[c];
        float kf[16];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float2 f = __half22float2(e4m3x2_to_h2(kb.s[j]));
          kf[2 * j] = f.x;
          kf[2 * j + 1] = f.y;
        }
#pragma unroll
        for (int g = 0; g < G; ++g) {
#pragma unroll
          for (int j = 0; j < 16; ++j) s[g] = fmaf(kf[j], q_s[g][c * 16 + j], s[g]);
        }
      }
      const float ks = p.k_scale[tok];
#pragma unroll
      for (int g = 0; g < G; ++g) s[g] *= ks;
    } else {
      const uint4* kr = reinterpret_cast<const uint4*>(reinterpret_cast<const bf16*>(p.k_cache) + tok * D);
#pragma unroll 2
      for (int c = 0; c < D / 8; ++c) {
        Pack16 kb;
        kb.u = kr[c];
#pragma unroll
        for (int g = 0; g < G; ++g) {
#pragma unroll
          for (int j = 0; j < 8; ++j) s[g] = fmaf(bf16_to_f32(kb.h[j]), q_s[g][c * 8 + j], s[g]);
        }
      }
    }
    // online softmax update for this 32-token tile
    float pr[G];
    const float vs = (p.kv_fp8 && valid) ? p.v_scale[tok] : 1.f;
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float sv = valid ? s[g] : -INFINITY;
      float tm = sv;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, o));
      const float mn = fmaxf(m[g], tm);
      const float corr = m[g] == -INFINITY ? 0.f : __expf(m[g] - mn);
      const float e = valid ? __expf(sv - mn) : 0.f;
      float ts = e;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ts += __shfl_xor_sync(0xffffffffu, ts, o);
      l[g] = l[g] * corr + ts;
      m[g] = mn;
#pragma unroll
      for (int j = 0; j < PER; ++j) acc[g][j] *= corr;
      pr[g] = e * vs;
    }
    // weighted V accumulation: lane owns dims [lane*PER, lane*PER + PER)
    const int ntile = min(32, t_end - t0);
    for (int tt = 0; tt < ntile; ++tt) {
      const size_t vtok = __shfl_sync(0xffffffffu, static_cast<unsigned long long>(tok), tt);
      float vf[PER];
      if (p.kv_fp8) {
        const uint8_t* vr = p.v_cache + vtok * D + lane * PER;
        if (PER == 4) {
          const uint32_t w = *reinterpret_cast<const uint32_t*>(vr);
          const float2 a = __half22float2(e4m3x2_to_h2(static_cast<uint16_t>(w & 0xffff)));
          const float2 b = __half22float2(e4m3x2_to_h2(static_cast<uint16_t>(w >> 16)));
          vf[0] = a.x; vf[1] = a.y; vf[2] = b.x; vf[3] = b.y;
        } else if (PER == 8) {
          const uint2 w = *reinterpret_cast<const uint2*>(vr);
          const float2 a = __half22float2(e4m3x2_to_h2(static_cast<uint16_t>(w.x & 0xffff)));
          const float2 b = __half22float2(e4m3x2_to_h2(static_cast<uint16_t>(w.x >> 16)));
          const float2 c = __half22float2(e4m3x2_to_h2(static_cast<uint16_t>(w.y & 0xffff)));
          const float2 d = __half22float2(e4m3x2_to_h2(static_cast<uint16_t>(w.y >> 16)));
          vf[0] = a.x; vf[1] = a.y; vf[2] = b.x; vf[3] = b.y;
          vf[4 % PER] = c.x; vf[5 % PER] = c.y; vf[6 % PER] = d.x; vf[7 % PER] = d.y;
        } else {
          const uint16_t w = *reinterpret_cast<const uint16_t*>(vr);
          const float2 a = __half22float2(e4m3x2_to_h2(w));
          vf[0] = a.x; vf[1 % PER] = a.y;
        }
      } else {
        const bf16* vr = reinterpret_cast<const bf16*>(p.v_cache) + vtok * D + lane * PER;
#pragma unroll
        for (int j = 0; j < PER; ++j) vf[j] = bf16_to_f32(vr[j]);
      }
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const float pg = __shfl_sync(0xffffffffu, pr[g], tt);
#pragma unroll
        for (int j = 0; j < PER; ++j) acc[g][j] = fmaf(pg, vf[j], acc[g][j]);
      }
    }
  }

  // merge the warps of this CTA in ascending warp order
  if (lane == 0) {
#pragma unroll
    for (int g = 0; g < G; ++g) {
      red_m[warp][g] = m[g];
      red_l[warp][g] = l[g];
    }
  }
#pragma unroll
  for (int g = 0; g < G; ++g)
#pragma unroll
    for (int j = 0; j < PER; ++j) red_acc[warp][g][lane * PER + j] = acc[g][j];
  __syncthreads();
  for (int i = threadIdx.x; i < G * D; i += blockDim.x) {
    const int g = i / D, d = i % D;
    float mm = -INFINITY;
    for (int w = 0; w < kDecWarps; ++w) mm = fmaxf(mm, red_m[w][g]);
    float ll = 0.f, a = 0.f;
    for (int w = 0; w < kDecWarps; ++w) {
      const float c = red_m[w][g] == -INFINITY ? 0.f : __expf(red_m[w][g] - mm);
      ll += red_l[w][g] * c;
      a += red_acc[w][g][d] * c;
    }
    const int h = kvh * G + g;
    if (p.splits == 1) {
      p.out[(static_cast<size_t>(row) * p.hq + h) * D + d] = f32_to_bf16(finish_softmax(a, ll, mm, p.sink, h));
    } else {
      const size_t pi = (static_cast<size_t>(row) * p.hq + h) * p.splits + split;
      p.part_acc[pi * D + d] = a;
      if (d == 0) {
        p.part_ml[pi * 2] = mm;
        p.part_ml[pi * 2 + 1] = ll;
      }
    }
  }
}

template <int D>
__global__ void attn_decode_combine_kernel(const float* __restrict__ part_ml, const float* __restrict__ part_acc,
                                           bf16* __restrict__ out, int splits, const float* __restrict__ sink, int hq) {
  pdl_wait();
  const size_t rh = blockIdx.x;  // row * hq + h
  const int d = threadIdx.x;
  float mm = -INFINITY;
  for (int s = 0; s < splits; ++s) mm = fmaxf(mm, part_ml[(rh * splits + s) * 2]);
  float ll = 0.f, a = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float ms = part_ml[(rh * splits + s) * 2];
    const float c = ms == -INFINITY ? 0.f : __expf(ms - mm);
    ll += part_ml[(rh * splits + s) * 2 + 1] * c;
    a += part_acc[(rh * splits + s) * D + d] * c;
  }
  out[rh * D + d] = f32_to_bf16(finish_softmax(a, ll, mm, sink, static_cast<int>(rh % hq)));
}

template <int D, int G>
static int launch_decode(const AttnDecodeParams& p, cudaStream_t st) {
  dim3 grid(p.hkv, p.splits, p.rows);
  attn_decode_kernel<D, G><<<grid, kDecWarps * 32, 0, st>>>(p);
  DGPP_CUDA_OK(cudaGetLastError());
  if (p.splits > 1) {
    attn_decode_combine_kernel<D><<<p.rows * p.hq, D, 0, st>>>(p.part_ml, p.part_acc, p.out, p.splits, p.sink, p.hq);
    DGPP_CUDA_OK(cudaGetLastError());
  }
  return 0;
}

}  // namespace dgpp

using namespace dgpp;

// Scratch needed for `splits` > 1: part_ml rows*hq*splits*2 floats, part_acc rows*hq*splits*d floats.
static int attn_decode_impl(const void* q, int64_t q_stride, const void* k_cache, const void* v_cache,
                            const void* k_scale, const void* v_scale, const void* block_table,
                            const void* row_req, const void* positions, void* part_ml, void* part_acc, void* out,
                            int rows, int hq, int hkv, int d, int page, int max_blocks, int splits, int kv_fp8,
                            float scale, int window, const void* sink, const void* sel, int sel_k, int sel_block,
                            cudaStream_t st) {
  DGPP_REQUIRE(hkv > 0 && hq % hkv == 0, "attn_decode: hq %d not a multiple of hkv %d", hq, hkv);
  DGPP_REQUIRE(sel == nullptr || (sel_k >= 1 && sel_block >= 1 && window == 0),
               "attn_decode: a block selection needs sel_k >= 1, sel_block >= 1 and no sliding window");
  DGPP_REQUIRE(splits >= 1, "attn_decode: splits must be >= 1");
  DGPP_REQUIRE(splits == 1 || (part_ml && part_acc), "attn_decode: scratch required when splits > 1");
  if (rows == 0) return 0;
  AttnDecodeParams p;
  p.q = static_cast<const bf16*>(q);
  p.q_stride = q_stride;
  p.k_cache = static_cast<const uint8_t*>(k_cache);
  p.v_cache = static_cast<const uint8_t*>(v_cache);
  p.k_scale = static_cast<const float*>(k_scale);
  p.v_scale = static_cast<const float*>(v_scale);
  p.block_table = static_cast<const int32_t*>(block_table);
  p.row_req = static_cast<const int32_t*>(row_req);
  p.positions = static_cast<const int32_t*>(positions);
  p.part_ml = static_cast<float*>(part_ml);
  p.part_acc = static_cast<float*>(part_acc);
  p.out = static_cast<bf16*>(out);
  p.rows = rows; p.hq = hq; p.hkv = hkv; p.page = page; p.max_blocks = max_blocks; p.splits = splits;
  p.kv_fp8 = kv_fp8; p.scale = scale; p.window = window;
  p.sink = static_cast<const float*>(sink);
  p.sel = static_cast<const int32_t*>(sel);
  p.sel_k = sel_k; p.sel_block = sel_block;
  const int g = hq / hkv;
#define DGPP_DEC_CASE(DD, GG) \
  if (d == DD && g == GG) return launch_decode<DD, GG>(p, st);
  DGPP_DEC_CASE(64, 1) DGPP_DEC_CASE(64, 2) DGPP_DEC_CASE(64, 4) DGPP_DEC_CASE(64, 8)
  DGPP_DEC_CASE(128, 1) DGPP_DEC_CASE(128, 2) DGPP_DEC_CASE(128, 4) DGPP_DEC_CASE(128, 5) DGPP_DEC_CASE(128, 8)
  DGPP_DEC_CASE(256, 1) DGPP_DEC_CASE(256, 2) DGPP_DEC_CASE(256, 4) DGPP_DEC_CASE(256, 8)
#undef DGPP_DEC_CASE
  dgpp_set_error("attn_decode: unsupported head_dim %d / group %d", d, g);
  return -1;
}

DGPP_API int dgpp_attn_decode(const void* q, int64_t q_stride, const void* k_cache, const void* v_cache,
                              const void* k_scale, const void* v_scale, const void* block_table,
                              const void* row_req, const void* positions, void* part_ml, void* part_acc, void* out,
                              int rows, int hq, int hkv, int d, int page, int max_blocks, int splits, int kv_fp8,
                              float scale, int window, cudaStream_t st) {
  return attn_decode_impl(q, q_stride, k_cache, v_cache, k_scale, v_scale, block_table, row_req, positions, part_ml,
                          part_acc, out, rows, hq, hkv, d, page, max_blocks, splits, kv_fp8, scale, window, nullptr, nullptr, 0, 0, st);
}

// Block-sparse attention: sel [rows, hkv, sel_k] int32 as described at the top of this file.
// (reference counterpart: src/kernels/minimax.hpp minimax_attn_partial + the partial merge.)
DGPP_API int dgpp_attn_decode_sparse(const void* q, int64_t q_stride, const void* k_cache, const void* v_cache,
                                     const void* k_scale, const void* v_scale, const void* block_table,
                                     const void* row_req, const void* positions, void* part_ml, void* part_acc,
                                     void* out, int rows, int hq, int hkv, int d, int page, int max_blocks, int splits,
                                     int kv_fp8, float scale, const void* sel, int sel_k, int sel_block,
                                     cudaStream_t st) {
  DGPP_REQUIRE(sel != nullptr, "attn_decode_sparse: no selection list");
  return attn_decode_impl(q, q_stride, k_cache, v_cache, k_scale, v_scale, block_table, row_req, positions, part_ml,
                          part_acc, out, rows, hq, hkv, d, page, max_blocks, splits, kv_fp8, scale, 0, nullptr, sel,
                          sel_k, sel_block, st);
}

// Sliding-window attention with per-head sink logits (sink: [hq] fp32, the logit of a value-less softmax column).
// (reference counterpart: src/kernels/sink_attn_impl.cuh:394-398.)
DGPP_API int dgpp_attn_decode_sink(const void* q, int64_t q_stride, const void* k_cache, const void* v_cache,
                                   const void* k_scale, const void* v_scale, const void* block_table,
                                   const void* row_req, const void* positions, void* part_ml, void* part_acc, void* out,
                                   int rows, int hq, int hkv, int d, int page, int max_blocks, int splits, int kv_fp8,
                                   float scale, int window, const void* sink, cudaStream_t st) {
  return attn_decode_impl(q, q_stride, k_cache, v_cache, k_scale, v_scale, block_table, row_req, positions, part_ml,
                          part_acc, out, rows, hq, hkv, d, page, max_blocks, splits, kv_fp8, scale, window, sink, nullptr, 0, 0, st);
}

// ------------------------------------------------------------------------------------------------------------
// Fixed-scratch variant: see attn_decode_static.h for the contract (no allocation, 4 MiB device array).
#include "kernels/attn_decode_static.h"

namespace dgpp {

constexpr size_t kAttnStaticScratchFloats = DGPP_ATTN_STATIC_SCRATCH_FLOATS;
static __device__ __align__(256) float g_attn_static_scratch[kAttnStaticScratchFloats];

// Address of the array on the current device; resolved once per device (first call: before any stream capture).
static float* attn_static_scratch_ptr() {
  static float* cache[64] = {nullptr};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) {
    dgpp_set_error("attn_decode_static: cudaGetDevice failed or device %d out of range: %s", dev, cudaGetErrorString(e));
    return nullptr;
  }
  if (!cache[dev]) {
    float* ptr = nullptr;
    e = cudaGetSymbolAddress((void**)&ptr, g_attn_static_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      dgpp_set_error("attn_decode_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      return nullptr;
    }
    cache[dev] = ptr;
  }
  return cache[dev];
}

}  // namespace dgpp

int dgpp_attn_decode_static(const void* q, int64_t q_stride, const void* k_cache, const void* v_cache,
                            const void* k_scale, const void* v_scale, const void* block_table, const void* row_req,
                            const void* positions, void* out, int rows, int hq, int hkv, int d, int page,
                            int max_blocks, int splits, int kv_fp8, float scale, int window, cudaStream_t st) {
  DGPP_REQUIRE(rows >= 0 && hq > 0 && d > 0 && splits >= 1, "attn_decode_static: bad sizes rows %d hq %d d %d splits %d",
               rows, hq, d, splits);
  const size_t parts = static_cast<size_t>(rows) * hq * splits;
  const size_t ml_floats = (parts * 2 + 63) & ~static_cast<size_t>(63);      // keeps the second region 256-byte aligned
  const size_t need = splits > 1 ? ml_floats + parts * d : 0;
  DGPP_REQUIRE(need <= kAttnStaticScratchFloats,
               "attn_decode_static: rows %d x heads %d x splits %d x head_dim %d needs %zu scratch floats, the fixed "
               "array holds %zu; use fewer splits or rows, or dgpp_attn_decode with caller-owned scratch",
               rows, hq, splits, d, need, static_cast<size_t>(kAttnStaticScratchFloats));
  float* ptr = attn_static_scratch_ptr();
  if (ptr == nullptr) return -1;
  return dgpp_attn_decode(q, q_stride, k_cache, v_cache, k_scale, v_scale, block_table, row_req, positions,
                          splits > 1 ? ptr : nullptr, splits > 1 ? ptr + ml_floats : nullptr, out, rows, hq, hkv, d,
                          page, max_blocks, splits, kv_fp8, scale, window, st);
}
