// Glue of a latent-attention layer around its projections and the attention kernel (mla.cu / mla_tc.cu):
//
//   mla_kv_prep_kernel    one CTA per row: RMSNorm of the compressed latent (bf16(w * bf16(x * rstd))), rotate-half RoPE
//                         of the shared rotary key, both written straight into the row's slot of the paged latent cache
//   mla_q_absorb_kernel   q_full[row, head] = [ W_uk[head]^T q_nope | rope(q_rot) ]: the key up-projection folded into the
//                         query (fp32 accumulation over nope in ascending order, one rounding), rotary part appended
//   mla_v_up_kernel       a[row, head, :] = W_uv[head] . latent_out[row, head, :] (value up-projection after attention)
//
// The two per-head products are weight-streaming on the CUDA cores: a CTA owns one head and eight rows, so a decode
// step reads every head's 128 KB matrix once; prefill chunks walk row groups of eight.
// (reference counterparts: src/models/dsa_layer.cu absorbed projections; src/kernels/dsa.cu latent append.)
#include <math.h>

#include "common/common.h"
#include "common/dtypes.cuh"
#include "common/ptx.cuh"

namespace dgpp {

constexpr int kGlueRows = 8;

// kv: [rows, kv_stride] bf16 = [dc latent | dr rotary key] before norm / rotation.  128 threads.
__global__ void __launch_bounds__(128) mla_kv_prep_kernel(const bf16* __restrict__ kv, int64_t kv_stride,
                                                          const bf16* __restrict__ norm_w, float eps,
                                                          const float* __restrict__ inv_freq,
                                                          const int32_t* __restrict__ positions,
                                                          const int32_t* __restrict__ row_req,
                                                          const int32_t* __restrict__ block_table, int max_blocks, int page,
                                                          bf16* __restrict__ cache, int dc, int dr) {
  __shared__ float wsum[4];
  pdl_wait();
  const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  const bf16* src = kv + static_cast<size_t>(row) * kv_stride;
  const int pos = positions[row], req = row_req[row];
  const int blk = block_table[static_cast<size_t>(req) * max_blocks + pos / page];
  bf16* dst = cache + (static_cast<size_t>(blk) * page + pos % page) * (dc + dr);
  float ss = 0.f;
  for (int i = tid; i < dc; i += 128) {
    const float v = bf16_to_f32(src[i]);
    ss = fmaf(v, v, ss);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if (lane == 0) wsum[wid] = ss;
  __syncthreads();
  const float rstd = rsqrtf((wsum[0] + wsum[1] + wsum[2] + wsum[3]) / static_cast<float>(dc) + eps);
  for (int i = tid; i < dc; i += 128) {
    const float n = bf16_to_f32(f32_to_bf16(bf16_to_f32(src[i]) * rstd));
    dst[i] = f32_to_bf16(n * bf16_to_f32(norm_w[i]));
  }
  const int half = dr / 2;
  for (int i = tid; i < half; i += 128) {
    const float a = bf16_to_f32(src[dc + i]), b = bf16_to_f32(src[dc + half + i]);
    float s, c;
    sincosf(static_cast<float>(pos) * inv_freq[i], &s, &c);
    dst[dc + i] = f32_to_bf16(a * c - b * s);
    dst[dc + half + i] = f32_to_bf16(b * c + a * s);
  }
}

// q: [rows, heads, nope + dr] bf16; w_uk: [heads, nope, dc] bf16; out: [rows, heads, dc + dr] bf16.
// grid (heads, ceil(rows / 8), ceil(dc / 64)), 256 threads: a CTA owns 64 latent dims of one head for up to 8 rows.
// Warp w sums its eighth of the nope rows of W_uk (lane = two adjacent dims, 128-byte coalesced loads, sixteen of them in
// flight: one thread walking all nope rows was a chain of dependent loads), the eight partial sums are added in
// ascending warp order.
__global__ void __launch_bounds__(256) mla_q_absorb_kernel(const bf16* __restrict__ q, const bf16* __restrict__ w_uk,
                                                           const float* __restrict__ inv_freq,
                                                           const int32_t* __restrict__ positions, bf16* __restrict__ out,
                                                           int rows, int heads, int nope, int dc, int dr) {
  extern __shared__ float sm_q[];
  float* qs = sm_q;                              // [8][nope]
  float* part = sm_q + kGlueRows * nope;         // [8 warps][8 rows][64]
  pdl_wait();
  const int h = blockIdx.x, r0 = blockIdx.y * kGlueRows, tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int nr = min(kGlueRows, rows - r0);
  const int dq = nope + dr;
  for (int i = tid; i < kGlueRows * nope; i += 256) {
    const int r = i / nope, n = i % nope;
    qs[i] = r < nr ? bf16_to_f32(q[(static_cast<size_t>(r0 + r) * heads + h) * dq + n]) : 0.f;
  }
  __syncthreads();
  const int d0 = blockIdx.z * 64 + lane * 2;
  const bool live = d0 < dc;
  const int per = (nope + 7) / 8;
  const int n0 = warp * per, n1 = min(nope, n0 + per);
  float acc[kGlueRows][2];
#pragma unroll
  for (int r = 0; r < kGlueRows; ++r) { acc[r][0] = 0.f; acc[r][1] = 0.f; }
  const bf16* wp = w_uk + static_cast<size_t>(h) * nope * dc + (live ? d0 : 0);
#pragma unroll 16
  for (int n = n0; n < (live ? n1 : n0); ++n) {
    const uint32_t w2 = *reinterpret_cast<const uint32_t*>(wp + static_cast<size_t>(n) * dc);
    const float w0 = __uint_as_float(w2 << 16), w1 = __uint_as_float(w2 & 0xffff0000u);
#pragma unroll
    for (int r = 0; r < kGlueRows; ++r) {
      const float qv = qs[r * nope + n];
      acc[r][0] = fmaf(qv, w0, acc[r][0]);
      acc[r][1] = fmaf(qv, w1, acc[r][1]);
    }
  }
#pragma unroll
  for (int r = 0; r < kGlueRows; ++r) {
    part[(warp * kGlueRows + r) * 64 + lane * 2] = acc[r][0];
    part[(warp * kGlueRows + r) * 64 + lane * 2 + 1] = acc[r][1];
  }
  __syncthreads();
  for (int i = tid; i < nr * 64; i += 256) {
    const int r = i / 64, d = i % 64;
    if (blockIdx.z * 64 + d >= dc) continue;
    float sum = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) sum += part[(w * kGlueRows + r) * 64 + d];
    out[(static_cast<size_t>(r0 + r) * heads + h) * (dc + dr) + blockIdx.z * 64 + d] = f32_to_bf16(sum);
  }
  if (blockIdx.z == 0) {
    const int half = dr / 2;
    for (int i = tid; i < nr * half; i += 256) {
      const int r = i / half, j = i % half;
      const bf16* qr = q + (static_cast<size_t>(r0 + r) * heads + h) * dq + nope;
      const float a = bf16_to_f32(qr[j]), b = bf16_to_f32(qr[half + j]);
      float s, c;
      sincosf(static_cast<float>(positions[r0 + r]) * inv_freq[j], &s, &c);
      bf16* o = out + (static_cast<size_t>(r0 + r) * heads + h) * (dc + dr) + dc;
      o[j] = f32_to_bf16(a * c - b * s);
      o[half + j] = f32_to_bf16(b * c + a * s);
    }
  }
}

// lat: [rows, heads, dc] bf16; w_uv: [heads, v, dc] bf16; out: [rows, heads * v] bf16.
// grid (heads, ceil(rows / 8), ceil(v / 16)), 256 threads: a CTA owns 16 outputs of one head for up to 8 rows.  A warp
// holds two outputs x 16 dim groups: lane (vl, g) reads the 16-byte chunks g, g + 16, g + 32, ... of its weight row (the
// sixteen lanes of an output read consecutive chunks; all of a thread's loads are issued before the first use), the
// sixteen partial sums of an output are folded by xor shuffles 8, 4, 2, 1.
__global__ void __launch_bounds__(256) mla_v_up_kernel(const bf16* __restrict__ lat, const bf16* __restrict__ w_uv,
                                                       bf16* __restrict__ out, int rows, int heads, int vdim, int dc) {
  extern __shared__ float ls[];                // [8][chunks][9]: one latent row = dc / 8 chunks of 8 values, padded
  pdl_wait();
  const int h = blockIdx.x, r0 = blockIdx.y * kGlueRows, tid = threadIdx.x;
  const int nr = min(kGlueRows, rows - r0);
  const int chunks = dc / 8;
  for (int i = tid; i < kGlueRows * dc; i += 256) {
    const int r = i / dc, d = i % dc;
    ls[(r * chunks + d / 8) * 9 + d % 8] = r < nr ? bf16_to_f32(lat[(static_cast<size_t>(r0 + r) * heads + h) * dc + d]) : 0.f;
  }
  __syncthreads();
  const int warp = tid >> 5, lane = tid & 31;
  const int g = lane & 15;
  const int v = blockIdx.z * 16 + warp * 2 + (lane >> 4);
  const bool live = v < vdim;
  const bf16* wp = w_uv + (static_cast<size_t>(h) * vdim + (live ? v : 0)) * dc;
  float acc[kGlueRows];
#pragma unroll
  for (int r = 0; r < kGlueRows; ++r) acc[r] = 0.f;
  for (int c0 = 0; c0 < chunks; c0 += 64) {          // up to four chunks per thread and round
    Pack16 w[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int c = c0 + g + 16 * k;
      w[k].u = (c < chunks) ? *reinterpret_cast<const uint4*>(wp + c * 8) : make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int c = c0 + g + 16 * k;
      if (c >= chunks) continue;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float wv = bf16_to_f32(w[k].h[j]);
#pragma unroll
        for (int r = 0; r < kGlueRows; ++r) acc[r] = fmaf(ls[(r * chunks + c) * 9 + j], wv, acc[r]);
      }
    }
  }
#pragma unroll
  for (int r = 0; r < kGlueRows; ++r) {
    float a = acc[r];
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
    if (g == 0 && live && r < nr) out[(static_cast<size_t>(r0 + r) * heads + h) * vdim + v] = f32_to_bf16(a);
  }
}

}  // namespace dgpp

using namespace dgpp;

DGPP_API int dgpp_mla_kv_prep(const void* kv, int64_t kv_stride, const void* norm_w, float eps, const void* inv_freq,
                              const void* positions, const void* row_req, const void* block_table, int max_blocks,
                              int page, void* cache, int rows, int dc, int dr, cudaStream_t st) {
  DGPP_REQUIRE(dr % 2 == 0 && dc >= 1, "mla_kv_prep: bad latent geometry %d + %d", dc, dr);
  if (rows == 0) return 0;
  mla_kv_prep_kernel<<<rows, 128, 0, st>>>(static_cast<const bf16*>(kv), kv_stride, static_cast<const bf16*>(norm_w), eps,
                                           static_cast<const float*>(inv_freq), static_cast<const int32_t*>(positions),
                                           static_cast<const int32_t*>(row_req), static_cast<const int32_t*>(block_table),
                                           max_blocks, page, static_cast<bf16*>(cache), dc, dr);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

DGPP_API int dgpp_mla_q_absorb(const void* q, const void* w_uk, const void* inv_freq, const void* positions, void* out,
                               int rows, int heads, int nope, int dc, int dr, cudaStream_t st) {
  DGPP_REQUIRE(dc % 2 == 0 && dr % 2 == 0 && nope >= 1 && nope <= 512, "mla_q_absorb: geometry %d / %d / %d", nope, dc, dr);
  if (rows == 0) return 0;
  dim3 grid(heads, dgpp_ceil_div(rows, kGlueRows), dgpp_ceil_div(dc, 64));
  mla_q_absorb_kernel<<<grid, 256, (kGlueRows * nope + 8 * kGlueRows * 64) * sizeof(float), st>>>(
      static_cast<const bf16*>(q), static_cast<const bf16*>(w_uk), static_cast<const float*>(inv_freq),
      static_cast<const int32_t*>(positions), static_cast<bf16*>(out), rows, heads, nope, dc, dr);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

DGPP_API int dgpp_mla_v_up(const void* lat, const void* w_uv, void* out, int rows, int heads, int vdim, int dc,
                           cudaStream_t st) {
  DGPP_REQUIRE(vdim >= 1 && dc % 8 == 0 && dc <= 1024, "mla_v_up: geometry %d / %d", vdim, dc);
  if (rows == 0) return 0;
  dim3 grid(heads, dgpp_ceil_div(rows, kGlueRows), dgpp_ceil_div(vdim, 16));
  const size_t smem = static_cast<size_t>(kGlueRows) * (dc / 8) * 9 * sizeof(float);
  mla_v_up_kernel<<<grid, 256, smem, st>>>(static_cast<const bf16*>(lat), static_cast<const bf16*>(w_uv),
                                                static_cast<bf16*>(out), rows, heads, vdim, dc);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}
