// Per-head post-processing of a fused QKV projection, in one pass over the qkv rows:
//   * optional per-head RMSNorm of q and k (weight of head_dim elements)
//   * rotary embedding (rotate-half / "neox" pairing, partial rotary supported) from an fp32
//     inverse-frequency table, so YaRN / linear scaling are just a different table + mscale
//   * q written back in place (bf16)
//   * k and v appended to the paged KV cache at the slot derived from (request, position):
//     FP8 e4m3 with one fp32 scale per (token, kv head) = amax / 448, or plain bf16.
// One warp per (row, head); head_dim is 64, 128 or 256.
// (operator family: src/kernels/qsa.cu:104-252 norm_rope / kv_append(_fp8) of the reference)
#include "common/common.h"
#include "common/dtypes.cuh"
#include "common/ptx.cuh"

namespace dgpp {

struct RopeKvParams {
  bf16* qkv;               // [rows, (hq + 2*hkv) * d]
  const int32_t* positions;  // [rows]
  const int32_t* row_req;    // [rows] request slot of each row
  const int32_t* block_table;  // [max_req, max_blocks]
  const float* inv_freq;     // [rot_dim / 2]
  const bf16* q_norm_w;      // [d] or null
  const bf16* k_norm_w;      // [d] or null
  uint8_t* k_cache;          // fp8: [blocks, hkv, page, d] bytes; bf16: same shape in bf16
  uint8_t* v_cache;
  float* k_scale;            // [blocks, hkv, page] (fp8 only)
  float* v_scale;
  int rows, hq, hkv, d, rot_dim, page, max_blocks;
  float mscale, eps;
  int kv_fp8, norm_one_plus_w;
};

template <int D>
__global__ void __launch_bounds__(128) rope_kv_kernel(RopeKvParams p) {
  pdl_wait();
  constexpr int PER = D / 32;  // elements per lane, element j of lane l is dim l + 32*j
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int heads = p.hq + 2 * p.hkv;
  if (warp >= p.rows * heads) return;
  const int row = warp / heads, head = warp % heads;
  bf16* src = p.qkv + static_cast<size_t>(row) * heads * D + static_cast<size_t>(head) * D;
  float v[PER];
#pragma unroll
  for (int j = 0; j < PER; ++j) v[j] = bf16_to_f32(src[lane + 32 * j]);

  const bool is_q = head < p.hq;
  const bool is_k = !is_q && head < p.hq + p.hkv;
  const bf16* nw = is_q ? p.q_norm_w : (is_k ? p.k_norm_w : nullptr);
  if (nw) {
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < PER; ++j) ss += v[j] * v[j];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float rstd = rsqrtf(ss / D + p.eps);
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      float g = bf16_to_f32(nw[lane + 32 * j]);
      if (p.norm_one_plus_w) g += 1.f;
      v[j] = bf16_to_f32(f32_to_bf16(bf16_to_f32(f32_to_bf16(v[j] * rstd)) * g));
    }
  }
  const int pos = p.positions[row];
  if (is_q || is_k) {
    // rotate-half pairing: dim i pairs with i + rot/2 for i < rot/2
    const int half = p.rot_dim / 2;
    float r[PER];
    if (p.rot_dim == D) {
      // the partner of lane element j (dim lane + 32 j) is element j + PER/2 of the same lane
#pragma unroll
      for (int j = 0; j < PER / 2; ++j) {
        float sn, cs;
        sincosf(static_cast<float>(pos) * p.inv_freq[lane + 32 * j], &sn, &cs);
        sn *= p.mscale;
        cs *= p.mscale;
        const float x0 = v[j], x1 = v[j + PER / 2];
        r[j] = x0 * cs - x1 * sn;
        r[j + PER / 2] = x1 * cs + x0 * sn;
      }
    } else {
      // partial rotary: the partner may live in another lane; fetch it with shuffles
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        const int a = lane + 32 * j;
        const int pd = a < half ? a + half : (a < p.rot_dim ? a - half : a);
        float partner = 0.f;
#pragma unroll
        for (int jj = 0; jj < PER; ++jj) {
          const float cand = __shfl_sync(0xffffffffu, v[jj], pd & 31);
          if ((pd >> 5) == jj) partner = cand;
        }
        if (a < p.rot_dim) {
          float sn, cs;
          sincosf(static_cast<float>(pos) * p.inv_freq[a < half ? a : a - half], &sn, &cs);
          sn *= p.mscale;
          cs *= p.mscale;
          r[j] = a < half ? v[j] * cs - partner * sn : v[j] * cs + partner * sn;
        } else {
          r[j] = v[j];
        }
      }
    }
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      v[j] = bf16_to_f32(f32_to_bf16(r[j]));
      src[lane + 32 * j] = f32_to_bf16(r[j]);  // rotated q / k stay visible in qkv (prefill attention reads them)
    }
  }
  if (is_q) return;
  // k or v: append to the paged cache
  const int req = p.row_req[row];
  const int blk = p.block_table[static_cast<size_t>(req) * p.max_blocks + pos / p.page];
  const int off = pos % p.page;
  const int kvh = is_k ? head - p.hq : head - p.hq - p.hkv;
  const size_t tok = (static_cast<size_t>(blk) * p.hkv + kvh) * p.page + off;
  if (p.kv_fp8) {
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < PER; ++j) amax = fmaxf(amax, fabsf(v[j]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float scale = amax > 0.f ? amax / 448.f : 1.f;
    const float inv = 1.f / scale;
    uint8_t* dst = (is_k ? p.k_cache : p.v_cache) + tok * D;
#pragma unroll
    for (int j = 0; j < PER; ++j) dst[lane + 32 * j] = f32_to_e4m3(v[j] * inv);
    if (lane == 0) (is_k ? p.k_scale : p.v_scale)[tok] = scale;
  } else {
    bf16* dst = reinterpret_cast<bf16*>(is_k ? p.k_cache : p.v_cache) + tok * D;
#pragma unroll
    for (int j = 0; j < PER; ++j) dst[lane + 32 * j] = f32_to_bf16(v[j]);
  }
}

}  // namespace dgpp

using namespace dgpp;

DGPP_API int dgpp_rope_kv_write(void* qkv, const void* positions, const void* row_req, const void* block_table,
                                const void* inv_freq, const void* q_norm_w, const void* k_norm_w, void* k_cache,
                                void* v_cache, void* k_scale, void* v_scale, int rows, int hq, int hkv, int d,
                                int rot_dim, int page, int max_blocks, float mscale, float eps, int kv_fp8,
                                int norm_one_plus_w, cudaStream_t st) {
  DGPP_REQUIRE(d == 64 || d == 128 || d == 256, "rope_kv: head_dim %d not in {64,128,256}", d);
  DGPP_REQUIRE(rot_dim % 2 == 0 && rot_dim <= d, "rope_kv: bad rot_dim %d", rot_dim);
  if (rows == 0) return 0;
  RopeKvParams p;
  p.qkv = static_cast<bf16*>(qkv);
  p.positions = static_cast<const int32_t*>(positions);
  p.row_req = static_cast<const int32_t*>(row_req);
  p.block_table = static_cast<const int32_t*>(block_table);
  p.inv_freq = static_cast<const float*>(inv_freq);
  p.q_norm_w = static_cast<const bf16*>(q_norm_w);
  p.k_norm_w = static_cast<const bf16*>(k_norm_w);
  p.k_cache = static_cast<uint8_t*>(k_cache);
  p.v_cache = static_cast<uint8_t*>(v_cache);
  p.k_scale = static_cast<float*>(k_scale);
  p.v_scale = static_cast<float*>(v_scale);
  p.rows = rows; p.hq = hq; p.hkv = hkv; p.d = d; p.rot_dim = rot_dim; p.page = page; p.max_blocks = max_blocks;
  p.mscale = mscale; p.eps = eps; p.kv_fp8 = kv_fp8; p.norm_one_plus_w = norm_one_plus_w;
  const int warps = rows * (hq + 2 * hkv);
  const int blocks = dgpp_ceil_div(warps, 4);
  if (d == 64) rope_kv_kernel<64><<<blocks, 128, 0, st>>>(p);
  else if (d == 128) rope_kv_kernel<128><<<blocks, 128, 0, st>>>(p);
  else rope_kv_kernel<256><<<blocks, 128, 0, st>>>(p);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}
