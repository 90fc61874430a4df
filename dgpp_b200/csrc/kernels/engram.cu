// Hashed n-gram memory ("Engram") for residual-stream models: every token looks up, per n-gram size n = 2 .. max_ngram
// and per head, one row of a large table addressed by a hash of its last n token classes; the gathered rows are
// projected to one key per stream and one shared value, and every stream takes the value in through its own gate.
//
//   engram_embed   hash + gather + dequantise in one launch.  Classes y[0..] = class of the token and of the tokens
//                  before it (pad class before the start of the sequence).  Per layer:
//                      rolling_1 = y[0] * mult[0] ^ y[1] * mult[1],  rolling_n = rolling_{n-1} ^ y[n] * mult[n]
//                  (64-bit wrapping products), id(n, h) = rolling_n mod prime(n, h) (non-negative) + offset(n, h).
//                  Table rows are e4m3 with one e8m0 scale per 32 values; out [rows, (max_ngram - 1) * heads * D] bf16
//                  = bf16(e4m3 x 2^(s - 127)) (exact).  The table lives in device memory.
//   engram_gate    x [rows, hc, H] bf16 in place, kv [rows, (hc + 1) * H] bf16 = key_0 .. key_{hc-1} | value:
//                      w    = q_weight[i] * k_weight[i]
//                      rstd = rsqrt(mean(x_i^2) + eps) * rsqrt(mean(key_i^2) + eps)
//                      dot  = sum_d x_i[d] w[d] key_i[d] * rstd / sqrt(H)
//                      gate = sigmoid(sign(dot) sqrt(max(|dot|, 1e-6)));   x_i += gate * value   (one bf16 rounding)
// (reference counterparts: src/kernels/dsv41_engram.cu hash_ids_rows_kernel, gather_staged_bf16, gate_rows;
//  src/models/dsv41/engram_layer.cpp.  There the tables stay on NVMe and a host node gathers the rows; here they are
//  resident in HBM and the gather is part of the kernel.)
#include <math.h>

#include "common/common.h"
#include "common/dtypes.cuh"
#include "common/ptx.cuh"

namespace dgpp {

constexpr int kEngramMaxNgram = 8;

struct EngramEmbedParams {
  const int32_t* tokens;        // [rows]
  const int32_t* prev;          // [max_ngram - 1, rows]: row k holds the token k + 1 positions back, -1 before the start
  const int32_t* token_map;     // [vocab] token id -> class
  const int64_t* multipliers;   // [max_ngram]
  const int64_t* primes;        // [max_ngram - 1, heads]
  const int64_t* offsets;       // [max_ngram - 1, heads]
  const uint8_t* table;         // [table_rows, D] e4m3
  const uint8_t* table_sf;      // [table_rows, D / 32] e8m0
  bf16* out;                    // [rows, (max_ngram - 1) * heads * D]
  int32_t* ids;                 // optional [rows, (max_ngram - 1) * heads]
  int rows, max_ngram, heads, head_dim, pad_class, vocab;
  long long table_rows;
};

// one warp per (row, n-gram size, head)
__global__ void __launch_bounds__(128) engram_embed_kernel(EngramEmbedParams p) {
  pdl_wait();
  const int slots = (p.max_ngram - 1) * p.heads;
  const long long warp = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= static_cast<long long>(p.rows) * slots) return;
  const int row = static_cast<int>(warp / slots), slot = static_cast<int>(warp % slots);
  const int n = slot / p.heads + 1, hd = slot % p.heads;        // n predecessors take part: an (n + 1)-gram
  auto cls = [&](int tok) { return (tok < 0 || tok >= p.vocab) ? p.pad_class : p.token_map[tok]; };
  unsigned long long rolling = static_cast<unsigned long long>(static_cast<long long>(cls(p.tokens[row]))) *
                               static_cast<unsigned long long>(p.multipliers[0]);
  for (int k = 1; k <= n; ++k)
    rolling ^= static_cast<unsigned long long>(static_cast<long long>(cls(p.prev[static_cast<size_t>(k - 1) * p.rows + row]))) *
               static_cast<unsigned long long>(p.multipliers[k]);
  const long long prime = p.primes[slot];
  long long r = static_cast<long long>(rolling) % prime;
  if (r < 0) r += prime;
  long long id = r + p.offsets[slot];
  if (id < 0 || id >= p.table_rows) id = 0;                      // (a damaged constant table: stay inside)
  if (lane == 0 && p.ids != nullptr) p.ids[static_cast<size_t>(row) * slots + slot] = static_cast<int32_t>(id);
  const int D = p.head_dim;
  const uint8_t* src = p.table + static_cast<size_t>(id) * D;
  const uint8_t* sf = p.table_sf + static_cast<size_t>(id) * (D / 32);
  bf16* dst = p.out + (static_cast<size_t>(row) * slots + slot) * D;
  for (int d2 = lane; d2 < D / 2; d2 += 32) {
    const uint16_t pair = *reinterpret_cast<const uint16_t*>(src + 2 * d2);
    const float2 f = __half22float2(e4m3x2_to_h2(pair));
    const float s = e8m0_to_f32(sf[(2 * d2) / 32]);
    dst[2 * d2] = f32_to_bf16(f.x * s);
    dst[2 * d2 + 1] = f32_to_bf16(f.y * s);
  }
}

// grid (hc, rows), 256 threads
__global__ void __launch_bounds__(256) engram_gate_kernel(bf16* __restrict__ x, const bf16* __restrict__ kv,
                                                          const bf16* __restrict__ q_weight, const bf16* __restrict__ k_weight,
                                                          int hc, int H, float eps) {
  __shared__ float red[3][8];
  __shared__ float gate_s;
  pdl_wait();
  const int i = blockIdx.x, row = blockIdx.y;
  bf16* xi = x + (static_cast<size_t>(row) * hc + i) * H;
  const bf16* key = kv + static_cast<size_t>(row) * (hc + 1) * H + static_cast<size_t>(i) * H;
  const bf16* val = kv + static_cast<size_t>(row) * (hc + 1) * H + static_cast<size_t>(hc) * H;
  const bf16* qw = q_weight + static_cast<size_t>(i) * H;
  const bf16* kw = k_weight + static_cast<size_t>(i) * H;
  float sx = 0.f, sk = 0.f, dot = 0.f;
  for (int d = threadIdx.x; d < H; d += 256) {
    const float xv = bf16_to_f32(xi[d]), kvv = bf16_to_f32(key[d]);
    sx = fmaf(xv, xv, sx);
    sk = fmaf(kvv, kvv, sk);
    dot = fmaf(xv * (bf16_to_f32(qw[d]) * bf16_to_f32(kw[d])), kvv, dot);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    sx += __shfl_xor_sync(0xffffffffu, sx, o);
    sk += __shfl_xor_sync(0xffffffffu, sk, o);
    dot += __shfl_xor_sync(0xffffffffu, dot, o);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) { red[0][warp] = sx; red[1][warp] = sk; red[2][warp] = dot; }
  __syncthreads();
  if (threadIdx.x == 0) {
    float a = 0.f, b = 0.f, c = 0.f;
    for (int w = 0; w < 8; ++w) { a += red[0][w]; b += red[1][w]; c += red[2][w]; }
    const float rstd = rsqrtf(a / H + eps) * rsqrtf(b / H + eps);
    const float dv = c * rstd * rsqrtf(static_cast<float>(H));
    const float sg = copysignf(sqrtf(fmaxf(fabsf(dv), 1e-6f)), dv);
    gate_s = 1.f / (1.f + __expf(-sg));
  }
  __syncthreads();
  const float g = gate_s;
  for (int d = threadIdx.x; d < H; d += 256) xi[d] = f32_to_bf16(fmaf(g, bf16_to_f32(val[d]), bf16_to_f32(xi[d])));
}

}  // namespace dgpp

using namespace dgpp;

DGPP_API int dgpp_engram_embed(const void* tokens, const void* prev, const void* token_map, const void* multipliers,
                               const void* primes, const void* offsets, const void* table, const void* table_sf,
                               void* out, void* ids, int rows, int max_ngram, int heads, int head_dim, int pad_class,
                               int vocab, long long table_rows, cudaStream_t st) {
  DGPP_REQUIRE(max_ngram >= 2 && max_ngram <= kEngramMaxNgram, "engram_embed: max_ngram %d outside 2..%d", max_ngram,
               kEngramMaxNgram);
  DGPP_REQUIRE(heads >= 1 && head_dim >= 32 && head_dim % 32 == 0, "engram_embed: bad heads %d / head_dim %d", heads,
               head_dim);
  DGPP_REQUIRE(table_rows >= 1 && vocab >= 1, "engram_embed: empty table");
  if (rows == 0) return 0;
  EngramEmbedParams p;
  p.tokens = static_cast<const int32_t*>(tokens);
  p.prev = static_cast<const int32_t*>(prev);
  p.token_map = static_cast<const int32_t*>(token_map);
  p.multipliers = static_cast<const int64_t*>(multipliers);
  p.primes = static_cast<const int64_t*>(primes);
  p.offsets = static_cast<const int64_t*>(offsets);
  p.table = static_cast<const uint8_t*>(table);
  p.table_sf = static_cast<const uint8_t*>(table_sf);
  p.out = static_cast<bf16*>(out);
  p.ids = static_cast<int32_t*>(ids);
  p.rows = rows; p.max_ngram = max_ngram; p.heads = heads; p.head_dim = head_dim; p.pad_class = pad_class;
  p.vocab = vocab; p.table_rows = table_rows;
  const long long warps = static_cast<long long>(rows) * (max_ngram - 1) * heads;
  engram_embed_kernel<<<static_cast<unsigned>((warps + 3) / 4), 128, 0, st>>>(p);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

DGPP_API int dgpp_engram_gate(void* x, const void* kv, const void* q_weight, const void* k_weight, int rows, int hc,
                              int hidden, float eps, cudaStream_t st) {
  DGPP_REQUIRE(hc >= 1 && hc <= 65535 && hidden >= 1 && rows <= 65535, "engram_gate: bad geometry");
  if (rows == 0) return 0;
  engram_gate_kernel<<<dim3(hc, rows), 256, 0, st>>>(static_cast<bf16*>(x), static_cast<const bf16*>(kv),
                                                     static_cast<const bf16*>(q_weight), static_cast<const bf16*>(k_weight),
                                                     hc, hidden, eps);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}
