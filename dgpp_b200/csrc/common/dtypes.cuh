// Device-side codecs for the storage formats the engine reads as-is: e2m1 (fp4) pairs,
// e4m3 (fp8), e8m0 block exponents, bf16.  Host-side twins live in rt/codec.h.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <stdint.h>

namespace dgpp {

typedef __nv_bfloat16 bf16;
typedef __nv_bfloat162 bf162;

__device__ __forceinline__ float bf16_to_f32(bf16 v) { return __bfloat162float(v); }
__device__ __forceinline__ bf16 f32_to_bf16(float v) { return __float2bfloat16_rn(v); }

// e4m3 byte -> float (exact).
__device__ __forceinline__ float e4m3_to_f32(uint8_t v) {
  const __half h(__nv_cvt_fp8_to_halfraw(v, __NV_E4M3));   // converting constructor: no pointer punning
  return __half2float(h);
}
// two e4m3 bytes (low byte first) -> half2 (exact).
__device__ __forceinline__ __half2 e4m3x2_to_h2(uint16_t v) {
  return __half2(__nv_cvt_fp8x2_to_halfraw2(v, __NV_E4M3));
}
// float -> e4m3 byte, round-to-nearest-even, saturating to +-448.
__device__ __forceinline__ uint8_t f32_to_e4m3(float v) {
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
}
// e8m0 exponent byte -> float 2^(e-127); 255 is NaN by the MX spec.
__device__ __forceinline__ float e8m0_to_f32(uint8_t e) {
  if (e == 255) return __int_as_float(0x7fc00000);
  if (e == 0) return __int_as_float(0x00400000);  // 2^-127 (subnormal)
  return __int_as_float(static_cast<int>(e) << 23);
}

// One byte holding two e2m1 codes (low nibble = even element) -> half2 {even, odd}, exact.
__device__ __forceinline__ __half2 e2m1x2_to_h2(uint8_t b) {
  uint32_t out;
  uint16_t in = b;
  asm("{\n\t.reg .b8 lo, hi;\n\t"
      "mov.b16 {lo, hi}, %1;\n\t"
      "cvt.rn.f16x2.e2m1x2 %0, lo;\n\t}\n"
      : "=r"(out)
      : "h"(in));
  __half2_raw r;
  r.x = static_cast<unsigned short>(out & 0xffffu);
  r.y = static_cast<unsigned short>(out >> 16);
  return __half2(r);
}
// Software decode of one e2m1 code (sign, 2-bit exponent, 1-bit mantissa).
__host__ __device__ __forceinline__ float e2m1_to_f32(uint32_t c) {
  const float mag[8] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
  float m = mag[c & 7];
  return (c & 8) ? -m : m;
}
// Round a float (already divided by its block scale) to the nearest e2m1 code, ties to even code.
__host__ __device__ __forceinline__ uint32_t f32_to_e2m1(float v) {
  uint32_t s = v < 0.f ? 8u : 0u;
  float a = v < 0.f ? -v : v;
  uint32_t c;
  if (a <= 0.25f) c = 0;            // 0 | 0.5 midpoint 0.25 -> even code 0
  else if (a < 0.75f) c = 1;        // 0.5 | 1.0 midpoint 0.75 -> even code 2
  else if (a <= 1.25f) c = 2;       // 1.0 | 1.5 midpoint 1.25 -> even code 2
  else if (a < 1.75f) c = 3;        // 1.5 | 2.0 midpoint 1.75 -> even code 4
  else if (a <= 2.5f) c = 4;        // 2 | 3 midpoint 2.5 -> even code 4
  else if (a < 3.5f) c = 5;         // 3 | 4 midpoint 3.5 -> even code 6
  else if (a <= 5.f) c = 6;         // 4 | 6 midpoint 5 -> even code 6
  else c = 7;
  return s | c;
}

// Eight floats -> eight e2m1 codes in one word (element 0 in the lowest nibble), round-to-nearest-even on the
// e2m1 grid, saturating at +-6: the hardware conversion (two values per instruction).
__device__ __forceinline__ uint32_t f32x8_to_e2m1x8(const float* v) {
  uint32_t out;
  asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n\t"
      "mov.b32 %0, {b0, b1, b2, b3};\n\t}\n"
      : "=r"(out)
      : "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7]));
  return out;
}
// Subtract the decoded codes (times s) from the eight values they were produced from.
__device__ __forceinline__ void e2m1x8_residual(uint32_t codes, float s, float* v) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 d = __half22float2(e2m1x2_to_h2(static_cast<uint8_t>((codes >> (8 * i)) & 0xffu)));
    v[2 * i] -= d.x * s;
    v[2 * i + 1] -= d.y * s;
  }
}

// Value of x after round-to-nearest-even onto the e4m3 grid (3 mantissa bits), computed with integer arithmetic on
// the fp32 bits: no fp8 decode instruction is involved.  Saturates at +-448.  Below 2^-6 (the e4m3 subnormal range)
// the result keeps 3 mantissa bits instead of the fixed 2^-9 step; callers use it for residuals, where that
// difference is far below the second term's own rounding.
__device__ __forceinline__ float e4m3_round_f32(float x) {
  const uint32_t u = __float_as_uint(x);
  const uint32_t r = (u + 0x0007FFFFu + ((u >> 20) & 1u)) & 0xFFF00000u;
  return fminf(fmaxf(__uint_as_float(r), -448.f), 448.f);
}
// Exact value of the e4m3 code that a saturating round-to-nearest-even conversion of x produces, subnormal range
// (|x| < 2^-6, step 2^-9) included; checked against a reference conversion over 10^7 values.  Used where a value
// is encoded and its decoded value is needed right away (block scales, residual terms).
__device__ __forceinline__ float e4m3_value_f32(float x) {
  const uint32_t u = __float_as_uint(x);
  const float normal = __uint_as_float((u + 0x0007FFFFu + ((u >> 20) & 1u)) & 0xFFF00000u);
  const float sub = rintf(x * 512.f) * (1.f / 512.f);
  const float y = fabsf(x) >= 0.015625f ? normal : sub;
  return fminf(fmaxf(y, -448.f), 448.f);
}
// Two floats -> two e4m3 terms each (value + residual), packed: a = {e4m3(x0), e4m3(x1)} (x0 in the low byte),
// b = e4m3 of what a left, so the pair keeps ~2^-8 relative error.  The value of the first term is recomputed
// arithmetically (e4m3_round_f32) rather than decoded from `a`: chaining the packed e4m3x2 -> f16x2 conversion to
// the packing conversion returned wrong values for every other pair on B200 in this kernel family.
__device__ __forceinline__ void f32x2_to_e4m3x2_two_term(float x0, float x1, uint16_t& a, uint16_t& b) {
  a = __nv_cvt_float2_to_fp8x2(make_float2(x0, x1), __NV_SATFINITE, __NV_E4M3);
  b = __nv_cvt_float2_to_fp8x2(make_float2(x0 - e4m3_round_f32(x0), x1 - e4m3_round_f32(x1)), __NV_SATFINITE, __NV_E4M3);
}
// 2^x, one MUFU; flushes denormals, ex2(-inf) = 0.
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

union Pack16 {
  uint4 u;
  bf16 h[8];
  bf162 h2[4];
  uint8_t b[16];
  uint16_t s[8];
  uint32_t w[4];
};

}  // namespace dgpp
