// Deterministic exp / log for the sampler: the same sequence of IEEE single-precision multiplies and adds on
// the host and on the device (no library calls, no fused multiply-add), so the host oracle and the device
// sampler agree bit for bit.  Translation units that include this for sampling are built with contraction
// off (-ffp-contract=off for g++, --fmad=false for nvcc).
// Accuracy: about 2 ulp for exp on [-87, 88], about 3 ulp for log on normal inputs.
// (same role as src/common/det_math.hpp of the reference.)
#pragma once
#include <stdint.h>
#include <string.h>

#if defined(__CUDACC__)
#define DGPP_HD __host__ __device__ __forceinline__
#else
#define DGPP_HD inline
#endif

namespace dgpp {
namespace det {

DGPP_HD float bits_to_f(uint32_t u) {
  float f;
  memcpy(&f, &u, 4);
  return f;
}
DGPP_HD uint32_t f_to_bits(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  return u;
}

// e^x.  x is split as n * ln2 + r with |r| <= ln2 / 2; e^r by a degree-6 polynomial; scaling by exponent bits.
DGPP_HD float exp(float x) {
  if (x > 88.5f) return bits_to_f(0x7f800000u);
  if (x < -103.0f) return 0.0f;
  const float t = x * 1.44269504088896341f;
  const float nf = (t >= 0.0f) ? static_cast<float>(static_cast<int>(t + 0.5f)) : static_cast<float>(static_cast<int>(t - 0.5f));
  // two-constant Cody-Waite reduction
  float r = x - nf * 0.693145751953125f;
  r = r - nf * 1.42860682030941723e-6f;
  float p = 1.3888889e-3f;
  p = p * r + 8.3333338e-3f;
  p = p * r + 4.1666668e-2f;
  p = p * r + 1.6666667e-1f;
  p = p * r + 5.0e-1f;
  p = p * r + 1.0f;
  p = p * r + 1.0f;
  int n = static_cast<int>(nf);
  // scale in two steps so that results in the subnormal range stay correct
  float s1 = 1.0f, s2 = 1.0f;
  if (n > 127) { s1 = bits_to_f(0x7f000000u); n -= 127; }
  else if (n < -126) { s1 = bits_to_f(0x00800000u); n += 126; }
  if (n < -126) n = -126;
  s2 = bits_to_f(static_cast<uint32_t>(n + 127) << 23);
  return p * s2 * s1;
}

// ln(x) for x > 0 (returns -inf for 0, the input for inf / nan-free use).
DGPP_HD float log(float x) {
  if (x <= 0.0f) return bits_to_f(0xff800000u);
  uint32_t u = f_to_bits(x);
  int e = 0;
  if ((u >> 23) == 0) {  // subnormal: normalise
    x = x * 8388608.0f;
    u = f_to_bits(x);
    e = -23;
  }
  e += static_cast<int>(u >> 23) - 127;
  float m = bits_to_f((u & 0x007fffffu) | 0x3f800000u);  // [1, 2)
  if (m > 1.41421356f) { m = m * 0.5f; e += 1; }
  const float f = m - 1.0f;
  const float s = f / (2.0f + f);
  const float z = s * s;
  float p = 0.2222222222f;  // 2/9
  p = p * z + 0.2857142857f;  // 2/7
  p = p * z + 0.4f;
  p = p * z + 0.6666666667f;
  p = p * z + 2.0f;
  const float ln_m = s * p;
  const float ef = static_cast<float>(e);
  return ef * 0.693145751953125f + (ln_m + ef * 1.42860682030941723e-6f);
}

// SplitMix64: counter-based, so a draw depends only on (seed, counter).
DGPP_HD uint64_t splitmix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}
// Uniform in [0, 1) with 24 bits.
DGPP_HD float uniform01(uint64_t seed, uint64_t counter) {
  const uint64_t r = splitmix64(seed ^ splitmix64(counter));
  return static_cast<float>(r >> 40) * (1.0f / 16777216.0f);
}

}  // namespace det
}  // namespace dgpp
