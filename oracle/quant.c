/*
 * TEST INFRASTRUCTURE — not part of the product.  Only tests/ and bench.py's CPU legs may load this code.
 *
 * CPU restatement of the activation quantiser upstream of the layer: bf16 [T,7168] -> e4m3 [T,7168] + one float32
 * scale per token per 128 columns, stored [56,T].  The reference has no operator for this step; its profiling script
 * builds the pair with torch by MULTIPLYING with 448/amax (scripts/yjl_ncu.py:413-416).  The specification restated
 * here, operation for operation in IEEE float32 (round to nearest even, no contraction):
 *     amax = max |x| over the 128 columns          s = max(amax * (1/448), 1e-12)
 *     inv  = 1 / s                                   q = e4m3(x * inv)   (round to nearest even, saturating at +-448)
 * Pinned by tests/test_oracle.py against torch's own float32 -> float8_e4m3fn conversion on the CPU.
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

#define H 7168
#define QB 128

/* float32 -> e4m3fn (1 sign, 4 exponent bits with bias 7, 3 mantissa bits; largest finite 448; S.1111.111 = NaN),
 * round to nearest even; magnitudes above 448 saturate to 448 (the "satfinite" conversion). */
uint8_t oracle_f32_to_e4m3(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  const uint8_t sign = (uint8_t)((u >> 24) & 0x80);
  u &= 0x7fffffffu;
  if (u > 0x7f800000u) return (uint8_t)(sign | 0x7f);              /* NaN */
  float a;
  memcpy(&a, &u, 4);
  if (a > 448.0f) return (uint8_t)(sign | 0x7e);                   /* saturate (also +-inf) */
  if (a < 0.015625f) {                                             /* below 2^-6: subnormal grid of 2^-9 */
    const float q = nearbyintf(a * 512.0f);                        /* exact product; ties to even */
    return (uint8_t)(sign | (uint8_t)q);                           /* q == 8 is the smallest normal, code 0x08 */
  }
  int e = (int)(u >> 23) - 127;
  uint32_t man = u & 0x7fffffu, m3 = man >> 20, rem = man & 0xfffffu;
  if (rem > 0x80000u || (rem == 0x80000u && (m3 & 1u))) ++m3;
  if (m3 == 8) { m3 = 0; ++e; }
  if (e > 8 || (e == 8 && m3 == 7)) return (uint8_t)(sign | 0x7e); /* rounded past 448 */
  return (uint8_t)(sign | ((uint32_t)(e + 7) << 3) | m3);
}

static float bf16_to_f32(uint16_t b) {
  uint32_t u = (uint32_t)b << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

/* x [T,7168] bf16 bit patterns -> q [T,7168] e4m3 bytes, scale [56,T] float32 */
void oracle_quantize_act(const uint16_t* x, int T, uint8_t* q, float* scale) {
  const float inv448 = 1.0f / 448.0f;
  for (int t = 0; t < T; ++t)
    for (int kb = 0; kb < H / QB; ++kb) {
      const uint16_t* row = x + (size_t)t * H + (size_t)kb * QB;
      float amax = 0.0f;
      for (int j = 0; j < QB; ++j) {
        const float v = fabsf(bf16_to_f32(row[j]));
        if (v > amax) amax = v;
      }
      float s = amax * inv448;
      if (!(s > 1e-12f)) s = 1e-12f;
      const float inv = 1.0f / s;
      scale[(size_t)kb * T + t] = s;
      for (int j = 0; j < QB; ++j) q[(size_t)t * H + (size_t)kb * QB + j] = oracle_f32_to_e4m3(bf16_to_f32(row[j]) * inv);
    }
}
