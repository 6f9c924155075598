// The half form of un-rounded result rows (B200MOE_PARTIAL_HALF in the C interface): a row of 7168 values is 896 groups
// of eight consecutive columns, each group stored as eight float16 that share one power-of-two scale (14336 bytes),
// followed by the 896 scale bytes.  Used for the partial rows an expert-parallel shard returns over NVLink and for the
// GEMM2 rows the reduce reads back inside one layer call: 15232 instead of 28672 bytes per row, 11 significant bits per
// value (the result is rounded to bfloat16, 8 bits, after at most eight such rows are added).
#pragma once
#include <cuda_fp16.h>
#include "common.cuh"

namespace b200moe {

constexpr int HALF_ROW_BYTES = B200MOE_HALF_ROW_BYTES;
constexpr int HALF_ROW_SCALES = H * 2;            // byte offset of the 896 scale bytes
static_assert(HALF_ROW_BYTES == H * 2 + H / 8 && HALF_ROW_BYTES % 16 == 0, "half-row layout");

// Scale byte eb and multiplier k of one group.  eb = biased float32 exponent of the group's largest magnitude, clamped
// to [14, 254] so that k = 2^(141 - eb) is a normal float (inf/nan stay inf/nan); k puts that magnitude in
// [2^14, 2^15), below the float16 maximum, and every value down to 2^-28 of it keeps 11 significant bits.
__device__ __forceinline__ uint32_t half_group_scale(float max_abs, float& k) {
  uint32_t eb = __float_as_uint(max_abs) >> 23;   // the sign bit is clear
  eb = eb < 14u ? 14u : (eb > 254u ? 254u : eb);
  k = __uint_as_float((268u - eb) << 23);
  return eb;
}
// Eight values -> the group's 16 bytes of float16 (returned) and its scale byte.
__device__ __forceinline__ uint4 encode_half_group(const float (&x)[8], uint32_t& eb) {
  float m = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) m = fmaxf(m, fabsf(x[j]));
  float k;
  eb = half_group_scale(m, k);
  uint32_t o[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    __half2 h = __floats2half2_rn(x[2 * j] * k, x[2 * j + 1] * k);
    o[j] = *reinterpret_cast<uint32_t*>(&h);
  }
  return make_uint4(o[0], o[1], o[2], o[3]);
}
// Group v of the half row at `row` <- acc.
__device__ __forceinline__ void store_half_group(uint8_t* row, int v, const float (&acc)[8]) {
  uint32_t eb;
  reinterpret_cast<uint4*>(row)[v] = encode_half_group(acc, eb);
  row[HALF_ROW_SCALES + v] = static_cast<uint8_t>(eb);
}
// acc += w * (group v of the half row at `row`).  2^(eb - 141) * w is exact (eb = 14 decodes to zero).
__device__ __forceinline__ void fma_half_group(const uint8_t* row, int v, float w, float (&acc)[8]) {
  const uint4 q = __ldg(reinterpret_cast<const uint4*>(row) + v);
  const uint32_t eb = __ldg(row + HALF_ROW_SCALES + v);
  const float k = __uint_as_float((eb - 14u) << 23) * w;
  const uint32_t x[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&x[j]));
    acc[2 * j] = fmaf(f.x, k, acc[2 * j]);
    acc[2 * j + 1] = fmaf(f.y, k, acc[2 * j + 1]);
  }
}

}  // namespace b200moe
