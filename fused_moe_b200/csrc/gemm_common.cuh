// Pieces shared by the two grouped FP8 GEMM kernels (128-token tiles in gemm.cu, token-minor tiles in gemm_skinny.cu).
#pragma once
#include <cuda.h>
#include <cuda_fp8.h>
#include <cuda_fp16.h>
#include "common.cuh"

namespace b200moe {

struct GemmArgs {
  const int* block_offsets;  // [E+1]
  const int* counts;         // [E]
  const float* row_scale;    // MODE1: a_scale_sorted [56,R_max]; MODE2: inter_scale [16,R_max]
  const float* w_scale;      // MODE1: [E,32,56]; MODE2: [E,56,16]
  const uint8_t* weights;    // token-minor kernels: MODE1 [E,4096,7168], MODE2 [E,7168,2048] e4m3 (read without TMA)
  uint8_t* inter_q;          // MODE1 out: [2,R_max,2048]
  float* inter_scale;        // MODE1 out: [16,R_max]
  float* expert_out;         // MODE2 out: [R_max,7168] float32
  int* status;
  int* tile_ctr;             // token-minor kernels: tickets of tiles shared by several CTAs (zero between launches)
  float* partial;            // token-minor kernels: partial sums of shared tiles, two slots per CTA
  int E_local;
  int R_max;
  int early_weights;         // token-minor kernels inside b200moe_forward: weight stream starts before the dependency
                             // wait, see gemm_skinny.cu
  int out_half;              // tile GEMM2: expert_out rows in the half form (half_rows.cuh) instead of float32
};

__device__ __forceinline__ float silu_mul(float gate, float up) {
  return __fdividef(gate, 1.0f + __expf(-gate)) * up;
}

__device__ __forceinline__ uint32_t pack4_e4m3(float a, float b, float c, float d) {
  uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return lo | (hi << 16);
}
__device__ __forceinline__ void unpack4_e4m3(uint32_t v, float (&f)[4]) {
  __half2_raw lo = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(v & 0xffffu), __NV_E4M3);
  __half2_raw hi = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(v >> 16), __NV_E4M3);
  float2 a = __half22float2(*reinterpret_cast<__half2*>(&lo));
  float2 b = __half22float2(*reinterpret_cast<__half2*>(&hi));
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}

// The deal.  Whole rounds first: tile r G + c goes to CTA c as one piece (r < rounds).  The tiles that are left (fewer
// than G, numbered from first_tile) are dealt in 128-K chunk units: CTA c owns units [begin(c), begin(c + 1)) of the
// U = left-over tiles x chunks per tile, so the last round keeps every SM busy for the same time.  With fewer units
// than CTAs only the first U CTAs take part, so the owners of a tile's units are always consecutive CTAs.
struct Deal {
  long long U;      // chunk units of the left-over tiles
  int G;            // CTAs
  int rounds;       // whole tiles per CTA
  int first_tile;   // = rounds * G
  int Gu;           // CTAs that take part in the unit deal = min(G, U): every one of them owns at least one unit
  __device__ __forceinline__ long long begin(int c) const { return c >= Gu ? U : U * c / Gu; }
  // the CTA that owns unit u: the largest c < Gu with begin(c) <= u
  __device__ __forceinline__ int owner(long long u) const { return static_cast<int>(((u + 1) * Gu + U - 1) / U) - 1; }
};

struct Item {
  int tile, kb0, kb1;   // chunks [kb0, kb1) of the tile
};

// Fills a Deal for `total_tiles` tiles of `k_chunks` chunks each on G CTAs.
__device__ __forceinline__ Deal make_deal(int total_tiles, int k_chunks, int G) {
  Deal d;
  d.G = G;
  d.rounds = total_tiles / G;
  d.first_tile = d.rounds * G;
  d.U = static_cast<long long>(total_tiles - d.first_tile) * k_chunks;
  d.Gu = d.U < G ? static_cast<int>(d.U) : G;
  return d;
}

// Work item number `v` in CTA `cta`'s sequence of chunk positions (its whole tiles first, then its run of left-over
// units [u_begin, u_end)); v_whole = rounds * k_chunks.
__device__ __forceinline__ Item deal_item(const Deal& d, int k_chunks, int cta, long long v, long long v_whole,
                                          long long u_begin, long long u_end) {
  Item it;
  if (v < v_whole) {
    it.tile = static_cast<int>(v / k_chunks) * d.G + cta;
    it.kb0 = 0;
    it.kb1 = k_chunks;
  } else {
    const long long u = u_begin + (v - v_whole);
    const int lt = static_cast<int>(u / k_chunks);
    it.tile = d.first_tile + lt;
    it.kb0 = static_cast<int>(u - static_cast<long long>(lt) * k_chunks);
    const long long left = u_end - u;
    it.kb1 = (left < k_chunks - it.kb0) ? it.kb0 + static_cast<int>(left) : k_chunks;
  }
  return it;
}

// 2-D byte tensor [rows, cols] (row pitch = cols), box [box_rows, 128 bytes], 128-byte swizzle.  Defined in gemm.cu.
int make_map_u8(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows);

}  // namespace b200moe
