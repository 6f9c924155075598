// Decode path (T <= B200MOE_DECODE_MAX_T tokens): the two expert matrices applied as matrix-vector products on the CUDA
// cores, one warp per output element, weights streamed from HBM exactly once per (token, expert) pair.
//
// With a handful of tokens every expert sees one or two rows, a 128-row tensor-core tile is >98 % padding and — worse —
// only (active experts x 16) CTAs have work, so the tile kernels pull a few hundred GB/s.  Here every SM streams
// weights: 14 336 bytes of W13 per warp task in GEMV1 (rows n and 2048+n, fused SwiGLU), 2 048 bytes of W2 per expert in
// GEMV2, which also applies the routing weights and sums the token's local experts, so the sort, the gather and the
// reduce are not needed at all.  The intermediate is kept in fp32 and enters GEMV2 as f16 scaled by its row maximum.
// Reference counterpart: the T = 1 path, solution/python/pure_triton_impl.py:2025-2123 (_kernel_t1) with
// _t1_fused_gemm2_reduce_kernel (:1676-1750); oracle math solution/cuda/binding.py:157-182.
#include "common.cuh"

namespace b200moe {

// Arithmetic: e4m3 -> f16 is exact, so 16-element partial dot products run on the packed half-precision FMA with the
// activation pre-scaled by 2^-6 (|a| <= 7, |w| <= 448: eight products per lane sum to < 2^15, no overflow; each
// product is rounded to 11 bits, far below the output tolerance) and are then added in fp32.  This needs 8 conversions
// per 16 weights instead of 24 and is what keeps the kernels at the memory system's pace.
struct Half2x8 {
  __half2 v[8];
};
__device__ __forceinline__ Half2x8 cvt16_h2(const uint4& q) {
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
  Half2x8 r;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __half2_raw lo = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(w[i] & 0xffffu), __NV_E4M3);
    __half2_raw hi = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(w[i] >> 16), __NV_E4M3);
    r.v[2 * i] = *reinterpret_cast<__half2*>(&lo);
    r.v[2 * i + 1] = *reinterpret_cast<__half2*>(&hi);
  }
  return r;
}
__device__ __forceinline__ float dot16_h2(const Half2x8& a, const uint4& wq) {
  const Half2x8 w = cvt16_h2(wq);
  __half2 acc = __hmul2(a.v[0], w.v[0]);
#pragma unroll
  for (int i = 1; i < 8; ++i) acc = __hfma2(a.v[i], w.v[i], acc);
  const float2 f = __half22float2(acc);
  return f.x + f.y;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
  return v;
}
// streaming 16-byte load: weights are read once, keep them out of L1
__device__ __forceinline__ uint4 ld_stream(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

constexpr int GEMV1_WARPS = 8;
constexpr int GEMV1_N_PER_CTA = 8;    // one column pair (n, 2048 + n) per warp; 2048 / 8 = 256 CTAs per (token, expert)
                                      // pair (measured at T = 1: 17.9 us against 21.3 us with 16 columns per CTA)
constexpr int GEMV2_N_PER_CTA = 32;   // 7168 / 32 = 224 CTAs per token, 4 columns per warp (16 or 8 columns per CTA
                                      // measured slower: every CTA stages the token's rows first)

// inter[p, n] = silu(x . W3[n]) * (x . W1[n]) for the local pair p = t*8+k of this CTA; the activation row is
// converted once per CTA into shared memory (f16, pre-scaled by 2^-6), each warp then streams rows n and 2048+n.
__global__ void __launch_bounds__(GEMV1_WARPS * 32)
k_gemv1_swiglu(const uint8_t* __restrict__ hidden, const float* __restrict__ hidden_scale,
               const int* __restrict__ topk_idx, int T, int local_offset, int E_local,
               const uint8_t* __restrict__ w13, const float* __restrict__ w13_scale, float* __restrict__ inter) {
  __shared__ __align__(16) __half2 s_a[H / 2];   // 14 KB
  __shared__ float s_as[H_BLOCKS];               // activation scales x 64
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  constexpr int CTAS_PER_PAIR = I / GEMV1_N_PER_CTA;
  const int p = blockIdx.x / CTAS_PER_PAIR;
  const int n0 = (blockIdx.x - p * CTAS_PER_PAIR) * GEMV1_N_PER_CTA;
  pdl_launch_dependents();
  pdl_wait();
  const int e = __ldg(topk_idx + p) - local_offset;
  if (e < 0 || e >= E_local) return;
  const int t = p / TOP_K;
  {
    const uint4* a_row = reinterpret_cast<const uint4*>(hidden + static_cast<size_t>(t) * H);
    const __half2 pre = __float2half2_rn(0.015625f);  // 2^-6, undone in s_as
    for (int c = threadIdx.x; c < H / 16; c += blockDim.x) {
      Half2x8 a = cvt16_h2(__ldg(a_row + c));
#pragma unroll
      for (int j = 0; j < 8; ++j) s_a[c * 8 + j] = __hmul2(a.v[j], pre);
    }
    if (threadIdx.x < H_BLOCKS)
      s_as[threadIdx.x] = 64.0f * __ldg(hidden_scale + static_cast<size_t>(threadIdx.x) * T + t);
  }
  __syncthreads();
  for (int n = n0 + warp; n < n0 + GEMV1_N_PER_CTA; n += GEMV1_WARPS) {
    const uint4* w1_row = reinterpret_cast<const uint4*>(w13 + (static_cast<size_t>(e) * 2 * I + n) * H);
    const uint4* w3_row = reinterpret_cast<const uint4*>(w13 + (static_cast<size_t>(e) * 2 * I + I + n) * H);
    const float* s1 = w13_scale + (static_cast<size_t>(e) * 32 + (n >> 7)) * H_BLOCKS;
    const float* s3 = w13_scale + (static_cast<size_t>(e) * 32 + 16 + (n >> 7)) * H_BLOCKS;
    float acc1 = 0.f, acc3 = 0.f;
#pragma unroll
    for (int i = 0; i < H / 16 / 32; ++i) {
      const int c = i * 32 + lane;       // 16-byte chunk of the row; 8 chunks per 128-column scale block
      const int kb = c >> 3;
      const uint4 wa = ld_stream(w1_row + c);
      const uint4 wb = ld_stream(w3_row + c);
      Half2x8 a;
      const uint4* sa = reinterpret_cast<const uint4*>(s_a + c * 8);
      *reinterpret_cast<uint4*>(&a.v[0]) = sa[0];
      *reinterpret_cast<uint4*>(&a.v[4]) = sa[1];
      const float as = s_as[kb];
      acc1 = fmaf(dot16_h2(a, wa), as * __ldg(s1 + kb), acc1);
      acc3 = fmaf(dot16_h2(a, wb), as * __ldg(s3 + kb), acc3);
    }
    acc1 = warp_sum(acc1);
    acc3 = warp_sum(acc3);
    if (lane == 0) inter[static_cast<size_t>(p) * I + n] = acc3 / (1.0f + expf(-acc3)) * acc1;
  }
}

// out[t, n] = sum over the token's local experts of weight * (inter[p] . W2[e][n]).  One CTA = one token and 32
// output columns; the token's (at most 8) intermediate rows are brought into shared memory once, as f16 scaled to
// |x| <= 7 by the row's own maximum (11-bit rounding of each element; the dot products then run on packed half FMAs
// like GEMV1).
__global__ void __launch_bounds__(256)
k_gemv2_reduce(const float* __restrict__ inter, const int* __restrict__ topk_idx, const float* __restrict__ topk_w,
               int T, int local_offset, int E_local, const uint8_t* __restrict__ w2, const float* __restrict__ w2_scale,
               uint16_t* __restrict__ out, float* __restrict__ out_f32) {
  __shared__ __align__(16) __half2 s_x[TOP_K][I / 2];   // 32 KB
  __shared__ float s_back[TOP_K];                       // weight * row maximum / 7
  __shared__ int s_e[TOP_K];
  __shared__ float s_red[TOP_K][8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  constexpr int CTAS_PER_TOKEN = H / GEMV2_N_PER_CTA;
  const int t = blockIdx.x / CTAS_PER_TOKEN;
  const int n0 = (blockIdx.x - t * CTAS_PER_TOKEN) * GEMV2_N_PER_CTA;
  pdl_launch_dependents();
  pdl_wait();
  // Stage the token's local rows: all loads first (up to 8 rows x 8 floats per thread), one block-wide maximum for all
  // rows at once, then the scaled f16 copies.  (Row by row this was a chain of 8 x (load, two barriers) before the first
  // weight byte was requested.)
  int e_k[TOP_K];
  float4 v[TOP_K][2];
  float m[TOP_K];
#pragma unroll
  for (int k = 0; k < TOP_K; ++k) {
    const int p = t * TOP_K + k;
    const int e = __ldg(topk_idx + p) - local_offset;
    e_k[k] = (e >= 0 && e < E_local) ? e : -1;   // CTA-uniform
    m[k] = 0.f;
    if (e_k[k] >= 0) {
      const float4* x = reinterpret_cast<const float4*>(inter + static_cast<size_t>(p) * I);
#pragma unroll
      for (int j = 0; j < 2; ++j) v[k][j] = __ldg(x + threadIdx.x * 2 + j);   // 256 threads x 8 floats = 2048
    }
  }
#pragma unroll
  for (int k = 0; k < TOP_K; ++k) {
    if (e_k[k] < 0) continue;
#pragma unroll
    for (int j = 0; j < 2; ++j)
      m[k] = fmaxf(m[k], fmaxf(fmaxf(fabsf(v[k][j].x), fabsf(v[k][j].y)), fmaxf(fabsf(v[k][j].z), fabsf(v[k][j].w))));
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) m[k] = fmaxf(m[k], __shfl_xor_sync(0xffffffffu, m[k], d));
    if (lane == 0) s_red[k][warp] = m[k];
  }
  if (threadIdx.x < TOP_K) s_e[threadIdx.x] = e_k[threadIdx.x];
  __syncthreads();
#pragma unroll
  for (int k = 0; k < TOP_K; ++k) {
    if (e_k[k] < 0) continue;
    float mk = s_red[k][0];
#pragma unroll
    for (int j = 1; j < 8; ++j) mk = fmaxf(mk, s_red[k][j]);
    const float r = mk > 0.f ? 7.0f / mk : 0.f;
    __half2* dst = &s_x[k][threadIdx.x * 4];
    dst[0] = __floats2half2_rn(v[k][0].x * r, v[k][0].y * r);
    dst[1] = __floats2half2_rn(v[k][0].z * r, v[k][0].w * r);
    dst[2] = __floats2half2_rn(v[k][1].x * r, v[k][1].y * r);
    dst[3] = __floats2half2_rn(v[k][1].z * r, v[k][1].w * r);
    if (threadIdx.x == 0) s_back[k] = __ldg(topk_w + t * TOP_K + k) * mk * (1.0f / 7.0f);
  }
  __syncthreads();
  // Each warp owns 4 output columns (n0 + warp + 8 j).  Per local expert it first requests all 16 weight loads of its
  // four rows (2 KB each), then consumes them: 8 KB in flight per warp instead of 2.
  constexpr int COLS = GEMV2_N_PER_CTA / 8;
  float total[COLS];   // per-lane shares; lanes are added once per column, after all of the token's experts
#pragma unroll
  for (int j = 0; j < COLS; ++j) total[j] = 0.f;
  for (int k = 0; k < TOP_K; ++k) {
    const int e = s_e[k];
    if (e < 0) continue;
    const float* sc = w2_scale + (static_cast<size_t>(e) * H_BLOCKS + (n0 >> 7)) * I_BLOCKS;
    uint4 w[COLS][I / 16 / 32];
#pragma unroll
    for (int j = 0; j < COLS; ++j) {
      const uint4* w_row = reinterpret_cast<const uint4*>(w2 + (static_cast<size_t>(e) * H + n0 + warp + 8 * j) * I);
#pragma unroll
      for (int i = 0; i < I / 16 / 32; ++i) w[j][i] = ld_stream(w_row + i * 32 + lane);
    }
    float acc[COLS];
#pragma unroll
    for (int j = 0; j < COLS; ++j) acc[j] = 0.f;
#pragma unroll
    for (int i = 0; i < I / 16 / 32; ++i) {
      const int c = i * 32 + lane;
      Half2x8 a;
      const uint4* sa = reinterpret_cast<const uint4*>(&s_x[k][c * 8]);
      *reinterpret_cast<uint4*>(&a.v[0]) = sa[0];
      *reinterpret_cast<uint4*>(&a.v[4]) = sa[1];
      const float scale = __ldg(sc + (c >> 3));
#pragma unroll
      for (int j = 0; j < COLS; ++j) acc[j] = fmaf(dot16_h2(a, w[j][i]), scale, acc[j]);
    }
    const float back = s_back[k];
#pragma unroll
    for (int j = 0; j < COLS; ++j) total[j] = fmaf(back, acc[j], total[j]);
  }
#pragma unroll
  for (int j = 0; j < COLS; ++j) {
    const float sum = warp_sum(total[j]);
    const int n = n0 + warp + 8 * j;
    if (lane == 0) {
      if (out) {
        __nv_bfloat16 b = __float2bfloat16_rn(sum);
        out[static_cast<size_t>(t) * H + n] = *reinterpret_cast<uint16_t*>(&b);
      }
      if (out_f32) out_f32[static_cast<size_t>(t) * H + n] = sum;
    }
  }
}

// `inter` lives in the workspace's expert_out array (unused by this path): [T*8, 2048] floats.
int launch_gemv1(const b200moe_problem* p, const b200moe_workspace* ws, int num_sms, cudaStream_t st) {
  if (p->T == 0) return B200MOE_OK;
  (void)num_sms;
  const unsigned grid = static_cast<unsigned>(p->T) * TOP_K * (I / GEMV1_N_PER_CTA);
  B200MOE_CUDA_TRY(launch_pdl(k_gemv1_swiglu, dim3(grid), dim3(GEMV1_WARPS * 32), 0, st, p->hidden_states,
                              p->hidden_states_scale, ws->topk_idx, p->T, p->local_expert_offset, p->E_local,
                              p->gemm1_weights, p->gemm1_weights_scale, ws->expert_out));
  return B200MOE_OK;
}

int launch_gemv2(const b200moe_problem* p, const b200moe_workspace* ws, int num_sms, cudaStream_t st) {
  if (p->T == 0) return B200MOE_OK;
  (void)num_sms;
  const unsigned grid = static_cast<unsigned>(p->T) * (H / GEMV2_N_PER_CTA);
  B200MOE_CUDA_TRY(launch_pdl(k_gemv2_reduce, dim3(grid), dim3(256), 0, st, ws->expert_out, ws->topk_idx, ws->topk_w,
                              p->T, p->local_expert_offset, p->E_local, p->gemm2_weights, p->gemm2_weights_scale,
                              p->output, p->output_f32));
  return B200MOE_OK;
}

}  // namespace b200moe
