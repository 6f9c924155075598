// DeepSeek-V3 no-aux routing, one warp per token.
//
// Behaviour follows the reference routing (solution/cuda/binding.py:38-61, the torch statement; and
// solution/python/pure_triton_impl.py:96-190, the Triton kernel):
//   s = sigmoid(logit); sb = s + bias; group score = sum of the two largest sb of each 32-expert group
//   (duplicates count, as torch.topk(2).sum does); keep the 4 best groups; take the 8 best sb among them;
//   weight_k = s_k / (sum_k s_k + 1e-20) * routed_scaling_factor  (the bias is not part of the weight).
// Ties always go to the lower index (tl.argmax first-occurrence rule); experts come out in descending sb.
//
// Layout: lane l holds experts {l, l+32, ..., l+224}, so register slot g of every lane belongs to routing group g.
// Group top-2 and the global arg-max are REDUX (warp reduce) operations on order-preserving integer keys.
//
// One CTA = 32 warps = one 32-token chunk; the CTA also records, per local expert, which of its tokens selected it
// (chunk_bits), which the stable ranking in sort.cu consumes.
#include "common.cuh"

namespace b200moe {

// exp(-x) and the sigmoid are built from individually rounded IEEE operations only (no fast-math, no contraction
// left to the compiler), so that a host restatement with fmaf() produces the same bits.
__device__ __forceinline__ float exp_neg_exact_ops(float x) {
  float z = fminf(fmaxf(-x, -87.0f), 88.0f);
  float t = __fmul_rn(z, 1.44269504088896341f);
  float n = rintf(t);
  float r = __fmaf_rn(n, -0.693145751953125f, z);           // ln2 high part (exact product for |n| < 2^11)
  r = __fmaf_rn(n, -1.42860682030941723e-6f, r);            // ln2 low part
  float p = 1.0f / 5040.0f;
  p = __fmaf_rn(p, r, 1.0f / 720.0f);
  p = __fmaf_rn(p, r, 1.0f / 120.0f);
  p = __fmaf_rn(p, r, 1.0f / 24.0f);
  p = __fmaf_rn(p, r, 1.0f / 6.0f);
  p = __fmaf_rn(p, r, 0.5f);
  p = __fmaf_rn(p, r, 1.0f);
  p = __fmaf_rn(p, r, 1.0f);
  float scale = __int_as_float((static_cast<int>(n) + 127) << 23);
  return __fmul_rn(p, scale);
}
__device__ __forceinline__ float sigmoid_exact_ops(float x) {
  return __fdiv_rn(1.0f, __fadd_rn(1.0f, exp_neg_exact_ops(x)));
}

// float <-> unsigned key with the same ordering (larger float = larger key); key 0 is below every float.
__device__ __forceinline__ uint32_t f2key(float f) {
  uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key2f(uint32_t k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

__global__ void __launch_bounds__(1024, 1)
k_route(const float* __restrict__ logits, const uint16_t* __restrict__ bias, int T, float scale_factor,
        int local_offset, int E_local, int* __restrict__ topk_idx, float* __restrict__ topk_w,
        uint32_t* __restrict__ chunk_bits) {
  __shared__ uint32_t s_bits[E_GLOBAL];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int chunk = blockIdx.x;
  const int t = chunk * 32 + warp;

  pdl_launch_dependents();
  if (threadIdx.x < E_GLOBAL) s_bits[threadIdx.x] = 0;
  pdl_wait();
  __syncthreads();

  if (t < T) {
    float s[N_GROUP];
    uint32_t key[N_GROUP];
#pragma unroll
    for (int g = 0; g < N_GROUP; ++g) {
      float x = __ldg(logits + static_cast<size_t>(t) * E_GLOBAL + g * 32 + lane);
      float b = bf16_bits_to_float(__ldg(bias + g * 32 + lane));
      s[g] = sigmoid_exact_ops(x);
      key[g] = f2key(__fadd_rn(s[g], b));
    }
    // group scores (warp-uniform)
    float gs[N_GROUP];
#pragma unroll
    for (int g = 0; g < N_GROUP; ++g) {
      uint32_t m1 = __reduce_max_sync(0xffffffffu, key[g]);
      uint32_t hit = __ballot_sync(0xffffffffu, key[g] == m1);
      int first = __ffs(hit) - 1;
      uint32_t m2 = __reduce_max_sync(0xffffffffu, lane == first ? 0u : key[g]);
      gs[g] = __fadd_rn(key2f(m1), key2f(m2));
    }
    // top-4 groups, lower index wins ties
    uint32_t gmask = 0;
#pragma unroll
    for (int r = 0; r < TOPK_GROUP; ++r) {
      int best = -1;
      float bv = 0.f;
#pragma unroll
      for (int g = 0; g < N_GROUP; ++g) {
        bool free_g = !((gmask >> g) & 1u);
        if (free_g && (best < 0 || gs[g] > bv)) { best = g; bv = gs[g]; }
      }
      gmask |= 1u << best;
    }
#pragma unroll
    for (int g = 0; g < N_GROUP; ++g)
      if (!((gmask >> g) & 1u)) key[g] = 0u;

    // top-8 experts by repeated arg-max with removal
    int my_idx = 0;
    float my_s = 0.f;
    float sum = 0.f;
#pragma unroll
    for (int k = 0; k < TOP_K; ++k) {
      uint32_t bk = key[0];
      int bg = 0;
#pragma unroll
      for (int g = 1; g < N_GROUP; ++g)
        if (key[g] > bk) { bk = key[g]; bg = g; }
      uint32_t vmax = __reduce_max_sync(0xffffffffu, bk);
      uint32_t cand = (bk == vmax) ? static_cast<uint32_t>(bg * 32 + lane) : 0xffffu;
      uint32_t widx = __reduce_min_sync(0xffffffffu, cand);
      int owner = widx & 31, slot = widx >> 5;
      float sv = 0.f;
#pragma unroll
      for (int g = 0; g < N_GROUP; ++g)
        if (g == slot) {
          sv = s[g];
          if (lane == owner) key[g] = 0u;
        }
      sv = __shfl_sync(0xffffffffu, sv, owner);
      sum = __fadd_rn(sum, sv);
      if (lane == k) { my_idx = static_cast<int>(widx); my_s = sv; }
    }
    if (lane < TOP_K) {
      float w = __fmul_rn(__fdiv_rn(my_s, __fadd_rn(sum, 1e-20f)), scale_factor);
      topk_idx[static_cast<size_t>(t) * TOP_K + lane] = my_idx;
      topk_w[static_cast<size_t>(t) * TOP_K + lane] = w;
      int le = my_idx - local_offset;
      if (le >= 0 && le < E_local) atomicOr(&s_bits[le], 1u << warp);
    }
  }
  __syncthreads();
  if (threadIdx.x < E_local) chunk_bits[static_cast<size_t>(chunk) * E_local + threadIdx.x] = s_bits[threadIdx.x];
}

// chunk_bits from an existing topk_idx: one warp per 32-token chunk, lane = token.
__global__ void __launch_bounds__(128)
k_topk_bits(const int* __restrict__ topk_idx, long long idx_stride, int T, int local_offset, int E_local, int n_chunks,
            uint32_t* __restrict__ chunk_bits) {
  const int lane = threadIdx.x & 31;
  const int chunk = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  pdl_launch_dependents();
  pdl_wait();
  if (chunk >= n_chunks) return;
  const int t = chunk * 32 + lane;
  uint32_t mask[E_GLOBAL / 32];
#pragma unroll
  for (int i = 0; i < E_GLOBAL / 32; ++i) mask[i] = 0;
  if (t < T) {
#pragma unroll
    for (int k = 0; k < TOP_K; ++k) {
      int le = __ldg(topk_idx + static_cast<size_t>(t) * idx_stride + k) - local_offset;
      if (le >= 0 && le < E_local) {
#pragma unroll
        for (int i = 0; i < E_GLOBAL / 32; ++i)
          if (i == (le >> 5)) mask[i] |= 1u << (le & 31);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < E_GLOBAL / 32; ++i) {
    if (i * 32 >= E_local) break;
    uint32_t mine = 0;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      uint32_t w = __ballot_sync(0xffffffffu, (mask[i] >> j) & 1u);
      if (lane == j) mine = w;
    }
    int e = i * 32 + lane;
    if (e < E_local) chunk_bits[static_cast<size_t>(chunk) * E_local + e] = mine;
  }
}

int launch_route(const b200moe_problem* p, const b200moe_workspace* ws, cudaStream_t st) {
  if (p->T == 0) return B200MOE_OK;
  B200MOE_CUDA_TRY(launch_pdl(k_route, dim3(ws->n_chunks), dim3(1024), 0, st, p->routing_logits, p->routing_bias, p->T,
                              p->routed_scaling_factor, p->local_expert_offset, p->E_local, ws->topk_idx, ws->topk_w,
                              ws->chunk_bits));
  return B200MOE_OK;
}

int launch_topk_bits(const b200moe_problem* p, const b200moe_workspace* ws, cudaStream_t st) {
  if (p->T == 0) return B200MOE_OK;
  int grid = (ws->n_chunks + 3) / 4;
  const int* idx = p->routing_logits ? ws->topk_idx : p->topk_idx_in;
  B200MOE_CUDA_TRY(launch_pdl(k_topk_bits, dim3(grid), dim3(128), 0, st, idx,
                              p->topk_row_stride ? p->topk_row_stride : static_cast<long long>(TOP_K), p->T, p->local_expert_offset, p->E_local,
                              ws->n_chunks, ws->chunk_bits));
  return B200MOE_OK;
}

}  // namespace b200moe
