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
// One CTA = 8 warps = a quarter of a 32-token chunk; the CTA also records, per local expert, which of its tokens
// selected it (its byte of the chunk's chunk_bits words), which the stable ranking in sort.cu consumes.
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

// Routing of one token by one warp.  Lane k < 8 returns the k-th selected expert in `my_idx` and its final weight in
// `my_w` (other lanes return 0).
__device__ __forceinline__ void route_token(const float* __restrict__ logits_row, const uint16_t* __restrict__ bias,
                                            float scale_factor, int lane, int& my_idx, float& my_w) {
  float s[N_GROUP];
  uint32_t key[N_GROUP];
#pragma unroll
  for (int g = 0; g < N_GROUP; ++g) {
    float x = __ldg(logits_row + g * 32 + lane);
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
  my_idx = 0;
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
  my_w = __fmul_rn(__fdiv_rn(my_s, __fadd_rn(sum, 1e-20f)), scale_factor);
}

// One CTA routes 8 tokens (a quarter of a 32-token chunk), one warp each: a token costs ~1000-1500 instructions on its
// warp, so a CTA per whole chunk kept 32 such warps on one SM (12 us of kernel time for 80 tokens with 145 SMs idle).
// The quarter's 8 selection bits per local expert are byte `quarter` of the chunk's 32-bit mask word: the four CTAs of
// a chunk write disjoint bytes, so the mask needs neither atomics nor clearing.  The grid covers whole chunks
// (4 CTAs each), so every byte of every mask word is written even where the last chunk is ragged.
constexpr int ROUTE_WARPS = 8;
__global__ void __launch_bounds__(ROUTE_WARPS * 32)
k_route(const float* __restrict__ logits, const uint16_t* __restrict__ bias, int T, float scale_factor,
        int local_offset, int E_local, int* __restrict__ topk_idx, float* __restrict__ topk_w,
        uint32_t* __restrict__ chunk_bits) {
  __shared__ uint32_t s_bits[E_GLOBAL];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int chunk = blockIdx.x >> 2;
  const int quarter = blockIdx.x & 3;
  const int t = blockIdx.x * ROUTE_WARPS + warp;

  pdl_launch_dependents();
  if (threadIdx.x < E_GLOBAL) s_bits[threadIdx.x] = 0;
  pdl_wait();
  __syncthreads();

  if (t < T) {
    int my_idx;
    float w;
    route_token(logits + static_cast<size_t>(t) * E_GLOBAL, bias, scale_factor, lane, my_idx, w);
    if (lane < TOP_K) {
      topk_idx[static_cast<size_t>(t) * TOP_K + lane] = my_idx;
      topk_w[static_cast<size_t>(t) * TOP_K + lane] = w;
      int le = my_idx - local_offset;
      if (le >= 0 && le < E_local) atomicOr(&s_bits[le], 1u << warp);
    }
  }
  __syncthreads();
  if (threadIdx.x < E_local) {
    uint8_t* word = reinterpret_cast<uint8_t*>(chunk_bits + static_cast<size_t>(chunk) * E_local + threadIdx.x);
    word[quarter] = static_cast<uint8_t>(s_bits[threadIdx.x]);   // little-endian: byte q = bits 8q .. 8q+7
  }
}

// Small batches (T <= B200MOE_PROLOGUE_MAX_T): routing, ranking, padded layout, scatter and the activation gather in ONE launch instead of
// four.  Same results, bit for bit, as k_route + k_rank_scan + k_scatter + k_gather.  Every CTA repeats the (cheap)
// routing and layout of the whole batch in shared memory, so no CTA waits for another; CTA 0 alone writes the metadata
// to global memory, and the row copies are dealt round-robin over all CTAs.  1024 threads: warp w routes token 32c + w
// of chunk c (chunks one after the other, which is why the limit is low: measured, one chunk costs ~9 us and the
// separate kernels win from the second chunk on) and keeps its eight pairs in lanes 0..7 for the placement.
constexpr int SMALL_T_MAX = B200MOE_PROLOGUE_MAX_T;
static_assert(SMALL_T_MAX % 32 == 0 && SMALL_T_MAX <= 128, "whole token chunks, at most 1024 (token, k) pairs");
__global__ void __launch_bounds__(1024, 1)
k_small_prologue(const float* __restrict__ logits, const uint16_t* __restrict__ bias, const uint8_t* __restrict__ hidden,
                 const float* __restrict__ hidden_scale, int T, float scale_factor, int local_offset, int E_local,
                 int R_max, int* __restrict__ topk_idx, float* __restrict__ topk_w, uint32_t* __restrict__ chunk_bits,
                 int* __restrict__ chunk_base, int* __restrict__ counts, int* __restrict__ block_offsets,
                 int* __restrict__ total_blocks, int* __restrict__ sorted_token_ids, float* __restrict__ sorted_weights,
                 int* __restrict__ scatter_map, uint8_t* __restrict__ a_sorted, float* __restrict__ a_scale_sorted) {
  __shared__ uint32_t s_bits[SMALL_T_MAX / 32][E_GLOBAL];
  __shared__ int s_base[SMALL_T_MAX / 32][E_GLOBAL];
  __shared__ int s_cnt[E_GLOBAL];
  __shared__ int s_row_base[E_GLOBAL + 1];   // in 128-row blocks
  __shared__ int s_dest[SMALL_T_MAX * TOP_K];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int n_chunks = (T + 31) / 32;
  const bool lead = blockIdx.x == 0;

  pdl_launch_dependents();
  for (int i = threadIdx.x; i < (SMALL_T_MAX / 32) * E_GLOBAL; i += blockDim.x) (&s_bits[0][0])[i] = 0;
  pdl_wait();
  __syncthreads();

  int my_idx[SMALL_T_MAX / 32];
  float my_w[SMALL_T_MAX / 32];
#pragma unroll
  for (int c = 0; c < SMALL_T_MAX / 32; ++c) {
    const int t = c * 32 + warp;
    my_idx[c] = -1;
    my_w[c] = 0.f;
    if (c < n_chunks && t < T) {
      route_token(logits + static_cast<size_t>(t) * E_GLOBAL, bias, scale_factor, lane, my_idx[c], my_w[c]);
      if (lane < TOP_K) {
        if (lead) {
          topk_idx[static_cast<size_t>(t) * TOP_K + lane] = my_idx[c];
          topk_w[static_cast<size_t>(t) * TOP_K + lane] = my_w[c];
        }
        const int le = my_idx[c] - local_offset;
        if (le >= 0 && le < E_local) atomicOr(&s_bits[c][le], 1u << warp);
      }
    }
  }
  __syncthreads();
  // per-expert prefix over chunks, counts
  if (threadIdx.x < E_local) {
    const int e = threadIdx.x;
    int run = 0;
    for (int c = 0; c < n_chunks; ++c) {
      s_base[c][e] = run;
      if (lead) {
        chunk_base[static_cast<size_t>(c) * E_local + e] = run;
        chunk_bits[static_cast<size_t>(c) * E_local + e] = s_bits[c][e];
      }
      run += __popc(s_bits[c][e]);
    }
    s_cnt[e] = run;
    if (lead) counts[e] = run;
  }
  __syncthreads();
  if (warp == 0) {
    int blocks[8], local = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int e = lane * 8 + i;
      blocks[i] = (e < E_local) ? (s_cnt[e] + BLOCK_M - 1) / BLOCK_M : 0;
      local += blocks[i];
    }
    int incl = local;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      int o = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += o;
    }
    int run = incl - local;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int e = lane * 8 + i;
      if (e < E_local) s_row_base[e] = run;
      run += blocks[i];
    }
    if (lane == 31) s_row_base[E_local] = incl;
  }
  __syncthreads();
  if (lead) {
    for (int e = threadIdx.x; e <= E_local; e += blockDim.x) block_offsets[e] = s_row_base[e];
    if (threadIdx.x == 0) *total_blocks = s_row_base[E_local];
  }
  // pad rows of every expert segment
  for (int e = warp; lead && e < E_local; e += 32) {
    const int begin = s_row_base[e] * BLOCK_M + s_cnt[e];
    const int end = s_row_base[e + 1] * BLOCK_M;
    for (int r = begin + lane; r < end; r += 32) {
      sorted_token_ids[r] = T;
      sorted_weights[r] = 0.f;
    }
  }
  // placement: warp w of chunk c still holds token 32c + w's routing in lanes 0..7
#pragma unroll
  for (int c = 0; c < SMALL_T_MAX / 32; ++c) {
    const int t = c * 32 + warp;
    if (c < n_chunks && t < T && lane < TOP_K) {
      const int le = my_idx[c] - local_offset;
      int d = -1;
      if (le >= 0 && le < E_local) {
        d = s_row_base[le] * BLOCK_M + s_base[c][le] + __popc(s_bits[c][le] & ((1u << warp) - 1u));
        if (lead) {
          sorted_token_ids[d] = t;
          sorted_weights[d] = my_w[c];
        }
      }
      if (lead) scatter_map[static_cast<size_t>(t) * TOP_K + lane] = d;
      s_dest[t * TOP_K + lane] = d;
    }
  }
  __syncthreads();
  // gather: one warp per local pair, pairs dealt over all CTAs
  for (int pair = blockIdx.x * 32 + warp; pair < T * TOP_K; pair += gridDim.x * 32) {
    const int d = s_dest[pair];
    if (d < 0) continue;
    const int tok = pair / TOP_K;
    const uint4* src = reinterpret_cast<const uint4*>(hidden + static_cast<size_t>(tok) * H);
    uint4* dst = reinterpret_cast<uint4*>(a_sorted + static_cast<size_t>(d) * H);
#pragma unroll
    for (int i = 0; i < H / 16 / 32; ++i) dst[i * 32 + lane] = __ldg(src + i * 32 + lane);
    for (int kb = lane; kb < H_BLOCKS; kb += 32)
      a_scale_sorted[static_cast<size_t>(kb) * R_max + d] = __ldg(hidden_scale + static_cast<size_t>(kb) * T + tok);
  }
}

// chunk_bits from an existing topk_idx: one warp per 32-token chunk, lane = token.
__global__ void __launch_bounds__(128)
k_topk_bits(const int* __restrict__ topk_idx, long long idx_stride, int T, int local_offset, int E_local, int n_chunks,
            uint32_t* __restrict__ chunk_bits, const b200moe_ep_plan* __restrict__ plan) {
  const int lane = threadIdx.x & 31;
  const int chunk = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  pdl_launch_dependents();
  pdl_wait();
  if (chunk >= n_chunks) return;
  if (plan) T = min(T, plan->n_recv);   // rows past the received count hold stale records: they select nothing
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
  B200MOE_CUDA_TRY(launch_pdl(k_route, dim3(ws->n_chunks * 4), dim3(ROUTE_WARPS * 32), 0, st, p->routing_logits, p->routing_bias, p->T,
                              p->routed_scaling_factor, p->local_expert_offset, p->E_local, ws->topk_idx, ws->topk_w,
                              ws->chunk_bits));
  return B200MOE_OK;
}

// Routing alone into caller-owned arrays (no workspace, no selection bits): what an expert-parallel rank runs on its own
// tokens before dispatch.
int launch_route_topk(const float* logits, const uint16_t* bias, int T, float scale, int* topk_idx, float* topk_w,
                      cudaStream_t st) {
  if (T == 0) return B200MOE_OK;
  const int n_chunks = (T + 31) / 32;
  B200MOE_CUDA_TRY(launch_pdl(k_route, dim3(n_chunks * 4), dim3(ROUTE_WARPS * 32), 0, st, logits, bias, T, scale, 0, 0,
                              topk_idx, topk_w, static_cast<uint32_t*>(nullptr)));
  return B200MOE_OK;
}

// route + sort + gather for T <= B200MOE_PROLOGUE_MAX_T in one launch (dense inputs only)
int launch_small_prologue(const b200moe_problem* p, const b200moe_workspace* ws, cudaStream_t st) {
  if (p->T == 0) return B200MOE_OK;
  // one CTA per 32 (token, k) pairs of the batch, at most 32
  const int ctas = p->T < 32 ? p->T : 32;
  B200MOE_CUDA_TRY(launch_pdl(k_small_prologue, dim3(ctas), dim3(1024), 0, st, p->routing_logits, p->routing_bias,
                              p->hidden_states, p->hidden_states_scale, p->T, p->routed_scaling_factor,
                              p->local_expert_offset, p->E_local, ws->R_max, ws->topk_idx, ws->topk_w, ws->chunk_bits,
                              ws->chunk_base, ws->counts, ws->block_offsets, ws->total_blocks, ws->sorted_token_ids,
                              ws->sorted_weights, ws->scatter_map, ws->a_sorted, ws->a_scale_sorted));
  return B200MOE_OK;
}

int launch_topk_bits(const b200moe_problem* p, const b200moe_workspace* ws, cudaStream_t st) {
  if (p->T == 0) return B200MOE_OK;
  int grid = (ws->n_chunks + 3) / 4;
  const int* idx = p->routing_logits ? ws->topk_idx : p->topk_idx_in;
  B200MOE_CUDA_TRY(launch_pdl(k_topk_bits, dim3(grid), dim3(128), 0, st, idx,
                              p->topk_row_stride ? p->topk_row_stride : static_cast<long long>(TOP_K), p->T, p->local_expert_offset, p->E_local,
                              ws->n_chunks, ws->chunk_bits, p->plan));
  return B200MOE_OK;
}

}  // namespace b200moe
