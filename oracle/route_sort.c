/*
 * TEST INFRASTRUCTURE — not part of the product.  Only the tests, the driver's smoke check and bench.py's CPU-baseline
 * legs may load this code; the CUDA library never calls it.
 *
 * CPU restatement of the reference's routing and sort metadata for the DeepSeek-V3 fused MoE layer.
 *
 *   oracle_route      follows solution/cuda/binding.py:38-61 (_ds_routing_impl) with the tie rule of
 *                     solution/python/pure_triton_impl.py:149-182 (tl.argmax: first occurrence = lower index).
 *   oracle_sort       follows solution/cuda/binding.py:134-154 (local mask + argsort(stable=True)) for the order and
 *                     solution/python/pure_triton_impl.py:512-531 for the padded layout (blocks = ceil(cnt/BM),
 *                     exclusive cumsum in block units, pad token id = T, pad weight = 0, scatter_map = -1 if non-local).
 *
 * The sigmoid is spelled out in individually rounded IEEE-754 single operations (fmaf, rintf, one division) so that it
 * gives the same bits on any conforming machine; compile this file with -ffp-contract=off.  It agrees with
 * torch.sigmoid to within a few ulp; the golden fixtures under tests/golden pin the selected expert sets against the
 * reference's own torch code.
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

#define E_GLOBAL 256
#define TOP_K 8
#define N_GROUP 8
#define GROUP_SIZE 32
#define TOPK_GROUP 4

static float bf16_to_f32(uint16_t b) {
  uint32_t u = (uint32_t)b << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

/* exp(-x): range reduction by ln2 (two-part constant), degree-7 Taylor polynomial, exponent re-insertion. */
static float exp_neg(float x) {
  float z = fminf(fmaxf(-x, -87.0f), 88.0f);
  float t = z * 1.44269504088896341f;
  float n = rintf(t);
  float r = fmaf(n, -0.693145751953125f, z);
  r = fmaf(n, -1.42860682030941723e-6f, r);
  float p = 1.0f / 5040.0f;
  p = fmaf(p, r, 1.0f / 720.0f);
  p = fmaf(p, r, 1.0f / 120.0f);
  p = fmaf(p, r, 1.0f / 24.0f);
  p = fmaf(p, r, 1.0f / 6.0f);
  p = fmaf(p, r, 0.5f);
  p = fmaf(p, r, 1.0f);
  p = fmaf(p, r, 1.0f);
  int32_t bits = ((int32_t)n + 127) << 23;
  float scale;
  memcpy(&scale, &bits, 4);
  return p * scale;
}

float oracle_sigmoid(float x) { return 1.0f / (1.0f + exp_neg(x)); }

/* binding.py:38-61.  topk_idx [T,8] int32 in descending biased score (ties: lower id first); topk_w [T,8] float32. */
void oracle_route(const float* logits, const uint16_t* bias_bf16, int T, float scale_factor, int32_t* topk_idx,
                  float* topk_w) {
  for (int t = 0; t < T; ++t) {
    float s[E_GLOBAL], sb[E_GLOBAL];
    for (int e = 0; e < E_GLOBAL; ++e) {
      s[e] = oracle_sigmoid(logits[(size_t)t * E_GLOBAL + e]);
      sb[e] = s[e] + bf16_to_f32(bias_bf16[e]);
    }
    /* group score = sum of the two largest entries (torch.topk(k=2).sum: duplicates count) */
    float gs[N_GROUP];
    for (int g = 0; g < N_GROUP; ++g) {
      int i1 = 0;
      for (int j = 1; j < GROUP_SIZE; ++j)
        if (sb[g * GROUP_SIZE + j] > sb[g * GROUP_SIZE + i1]) i1 = j;
      int i2 = -1;
      for (int j = 0; j < GROUP_SIZE; ++j) {
        if (j == i1) continue;
        if (i2 < 0 || sb[g * GROUP_SIZE + j] > sb[g * GROUP_SIZE + i2]) i2 = j;
      }
      gs[g] = sb[g * GROUP_SIZE + i1] + sb[g * GROUP_SIZE + i2];
    }
    int keep[N_GROUP] = {0};
    for (int r = 0; r < TOPK_GROUP; ++r) {
      int best = -1;
      for (int g = 0; g < N_GROUP; ++g)
        if (!keep[g] && (best < 0 || gs[g] > gs[best])) best = g;
      keep[best] = 1;
    }
    int taken[E_GLOBAL] = {0};
    float sel_s[TOP_K];
    float sum = 0.0f;
    for (int k = 0; k < TOP_K; ++k) {
      int best = -1;
      for (int e = 0; e < E_GLOBAL; ++e) {
        if (!keep[e / GROUP_SIZE] || taken[e]) continue;
        if (best < 0 || sb[e] > sb[best]) best = e;
      }
      taken[best] = 1;
      topk_idx[(size_t)t * TOP_K + k] = best;
      sel_s[k] = s[best];
      sum = sum + s[best];
    }
    for (int k = 0; k < TOP_K; ++k) topk_w[(size_t)t * TOP_K + k] = sel_s[k] / (sum + 1e-20f) * scale_factor;
  }
}

/* Stable counting sort of the local (token, k) pairs by local expert, padded to block_m rows per expert.
 * Arrays: counts[E], block_offsets[E+1] (block units), sorted_token_ids / sorted_weights [r_max], scatter_map [8T].
 * Rows of sorted_* beyond total_blocks*block_m are left untouched.  Returns total_blocks. */
int oracle_sort(const int32_t* topk_idx, const float* topk_w, int T, int E_local, int local_offset, int block_m,
                int32_t* counts, int32_t* block_offsets, int32_t* sorted_token_ids, float* sorted_weights,
                int32_t* scatter_map) {
  for (int e = 0; e < E_local; ++e) counts[e] = 0;
  for (size_t i = 0; i < (size_t)T * TOP_K; ++i) {
    int le = topk_idx[i] - local_offset;
    if (le >= 0 && le < E_local) counts[le]++;
  }
  int run = 0;
  for (int e = 0; e < E_local; ++e) {
    block_offsets[e] = run;
    run += (counts[e] + block_m - 1) / block_m;
  }
  block_offsets[E_local] = run;
  for (int r = 0; r < run * block_m; ++r) {
    sorted_token_ids[r] = T;
    sorted_weights[r] = 0.0f;
  }
  int32_t fill[E_GLOBAL];
  for (int e = 0; e < E_local; ++e) fill[e] = block_offsets[e] * block_m;
  for (size_t i = 0; i < (size_t)T * TOP_K; ++i) {
    int le = topk_idx[i] - local_offset;
    if (le >= 0 && le < E_local) {
      int d = fill[le]++;
      sorted_token_ids[d] = (int32_t)(i / TOP_K);
      sorted_weights[d] = topk_w[i];
      scatter_map[i] = d;
    } else {
      scatter_map[i] = -1;
    }
  }
  return run;
}
