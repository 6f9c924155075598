/*
 * TEST INFRASTRUCTURE — not part of the product.  Only the tests, the driver's smoke check and bench.py's CPU-baseline
 * legs may load this code; the CUDA library never calls it.
 *
 * CPU restatement of the reference's fp32-dequant expert path, solution/cuda/binding.py:96-185:
 *   dequantise activations (binding.py:74-78) and the hit experts' weights (binding.py:80-83) to float32,
 *   per expert  G = A W13^T (binding.py:166-167), inter = silu(G[:,2048:]) * G[:,:2048] (binding.py:170-175),
 *   O = inter W2^T (binding.py:178-179), out[token] += weight * O (binding.py:182), cast to bfloat16 (binding.py:185).
 * Sums are float32; their order is not that of torch's BLAS, so results agree to float32 rounding, not bit for bit.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define H 7168
#define I 2048
#define TOP_K 8
#define QB 128

static float g_lut[256];
static int g_lut_ready = 0;

/* float8 e4m3fn: 1 sign, 4 exponent (bias 7), 3 mantissa; no infinities; S.1111.111 is NaN. */
static void init_lut(void) {
  if (g_lut_ready) return;
  for (int b = 0; b < 256; ++b) {
    int sign = b >> 7, ex = (b >> 3) & 15, man = b & 7;
    float v;
    if (ex == 15 && man == 7) v = NAN;
    else if (ex == 0) v = ldexpf((float)man, -9);
    else v = ldexpf(1.0f + (float)man / 8.0f, ex - 7);
    g_lut[b] = sign ? -v : v;
  }
  g_lut_ready = 1;
}

float oracle_e4m3_to_f32(uint8_t b) {
  init_lut();
  return g_lut[b];
}

uint16_t oracle_f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40); /* NaN */
  u += 0x7fffu + ((u >> 16) & 1u);                                            /* round to nearest even */
  return (uint16_t)(u >> 16);
}

static float dotf(const float* a, const float* b, int n) {
  float acc = 0.0f;
#pragma omp simd reduction(+ : acc)
  for (int k = 0; k < n; ++k) acc += a[k] * b[k];
  return acc;
}

/*
 * topk_idx/topk_w [T,8] as produced by oracle_route (or by the implementation under test).
 * out_f32 [T,7168] receives the un-rounded sum (may be NULL); out_bf16 [T,7168] the bfloat16 result (may be NULL).
 * Returns the number of local (token, expert) pairs, or -1 when out of memory.
 */
long oracle_forward(const int32_t* topk_idx, const float* topk_w, int T, int E_local, int local_offset,
                    const uint8_t* hs, const float* hs_scale /* [56,T] */, const uint8_t* w13,
                    const float* w13s /* [E,32,56] */, const uint8_t* w2, const float* w2s /* [E,56,16] */,
                    float* out_f32, uint16_t* out_bf16, int num_threads) {
  init_lut();
#ifdef _OPENMP
  if (num_threads > 0) omp_set_num_threads(num_threads);
#else
  (void)num_threads;
#endif
  size_t TH = (size_t)T * H;
  float* acc = (float*)calloc(TH ? TH : 1, sizeof(float));
  int32_t* tok = (int32_t*)malloc(sizeof(int32_t) * (size_t)(T ? T : 1));
  float* wt = (float*)malloc(sizeof(float) * (size_t)(T ? T : 1));
  if (!acc || !tok || !wt) { free(acc); free(tok); free(wt); return -1; }
  long pairs = 0;
  for (int e = 0; e < E_local; ++e) {
    int cnt = 0;
    for (int t = 0; t < T; ++t)
      for (int k = 0; k < TOP_K; ++k)
        if (topk_idx[(size_t)t * TOP_K + k] - local_offset == e) { tok[cnt] = t; wt[cnt] = topk_w[(size_t)t * TOP_K + k]; ++cnt; }
    if (cnt == 0) continue;
    pairs += cnt;
    float* A = (float*)malloc(sizeof(float) * (size_t)cnt * H);
    float* G = (float*)malloc(sizeof(float) * (size_t)cnt * 2 * I);
    float* X = (float*)malloc(sizeof(float) * (size_t)cnt * I);
    if (!A || !G || !X) { free(A); free(G); free(X); free(acc); free(tok); free(wt); return -1; }
    for (int r = 0; r < cnt; ++r)
      for (int k = 0; k < H; ++k)
        A[(size_t)r * H + k] = g_lut[hs[(size_t)tok[r] * H + k]] * hs_scale[(size_t)(k / QB) * T + tok[r]];
    const uint8_t* W13 = w13 + (size_t)e * 2 * I * H;
    const float* S13 = w13s + (size_t)e * (2 * I / QB) * (H / QB);
#pragma omp parallel
    {
      float* wrow = (float*)malloc(sizeof(float) * H);
#pragma omp for schedule(static)
      for (int n = 0; n < 2 * I; ++n) {
        for (int k = 0; k < H; ++k) wrow[k] = g_lut[W13[(size_t)n * H + k]] * S13[(n / QB) * (H / QB) + k / QB];
        for (int r = 0; r < cnt; ++r) G[(size_t)r * 2 * I + n] = dotf(A + (size_t)r * H, wrow, H);
      }
      free(wrow);
    }
    for (int r = 0; r < cnt; ++r)
      for (int n = 0; n < I; ++n) {
        float gate = G[(size_t)r * 2 * I + I + n], up = G[(size_t)r * 2 * I + n];
        X[(size_t)r * I + n] = gate / (1.0f + expf(-gate)) * up;
      }
    const uint8_t* W2 = w2 + (size_t)e * H * I;
    const float* S2 = w2s + (size_t)e * (H / QB) * (I / QB);
#pragma omp parallel
    {
      float* wrow = (float*)malloc(sizeof(float) * I);
#pragma omp for schedule(static)
      for (int n = 0; n < H; ++n) {
        for (int k = 0; k < I; ++k) wrow[k] = g_lut[W2[(size_t)n * I + k]] * S2[(n / QB) * (I / QB) + k / QB];
        for (int r = 0; r < cnt; ++r) acc[(size_t)tok[r] * H + n] += wt[r] * dotf(X + (size_t)r * I, wrow, I);
      }
      free(wrow);
    }
    free(A); free(G); free(X);
  }
  if (out_f32) memcpy(out_f32, acc, sizeof(float) * TH);
  if (out_bf16)
    for (size_t i = 0; i < TH; ++i) out_bf16[i] = oracle_f32_to_bf16(acc[i]);
  free(acc); free(tok); free(wt);
  return pairs;
}
