// Grouped FP8 GEMMs for batches in which an expert sees few tokens: the operands of gemm.cu swapped.
//
// With a few rows per expert the 128-token x 256-column tiles of gemm.cu spend a full 128 x 256 x 128 MMA and a full
// 128 x 256 promotion on every 128-K chunk although almost all rows are padding, and the chunk rate of that chain
// (not HBM) sets the time of a tile.  Here the WEIGHT rows take the M side of the instruction and the tokens the N side:
//
//   D[n, t] = sum_k W[n, k] * X[t, k]      M = 128 weight rows (TMEM lanes), N = 16 / 32 / 64 tokens (TMEM columns)
//
// so MMA time and promotion work shrink with the number of tokens and a tile is bound by streaming its 256 weight rows
// from HBM.  A tile = (expert, sub-block of at most 64 sorted rows, n-tile); it covers 256 weight rows as two M = 128
// halves that accumulate into columns [0, N) and [128, 128 + N) of a TMEM stage:
//   GEMM1: half 0 = W1 rows nt*128.. ("up"), half 1 = W3 rows I + nt*128.. ("gate"): one thread owns up and gate of the
//          same (n, t), so SwiGLU needs no exchange, and the tile spans exactly one 128-wide quantisation block;
//   GEMM2: halves = W2 rows nt*256.. and nt*256 + 128..; two MMAs per K step (both terms of the intermediate).
// The per-token scale now varies along the columns, so each promotion FMA multiplies by (token scale x weight scale).
// An expert with more than 64 rows is split into several tiles that re-read its weights (adjacent tile numbers, so they
// run together and share L2); the host picks this kernel only for batches where that is rare.
//
// Whole tiles are dealt round-robin while a full round of them is left; the tiles of the last, incomplete round are
// dealt in 128-K CHUNKS instead: CTA c of G takes the contiguous run [U c / G, U (c + 1) / G) of their U (tile, chunk)
// units, so that round keeps every SM streaming for the same time (dealt whole, 176 tiles on 148 SMs take two full
// rounds).  A tile whose chunks are shared by several CTAs is finished by whichever of them completes last: each writes
// its promoted fp32 partial sums to its own slot of a scratch array (at most two such tiles per CTA: the first and the
// last of its run), takes a ticket from the tile's counter, and the CTA that draws the last ticket adds the partials in
// chunk order (its own included, so the sum does not depend on who came last) and runs the epilogue.  Nobody waits for
// another CTA.  The counter returns to zero for the next launch.
//
// The weight rows are copied by two loader warps with 16-byte cp.async (the token tiles stay on TMA).  Measured, either
// way of loading streams the weights at 4.5 - 5.3 TB/s (a plain read sweep reaches 5.9 - 6.0 TB/s on the same GPU), so
// the choice is not about speed: the cp.async path keeps the TMA unit free for the token tiles and needs no tensor map
// over the weights.  -DSKINNY_W_VIA_TMA=1 builds the TMA variant.
//
// Roles, pipeline, bounded waits and teardown are those of gemm.cu: 8 promotion warps (warp w: TMEM lanes 32*(w%4)..,
// token columns of half w/4), one TMA thread, one MMA thread, two TMEM stages, `setmaxnreg` 224 / 56.
// A tile that one CTA computes alone gives bit for bit what gemm.cu gives (same products, same order); a shared tile
// adds the same products in a different association (last-bit differences in fp32).
#include <cuda.h>

#include "common.cuh"
#include "gemm_common.cuh"

namespace b200moe {
namespace skinny {

constexpr int SUB_M = 64;                    // tokens per tile at most
constexpr int W_HALF_BYTES = 128 * 128;      // 128 weight rows x 128 K bytes
constexpr int W_BYTES = 2 * W_HALF_BYTES;
constexpr int X_BOX_ROWS = 32;               // token rows per TMA box
constexpr int X_BOX_BYTES = X_BOX_ROWS * 128;
constexpr int X_TILE_BYTES = SUB_M * 128;
constexpr int ACC_COLS = 256;                // TMEM columns per stage: half 0 at +0, half 1 at +128
constexpr int NUM_PROMO_WARPS = 8;
constexpr int PRODUCER_WARP = 8;
constexpr int MMA_WARP = 9;
constexpr int LOADER_WARP0 = 10;             // warps 10 and 11 copy the weight rows
constexpr int NUM_LOADER_WARPS = 2;
constexpr int THREADS = 384;
#ifndef SKINNY_W_VIA_TMA
#define SKINNY_W_VIA_TMA 0                   // 1: weight slabs by TMA like the token tiles (measured slower, see above)
#endif
constexpr int SLOT_FLOATS = 2 * SUB_M * 128;   // one tile's partial sums: [half][token column][weight row]

template <int MODE>
struct Cfg {
  static constexpr int X_TILES = (MODE == 1) ? 1 : 2;
  static constexpr int STAGE_BYTES = W_BYTES + X_TILES * X_TILE_BYTES;  // 40 KB / 48 KB
  static constexpr int STAGES = (MODE == 1) ? 5 : 4;
  static constexpr int K_CHUNKS = (MODE == 1) ? H_BLOCKS : I_BLOCKS;
  static constexpr int N_TILES = (MODE == 1) ? (I / 128) : (H / 256);   // 16, 28
};

struct __align__(8) Aux {
  uint64_t full[5];
  uint64_t empty[5];
  uint64_t tfull[2];
  uint64_t tempty[2];
  uint64_t xbar[2];
  uint64_t pbar[2];        // partial-tile hand-shake: [0] all promotion warps stored, [1] ticket drawn
  uint32_t tmem_base;
  int abort_flag;
  int last_flag;           // this CTA drew the last ticket of the tile it just stored
  int off[E_GLOBAL + 1];   // block_offsets (128-row blocks)
  int grp[E_GLOBAL + 1];   // sub-blocks before expert e
  int cnt[E_GLOBAL];
  float amax[2][4][SUB_M];
};

template <int MODE>
constexpr size_t smem_bytes() {
  return 1024 + static_cast<size_t>(Cfg<MODE>::STAGES) * Cfg<MODE>::STAGE_BYTES + sizeof(Aux);
}

struct Tile {
  int e, nt, row0, n_tok, nb;   // nb = 16 / 32 / 64: the N of the MMAs
};

// Tiles are numbered expert-major, then n-tile, then sub-block, so the tiles that stream the same weight rows are
// neighbours.
__device__ __forceinline__ Tile decode_tile(int tile, const Aux* aux, int E, int NT) {
  int lo = 0, hi = E - 1;
  while (lo < hi) {
    int mid = (lo + hi + 1) >> 1;
    if (aux->grp[mid] * NT <= tile) lo = mid; else hi = mid - 1;
  }
  Tile t;
  t.e = lo;
  const int local = tile - aux->grp[lo] * NT;
  const int groups = aux->grp[lo + 1] - aux->grp[lo];
  t.nt = local / groups;
  const int sub = local - t.nt * groups;
  t.row0 = aux->off[lo] * BLOCK_M + sub * SUB_M;
  const int left = aux->cnt[lo] - sub * SUB_M;
  t.n_tok = left < SUB_M ? left : SUB_M;
  t.nb = t.n_tok <= 16 ? 16 : (t.n_tok <= 32 ? 32 : 64);
  return t;
}

template <int NC>
__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, uint32_t (&r)[NC]) {
  if constexpr (NC == 8) tmem_ld8(taddr, r);
  else if constexpr (NC == 16) tmem_ld16(taddr, r);
  else tmem_ld32(taddr, r);
}

__device__ __forceinline__ uint32_t e4m3_of(float x) {
  return static_cast<uint32_t>(__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3));
}
__device__ __forceinline__ float e4m3_to_float(uint32_t b) {
  __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(b), __NV_E4M3);
  return __half2float(*reinterpret_cast<__half*>(&h));
}

// Per-thread state of a promotion warp that lives across work items.
struct PromoState {
  int acc = 0;
  uint32_t acc_phase = 0;
  int epi_iter = 0;    // epilogues run (selects the amax exchange buffer and its barrier phase)
  int part_iter = 0;   // partial tiles stored (phase of the hand-shake barriers)
};

// Promotion (and, when this CTA finishes the tile, epilogue) of one work item for a thread that owns NC token columns
// (NC = nb / 2) of weight row 32q + lane in both halves.  Returns false after a wait timed out.
template <int MODE, int NC>
__device__ __forceinline__ bool run_item(const GemmArgs& args, Aux* aux, const Tile& ti, const Item& it, const Deal& deal,
                                         uint32_t tmem_base, int warp, int lane, PromoState& ps,
                                         volatile int* abort_flag) {
  using C = Cfg<MODE>;
  const int q = warp & 3;    // TMEM lane quarter this warp may read = weight rows 32q..32q+31 of each half
  const int ch = warp >> 2;  // which half of the tile's token columns
  const int col0 = ch * NC;
  const float* xs_ptr = args.row_scale + ti.row0 + col0;
  const float* w0_ptr;
  const float* w1_ptr;
  if (MODE == 1) {
    w0_ptr = args.w_scale + (static_cast<size_t>(ti.e) * 32 + ti.nt) * H_BLOCKS;
    w1_ptr = args.w_scale + (static_cast<size_t>(ti.e) * 32 + 16 + ti.nt) * H_BLOCKS;
  } else {
    w0_ptr = args.w_scale + (static_cast<size_t>(ti.e) * H_BLOCKS + ti.nt * 2) * I_BLOCKS;
    w1_ptr = w0_ptr + I_BLOCKS;
  }
  float a0[NC], a1[NC];   // half 0 / half 1 accumulators (GEMM1: up / gate)
#pragma unroll
  for (int j = 0; j < NC; ++j) a0[j] = a1[j] = 0.f;

  float4 xs_n[NC / 4];
  {
    const float4* nx = reinterpret_cast<const float4*>(xs_ptr + static_cast<size_t>(it.kb0) * args.R_max);
#pragma unroll
    for (int v = 0; v < NC / 4; ++v) xs_n[v] = __ldg(nx + v);
  }
  float w0_n = __ldg(w0_ptr + it.kb0), w1_n = __ldg(w1_ptr + it.kb0);

  for (int kb = it.kb0; kb < it.kb1; ++kb) {
    float xs[NC];
#pragma unroll
    for (int v = 0; v < NC / 4; ++v) {
      xs[4 * v] = xs_n[v].x; xs[4 * v + 1] = xs_n[v].y; xs[4 * v + 2] = xs_n[v].z; xs[4 * v + 3] = xs_n[v].w;
    }
    const float w0 = w0_n, w1 = w1_n;
    if (kb + 1 < it.kb1) {
      const float4* nx = reinterpret_cast<const float4*>(xs_ptr + static_cast<size_t>(kb + 1) * args.R_max);
#pragma unroll
      for (int v = 0; v < NC / 4; ++v) xs_n[v] = __ldg(nx + v);
      w0_n = __ldg(w0_ptr + kb + 1);
      w1_n = __ldg(w1_ptr + kb + 1);
    }
    if (!mbar_wait_all(smem_u32(&aux->tfull[ps.acc]), ps.acc_phase, abort_flag, args.status, 4, kb)) return false;
    tc_fence_after();
    const uint32_t taddr =
        tmem_base + static_cast<uint32_t>(ps.acc * ACC_COLS + col0) + (static_cast<uint32_t>(q * 32) << 16);
    uint32_t t0[NC], t1[NC];
    tmem_ld_cols<NC>(taddr, t0);
    tmem_ld_cols<NC>(taddr + 128, t1);
    tc_wait_ld();
    // this warp's reads of the stage are complete: hand it back to the MMA issuer
    tc_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive_relaxed(smem_u32(&aux->tempty[ps.acc]));
#pragma unroll
    for (int j = 0; j < NC; ++j) {
      a0[j] = __fmaf_rn(__uint_as_float(t0[j]), xs[j] * w0, a0[j]);
      a1[j] = __fmaf_rn(__uint_as_float(t1[j]), xs[j] * w1, a1[j]);
    }
    ps.acc ^= 1;
    if (ps.acc == 0) ps.acc_phase ^= 1u;
  }

  if (it.kb0 != 0 || it.kb1 != C::K_CHUNKS) {
    // ---- the tile is shared with other CTAs: store the partial sums, draw a ticket, finish the tile if it is the last
    const int lt = it.tile - deal.first_tile;   // number among the left-over tiles
    const long long t_lo = static_cast<long long>(lt) * C::K_CHUNKS;
    const int c_first = deal.owner(t_lo), c_last = deal.owner(t_lo + C::K_CHUNKS - 1);
    const int my_slot = (deal.begin(blockIdx.x) / C::K_CHUNKS == lt) ? 0 : 1;
    float* mine = args.partial + static_cast<size_t>(blockIdx.x * 2 + my_slot) * SLOT_FLOATS + q * 32 + lane;
#pragma unroll
    for (int j = 0; j < NC; ++j) {
      __stcg(mine + (col0 + j) * 128, a0[j]);
      __stcg(mine + (SUB_M + col0 + j) * 128, a1[j]);
    }
    __threadfence();
    __syncwarp();
    const uint32_t par = static_cast<uint32_t>(ps.part_iter & 1);
    ++ps.part_iter;
    if (lane == 0) mbar_arrive(smem_u32(&aux->pbar[0]));
    if (warp == 0 && lane == 0) {
      if (mbar_wait(smem_u32(&aux->pbar[0]), par, abort_flag, args.status, 6, it.tile)) {
        __threadfence();
        const int old = atomicAdd(args.tile_ctr + it.tile, 1);
        const int last = (old == c_last - c_first) ? 1 : 0;
        if (last) args.tile_ctr[it.tile] = 0;   // every sharer has drawn: ready for the next launch
        __threadfence();
        aux->last_flag = last;
        mbar_arrive(smem_u32(&aux->pbar[1]));
      }
    }
    __syncwarp();
    if (!mbar_wait_all(smem_u32(&aux->pbar[1]), par, abort_flag, args.status, 7, it.tile)) return false;
    if (!aux->last_flag) return true;
    __threadfence();
    for (int c = c_first; c <= c_last; ++c) {
      const int slot = (deal.begin(c) / C::K_CHUNKS == lt) ? 0 : 1;
      const float* src = args.partial + static_cast<size_t>(c * 2 + slot) * SLOT_FLOATS + q * 32 + lane;
#pragma unroll
      for (int j = 0; j < NC; ++j) {
        const float v0 = __ldcg(src + (col0 + j) * 128);
        const float v1 = __ldcg(src + (SUB_M + col0 + j) * 128);
        a0[j] = (c == c_first) ? v0 : a0[j] + v0;
        a1[j] = (c == c_first) ? v1 : a1[j] + v1;
      }
    }
  }

  const int n_valid = ti.n_tok - col0;   // this thread's columns j < n_valid are real tokens
  if (MODE == 1) {
    // a0 <- silu(gate) * up; per-token maximum over the tile's 128 weight rows = 4 warps x 32 lanes
    const int buf = ps.epi_iter & 1;
    const uint32_t xpar = static_cast<uint32_t>((ps.epi_iter >> 1) & 1);
    ++ps.epi_iter;
    float* ex = &aux->amax[buf][0][0];
#pragma unroll
    for (int j = 0; j < NC; ++j) {
      a0[j] = silu_mul(a1[j], a0[j]);
      const uint32_t m = __reduce_max_sync(0xffffffffu, __float_as_uint(fabsf(a0[j])));
      if (lane == j) ex[q * SUB_M + col0 + j] = __uint_as_float(m);
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(smem_u32(&aux->xbar[buf]));
    if (!mbar_wait_all(smem_u32(&aux->xbar[buf]), xpar, abort_flag, args.status, 5, it.tile)) return false;
    uint8_t* q1 = args.inter_q + static_cast<size_t>(ti.row0 + col0) * I + ti.nt * 128 + q * 32 + lane;
    uint8_t* q2 = q1 + static_cast<size_t>(args.R_max) * I;
#pragma unroll
    for (int j = 0; j < NC; ++j) {
      const int c = col0 + j;
      const float amax = fmaxf(fmaxf(ex[c], ex[SUB_M + c]), fmaxf(ex[2 * SUB_M + c], ex[3 * SUB_M + c]));
      const float s = fmaxf(amax, 1e-20f) * (1.0f / 448.0f);
      const float inv = 1.0f / s;
      const uint32_t b1 = e4m3_of(a0[j] * inv);
      const uint32_t b2 = e4m3_of((a0[j] - e4m3_to_float(b1) * s) * inv);
      if (j < n_valid) {
        q1[static_cast<size_t>(j) * I] = static_cast<uint8_t>(b1);
        q2[static_cast<size_t>(j) * I] = static_cast<uint8_t>(b2);
        if (q == 0 && lane == j) args.inter_scale[static_cast<size_t>(ti.nt) * args.R_max + ti.row0 + c] = s;
      }
    }
  } else {
    // lanes hold consecutive output columns: every store instruction of a warp writes 128 contiguous bytes of one row
    float* o = args.expert_out + static_cast<size_t>(ti.row0 + col0) * H + ti.nt * 256 + q * 32 + lane;
#pragma unroll
    for (int j = 0; j < NC; ++j) {
      if (j < n_valid) {
        o[static_cast<size_t>(j) * H] = a0[j];
        o[static_cast<size_t>(j) * H + 128] = a1[j];
      }
    }
  }
  return true;
}

template <int MODE>
__global__ void __launch_bounds__(THREADS, 1)
k_grouped_gemm_skinny(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW,
                      const GemmArgs args) {
  using C = Cfg<MODE>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t tiles_addr = (raw_addr + 1023u) & ~1023u;
  uint8_t* tiles_ptr = smem_raw + (tiles_addr - raw_addr);
  Aux* aux = reinterpret_cast<Aux*>(tiles_ptr + C::STAGES * C::STAGE_BYTES);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int E = args.E_local;
  constexpr int NT = C::N_TILES;

  // Early weights (args.early_weights, set by b200moe_forward): the expert weights depend on no earlier kernel, and the
  // sort metadata that names the tiles is complete before this kernel can start at all — GEMM1 follows k_gather, which
  // releases its dependents only after it has seen the scatter finish, and GEMM2 follows GEMM1, which started under
  // that same condition.  So the metadata is read and the weight loaders start BEFORE the dependency wait; only the
  // roles that touch what the predecessor writes (token tiles, scales, tickets, partial sums) wait for it.  The first
  // weight stages are then in flight while the predecessor (the row gather, or the slowest GEMM1 CTAs) still runs.
  const bool early = args.early_weights != 0;
  if (MODE == 2 || early) pdl_launch_dependents();
  if (threadIdx.x == 0) aux->abort_flag = 0;
  if (warp == PRODUCER_WARP && lane == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(smem_u32(&aux->full[s]), SKINNY_W_VIA_TMA ? 1 : 1 + NUM_LOADER_WARPS);
      mbar_init(smem_u32(&aux->empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&aux->tfull[a]), 1);
      mbar_init(smem_u32(&aux->tempty[a]), NUM_PROMO_WARPS);
      mbar_init(smem_u32(&aux->xbar[a]), NUM_PROMO_WARPS);
    }
    mbar_init(smem_u32(&aux->pbar[0]), NUM_PROMO_WARPS);
    mbar_init(smem_u32(&aux->pbar[1]), 1);
    fence_mbar_init();
    tma_prefetch_desc(&tmX);
    tma_prefetch_desc(&tmW);
  }
  if (warp == MMA_WARP) {
    tmem_alloc(smem_u32(&aux->tmem_base), 512);
    tmem_relinquish();
  }
  // CTA-local set-up above may overlap the tail of the previous kernel; what that kernel wrote is read from here on
  if (!early) pdl_wait();
  if (MODE == 1 && !early) pdl_launch_dependents();
  for (int i = threadIdx.x; i <= E; i += THREADS) aux->off[i] = __ldg(args.block_offsets + i);
  for (int i = threadIdx.x; i < E; i += THREADS) aux->cnt[i] = __ldg(args.counts + i);
  __syncthreads();
  if (warp == 0) {
    // sub-blocks per expert = ceil(count / 64), exclusive prefix over experts; lane handles experts [8*lane, 8*lane+8)
    int g[8], local = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int e = lane * 8 + i;
      g[i] = (e < E) ? (aux->cnt[e] + SUB_M - 1) / SUB_M : 0;
      local += g[i];
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
      if (e < E) aux->grp[e] = run;
      run += g[i];
    }
    if (lane == 31) aux->grp[E] = incl;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  const uint32_t tmem_base = aux->tmem_base;
  const int total_tiles = aux->grp[E] * NT;
  volatile int* abort_flag = &aux->abort_flag;
  const Deal deal = make_deal(total_tiles, C::K_CHUNKS, static_cast<int>(gridDim.x));
  const long long u_begin = deal.begin(blockIdx.x), u_end = deal.begin(blockIdx.x + 1);
  // This CTA's work as one sequence of chunk positions: its whole tiles, then its run of left-over units.
  const long long v_whole = static_cast<long long>(deal.rounds) * C::K_CHUNKS;
  const long long v_end = v_whole + (u_end - u_begin);
  auto item_at = [&](long long v) {
    return deal_item(deal, C::K_CHUNKS, static_cast<int>(blockIdx.x), v, v_whole, u_begin, u_end);
  };

  if (warp >= NUM_PROMO_WARPS) {
    setmaxnreg_dec<56>();   // the loader warps keep 32 row addresses in flight
    if (warp == PRODUCER_WARP) {
      // ------------------------------------------------------------------ TMA producer (one thread)
      if (lane == 0) {
        if (early) pdl_wait();   // the token tiles are GEMM1's output
        int stage = 0;
        uint32_t phase = 0;
        long long issued = 0;
        bool ok = true;
        for (long long u = 0; ok && u < v_end;) {
          const Item it = item_at(u);
          u += it.kb1 - it.kb0;
          const Tile ti = decode_tile(it.tile, aux, E, NT);
          const int x_boxes = ti.nb > X_BOX_ROWS ? 2 : 1;
          const uint32_t bytes = (SKINNY_W_VIA_TMA ? W_BYTES : 0) + C::X_TILES * x_boxes * X_BOX_BYTES;
          for (int kb = it.kb0; kb < it.kb1; ++kb) {
            ok = mbar_wait(smem_u32(&aux->empty[stage]), phase ^ 1u, abort_flag, args.status, 1, kb);
            if (!ok) break;
            const uint32_t sW = tiles_addr + stage * C::STAGE_BYTES;
            const uint32_t sX = sW + W_BYTES;
            const uint32_t full = smem_u32(&aux->full[stage]);
            mbar_arrive_expect_tx(full, bytes);
#if SKINNY_W_VIA_TMA
            if (MODE == 1) {
              tma_load_2d(sW, &tmW, full, kb * 128, ti.e * (2 * I) + ti.nt * 128);
              tma_load_2d(sW + W_HALF_BYTES, &tmW, full, kb * 128, ti.e * (2 * I) + I + ti.nt * 128);
            } else {
              tma_load_2d(sW, &tmW, full, kb * 128, ti.e * H + ti.nt * 256);   // one 256-row box
            }
#endif
            for (int b = 0; b < x_boxes; ++b) {
              tma_load_2d(sX + b * X_BOX_BYTES, &tmX, full, kb * 128, ti.row0 + b * X_BOX_ROWS);
              if (MODE == 2)
                tma_load_2d(sX + X_TILE_BYTES + b * X_BOX_BYTES, &tmX, full, kb * 128,
                            args.R_max + ti.row0 + b * X_BOX_ROWS);
            }
            ++issued;
            if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
          }
        }
        if (!ok) {
          // Drain: every load already issued completes on its own; wait (bounded) so none lands after the CTA exits.
          for (int s = 0; s < C::STAGES; ++s) {
            long long n_s = issued / C::STAGES + ((issued % C::STAGES) > s ? 1 : 0);
            if (n_s == 0) continue;
            uint32_t par = static_cast<uint32_t>((n_s - 1) & 1);
            for (int spin = 0; spin < DRAIN_POLLS; ++spin)
              if (mbar_try_wait(smem_u32(&aux->full[s]), par)) break;
          }
        }
      }
      __syncwarp();
    } else if (warp == MMA_WARP) {
      // ------------------------------------------------------------------ MMA issuer (one thread)
      if (lane == 0) {
        int stage = 0, acc = 0;
        uint32_t phase = 0, acc_phase = 0;
        bool ok = true;
        for (long long u = 0; ok && u < v_end;) {
          const Item it = item_at(u);
          u += it.kb1 - it.kb0;
          const Tile ti = decode_tile(it.tile, aux, E, NT);
          const uint32_t idesc = umma_idesc_e4m3(128, ti.nb);
          for (int kb = it.kb0; kb < it.kb1; ++kb) {
            ok = mbar_wait(smem_u32(&aux->tempty[acc]), acc_phase ^ 1u, abort_flag, args.status, 2, kb);
            if (!ok) break;
            ok = mbar_wait(smem_u32(&aux->full[stage]), phase, abort_flag, args.status, 3, kb);
            if (!ok) break;
            tc_fence_after();
            const uint32_t sW = tiles_addr + stage * C::STAGE_BYTES;
            const uint64_t x0 = umma_desc_sw128(sW + W_BYTES);
#pragma unroll
            for (int half = 0; half < 2; ++half) {
              const uint32_t d = tmem_base + static_cast<uint32_t>(acc * ACC_COLS + half * 128);
              const uint64_t w = umma_desc_sw128(sW + half * W_HALF_BYTES);
#pragma unroll
              for (int k4 = 0; k4 < 4; ++k4) tc_mma_f8(d, w + 2 * k4, x0 + 2 * k4, idesc, k4 > 0 ? 1u : 0u);
              if (MODE == 2) {
                const uint64_t x1 = umma_desc_sw128(sW + W_BYTES + X_TILE_BYTES);
#pragma unroll
                for (int k4 = 0; k4 < 4; ++k4) tc_mma_f8(d, w + 2 * k4, x1 + 2 * k4, idesc, 1u);
              }
            }
            tc_commit(smem_u32(&aux->empty[stage]));
            tc_commit(smem_u32(&aux->tfull[acc]));
            if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
            acc ^= 1;
            if (acc == 0) acc_phase ^= 1u;
          }
        }
      }
      __syncwarp();
    }
#if !SKINNY_W_VIA_TMA
    else {
      // ------------------------------------------------------------------ weight loaders (warps 10-11, 64 threads)
      // Thread t copies 16-byte unit t % 8 of rows t / 8 + 8 i (i = 0..31) of the 256-row slab: 8 lanes cover one
      // 128-byte row piece, and the unit lands where the 128-byte swizzle of the MMA descriptors expects it
      // (unit ^ (row % 8); row % 8 = t / 8 for every row of the thread).  A chunk is signalled LAG chunks after it was
      // issued: by then its group has completed, the thread fences its writes towards the async proxy, and one lane
      // per warp arrives on the chunk's barrier.
      constexpr int LAG = C::STAGES - 2;
      constexpr int PITCH = (MODE == 1) ? H : I;
      const int lt = threadIdx.x - LOADER_WARP0 * 32;
      const int u = lt & 7, r8 = lt >> 3;
      const uint32_t dst_thread = static_cast<uint32_t>(r8 * 128 + ((u ^ r8) << 4));
      int stage = 0, arr_stage = 0;
      uint32_t phase = 0;
      int pending = 0;   // chunks issued and not yet signalled
      bool ok = true;
      for (long long uu = 0; ok && uu < v_end;) {
        const Item it = item_at(uu);
        uu += it.kb1 - it.kb0;
        const Tile ti = decode_tile(it.tile, aux, E, NT);
        const uint8_t* src0;
        const uint8_t* src1;
        if (MODE == 1) {
          src0 = args.weights + (static_cast<size_t>(ti.e) * (2 * I) + ti.nt * 128 + r8) * PITCH + u * 16;
          src1 = src0 + static_cast<size_t>(I) * PITCH;
        } else {
          src0 = args.weights + (static_cast<size_t>(ti.e) * H + ti.nt * 256 + r8) * PITCH + u * 16;
          src1 = src0 + static_cast<size_t>(128) * PITCH;
        }
        for (int kb = it.kb0; kb < it.kb1; ++kb) {
          ok = mbar_wait_all(smem_u32(&aux->empty[stage]), phase ^ 1u, abort_flag, args.status, 8, kb);
          if (!ok) break;
          const uint32_t dst = tiles_addr + stage * C::STAGE_BYTES + dst_thread;
          const uint8_t* s0 = src0 + kb * 128;
          const uint8_t* s1 = src1 + kb * 128;
#pragma unroll
          for (int i = 0; i < 16; ++i) cp_async16(dst + i * 1024, s0 + static_cast<size_t>(i) * 8 * PITCH);
#pragma unroll
          for (int i = 0; i < 16; ++i)
            cp_async16(dst + W_HALF_BYTES + i * 1024, s1 + static_cast<size_t>(i) * 8 * PITCH);
          cp_async_commit();
          if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
          if (++pending > LAG) {
            cp_async_wait_group<LAG>();
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&aux->full[arr_stage]));
            if (++arr_stage == C::STAGES) arr_stage = 0;
            --pending;
          }
        }
      }
      // drain: nothing of this thread may still be in flight when the CTA exits; signal what is left
      cp_async_wait_group<0>();
      fence_proxy_async_smem();
      __syncwarp();
      if (ok) {
        for (; pending > 0; --pending) {
          if (lane == 0) mbar_arrive(smem_u32(&aux->full[arr_stage]));
          if (++arr_stage == C::STAGES) arr_stage = 0;
        }
      }
    }
#endif
  } else {
    setmaxnreg_inc<224>();
    if (early) pdl_wait();   // scales, tickets and partial-sum slots are GEMM1's
    // ------------------------------------------------------------------ promotion + epilogue (8 warps)
    PromoState ps;
    bool ok = true;
    for (long long u = 0; ok && u < v_end;) {
      const Item it = item_at(u);
      u += it.kb1 - it.kb0;
      const Tile ti = decode_tile(it.tile, aux, E, NT);
      if (ti.nb == 16)
        ok = run_item<MODE, 8>(args, aux, ti, it, deal, tmem_base, warp, lane, ps, abort_flag);
      else if (ti.nb == 32)
        ok = run_item<MODE, 16>(args, aux, ti, it, deal, tmem_base, warp, lane, ps, abort_flag);
      else
        ok = run_item<MODE, 32>(args, aux, ti, it, deal, tmem_base, warp, lane, ps, abort_flag);
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (warp == MMA_WARP) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <int MODE>
static int launch(const b200moe_problem* p, const b200moe_workspace* ws, int num_sms, cudaStream_t st, bool early) {
  if (p->T == 0) return B200MOE_OK;
  static bool attr_set[64] = {};
  int dev = 0;
  B200MOE_CUDA_TRY(cudaGetDevice(&dev));
  constexpr size_t smem = smem_bytes<MODE>();
  if (dev < 64 && !attr_set[dev]) {
    B200MOE_CUDA_TRY(cudaFuncSetAttribute(k_grouped_gemm_skinny<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          static_cast<int>(smem)));
    attr_set[dev] = true;
  }
  CUtensorMap tmX, tmW;
  int rc;
  GemmArgs a;
  a.block_offsets = ws->block_offsets;
  a.counts = ws->counts;
  a.inter_q = ws->inter_q;
  a.inter_scale = ws->inter_scale;
  a.expert_out = ws->expert_out;
  a.status = ws->status;
  a.E_local = p->E_local;
  a.R_max = ws->R_max;
  a.tile_ctr = ws->gemm_tile_ctr;
  a.partial = ws->gemm_partial;
  a.early_weights = early ? 1 : 0;
  a.out_half = 0;
  a.weights = static_cast<const uint8_t*>(MODE == 1 ? p->gemm1_weights : p->gemm2_weights);
  if (!a.tile_ctr || !a.partial) return B200MOE_EWORKSPACE;
  if (MODE == 1) {
    if ((rc = make_map_u8(&tmX, ws->a_sorted, static_cast<uint64_t>(ws->R_max), H, X_BOX_ROWS))) return rc;
    if ((rc = make_map_u8(&tmW, p->gemm1_weights, static_cast<uint64_t>(p->E_local) * 2 * I, H, 128))) return rc;
    a.row_scale = ws->a_scale_sorted;
    a.w_scale = p->gemm1_weights_scale;
  } else {
    if ((rc = make_map_u8(&tmX, ws->inter_q, static_cast<uint64_t>(ws->R_max) * 2, I, X_BOX_ROWS))) return rc;
    if ((rc = make_map_u8(&tmW, p->gemm2_weights, static_cast<uint64_t>(p->E_local) * H, I, 256))) return rc;
    a.row_scale = ws->inter_scale;
    a.w_scale = p->gemm2_weights_scale;
  }
  const int grid = num_sms < B200MOE_GEMM_MAX_CTAS ? num_sms : B200MOE_GEMM_MAX_CTAS;   // one scratch slot pair per CTA
  B200MOE_CUDA_TRY(launch_pdl(k_grouped_gemm_skinny<MODE>, dim3(grid), dim3(THREADS), smem, st, tmX, tmW, a));
  return B200MOE_OK;
}

}  // namespace skinny

// behind_gather: the launch directly follows launch_gather on the same stream and workspace
int launch_gemm1_skinny(const b200moe_problem* p, const b200moe_workspace* ws, int num_sms, cudaStream_t st,
                        bool behind_gather) {
  return skinny::launch<1>(p, ws, num_sms, st, behind_gather);
}
// behind_gemm1: the launch directly follows launch_gemm1_skinny on the same stream and workspace
int launch_gemm2_skinny(const b200moe_problem* p, const b200moe_workspace* ws, int num_sms, cudaStream_t st,
                        bool behind_gemm1) {
  return skinny::launch<2>(p, ws, num_sms, st, behind_gemm1);
}

}  // namespace b200moe
