// Persistent grouped FP8 GEMMs on the 5th-generation tensor core (tcgen05), sm_100a.
//
//   MODE 1  GEMM1 + SwiGLU:  G = A_sorted[R,7168] x W13[e]^T, promoted with a_scale[row,kb] * w13_scale[e,nb,kb] every
//           128 K; inter = silu(G[:, 2048+n]) * G[:, n]; inter is re-quantised per row per 128 columns into TWO e4m3
//           terms with one shared scale (value + residual), so GEMM2 stays on the FP8 pipe at ~bf16 accuracy.
//           Reference: _fused_moe_gemm1_swiglu_kernel (solution/python/pure_triton_impl.py:886-1046), oracle math
//           solution/cuda/binding.py:166-175.
//   MODE 2  GEMM2:  O = inter[R,2048] x W2[e]^T, both e4m3 terms accumulate into the same TMEM tile, promoted with
//           inter_scale[row,kb] * w2_scale[e,nb,kb]; float32 rows out (eight of them
//           are later summed per token, so they are not rounded here).
//           Reference: _fused_moe_gemm2_kernel (solution/python/pure_triton_impl.py:1056-1196), oracle math
//           solution/cuda/binding.py:178-179.
//
// Tile: 128 sorted rows x 256 accumulator columns, K chunk = 128 bytes = one quantisation block = one 128-byte swizzle
// row.  MODE 1 uses two 128-row weight boxes per chunk (W1 rows n0.., W3 rows 2048+n0..) laid out back to back so a
// single N=256 MMA produces both SwiGLU operands; MODE 2 uses one 256-row box of W2 and two A boxes (the two terms).
//
// One CTA per tile.  What paces it (cycle stamps, probes): a TMEM stage goes round MMA -> completion signal -> promotion
// warps read it (two 64-column loads per warp) -> hand-back -> next MMA into it, and with 512 TMEM columns there are
// only two such stages of 256 columns.  A round costs ~600 cycles of tensor work (four MMAs of 128 cycles plus issue
// gaps) and ~1100-1300 cycles of latencies (barrier wake-ups of 190-280 cycles each way, 260 for the two loads, 150 to
// the hand-back, 170 to re-check the operands), so two stages keep the tensor pipe ~55 % busy: ~970 cycles per 128-K
// chunk.  Things that were built, measured and did NOT move it: CTA pairs (tcgen05.mma.cta_group::2, each CTA loading
// half of the weight tile: fewer L2 bytes, but the hand-back then crosses SMs; 485 vs 456 us, also 7 % of pair padding),
// a second MMA-issuing thread (one per TMEM stage; with it the issuer has slack and the promotion warps are busy
// ~850 of every ~980 cycles: wake-up, 64-column load, 32 packed FMAs, load, 32 FMAs, nothing overlapped because 128
// accumulators + 64 loaded values fill the 232 registers), the last promotion warp issuing the next MMAs itself (the
// issue of four MMAs blocks its thread for ~430 cycles: 38 % slower), parking barrier polls with a suspend-time hint,
// and a relaxed instead of a releasing hand-back.  The hand-back itself is a shared-memory counter polled by the
// issuer (2-7 % faster than an mbarrier).  In isolation the pieces run at 512 (MMA), 320 (promotion, 8 warps) and
// 610-690 (48 KB of loads per SM from L2, all SMs) cycles per chunk, and ~600 when all three run unsynchronised.
//
// Warp roles (384 threads): warps 0-7 promote TMEM partials into fp32 registers and run the epilogue (warp w owns TMEM
// lanes 32*(w%4).. and half of the columns), warp 8 issues TMA loads, warp 9 owns TMEM and issues the MMAs, warps 10-11
// only exist so that the third warpgroup can hand its registers to the other two (setmaxnreg 40 / 232).
// fp32 block scales are not power-of-two, so the hardware block-scaled MMA cannot apply them: each 128-K chunk is
// accumulated on its own into one of two 256-column TMEM stages and folded into registers with one FMA per element
// while the next chunk's MMAs run into the other stage.
//
// Every mbarrier wait is bounded (common.cuh: mbar_wait); on a timeout the CTA records the failure in the status word,
// raises a CTA-wide abort flag, drains its outstanding TMA loads, frees TMEM and returns.
#include <cuda.h>
#include <cstddef>

#include "common.cuh"
#include "gemm_common.cuh"
#include "half_rows.cuh"

namespace b200moe {

constexpr int TILE_N = 256;                    // TMEM columns per accumulator stage
constexpr int A_TILE_BYTES = BLOCK_M * 128;    // 16 KB
constexpr int NUM_PROMO_WARPS = 8;
constexpr int PRODUCER_WARP = 8;
constexpr int MMA_WARP = 9;
constexpr int GEMM_THREADS = 384;            // 3 warpgroups: 2 x promotion, 1 x {TMA, MMA, 2 idle warps}

template <int MODE>
struct Cfg {
  static constexpr int A_TILES = (MODE == 1) ? 1 : 2;
  static constexpr int B_BYTES = TILE_N * 128;         // the 256-row weight tile of one chunk
  static constexpr int STAGE_BYTES = A_TILES * A_TILE_BYTES + B_BYTES;
  static constexpr int STAGES = 196608 / STAGE_BYTES;  // 4 (GEMM1, 48 KB), 3 (GEMM2, 64 KB)
  static constexpr int K_CHUNKS = (MODE == 1) ? H_BLOCKS : I_BLOCKS;
  static constexpr int N_TILES = (MODE == 1) ? (I / 128) : (H / 256);  // 16, 28
};

struct TileInfo {
  int e, nt, mblk, m_local, cnt;
};

// Tiles are numbered expert-major, then n-tile, then 128-row block, so CTAs that run at the same time share weight
// tiles in L2.  s_off[e] = row blocks before expert e (block_offsets).
__device__ __forceinline__ TileInfo decode_tile(int tile, const int* s_off, const int* s_cnt, int E, int NT) {
  int lo = 0, hi = E - 1;
  while (lo < hi) {
    int mid = (lo + hi + 1) >> 1;
    if (s_off[mid] * NT <= tile) lo = mid; else hi = mid - 1;
  }
  TileInfo ti;
  ti.e = lo;
  int local = tile - s_off[lo] * NT;
  int groups = s_off[lo + 1] - s_off[lo];
  ti.nt = local / groups;
  ti.m_local = local - ti.nt * groups;
  ti.mblk = s_off[lo] + ti.m_local;
  ti.cnt = s_cnt[lo];
  return ti;
}

struct __align__(16) GemmAux {
  uint64_t full[4];
  uint64_t empty[4];
  uint64_t tfull[2];
  uint64_t xbar[2];
  uint32_t tmem_base;
  int abort_flag;
  // per TMEM stage: promotion warps that have finished reading it, counted up for ever (8 per fill).  The MMA issuer
  // polls it with plain loads; an mbarrier hand-back measured 2-7 % slower (the issuer's wake-up is on its serial path)
  uint32_t drained[2];
  int off[E_GLOBAL + 1];
  int cnt[E_GLOBAL];
  float amax[2][2][BLOCK_M];
  // GEMM2 epilogue: per promotion warp, 32 rows x 16 columns (+4 padding: conflict-free 16-byte accesses) through which
  // the thread-per-row accumulators are turned into stores of 64 contiguous bytes per row
  // (16-byte aligned: it is read and written with 16-byte accesses)
  alignas(16) float out_stage[NUM_PROMO_WARPS][32][20];
};
static_assert(offsetof(GemmAux, out_stage) % 16 == 0, "out_stage is accessed with 16-byte vectors");

template <int MODE>
constexpr size_t gemm_smem_bytes() {
  return 1024 + static_cast<size_t>(Cfg<MODE>::STAGES) * Cfg<MODE>::STAGE_BYTES + sizeof(GemmAux);
}

template <int MODE>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
k_grouped_gemm(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const GemmArgs args) {
  using C = Cfg<MODE>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t tiles_addr = (raw_addr + 1023u) & ~1023u;
  uint8_t* tiles_ptr = smem_raw + (tiles_addr - raw_addr);
  GemmAux* aux = reinterpret_cast<GemmAux*>(tiles_ptr + C::STAGES * C::STAGE_BYTES);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int E = args.E_local;
  constexpr int NT = C::N_TILES;
  const int group_id = blockIdx.x;            // tiles are dealt round-robin to the CTAs
  const int num_groups = gridDim.x;

  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    aux->abort_flag = 0;
    aux->drained[0] = 0;
    aux->drained[1] = 0;
  }

  if (warp == PRODUCER_WARP && lane == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(smem_u32(&aux->full[s]), 1);
      mbar_init(smem_u32(&aux->empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&aux->tfull[a]), 1);
      mbar_init(smem_u32(&aux->xbar[a]), NUM_PROMO_WARPS);
    }
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == MMA_WARP) {
    tmem_alloc(smem_u32(&aux->tmem_base), 512);
    tmem_relinquish();
  }
  // everything above is CTA-local set-up and may overlap the tail of the previous kernel; the layout it wrote is
  // read only from here on
  pdl_wait();
  for (int i = threadIdx.x; i <= E; i += GEMM_THREADS) aux->off[i] = __ldg(args.block_offsets + i);
  for (int i = threadIdx.x; i < E; i += GEMM_THREADS) aux->cnt[i] = __ldg(args.counts + i);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  const uint32_t tmem_base = aux->tmem_base;
  const int total_tiles = aux->off[E] * NT;
  volatile int* abort_flag = &aux->abort_flag;

  // Each register budget is set inside the branch it governs, so the compiler sees one budget per region.
  if (warp >= NUM_PROMO_WARPS) {
  setmaxnreg_dec_aux();
  if (warp == PRODUCER_WARP) {
    // ------------------------------------------------------------------ TMA producer (one thread per CTA)
    // The two single-thread roles run as lane 0 alone: one poller per barrier and no per-chunk warp votes.  (Measured:
    // all 32 lanes voting on every wait cost the MMA issuer ~300 idle cycles per chunk.)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      long long issued = 0;
      bool ok = true;
      for (int tile = group_id; ok && tile < total_tiles; tile += num_groups) {
        const TileInfo ti = decode_tile(tile, aux->off, aux->cnt, E, NT);
        for (int kb = 0; kb < C::K_CHUNKS; ++kb) {
          ok = mbar_wait(smem_u32(&aux->empty[stage]), phase ^ 1u, abort_flag, args.status, 1, kb);
          if (!ok) break;
          const uint32_t sbase = tiles_addr + stage * C::STAGE_BYTES;
          const uint32_t sB = sbase + C::A_TILES * A_TILE_BYTES;
          const uint32_t full = smem_u32(&aux->full[stage]);
          mbar_arrive_expect_tx(full, C::STAGE_BYTES);
          tma_load_2d(sbase, &tmA, full, kb * 128, ti.mblk * BLOCK_M);
          if (MODE == 1) {
            tma_load_2d(sB, &tmB, full, kb * 128, ti.e * (2 * I) + ti.nt * 128);
            tma_load_2d(sB + 128 * 128, &tmB, full, kb * 128, ti.e * (2 * I) + I + ti.nt * 128);
          } else {
            tma_load_2d(sbase + A_TILE_BYTES, &tmA, full, kb * 128, args.R_max + ti.mblk * BLOCK_M);
            tma_load_2d(sB, &tmB, full, kb * 128, ti.e * H + ti.nt * TILE_N);
          }
          ++issued;
          if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        // Drain: every load already issued completes on its own; wait (bounded) so none lands after the CTA exits.
        for (int s = 0; s < C::STAGES; ++s) {
          long long n_s = issued / C::STAGES + ((issued % C::STAGES) > s ? 1 : 0);  // loads issued to stage s
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
      constexpr uint32_t IDESC = umma_idesc_e4m3(BLOCK_M, TILE_N);
      int stage = 0, acc = 0;
      uint32_t phase = 0;
      uint32_t chunk = 0;                // chunks issued so far: chunk c is fill number c / 2 of TMEM stage c % 2
      bool ok = true;
      for (int tile = group_id; ok && tile < total_tiles; tile += num_groups) {
        for (int kb = 0; kb < C::K_CHUNKS; ++kb) {
          // operands first (they landed several chunks ago), the TMEM stage last: its hand-back is the critical
          // signal, and everything that can be prepared is ready when it comes
          const uint32_t sbase = tiles_addr + stage * C::STAGE_BYTES;
          const uint32_t d = tmem_base + static_cast<uint32_t>(acc * TILE_N);
          const uint64_t a0 = umma_desc_sw128(sbase);
          const uint64_t b0 = umma_desc_sw128(sbase + C::A_TILES * A_TILE_BYTES);
          ok = mbar_wait(smem_u32(&aux->full[stage]), phase, abort_flag, args.status, 3, kb);
          if (!ok) break;
          ok = counter_wait(&aux->drained[acc], (chunk >> 1) * NUM_PROMO_WARPS, abort_flag, args.status, 2, kb);
          if (!ok) break;
          ++chunk;
          tc_fence_after();
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4) tc_mma_f8(d, a0 + 2 * k4, b0 + 2 * k4, IDESC, k4 > 0 ? 1u : 0u);
          if (MODE == 2) {
            const uint64_t a1 = umma_desc_sw128(sbase + A_TILE_BYTES);
#pragma unroll
            for (int k4 = 0; k4 < 4; ++k4) tc_mma_f8(d, a1 + 2 * k4, b0 + 2 * k4, IDESC, 1u);
          }
          tc_commit(smem_u32(&aux->empty[stage]));
          tc_commit(smem_u32(&aux->tfull[acc]));
          if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
          acc ^= 1;
        }
      }
    }
    __syncwarp();
  }
  } else {
    setmaxnreg_inc_promo();
    // ------------------------------------------------------------------ promotion + epilogue (8 warps)
    const int q = warp & 3;       // TMEM lane quarter this warp may read
    const int h = warp >> 2;      // column half
    const int r_in_tile = q * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    int tile_iter = 0;
    bool ok = true;
    for (int tile = group_id; ok && tile < total_tiles; tile += num_groups, ++tile_iter) {
      const TileInfo ti = decode_tile(tile, aux->off, aux->cnt, E, NT);
      const int row = ti.mblk * BLOCK_M + r_in_tile;
      const bool valid = (ti.m_local * BLOCK_M + r_in_tile) < ti.cnt;
      // rows past the expert's last block (odd CTA of an incomplete pair) can lie outside the workspace: clamp reads
      const int row_rd = row < args.R_max ? row : 0;
      const float* rs_ptr = args.row_scale + row_rd;
      const float* ws0_ptr;
      const float* ws1_ptr;
      if (MODE == 1) {
        ws0_ptr = args.w_scale + (static_cast<size_t>(ti.e) * 32 + ti.nt) * H_BLOCKS;
        ws1_ptr = args.w_scale + (static_cast<size_t>(ti.e) * 32 + 16 + ti.nt) * H_BLOCKS;
      } else {
        ws0_ptr = args.w_scale + (static_cast<size_t>(ti.e) * H_BLOCKS + ti.nt * 2 + h) * I_BLOCKS;
        ws1_ptr = ws0_ptr;
      }
      // 128 fp32 accumulators per thread, kept as 64 pairs so the promotion runs on the packed FMA (2 lanes / issue)
      float2 acc2[64];
#pragma unroll
      for (int j = 0; j < 64; ++j) acc2[j] = make_float2(0.f, 0.f);
#define ACC(j) (((j) & 1) ? acc2[(j) >> 1].y : acc2[(j) >> 1].x)

      float rs_n = __ldg(rs_ptr);
      float w0_n = __ldg(ws0_ptr);
      float w1_n = __ldg(ws1_ptr);
      for (int kb = 0; kb < C::K_CHUNKS; ++kb) {
        const float sc0 = rs_n * w0_n;
        const float sc1 = rs_n * w1_n;
        if (kb + 1 < C::K_CHUNKS) {
          rs_n = __ldg(rs_ptr + static_cast<size_t>(kb + 1) * args.R_max);
          w0_n = __ldg(ws0_ptr + kb + 1);
          w1_n = __ldg(ws1_ptr + kb + 1);
        }
        ok = mbar_wait_all(smem_u32(&aux->tfull[acc]), acc_phase, abort_flag, args.status, 4, kb);
        if (!ok) break;
        tc_fence_after();
        const uint32_t taddr = tmem_base + static_cast<uint32_t>(acc * TILE_N) + (static_cast<uint32_t>(q * 32) << 16);
        // This warp's 128 accumulators are two runs of 64 TMEM columns — MODE 1: [64h, 64h+64) holds W1 ("up") and
        // [128+64h, 128+64h+64) holds W3 ("gate"); MODE 2: [128h, 128h+128) — each read with one 64-column load
        // (fewer, wider loads measured faster than four 32-column loads, pipelined or not).
#pragma unroll
        for (int run = 0; run < 2; ++run) {
          const uint32_t col = static_cast<uint32_t>((MODE == 1) ? (run * 128 + h * 64) : (h * 128 + run * 64));
          const float sc = (MODE == 1 && run == 1) ? sc1 : sc0;
          uint32_t tmp[64];
          tmem_ld64(taddr + col, tmp);
          tc_wait_ld();
          if (run == 1) {
            // all of this warp's reads of the stage are complete (tcgen05.wait::ld is warp-synchronous): hand it back
            // to the MMA issuer
            tc_fence_before();
            if (lane == 0) red_add_release_shared(&aux->drained[acc], 1u);
          }
          const float2 sc2 = make_float2(sc, sc);
#pragma unroll
          for (int j = 0; j < 32; ++j)
            acc2[run * 32 + j] = __ffma2_rn(make_float2(__uint_as_float(tmp[2 * j]), __uint_as_float(tmp[2 * j + 1])),
                                            sc2, acc2[run * 32 + j]);
        }
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
      if (!ok) break;

      if (MODE == 1) {
        // accumulators 0..63 = up (W1) columns 64h.., 64..127 = gate (W3) for the same columns.
        float amax = 0.f;
#pragma unroll
        for (int j = 0; j < 64; ++j) {
          ACC(j) = silu_mul(ACC(64 + j), ACC(j));
          amax = fmaxf(amax, fabsf(ACC(j)));
        }
        float* ex = &aux->amax[tile_iter & 1][0][0];
        ex[h * BLOCK_M + r_in_tile] = amax;
        // the other column half of each row lives in warp (w ^ 4): exchange through shared memory, bounded wait
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&aux->xbar[tile_iter & 1]));
        ok = mbar_wait_all(smem_u32(&aux->xbar[tile_iter & 1]), (tile_iter >> 1) & 1, abort_flag, args.status, 5,
                           tile_iter);
        if (!ok) break;
        amax = fmaxf(ex[r_in_tile], ex[BLOCK_M + r_in_tile]);
        const float s = fmaxf(amax, 1e-20f) * (1.0f / 448.0f);
        const float inv = 1.0f / s;
        // Quantise in registers (thread = row), then pass each term's 32 rows x 64 bytes through shared memory so that a
        // store instruction writes 64 contiguous bytes of 8 rows instead of 16 bytes of 32 rows.
        uint4 t1[4], t2[4];
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          uint32_t w1[4], w2[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int j = v * 16 + u * 4;
            w1[u] = pack4_e4m3(ACC(j) * inv, ACC(j + 1) * inv, ACC(j + 2) * inv, ACC(j + 3) * inv);
            float back[4];
            unpack4_e4m3(w1[u], back);
            w2[u] = pack4_e4m3((ACC(j) - back[0] * s) * inv, (ACC(j + 1) - back[1] * s) * inv,
                               (ACC(j + 2) - back[2] * s) * inv, (ACC(j + 3) - back[3] * s) * inv);
          }
          t1[v] = make_uint4(w1[0], w1[1], w1[2], w1[3]);
          t2[v] = make_uint4(w2[0], w2[1], w2[2], w2[3]);
        }
        float (*stg)[20] = aux->out_stage[warp];   // 80-byte row pitch: 64 bytes used
        const int rows_valid = ti.cnt - ti.m_local * BLOCK_M - q * 32;
        uint8_t* qbase = args.inter_q + static_cast<size_t>(ti.mblk * BLOCK_M + q * 32) * I + ti.nt * 128 + h * 64;
        const int rsub = lane >> 2, csub = lane & 3;
#pragma unroll
        for (int term = 0; term < 2; ++term) {
#pragma unroll
          for (int v = 0; v < 4; ++v) *reinterpret_cast<uint4*>(&stg[lane][4 * v]) = term == 0 ? t1[v] : t2[v];
          __syncwarp();
          uint8_t* dst = qbase + (term == 0 ? 0 : static_cast<size_t>(args.R_max) * I);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int r = rsub + 8 * j;
            const uint4 val = *reinterpret_cast<const uint4*>(&stg[r][4 * csub]);
            if (r < rows_valid) *reinterpret_cast<uint4*>(dst + static_cast<size_t>(r) * I + csub * 16) = val;
          }
          __syncwarp();
        }
        if (valid && h == 0) args.inter_scale[static_cast<size_t>(ti.nt) * args.R_max + row] = s;
      } else if (args.out_half) {
        // Rows in the half form: the thread's 128 columns are 16 groups of eight (one scale byte each).  Same staging
        // as below, 32 columns = four groups = 64 bytes of float16 per row at a time.
        uint32_t (*stg)[20] = reinterpret_cast<uint32_t (*)[20]>(aux->out_stage[warp]);
        const int rows_valid = ti.cnt - ti.m_local * BLOCK_M - q * 32;
        uint8_t* obase = reinterpret_cast<uint8_t*>(args.expert_out) +
                         static_cast<size_t>(ti.mblk * BLOCK_M + q * 32) * HALF_ROW_BYTES;
        const int g0 = ti.nt * (TILE_N / 8) + h * 16;   // this thread's first group within the row
        const int rsub = lane >> 2, csub = (lane & 3) * 4;
        uint32_t scale_bytes[4] = {0u, 0u, 0u, 0u};
#pragma unroll
        for (int piece = 0; piece < 4; ++piece) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            const int g = piece * 4 + v;
            const float x[8] = {ACC(8 * g), ACC(8 * g + 1), ACC(8 * g + 2), ACC(8 * g + 3),
                                ACC(8 * g + 4), ACC(8 * g + 5), ACC(8 * g + 6), ACC(8 * g + 7)};
            uint32_t eb;
            *reinterpret_cast<uint4*>(&stg[lane][4 * v]) = encode_half_group(x, eb);
            scale_bytes[piece] |= eb << (8 * v);
          }
          __syncwarp();
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int r = rsub + 8 * j;
            const uint4 val = *reinterpret_cast<const uint4*>(&stg[r][csub]);
            if (r < rows_valid)
              *reinterpret_cast<uint4*>(obase + static_cast<size_t>(r) * HALF_ROW_BYTES + (g0 + piece * 4) * 16 +
                                        csub * 4) = val;
          }
          __syncwarp();
        }
        if (lane < rows_valid)
          *reinterpret_cast<uint4*>(obase + static_cast<size_t>(lane) * HALF_ROW_BYTES + HALF_ROW_SCALES + g0) =
              make_uint4(scale_bytes[0], scale_bytes[1], scale_bytes[2], scale_bytes[3]);
      } else {
        // Thread-per-row stores would touch 32 rows with 16 bytes each per instruction.  Instead each warp passes its
        // 32 x 128 block through shared memory 16 columns at a time and stores 64 contiguous bytes per row (8 rows per
        // instruction), which halves the sectors L2 has to merge.
        float (*stg)[20] = aux->out_stage[warp];
        const int rows_valid = ti.cnt - ti.m_local * BLOCK_M - q * 32;   // valid rows of this warp's 32 (may be <= 0)
        float* obase = args.expert_out + static_cast<size_t>(ti.mblk * BLOCK_M + q * 32) * H + ti.nt * TILE_N + h * 128;
        const int rsub = lane >> 2, csub = (lane & 3) * 4;
#pragma unroll
        for (int piece = 0; piece < 8; ++piece) {
#pragma unroll
          for (int v = 0; v < 4; ++v)
            *reinterpret_cast<float4*>(&stg[lane][4 * v]) =
                make_float4(ACC(piece * 16 + 4 * v), ACC(piece * 16 + 4 * v + 1), ACC(piece * 16 + 4 * v + 2),
                            ACC(piece * 16 + 4 * v + 3));
          __syncwarp();
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int r = rsub + 8 * j;
            const float4 val = *reinterpret_cast<const float4*>(&stg[r][csub]);
            if (r < rows_valid)
              *reinterpret_cast<float4*>(obase + static_cast<size_t>(r) * H + piece * 16 + csub) = val;
          }
          __syncwarp();
        }
      }
    }
  }

#undef ACC
  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (warp == MMA_WARP) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ---------------------------------------------------------------------------------------------------------
// Host side: tensor maps and launches
// ---------------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void* p = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) != cudaSuccess ||
      qres != cudaDriverEntryPointSuccess)
    return nullptr;
  fn = reinterpret_cast<EncodeTiledFn>(p);
  return fn;
}

// 2-D byte tensor [rows, cols] (row pitch = cols), box [box_rows, 128 bytes], 128-byte swizzle.
int make_map_u8(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return record_cuda_error(cudaErrorNotSupported);
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols};
  cuuint32_t box[2] = {128, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return record_cuda_error(cudaErrorInvalidValue);
  return B200MOE_OK;
}

template <int MODE>
static int launch_gemm(const b200moe_problem* p, const b200moe_workspace* ws, int num_sms, cudaStream_t st,
                       bool half_out) {
  if (p->T == 0) return B200MOE_OK;
  static bool attr_set[64] = {};
  int dev = 0;
  B200MOE_CUDA_TRY(cudaGetDevice(&dev));
  constexpr size_t smem = gemm_smem_bytes<MODE>();
  if (dev < 64 && !attr_set[dev]) {
    B200MOE_CUDA_TRY(cudaFuncSetAttribute(k_grouped_gemm<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          static_cast<int>(smem)));
    attr_set[dev] = true;
  }
  CUtensorMap tmA, tmB;
  int rc;
  GemmArgs a;
  a.block_offsets = ws->block_offsets;
  a.counts = ws->counts;
  a.inter_q = ws->inter_q;
  a.inter_scale = ws->inter_scale;
  a.expert_out = ws->expert_out;
  a.status = ws->status;
  a.tile_ctr = nullptr;
  a.weights = nullptr;
  a.early_weights = 0;
  a.out_half = half_out ? 1 : 0;
  a.partial = nullptr;
  a.E_local = p->E_local;
  a.R_max = ws->R_max;
  // weight boxes: GEMM1 takes 128 W1 rows and 128 W3 rows as two boxes, GEMM2 its 256 W2 rows in one
  const uint32_t b_box_rows = (MODE == 2) ? TILE_N : 128;
  if (MODE == 1) {
    if ((rc = make_map_u8(&tmA, ws->a_sorted, static_cast<uint64_t>(ws->R_max), H, BLOCK_M))) return rc;
    if ((rc = make_map_u8(&tmB, p->gemm1_weights, static_cast<uint64_t>(p->E_local) * 2 * I, H, b_box_rows))) return rc;
    a.row_scale = ws->a_scale_sorted;
    a.w_scale = p->gemm1_weights_scale;
  } else {
    if ((rc = make_map_u8(&tmA, ws->inter_q, static_cast<uint64_t>(ws->R_max) * 2, I, BLOCK_M))) return rc;
    if ((rc = make_map_u8(&tmB, p->gemm2_weights, static_cast<uint64_t>(p->E_local) * H, I, b_box_rows))) return rc;
    a.row_scale = ws->inter_scale;
    a.w_scale = p->gemm2_weights_scale;
  }
  B200MOE_CUDA_TRY(launch_pdl(k_grouped_gemm<MODE>, dim3(num_sms), dim3(GEMM_THREADS), smem, st, tmA, tmB, a));
  return B200MOE_OK;
}

int launch_gemm1(const b200moe_problem* p, const b200moe_workspace* ws, int num_sms, cudaStream_t st) {
  return launch_gemm<1>(p, ws, num_sms, st, false);
}
int launch_gemm2(const b200moe_problem* p, const b200moe_workspace* ws, int num_sms, cudaStream_t st, bool half_out) {
  return launch_gemm<2>(p, ws, num_sms, st, half_out);
}

}  // namespace b200moe
