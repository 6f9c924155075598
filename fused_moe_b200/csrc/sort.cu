// Stable token ranking, BLOCK_M-padded expert layout, scatter, activation gather and the weighted top-8 reduce.
//
// What is produced equals the reference's sort metadata (solution/python/pure_triton_impl.py:474-551): padded
// per-expert segments, block_offsets in units of BLOCK_M rows, pad rows carrying token id T and weight 0,
// scatter_map = -1 for non-local pairs.  The ORDER inside an expert segment is ascending token id, which is what a
// stable sort of the flat (token*8+k) list by expert gives (solution/cuda/binding.py:138-150); the reference's
// Triton kernels take their positions from atomics and are not reproducible from run to run.
//
// A token selects an expert at most once, so the rank of pair (t, e) inside expert e is the number of earlier
// tokens that selected e.  chunk_bits[c][e] holds that selection as one bit per token of 32-token chunk c; the rank
// is chunk_base[c][e] + popc(bits & lanes_below).
#include "common.cuh"
#include "half_rows.cuh"

namespace b200moe {

// chunk_base[c][e] = local pairs of expert e in chunks < c; counts[e] = total.
//
// chunk_bits is expert-minor, so the lanes of a warp take 32 CONSECUTIVE EXPERTS (one 128-byte line per chunk row) and
// the 32 warps of a CTA take 32 contiguous runs of chunks.  Three steps: every thread sums its run (independent,
// coalesced loads), the run totals are prefixed over the warps through shared memory, every thread walks its run again
// and writes chunk_base.  (Two earlier layouts, one warp per expert with a lane per chunk or per run of chunks, touched
// 32 lines per load instruction and took 24 - 30 us at 512 chunks x 256 experts.)
__global__ void __launch_bounds__(1024)
k_rank_scan(const uint32_t* __restrict__ chunk_bits, int n_chunks, int E_local, int* __restrict__ chunk_base,
            int* __restrict__ counts) {
  __shared__ int s_run[32][33];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int e = blockIdx.x * 32 + lane;
  const bool live = e < E_local;
  pdl_launch_dependents();
  pdl_wait();
  const int per = (n_chunks + 31) >> 5;                 // chunks per warp
  const int c0 = warp * per < n_chunks ? warp * per : n_chunks;
  const int c1 = (c0 + per < n_chunks) ? c0 + per : n_chunks;
  const uint32_t* col = chunk_bits + e;
  int sum = 0;
  if (live) {
#pragma unroll 8
    for (int c = c0; c < c1; ++c) sum += __popc(__ldg(col + static_cast<size_t>(c) * E_local));
  }
  s_run[warp][lane] = sum;
  __syncthreads();
  int run = 0;
  for (int w = 0; w < warp; ++w) run += s_run[w][lane];
  if (live) {
    if (warp == 31) counts[e] = run + sum;
    int* out = chunk_base + e;
#pragma unroll 8
    for (int c = c0; c < c1; ++c) {
      out[static_cast<size_t>(c) * E_local] = run;
      run += __popc(__ldg(col + static_cast<size_t>(c) * E_local));
    }
  }
}

// Padded layout (every CTA recomputes it in shared memory; CTA 0 publishes it) and the scatter, one warp per chunk.
// SCAN = true (batches of at most 32 chunks): the CTA also derives the per-expert totals and the prefix for its four
// chunks from the bit matrix itself (at most 32 x E words, read with coalesced loads), so k_rank_scan is not launched
// and chunk_base is not used; CTA 0 publishes counts.
constexpr int SCATTER_SCAN_MAX_CHUNKS = 32;
template <bool SCAN>
__global__ void __launch_bounds__(128)
k_scatter(const int* __restrict__ topk_idx, const float* __restrict__ topk_w, long long topk_stride,
          const uint32_t* __restrict__ chunk_bits,
          const int* __restrict__ chunk_base, int* __restrict__ counts, int T, int local_offset, int E_local,
          int n_chunks, int* __restrict__ block_offsets, int* __restrict__ total_blocks,
          int* __restrict__ sorted_token_ids, float* __restrict__ sorted_weights, int* __restrict__ scatter_map,
          const b200moe_ep_plan* __restrict__ plan) {
  __shared__ int s_row_base[E_GLOBAL + 1];
  __shared__ int s_cnt[SCAN ? E_GLOBAL : 1];
  __shared__ int s_base[SCAN ? 4 : 1][SCAN ? E_GLOBAL : 1];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;

  pdl_launch_dependents();
  pdl_wait();
  if (SCAN) {
    const int c_first = blockIdx.x * 4;
    for (int e = threadIdx.x; e < E_local; e += blockDim.x) {
      int run = 0;
#pragma unroll 8
      for (int c = 0; c < n_chunks; ++c) {
        if (c >= c_first && c < c_first + 4) s_base[c - c_first][e] = run;
        run += __popc(__ldg(chunk_bits + static_cast<size_t>(c) * E_local + e));
      }
      s_cnt[e] = run;
      if (blockIdx.x == 0) counts[e] = run;
    }
    __syncthreads();
  }
  if (warp == 0) {
    // lane handles experts [8*lane, 8*lane+8)
    int blocks[8];
    int local = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      int e = lane * 8 + i;
      int c = (e < E_local) ? (SCAN ? s_cnt[e] : __ldg(counts + e)) : 0;
      blocks[i] = (c + BLOCK_M - 1) / BLOCK_M;
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
      int e = lane * 8 + i;
      if (e < E_local) s_row_base[e] = run;  // in blocks
      run += blocks[i];
    }
    if (lane == 31) s_row_base[E_local] = incl;  // total blocks
  }
  __syncthreads();
  const int tot_blocks = s_row_base[E_local];

  if (blockIdx.x == 0) {
    for (int e = threadIdx.x; e <= E_local; e += blockDim.x) block_offsets[e] = s_row_base[e];
    if (threadIdx.x == 0) *total_blocks = tot_blocks;
  }
  // pad rows: expert e is handled by CTA (e mod gridDim)
  for (int e = blockIdx.x; e < E_local; e += gridDim.x) {
    int begin = s_row_base[e] * BLOCK_M + (SCAN ? s_cnt[e] : __ldg(counts + e));
    int end = s_row_base[e + 1] * BLOCK_M;
    for (int r = begin + threadIdx.x; r < end; r += blockDim.x) {
      sorted_token_ids[r] = T;
      sorted_weights[r] = 0.f;
    }
  }

  const int chunk = blockIdx.x * (blockDim.x >> 5) + warp;
  if (chunk >= n_chunks) return;
  const int t = chunk * 32 + lane;
  // with a device-side plan only the received rows exist; pad rows keep the id T (the capacity) either way
  if (t >= (plan ? min(T, plan->n_recv) : T)) return;
  const uint32_t below = (1u << lane) - 1u;
  int dest[TOP_K];
#pragma unroll
  for (int k = 0; k < TOP_K; ++k) {
    int le = __ldg(topk_idx + static_cast<size_t>(t) * topk_stride + k) - local_offset;
    dest[k] = -1;
    if (le >= 0 && le < E_local) {
      uint32_t bits = __ldg(chunk_bits + static_cast<size_t>(chunk) * E_local + le);
      int rank = (SCAN ? s_base[warp][le] : __ldg(chunk_base + static_cast<size_t>(chunk) * E_local + le)) +
                 __popc(bits & below);
      int d = s_row_base[le] * BLOCK_M + rank;
      dest[k] = d;
      sorted_token_ids[d] = t;
      sorted_weights[d] = __ldg(topk_w + static_cast<size_t>(t) * topk_stride + k);
    }
  }
  int4* out = reinterpret_cast<int4*>(scatter_map + static_cast<size_t>(t) * TOP_K);
  out[0] = make_int4(dest[0], dest[1], dest[2], dest[3]);
  out[1] = make_int4(dest[4], dest[5], dest[6], dest[7]);
}

// Copy the e4m3 row and the 56 scales of each real sorted row; pad rows are left as they are (their products are
// never read).  One warp per row, grid-stride over the rows that exist.
__global__ void __launch_bounds__(256)
k_gather(const uint8_t* __restrict__ hidden, long long row_stride, const float* __restrict__ hidden_scale,
         long long scale_token_stride, long long scale_block_stride, int T,
         const int* __restrict__ sorted_token_ids, const int* __restrict__ total_blocks, int R_max,
         uint8_t* __restrict__ a_sorted, float* __restrict__ a_scale_sorted) {
  const int lane = threadIdx.x & 31;
  const int warps_per_cta = blockDim.x >> 5;
  // Dependents are released only AFTER this kernel's own dependency wait: a GEMM1 that starts because of this release
  // may then read the sort metadata (complete, since every CTA here has seen the scatter finish) and stream its first
  // weight stages while the rows are still being copied; the roles that read those rows wait for this kernel as usual.
  pdl_wait();
  pdl_launch_dependents();
  const int rows = __ldg(total_blocks) * BLOCK_M;
  for (int r = blockIdx.x * warps_per_cta + (threadIdx.x >> 5); r < rows; r += gridDim.x * warps_per_cta) {
    int tok = __ldg(sorted_token_ids + r);
    if (tok >= T) continue;
    const uint4* src = reinterpret_cast<const uint4*>(hidden + static_cast<size_t>(tok) * row_stride);
    uint4* dst = reinterpret_cast<uint4*>(a_sorted + static_cast<size_t>(r) * H);
#pragma unroll
    for (int i = 0; i < H / 16 / 32; ++i) dst[i * 32 + lane] = __ldg(src + i * 32 + lane);
    for (int kb = lane; kb < H_BLOCKS; kb += 32)
      a_scale_sorted[static_cast<size_t>(kb) * R_max + r] =
          __ldg(hidden_scale + static_cast<size_t>(kb) * scale_block_stride + static_cast<size_t>(tok) * scale_token_stride);
  }
}

struct OutSegments {
  int count;
  int start[9];
  float* base[8];
};

// out[t, :] = sum_k w[t,k] * expert_out[scatter_map[t,k], :] in fp32, k ascending; 16-byte loads and stores.
// Writes bf16 to `out` and/or the un-rounded sums to `out_f32` (either may be null).  topk_w == nullptr means weight 1
// (the expert-parallel combine adds rows that are already weighted).
// G = groups of eight columns a thread takes per round: 4 when the source rows are in the half form and a CTA owns a
// whole token, else 1.  With G = 4 a thread takes four ADJACENT groups: 64 contiguous bytes of float16 and one 4-byte
// word of scale bytes per source row (measured at T = 16384 / 256 experts: 397 us, against 496 with one group per
// thread and round and 533 with the four groups interleaved over the lanes of a warp).  Stores of half rows are another
// matter when the row lives in another GPU's memory: 16 bytes at a 64-byte stride per lane and instruction made the
// return of partial rows 1.6 x slower than whole 512-byte runs per instruction, so the encoded groups of a warp pass
// through shared memory (swizzled, conflict-free both ways) and leave in lane order.
__device__ __forceinline__ int swizzled_slot(int slot) {   // slot = 4 * lane + group; 16-byte units of a warp's 2 KB
  const int l = slot >> 2;
  return (slot & ~3) | ((slot & 3) ^ ((l >> 1) & 3));
}
template <int G>
__global__ void __launch_bounds__(128)
k_reduce(const float* __restrict__ expert_out, const int* __restrict__ scatter_map, const float* __restrict__ topk_w,
         long long w_stride, int T, uint16_t* __restrict__ out, float* __restrict__ out_f32, const OutSegments segs,
         const b200moe_ep_plan* __restrict__ plan, int* __restrict__ status, int* __restrict__ status_mirror,
         int half_rows, int half_src) {
  int t = blockIdx.x;
  // un-rounded rows: float32 [7168] or the half form; either way `pitch` floats apart
  const size_t pitch = half_rows ? HALF_ROW_BYTES / 4 : H;
  float* dst_row = out_f32 ? out_f32 + static_cast<size_t>(t) * pitch : nullptr;
  if (segs.count > 0) {
    // rows of segment i go to segs.base[i], which may be memory of another GPU (plain 16-byte stores)
    int i = 0;
#pragma unroll
    for (int j = 1; j < 8; ++j)
      if (j < segs.count && t >= segs.start[j]) i = j;
    out = nullptr;
    dst_row = segs.base[i] + static_cast<size_t>(t - segs.start[i]) * pitch;
  }
  __shared__ int s_pos[TOP_K];
  __shared__ float s_w[TOP_K];
  __shared__ uint4 s_stage[G > 1 ? 4 : 1][G > 1 ? 128 : 1];   // G = 4: one warp's encoded groups on their way out
  pdl_launch_dependents();
  pdl_wait();
  // This is the last kernel of a layer call: if an earlier kernel of the call gave up on a wait, copy the status word
  // to the host-visible mirror (plain stores into mapped host memory), where the host sees it without synchronising.
  if (status_mirror && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0 && status[0] != 0) {
    status_mirror[1] = status[1];
    status_mirror[2] = status[2];
    status_mirror[3] = status[3];
    __threadfence_system();
    status_mirror[0] = status[0];
  }
  if (plan) {
    // the row window and the destinations were decided on the device (expert-parallel receiver)
    const int n = plan->n_recv;
    if (t >= n) return;
    // CTAs are scheduled in index order and the rows of one sender are contiguous: start with the rows of the NEXT rank
    // and wrap around, so that the ranks return rows to different peers at any moment instead of all to rank 0 first
    // (one receiver's NVLink ingress shared by every sender), then all to rank 1, ...
    t += plan->seg_start[(plan->rank + 1) % plan->seg_count];
    if (t >= n) t -= n;
    int i = 0;
#pragma unroll
    for (int j = 1; j < 8; ++j)
      if (j < plan->seg_count && t >= plan->seg_start[j]) i = j;
    out = nullptr;
    dst_row = plan->seg_base[i] + static_cast<size_t>(t - plan->seg_start[i]) * pitch;
    if (reinterpret_cast<uintptr_t>(dst_row) & 15u) {
      // never store through an address that does not add up: record it (status code 4) and skip the row
      if (status && threadIdx.x == 0 && atomicCAS(status, 0, 4) == 0) {
        status[1] = 300 + i;
        status[2] = t;
        status[3] = static_cast<int>(reinterpret_cast<uintptr_t>(dst_row) & 0xffff);
      }
      return;
    }
  }
  if (threadIdx.x < TOP_K) {
    s_pos[threadIdx.x] = __ldg(scatter_map + static_cast<size_t>(t) * TOP_K + threadIdx.x);
    s_w[threadIdx.x] = topk_w ? __ldg(topk_w + static_cast<size_t>(t) * w_stride + threadIdx.x) : 1.0f;
  }
  __syncthreads();
  // gridDim.y CTAs share a token's 896 eight-column vectors (small batches: a token per CTA left most SMs idle and
  // made each thread walk seven dependent rounds of loads)
  const int per = (H / 8 / G) / gridDim.y;
  for (int u = blockIdx.y * per + threadIdx.x; u < (blockIdx.y + 1) * per; u += blockDim.x) {
    float acc[G][8];
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[g][j] = 0.f;
#pragma unroll
    for (int k = 0; k < TOP_K; ++k) {
      int pos = s_pos[k];
      if (pos < 0) continue;
      float w = s_w[k];
      if (G > 1) {
        // half-form source rows, four groups per thread (only launched with half_src)
        const uint8_t* row = reinterpret_cast<const uint8_t*>(expert_out) + static_cast<size_t>(pos) * HALF_ROW_BYTES;
        const uint32_t sc4 = __ldg(reinterpret_cast<const uint32_t*>(row + HALF_ROW_SCALES) + u);
#pragma unroll
        for (int g = 0; g < G; ++g) {
          const uint4 q = __ldg(reinterpret_cast<const uint4*>(row) + G * u + g);
          const float kw = __uint_as_float((((sc4 >> (8 * g)) & 0xffu) - 14u) << 23) * w;
          const uint32_t x[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&x[j]));
            acc[g][2 * j] = fmaf(f.x, kw, acc[g][2 * j]);
            acc[g][2 * j + 1] = fmaf(f.y, kw, acc[g][2 * j + 1]);
          }
        }
        continue;
      }
      if (half_src) {   // the tile GEMM2 of the same layer call left its rows in the half form (uniform branch)
        fma_half_group(reinterpret_cast<const uint8_t*>(expert_out) + static_cast<size_t>(pos) * HALF_ROW_BYTES, u, w,
                       acc[0]);
        continue;
      }
      const float4* src = reinterpret_cast<const float4*>(expert_out + static_cast<size_t>(pos) * H) + 2 * u;
      float4 a = __ldg(src), b = __ldg(src + 1);
      acc[0][0] = fmaf(w, a.x, acc[0][0]); acc[0][1] = fmaf(w, a.y, acc[0][1]);
      acc[0][2] = fmaf(w, a.z, acc[0][2]); acc[0][3] = fmaf(w, a.w, acc[0][3]);
      acc[0][4] = fmaf(w, b.x, acc[0][4]); acc[0][5] = fmaf(w, b.y, acc[0][5]);
      acc[0][6] = fmaf(w, b.z, acc[0][6]); acc[0][7] = fmaf(w, b.w, acc[0][7]);
    }
    if (G > 1 && dst_row && half_rows) {
      // encode, pass the warp's 128 groups through shared memory, store them in lane order (512 contiguous bytes per
      // instruction); the scale bytes of a thread's four groups are one aligned word
      uint8_t* row = reinterpret_cast<uint8_t*>(dst_row);
      const int lane = threadIdx.x & 31;
      uint4* stage = s_stage[threadIdx.x >> 5];
      uint32_t sc4 = 0;
#pragma unroll
      for (int g = 0; g < G; ++g) {
        uint32_t eb;
        stage[swizzled_slot(4 * lane + g)] = encode_half_group(acc[g], eb);
        sc4 |= eb << (8 * g);
      }
      __syncwarp();
      const int first = (u >> 5) * 128;   // the warp's first group
#pragma unroll
      for (int g = 0; g < G; ++g) reinterpret_cast<uint4*>(row)[first + 32 * g + lane] = stage[swizzled_slot(32 * g + lane)];
      __syncwarp();
      reinterpret_cast<uint32_t*>(row + HALF_ROW_SCALES)[u] = sc4;
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const int v = G * u + g;
      if (out) {
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          __nv_bfloat162 b = __floats2bfloat162_rn(acc[g][2 * j], acc[g][2 * j + 1]);
          o[j] = *reinterpret_cast<uint32_t*>(&b);
        }
        reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * H)[v] = make_uint4(o[0], o[1], o[2], o[3]);
      }
      if (dst_row && half_rows) {
        if (G == 1) store_half_group(reinterpret_cast<uint8_t*>(dst_row), v, acc[g]);
      } else if (dst_row) {
        float4* dst = reinterpret_cast<float4*>(dst_row) + 2 * v;
        dst[0] = make_float4(acc[g][0], acc[g][1], acc[g][2], acc[g][3]);
        dst[1] = make_float4(acc[g][4], acc[g][5], acc[g][6], acc[g][7]);
      }
    }
  }
  if (segs.count > 0 || plan) __threadfence_system();  // peer stores are visible system-wide before the barrier that follows
}

// out[t, :] = bf16(sum over the token's returned half rows, in slot order): the expert-parallel combine when the
// partial rows travelled in the half form.  Same work split as k_reduce (G groups of eight columns per thread).
template <int G>
__global__ void __launch_bounds__(128)
k_combine_half(const uint8_t* __restrict__ rows, const int* __restrict__ slot_map, int T, uint16_t* __restrict__ out) {
  const int t = blockIdx.x;
  __shared__ int s_pos[TOP_K];
  pdl_launch_dependents();
  pdl_wait();
  if (threadIdx.x < TOP_K) s_pos[threadIdx.x] = __ldg(slot_map + static_cast<size_t>(t) * TOP_K + threadIdx.x);
  __syncthreads();
  const int per = (H / 8 / G) / gridDim.y;
  for (int u = blockIdx.y * per + threadIdx.x; u < (blockIdx.y + 1) * per; u += blockDim.x) {
    float acc[G][8];
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[g][j] = 0.f;
#pragma unroll
    for (int k = 0; k < TOP_K; ++k) {
      const int pos = s_pos[k];
      if (pos < 0) continue;
      const uint8_t* row = rows + static_cast<size_t>(pos) * HALF_ROW_BYTES;
      if (G == 1) {
        fma_half_group(row, u, 1.0f, acc[0]);
        continue;
      }
      // four adjacent groups per thread: 64 contiguous bytes and one word of scale bytes (see k_reduce)
      const uint32_t sc4 = __ldg(reinterpret_cast<const uint32_t*>(row + HALF_ROW_SCALES) + u);
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const uint4 q = __ldg(reinterpret_cast<const uint4*>(row) + G * u + g);
        const float kw = __uint_as_float((((sc4 >> (8 * g)) & 0xffu) - 14u) << 23);
        const uint32_t x[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&x[j]));
          acc[g][2 * j] = fmaf(f.x, kw, acc[g][2 * j]);
          acc[g][2 * j + 1] = fmaf(f.y, kw, acc[g][2 * j + 1]);
        }
      }
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        __nv_bfloat162 b = __floats2bfloat162_rn(acc[g][2 * j], acc[g][2 * j + 1]);
        o[j] = *reinterpret_cast<uint32_t*>(&b);
      }
      reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * H)[G * u + g] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

// CTAs per token of k_reduce: 7 x 128 threads = one vector per thread while the batch alone cannot fill the GPU
static unsigned reduce_splits(int T) { return T <= 512 ? 7u : 1u; }

// Entry points for the expert-parallel code (ep.cu), which ranks (token, destination) pairs with the same scan and adds
// returned rows with the same reduce.
int launch_rank_scan(const uint32_t* bits, int n_chunks, int E, int* base, int* counts, cudaStream_t st) {
  B200MOE_CUDA_TRY(launch_pdl(k_rank_scan, dim3((E + 31) / 32), dim3(1024), 0, st, bits, n_chunks, E, base, counts));
  return B200MOE_OK;
}
int launch_reduce_rows(const float* rows, const int* slot_map, int T, uint16_t* out, cudaStream_t st) {
  OutSegments none = {};
  B200MOE_CUDA_TRY(launch_pdl(k_reduce<1>, dim3(T, reduce_splits(T)), dim3(128), 0, st, rows, slot_map, static_cast<const float*>(nullptr),
                              static_cast<long long>(TOP_K), T, out, static_cast<float*>(nullptr), none,
                              static_cast<const b200moe_ep_plan*>(nullptr), static_cast<int*>(nullptr),
                              static_cast<int*>(nullptr), 0, 0));
  return B200MOE_OK;
}
int launch_combine_half(const void* rows, const int* slot_map, int T, uint16_t* out, cudaStream_t st) {
  auto kern = reduce_splits(T) == 1u ? k_combine_half<4> : k_combine_half<1>;
  B200MOE_CUDA_TRY(launch_pdl(kern, dim3(T, reduce_splits(T)), dim3(128), 0, st,
                              static_cast<const uint8_t*>(rows), slot_map, T, out));
  return B200MOE_OK;
}

int launch_sort(const b200moe_problem* p, const b200moe_workspace* ws, cudaStream_t st) {
  const int* idx = p->routing_logits ? ws->topk_idx : p->topk_idx_in;
  const float* w = p->routing_logits ? ws->topk_w : p->topk_w_in;
  if (p->T == 0) {
    B200MOE_CUDA_TRY(cudaMemsetAsync(ws->block_offsets, 0, sizeof(int) * (p->E_local + 1), st));
    B200MOE_CUDA_TRY(cudaMemsetAsync(ws->total_blocks, 0, sizeof(int), st));
    B200MOE_CUDA_TRY(cudaMemsetAsync(ws->counts, 0, sizeof(int) * p->E_local, st));
    return B200MOE_OK;
  }
  const long long tstride = (!p->routing_logits && p->topk_row_stride) ? p->topk_row_stride : TOP_K;
  int grid = (ws->n_chunks + 3) / 4;
  if (ws->n_chunks <= SCATTER_SCAN_MAX_CHUNKS) {
    // small batch: the scatter CTAs do the scan themselves, one launch less
    B200MOE_CUDA_TRY(launch_pdl(k_scatter<true>, dim3(grid), dim3(128), 0, st, idx, w, tstride, ws->chunk_bits,
                                ws->chunk_base, ws->counts, p->T, p->local_expert_offset, p->E_local, ws->n_chunks,
                                ws->block_offsets, ws->total_blocks, ws->sorted_token_ids, ws->sorted_weights,
                                ws->scatter_map, p->plan));
    return B200MOE_OK;
  }
  int scan_grid = (p->E_local + 31) / 32;
  B200MOE_CUDA_TRY(launch_pdl(k_rank_scan, dim3(scan_grid), dim3(1024), 0, st, ws->chunk_bits, ws->n_chunks, p->E_local,
                              ws->chunk_base, ws->counts));
  B200MOE_CUDA_TRY(launch_pdl(k_scatter<false>, dim3(grid), dim3(128), 0, st, idx, w, tstride, ws->chunk_bits,
                              ws->chunk_base, ws->counts, p->T, p->local_expert_offset, p->E_local, ws->n_chunks,
                              ws->block_offsets, ws->total_blocks, ws->sorted_token_ids, ws->sorted_weights,
                              ws->scatter_map, p->plan));
  return B200MOE_OK;
}

int launch_gather(const b200moe_problem* p, const b200moe_workspace* ws, int num_sms, cudaStream_t st) {
  if (p->T == 0) return B200MOE_OK;
  long long max_rows = ws->R_max;
  int grid = static_cast<int>((max_rows + 7) / 8);
  if (grid > num_sms * 8) grid = num_sms * 8;
  if (grid < 1) grid = 1;
  B200MOE_CUDA_TRY(launch_pdl(k_gather, dim3(grid), dim3(256), 0, st, p->hidden_states,
                              p->hidden_row_stride ? p->hidden_row_stride : static_cast<long long>(H),
                              p->hidden_states_scale, p->scale_token_stride ? p->scale_token_stride : 1LL,
                              p->scale_block_stride ? p->scale_block_stride : static_cast<long long>(p->T), p->T,
                              ws->sorted_token_ids, ws->total_blocks, ws->R_max, ws->a_sorted, ws->a_scale_sorted));
  return B200MOE_OK;
}

int launch_reduce(const b200moe_problem* p, const b200moe_workspace* ws, cudaStream_t st, bool half_src) {
  if (p->T == 0) return B200MOE_OK;
  const float* w = p->routing_logits ? ws->topk_w : p->topk_w_in;
  OutSegments segs = {};
  segs.count = p->out_seg_count;
  for (int i = 0; i < 8; ++i) segs.base[i] = p->out_seg_base[i];
  for (int i = 0; i < 9; ++i) segs.start[i] = p->out_seg_start[i];
  // half-form source rows and one CTA per token: four groups per thread (see k_reduce)
  auto kern = (half_src && reduce_splits(p->T) == 1u) ? k_reduce<4> : k_reduce<1>;
  B200MOE_CUDA_TRY(launch_pdl(kern, dim3(p->T, reduce_splits(p->T)), dim3(128), 0, st, ws->expert_out, ws->scatter_map, w,
                              (!p->routing_logits && p->topk_row_stride) ? p->topk_row_stride : static_cast<long long>(TOP_K), p->T,
                              p->output, p->output_f32, segs, p->plan, ws->status,
                              ws->status_mirror, p->partial_format == B200MOE_PARTIAL_HALF ? 1 : 0,
                              half_src ? 1 : 0));
  return B200MOE_OK;
}

}  // namespace b200moe
