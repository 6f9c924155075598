// Expert-parallel dispatch and combine (the reference is single-GPU and has neither).
//
// Dispatch: a token goes once to every rank that owns one of its eight experts.  The (token, destination) pairs are
// ranked with the same bit-matrix trick as the expert sort (sort.cu): chunk_bits[c][d] has bit j set when token 32c+j
// needs rank d, the per-destination prefix over chunks gives each pair its position, and the order — by destination,
// then by token id — is deterministic.  One warp then writes each 7456-byte record (activations, 56 scales, the eight
// expert ids and weights) into the send buffer, laid out so that a plain all-to-all with `send_counts` rows per
// destination delivers contiguous segments.  The receiver's kernels read the records in place through the strides of
// b200moe_problem.
//
// Combine: the float32 rows that come back in the same order are summed per token in slot order and rounded once.
#include "common.cuh"

namespace b200moe {

constexpr int EP_RECORD = B200MOE_EP_RECORD_BYTES;  // 7168 + 224 + 32 + 32
constexpr int ST_BAD_ADDRESS = 4;     // a kernel found a misaligned or out-of-range destination and skipped the access

int launch_rank_scan(const uint32_t* bits, int n_chunks, int E, int* base, int* counts, cudaStream_t st);
int launch_reduce_rows(const float* rows, const int* slot_map, int T, uint16_t* out, cudaStream_t st);
int launch_combine_half(const void* rows, const int* slot_map, int T, uint16_t* out, cudaStream_t st);

// chunk_bits over destination ranks: one warp per 32-token chunk, lane = token.
__global__ void __launch_bounds__(128)
k_dest_bits(const int* __restrict__ topk_idx, int T, int experts_per_rank, int world, int n_chunks,
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
      const int d = __ldg(topk_idx + static_cast<size_t>(t) * TOP_K + k) / experts_per_rank;
#pragma unroll
      for (int i = 0; i < E_GLOBAL / 32; ++i)
        if (i == (d >> 5)) mask[i] |= 1u << (d & 31);
    }
  }
#pragma unroll
  for (int i = 0; i < E_GLOBAL / 32; ++i) {
    if (i * 32 >= world) break;
    uint32_t mine = 0;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      uint32_t w = __ballot_sync(0xffffffffu, (mask[i] >> j) & 1u);
      if (lane == j) mine = w;
    }
    const int d = i * 32 + lane;
    if (d < world) chunk_bits[static_cast<size_t>(chunk) * world + d] = mine;
  }
}

// Record index of every (token, destination) pair: segment start of the destination + rank of the token inside it.
// slot_map[t,k] gets the index for the FIRST of the token's experts that lives on that destination, -1 for the others.
__global__ void __launch_bounds__(128)
k_dispatch_slots(const int* __restrict__ topk_idx, const uint32_t* __restrict__ chunk_bits,
                 const int* __restrict__ chunk_base, const int* __restrict__ counts, int T, int experts_per_rank,
                 int world, int n_chunks, int* __restrict__ send_counts, int* __restrict__ slot_token,
                 int* __restrict__ slot_map) {
  __shared__ int s_seg[E_GLOBAL + 1];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  pdl_launch_dependents();
  pdl_wait();
  if (warp == 0) {
    int c[8], local = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int d = lane * 8 + i;
      c[i] = (d < world) ? __ldg(counts + d) : 0;
      local += c[i];
    }
    int incl = local;
#pragma unroll
    for (int s = 1; s < 32; s <<= 1) {
      int o = __shfl_up_sync(0xffffffffu, incl, s);
      if (lane >= s) incl += o;
    }
    int run = incl - local;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int d = lane * 8 + i;
      if (d < world) s_seg[d] = run;
      run += c[i];
    }
  }
  __syncthreads();
  if (blockIdx.x == 0)
    for (int d = threadIdx.x; d < world; d += blockDim.x) send_counts[d] = __ldg(counts + d);

  const int chunk = blockIdx.x * (blockDim.x >> 5) + warp;
  if (chunk >= n_chunks) return;
  const int t = chunk * 32 + lane;
  if (t >= T) return;
  const uint32_t below = (1u << lane) - 1u;
  int dest[TOP_K], slot[TOP_K];
#pragma unroll
  for (int k = 0; k < TOP_K; ++k) {
    dest[k] = __ldg(topk_idx + static_cast<size_t>(t) * TOP_K + k) / experts_per_rank;
    bool first = true;
#pragma unroll
    for (int j = 0; j < k; ++j) first = first && (dest[j] != dest[k]);
    slot[k] = -1;
    if (first) {
      const int d = dest[k];
      const uint32_t bits = __ldg(chunk_bits + static_cast<size_t>(chunk) * world + d);
      const int s = s_seg[d] + __ldg(chunk_base + static_cast<size_t>(chunk) * world + d) + __popc(bits & below);
      slot[k] = s;
      slot_token[s] = t;
    }
  }
  int4* out = reinterpret_cast<int4*>(slot_map + static_cast<size_t>(t) * TOP_K);
  out[0] = make_int4(slot[0], slot[1], slot[2], slot[3]);
  out[1] = make_int4(slot[4], slot[5], slot[6], slot[7]);
}

// Where records go when they are written straight into the destinations' memory: segment d (records for rank d)
// starts at row row0[d] of base[d].
struct PeerTargets {
  uint8_t* base[8];
  int row0[8];
};

// One warp per record.  With send_rows the records form one local buffer in slot order; with send_rows == nullptr
// (world <= 8) each record is stored into its destination rank's receive buffer, which may be another GPU's memory.
__global__ void __launch_bounds__(256)
k_pack_records(const uint8_t* __restrict__ hidden, const float* __restrict__ hidden_scale,
               const int* __restrict__ topk_idx, const float* __restrict__ topk_w, int T, const int* __restrict__ counts,
               int world, const int* __restrict__ slot_token, uint8_t* __restrict__ send_rows, const PeerTargets peers,
               const b200moe_ep_plan* __restrict__ plan, int cap_recv, int* __restrict__ check) {
  const int lane = threadIdx.x & 31;
  const int warps_per_cta = blockDim.x >> 5;
  pdl_launch_dependents();
  pdl_wait();
  if (plan && !plan->ok) return;   // the counts did not fit the buffers (or the exchange timed out): store nothing
  int total = 0;
  int seg[9];
#pragma unroll
  for (int d = 0; d < 8; ++d) {
    seg[d] = total;
    if (d < world) total += __ldg(counts + d);
  }
  seg[8] = total;
  if (world > 8)
    for (int d = 8; d < world; ++d) total += __ldg(counts + d);
  // Peer stores: every rank starts with the records for the NEXT rank and wraps around.  In destination order all ranks
  // would write to rank 0 first, then all to rank 1, ...: one receiver's NVLink ingress shared by every sender.
  const int rot = (plan && !send_rows) ? seg[(plan->rank + 1) % world] : 0;
  for (int s0 = blockIdx.x * warps_per_cta + (threadIdx.x >> 5); s0 < total; s0 += gridDim.x * warps_per_cta) {
    const int s = (s0 + rot < total) ? s0 + rot : s0 + rot - total;
    const int tok = __ldg(slot_token + s);
    uint8_t* rec;
    if (send_rows) {
      rec = send_rows + static_cast<size_t>(s) * EP_RECORD;
    } else {
      int d = 0;
#pragma unroll
      for (int j = 1; j < 8; ++j)
        if (s >= seg[j]) d = j;
      const int row0 = plan ? plan->dst_row0[d] : peers.row0[d];
      rec = peers.base[d] + static_cast<size_t>(row0 + (s - seg[d])) * EP_RECORD;
      if (check && ((reinterpret_cast<uintptr_t>(rec) & 15u) || row0 < 0 || row0 + (s - seg[d]) >= cap_recv)) {
        // never store through an address that does not add up: record it and skip the record
        if (lane == 0 && atomicCAS(check, ST_OK, ST_BAD_ADDRESS) == ST_OK) {
          check[1] = 100 + d;
          check[2] = row0 + (s - seg[d]);
          check[3] = static_cast<int>(reinterpret_cast<uintptr_t>(rec) & 0xffff);
        }
        continue;
      }
    }
    const uint4* src = reinterpret_cast<const uint4*>(hidden + static_cast<size_t>(tok) * H);
    uint4* dst = reinterpret_cast<uint4*>(rec);
#pragma unroll
    for (int i = 0; i < H / 16 / 32; ++i) dst[i * 32 + lane] = __ldg(src + i * 32 + lane);
    float* sc = reinterpret_cast<float*>(rec + H);
    for (int kb = lane; kb < H_BLOCKS; kb += 32) sc[kb] = __ldg(hidden_scale + static_cast<size_t>(kb) * T + tok);
    if (lane < TOP_K) {
      reinterpret_cast<int*>(rec + H + 4 * H_BLOCKS)[lane] = __ldg(topk_idx + static_cast<size_t>(tok) * TOP_K + lane);
      reinterpret_cast<float*>(rec + H + 4 * H_BLOCKS + 4 * TOP_K)[lane] =
          __ldg(topk_w + static_cast<size_t>(tok) * TOP_K + lane);
    }
  }
  if (!send_rows) __threadfence_system();  // peer stores are visible system-wide before the barrier that follows
}

// Bounded all-rank barrier on flags mapped into every rank: publish `epoch`, then wait for everybody's.
constexpr int ST_BARRIER_TIMEOUT = 2;
constexpr int ST_PLAN_OVERFLOW = 3;
static long long g_wait_limit_cycles = WAIT_LIMIT_CYCLES;   // host side: limit handed to the barrier kernels

__global__ void __launch_bounds__(32)
k_ep_barrier(const PeerTargets flags /* base[r] = rank r's int flags[world] */, int world, int rank, int epoch,
             long long limit_cycles, int* __restrict__ status) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x;
  __threadfence_system();
  if (lane < world) {
    volatile int* remote = reinterpret_cast<volatile int*>(flags.base[lane]) + rank;
    *remote = epoch;
  }
  __threadfence_system();
  if (lane < world) {
    volatile int* mine = reinterpret_cast<volatile int*>(flags.base[rank]) + lane;
    const long long t0 = clock64();
    while (*mine < epoch) {
      if (clock64() - t0 > limit_cycles) {
        if (atomicCAS(status, ST_OK, ST_BARRIER_TIMEOUT) == ST_OK) {
          status[1] = rank;
          status[2] = lane;
          status[3] = epoch;
        }
        break;
      }
    }
  }
  __threadfence_system();
}

// The count exchange: row `rank` of every rank's count matrix <- send_counts, the flag barrier above, then thread 0
// turns this rank's (complete) matrix into the plan the following kernels read.  One CTA of 64 threads.
struct ExchangeTargets {
  int* flags[8];
  int* counts[8];
  float* back[8];
};
__global__ void __launch_bounds__(64)
k_ep_exchange(const ExchangeTargets tg, const int* __restrict__ send_counts, int world, int rank, int epoch,
              int cap_recv, int cap_back, int back_row_floats, long long limit_cycles,
              b200moe_ep_plan* __restrict__ plan, int* __restrict__ status) {
  __shared__ int s_timeout;
  pdl_launch_dependents();
  pdl_wait();
  const int tid = threadIdx.x;
  if (tid == 0) s_timeout = 0;
  if (tid < world * world) {
    const int d = tid / world, j = tid - d * world;
    volatile int* remote = reinterpret_cast<volatile int*>(tg.counts[d]) + rank * 8 + j;
    *remote = __ldg(send_counts + j);
  }
  __threadfence_system();
  __syncthreads();
  if (tid < world) {
    volatile int* remote = reinterpret_cast<volatile int*>(tg.flags[tid]) + rank;
    *remote = epoch;
  }
  __threadfence_system();
  if (tid < world) {
    volatile int* mine = reinterpret_cast<volatile int*>(tg.flags[rank]) + tid;
    const long long t0 = clock64();
    while (*mine < epoch) {
      if (clock64() - t0 > limit_cycles) {
        if (atomicCAS(status, ST_OK, ST_BARRIER_TIMEOUT) == ST_OK) {
          status[1] = rank;
          status[2] = tid;
          status[3] = epoch;
        }
        s_timeout = 1;
        break;
      }
    }
  }
  __threadfence_system();
  __syncthreads();
  if (tid == 0) {
    volatile const int* m = reinterpret_cast<volatile const int*>(tg.counts[rank]);
    int mm[8][8];
    bool ok = s_timeout == 0;
#pragma unroll
    for (int s = 0; s < 8; ++s)
#pragma unroll
      for (int d = 0; d < 8; ++d) {
        const int v = (s < world && d < world) ? m[s * 8 + d] : 0;
        mm[s][d] = v;
        if (v < 0) ok = false;
      }
    for (int x = 0; x < world && ok; ++x) {
      long long col = 0, row = 0;
      for (int y = 0; y < world; ++y) { col += mm[y][x]; row += mm[x][y]; }
      if (col > cap_recv || row > cap_back) ok = false;
    }
    if (!ok && s_timeout == 0 && atomicCAS(status, ST_OK, ST_PLAN_OVERFLOW) == ST_OK) {
      status[1] = rank;
      status[2] = cap_recv;
      status[3] = cap_back;
    }
    for (int x = 0; x < world; ++x)
      if ((reinterpret_cast<uintptr_t>(tg.back[x]) & 15u) || (reinterpret_cast<uintptr_t>(tg.counts[x]) & 3u)) {
        if (atomicCAS(status, ST_OK, ST_BAD_ADDRESS) == ST_OK) {
          status[1] = 200 + x;
          status[2] = static_cast<int>(reinterpret_cast<uintptr_t>(tg.back[x]) & 0xffff);
          status[3] = static_cast<int>(reinterpret_cast<uintptr_t>(tg.counts[x]) & 0xffff);
        }
        ok = false;
      }
    plan->ok = ok ? 1 : 0;
    plan->seg_count = world;
    plan->rank = rank;
    int n_recv = 0, n_send = 0;
    for (int s = 0; s < 8; ++s) {
      plan->seg_start[s] = n_recv;
      int before_me = 0;   // rows rank s sends to the ranks before this one: its return buffer keeps them first
      for (int d = 0; d < 8; ++d) {
        if (d < rank) before_me += ok ? mm[s][d] : 0;
        plan->matrix[s * 8 + d] = ok ? mm[s][d] : 0;
      }
      plan->seg_base[s] = (s < world) ? tg.back[s] + static_cast<size_t>(before_me) * back_row_floats : nullptr;
      if (ok && s < world) n_recv += mm[s][rank];
    }
    plan->seg_start[8] = n_recv;
    for (int d = 0; d < 8; ++d) {
      int r0 = 0;
      for (int s = 0; s < rank; ++s) r0 += ok ? mm[s][d] : 0;
      plan->dst_row0[d] = r0;
      if (ok && d < world) n_send += mm[rank][d];
    }
    plan->n_recv = n_recv;
    plan->n_send = n_send;
  }
}

}  // namespace b200moe

using namespace b200moe;

extern "C" {

int b200moe_ep_scratch_bytes(int32_t T, int32_t world, size_t* bytes) {
  if (!bytes || T < 0 || world < 1 || world > E_GLOBAL || E_GLOBAL % world) return B200MOE_EINVAL;
  const size_t n_chunks = (static_cast<size_t>(T) + 31) / 32;
  const size_t pairs = static_cast<size_t>(T) * (world < TOP_K ? world : TOP_K);
  // chunk_bits, chunk_base [n_chunks, world]; counts [world]; slot_token [pairs]; each rounded up to 256 bytes
  auto up = [](size_t x) { return (x + 255) / 256 * 256; };
  *bytes = 2 * up(4 * n_chunks * world) + up(4 * static_cast<size_t>(world)) + up(4 * pairs);
  return B200MOE_OK;
}

namespace {
struct Scratch {
  uint32_t* bits;
  int* cbase;
  int* counts;
  int* slot_token;
};
Scratch carve_scratch(void* scratch, int T, int world) {
  const size_t n_chunks = (static_cast<size_t>(T) + 31) / 32;
  auto up = [](size_t x) { return (x + 255) / 256 * 256; };
  uint8_t* base = static_cast<uint8_t*>(scratch);
  Scratch s;
  s.bits = reinterpret_cast<uint32_t*>(base);
  s.cbase = reinterpret_cast<int*>(base + up(4 * n_chunks * world));
  s.counts = reinterpret_cast<int*>(base + 2 * up(4 * n_chunks * world));
  s.slot_token = reinterpret_cast<int*>(base + 2 * up(4 * n_chunks * world) + up(4 * static_cast<size_t>(world)));
  return s;
}
int check_scratch(int32_t T, int32_t world, const void* scratch, size_t scratch_bytes) {
  size_t need = 0;
  int rc = b200moe_ep_scratch_bytes(T, world, &need);
  if (rc) return rc;
  if (T > 0 && (!scratch || scratch_bytes < need || (reinterpret_cast<uintptr_t>(scratch) & 255u)))
    return B200MOE_EWORKSPACE;
  return B200MOE_OK;
}
int launch_pack(const int32_t* topk_idx, const float* topk_w, const uint8_t* hidden_states,
                const float* hidden_states_scale, int32_t T, int32_t world, const Scratch& sc, uint8_t* send_rows,
                const PeerTargets& peers, const b200moe_ep_plan* plan, int cap_recv, int* check, cudaStream_t st) {
  long long max_pairs = static_cast<long long>(T) * (world < TOP_K ? world : TOP_K);
  int pgrid = static_cast<int>((max_pairs + 7) / 8);
  if (pgrid > 148 * 8) pgrid = 148 * 8;
  B200MOE_CUDA_TRY(launch_pdl(k_pack_records, dim3(pgrid), dim3(256), 0, st, hidden_states, hidden_states_scale,
                              topk_idx, topk_w, T, sc.counts, world, sc.slot_token, send_rows, peers, plan, cap_recv,
                              check));
  return B200MOE_OK;
}
}  // namespace

int b200moe_ep_rank(const int32_t* topk_idx, int32_t T, int32_t world, void* scratch, size_t scratch_bytes,
                    int32_t* send_counts, int32_t* slot_map, void* stream) {
  int rc = check_scratch(T, world, scratch, scratch_bytes);
  if (rc) return rc;
  if (!send_counts) return B200MOE_EINVAL;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (T == 0) {
    B200MOE_CUDA_TRY(cudaMemsetAsync(send_counts, 0, sizeof(int32_t) * world, st));
    return B200MOE_OK;
  }
  if (!topk_idx || !slot_map || (reinterpret_cast<uintptr_t>(slot_map) & 15u)) return B200MOE_EINVAL;
  const Scratch sc = carve_scratch(scratch, T, world);
  const int n_chunks = (T + 31) / 32;
  const int epr = E_GLOBAL / world;
  const int grid = (n_chunks + 3) / 4;
  B200MOE_CUDA_TRY(launch_pdl(k_dest_bits, dim3(grid), dim3(128), 0, st, topk_idx, T, epr, world, n_chunks, sc.bits));
  if ((rc = launch_rank_scan(sc.bits, n_chunks, world, sc.cbase, sc.counts, st))) return rc;
  B200MOE_CUDA_TRY(launch_pdl(k_dispatch_slots, dim3(grid), dim3(128), 0, st, topk_idx, sc.bits, sc.cbase, sc.counts, T,
                              epr, world, n_chunks, send_counts, sc.slot_token, slot_map));
  return B200MOE_OK;
}

int b200moe_ep_dispatch(const int32_t* topk_idx, const float* topk_w, const uint8_t* hidden_states,
                        const float* hidden_states_scale, int32_t T, int32_t world, void* scratch, size_t scratch_bytes,
                        uint8_t* send_rows, int32_t* send_counts, int32_t* slot_map, void* stream) {
  int rc = b200moe_ep_rank(topk_idx, T, world, scratch, scratch_bytes, send_counts, slot_map, stream);
  if (rc || T == 0) return rc;
  if (!topk_w || !hidden_states || !hidden_states_scale || !send_rows) return B200MOE_EINVAL;
  if ((reinterpret_cast<uintptr_t>(send_rows) & 15u) || (reinterpret_cast<uintptr_t>(hidden_states) & 15u))
    return B200MOE_EINVAL;
  PeerTargets none = {};
  return launch_pack(topk_idx, topk_w, hidden_states, hidden_states_scale, T, world, carve_scratch(scratch, T, world),
                     send_rows, none, nullptr, 0, nullptr, static_cast<cudaStream_t>(stream));
}

int b200moe_ep_pack_peers(const int32_t* topk_idx, const float* topk_w, const uint8_t* hidden_states,
                          const float* hidden_states_scale, int32_t T, const b200moe_ep_peers* peers,
                          const int32_t* dst_row0, void* scratch, size_t scratch_bytes, void* stream) {
  if (!peers || !dst_row0 || peers->world < 1 || peers->world > 8) return B200MOE_EINVAL;
  int rc = check_scratch(T, peers->world, scratch, scratch_bytes);
  if (rc || T == 0) return rc;
  if (!topk_idx || !topk_w || !hidden_states || !hidden_states_scale) return B200MOE_EINVAL;
  if (reinterpret_cast<uintptr_t>(hidden_states) & 15u) return B200MOE_EINVAL;
  PeerTargets tg = {};
  for (int d = 0; d < peers->world; ++d) {
    if (!peers->recv_records[d] || (reinterpret_cast<uintptr_t>(peers->recv_records[d]) & 15u) || dst_row0[d] < 0)
      return B200MOE_EINVAL;
    tg.base[d] = peers->recv_records[d];
    tg.row0[d] = dst_row0[d];
  }
  return launch_pack(topk_idx, topk_w, hidden_states, hidden_states_scale, T, peers->world,
                     carve_scratch(scratch, T, peers->world), nullptr, tg, nullptr, 0, nullptr,
                     static_cast<cudaStream_t>(stream));
}

int b200moe_ep_pack_peers_planned(const int32_t* topk_idx, const float* topk_w, const uint8_t* hidden_states,
                                  const float* hidden_states_scale, int32_t T, const b200moe_ep_peers* peers,
                                  const b200moe_ep_plan* plan, void* scratch, size_t scratch_bytes, int32_t* status,
                                  void* stream) {
  if (!peers || !plan || !status || peers->world < 1 || peers->world > 8) return B200MOE_EINVAL;
  int rc = check_scratch(T, peers->world, scratch, scratch_bytes);
  if (rc || T == 0) return rc;
  if (!topk_idx || !topk_w || !hidden_states || !hidden_states_scale) return B200MOE_EINVAL;
  if (reinterpret_cast<uintptr_t>(hidden_states) & 15u) return B200MOE_EINVAL;
  PeerTargets tg = {};
  for (int d = 0; d < peers->world; ++d) {
    if (!peers->recv_records[d] || (reinterpret_cast<uintptr_t>(peers->recv_records[d]) & 15u)) return B200MOE_EINVAL;
    tg.base[d] = peers->recv_records[d];
  }
  return launch_pack(topk_idx, topk_w, hidden_states, hidden_states_scale, T, peers->world,
                     carve_scratch(scratch, T, peers->world), nullptr, tg, plan, peers->cap_recv, status,
                     static_cast<cudaStream_t>(stream));
}

int b200moe_ep_exchange_counts(const b200moe_ep_peers* peers, const int32_t* send_counts, int32_t epoch,
                               b200moe_ep_plan* plan, int32_t* status, void* stream) {
  if (!peers || !send_counts || !plan || !status || peers->world < 1 || peers->world > 8 || peers->rank < 0 ||
      peers->rank >= peers->world || peers->cap_recv < 0 || peers->cap_back < 0 ||
      (peers->back_row_bytes != 0 && peers->back_row_bytes != H * 4 && peers->back_row_bytes != B200MOE_HALF_ROW_BYTES))
    return B200MOE_EINVAL;
  if (reinterpret_cast<uintptr_t>(plan) & 7u) return B200MOE_EINVAL;
  ExchangeTargets tg = {};
  for (int d = 0; d < peers->world; ++d) {
    if (!peers->flags[d] || !peers->counts[d] || !peers->back_rows[d] ||
        (reinterpret_cast<uintptr_t>(peers->back_rows[d]) & 15u))
      return B200MOE_EINVAL;
    tg.flags[d] = peers->flags[d];
    tg.counts[d] = peers->counts[d];
    tg.back[d] = peers->back_rows[d];
  }
  B200MOE_CUDA_TRY(launch_pdl(k_ep_exchange, dim3(1), dim3(64), 0, static_cast<cudaStream_t>(stream), tg, send_counts,
                              peers->world, peers->rank, epoch, peers->cap_recv, peers->cap_back,
                              (peers->back_row_bytes ? peers->back_row_bytes : H * 4) / 4, g_wait_limit_cycles,
                              plan, status));
  return B200MOE_OK;
}

int b200moe_set_wait_limit_cycles(int64_t cycles) {
  if (cycles < 0) return B200MOE_EINVAL;
  g_wait_limit_cycles = cycles == 0 ? WAIT_LIMIT_CYCLES : static_cast<long long>(cycles);
  return B200MOE_OK;
}

int b200moe_ep_barrier(const b200moe_ep_peers* peers, int32_t epoch, int32_t* status, void* stream) {
  if (!peers || !status || peers->world < 1 || peers->world > 8 || peers->rank < 0 || peers->rank >= peers->world)
    return B200MOE_EINVAL;
  PeerTargets fl = {};
  for (int d = 0; d < peers->world; ++d) {
    if (!peers->flags[d]) return B200MOE_EINVAL;
    fl.base[d] = reinterpret_cast<uint8_t*>(peers->flags[d]);
  }
  B200MOE_CUDA_TRY(launch_pdl(k_ep_barrier, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream), fl, peers->world,
                              peers->rank, epoch, g_wait_limit_cycles, status));
  return B200MOE_OK;
}

int b200moe_ep_record_layout(const uint8_t* records, int32_t n, b200moe_problem* p) {
  if (!p || n < 0 || (n > 0 && !records)) return B200MOE_EINVAL;
  p->T = n;
  p->routing_logits = nullptr;
  p->routing_bias = nullptr;
  p->hidden_states = records;
  p->hidden_row_stride = EP_RECORD;
  p->hidden_states_scale = reinterpret_cast<const float*>(records + H);
  p->scale_token_stride = EP_RECORD / 4;
  p->scale_block_stride = 1;
  p->topk_idx_in = reinterpret_cast<const int32_t*>(records + H + 4 * H_BLOCKS);
  p->topk_w_in = reinterpret_cast<const float*>(records + H + 4 * H_BLOCKS + 4 * TOP_K);
  p->topk_row_stride = EP_RECORD / 4;
  return B200MOE_OK;
}

int b200moe_ep_combine(const float* returned_rows, const int32_t* slot_map, int32_t T, uint16_t* output,
                       void* stream) {
  if (T < 0) return B200MOE_EINVAL;
  if (T == 0) return B200MOE_OK;
  if (!returned_rows || !slot_map || !output) return B200MOE_EINVAL;
  if ((reinterpret_cast<uintptr_t>(returned_rows) & 15u) || (reinterpret_cast<uintptr_t>(output) & 15u))
    return B200MOE_EINVAL;
  return launch_reduce_rows(returned_rows, slot_map, T, output, static_cast<cudaStream_t>(stream));
}

int b200moe_ep_combine_half(const void* returned_rows, const int32_t* slot_map, int32_t T, uint16_t* output,
                            void* stream) {
  if (T < 0) return B200MOE_EINVAL;
  if (T == 0) return B200MOE_OK;
  if (!returned_rows || !slot_map || !output) return B200MOE_EINVAL;
  if ((reinterpret_cast<uintptr_t>(returned_rows) & 15u) || (reinterpret_cast<uintptr_t>(output) & 15u))
    return B200MOE_EINVAL;
  return launch_combine_half(returned_rows, slot_map, T, output, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
