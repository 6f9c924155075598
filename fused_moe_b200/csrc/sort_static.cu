// b200moe_sort_static: the token sort (chunk bits -> per-expert prefix -> padded layout -> stable scatter) for callers
// that may not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc at all: a serving process that has handed every byte of HBM to its
// own pool allocator, a plugin loaded into a process whose memory budget is fixed at start-up, code that runs inside a
// region where allocation is forbidden.  b200moe_sort needs two scratch tables (which tokens of each 32-token chunk
// chose each local expert, and the running per-expert counts before each chunk); here they live in a fixed array that
// is part of the library image, so the call touches no allocator — not cudaMalloc, not cudaFree, not torch's.
//
// The price: the array has a fixed capacity (B200MOE_SORT_STATIC_MAX_ENTRIES chunk-expert pairs; larger problems are
// refused with B200MOE_ETOOLARGE), every GPU that loads the library holds its 256 KB until the process exits, and all
// calls on one GPU share it — two calls whose kernels overlap on the device race on it; run them on one stream or
// order them yourself.  Nothing in the array has to start at zero: every entry a call reads is written by that call
// first, so leftovers from the previous call are harmless.
#include "common.cuh"

namespace b200moe {

int launch_topk_bits(const b200moe_problem*, const b200moe_workspace*, cudaStream_t);
int launch_sort(const b200moe_problem*, const b200moe_workspace*, cudaStream_t);

// [0, MAX) = chunk_bits, [MAX, 2*MAX) = chunk_base.  In host code this name is only a handle for
// cudaGetSymbolAddress; the device address is looked up once per GPU below.
static __device__ __align__(256) uint32_t g_sort_scratch[2 * B200MOE_SORT_STATIC_MAX_ENTRIES];

static uint32_t* g_scratch_addr[64] = {};

// Device address of the scratch array on the CURRENT device, resolved on first use.
static int scratch_for_current_device(uint32_t** out) {
  int dev = 0;
  B200MOE_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return B200MOE_EINVAL;
  if (!g_scratch_addr[dev]) {
    void* p = nullptr;
    B200MOE_CUDA_TRY(cudaGetSymbolAddress(&p, g_sort_scratch));
    if (!p) return record_cuda_error(cudaErrorInvalidSymbol);
    g_scratch_addr[dev] = static_cast<uint32_t*>(p);
  }
  *out = g_scratch_addr[dev];
  return B200MOE_OK;
}

}  // namespace b200moe

using namespace b200moe;

extern "C" int b200moe_sort_static(const int32_t* topk_idx, const float* topk_w, int32_t T, int32_t E_local,
                                   int32_t local_expert_offset, int32_t* counts, int32_t* block_offsets,
                                   int32_t* total_blocks, int32_t* sorted_token_ids, float* sorted_weights,
                                   int32_t* scatter_map, void* stream) {
  if (T < 0 || E_local < 1 || E_local > E_GLOBAL) return B200MOE_EINVAL;
  if (local_expert_offset < 0 || local_expert_offset + E_local > E_GLOBAL) return B200MOE_EINVAL;
  if (!counts || !block_offsets || !total_blocks) return B200MOE_EINVAL;
  if (T > 0 && (!topk_idx || !topk_w || !sorted_token_ids || !sorted_weights || !scatter_map)) return B200MOE_EINVAL;
  if (T > 0 && (reinterpret_cast<uintptr_t>(scatter_map) & 15u)) return B200MOE_EINVAL;
  const long long n_chunks = (static_cast<long long>(T) + 31) / 32;
  if (n_chunks * E_local > B200MOE_SORT_STATIC_MAX_ENTRIES) return B200MOE_ETOOLARGE;

  int major = 0, dev = 0;
  B200MOE_CUDA_TRY(cudaGetDevice(&dev));
  B200MOE_CUDA_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
  if (major != 10) return B200MOE_EUNSUPPORTED;

  uint32_t* scratch = nullptr;
  int rc = scratch_for_current_device(&scratch);
  if (rc) return rc;

  b200moe_problem p = {};
  p.T = T;
  p.E_local = E_local;
  p.local_expert_offset = local_expert_offset;
  p.topk_idx_in = topk_idx;
  p.topk_w_in = topk_w;  // routing_logits stays NULL: the sort reads the caller's (ids, weights)

  b200moe_workspace ws = {};
  ws.T = T;
  ws.E_local = E_local;
  ws.n_chunks = static_cast<int32_t>(n_chunks);
  ws.chunk_bits = scratch;
  ws.chunk_base = reinterpret_cast<int32_t*>(scratch + B200MOE_SORT_STATIC_MAX_ENTRIES);
  ws.counts = counts;
  ws.block_offsets = block_offsets;
  ws.total_blocks = total_blocks;
  ws.sorted_token_ids = sorted_token_ids;
  ws.sorted_weights = sorted_weights;
  ws.scatter_map = scatter_map;

  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if ((rc = launch_topk_bits(&p, &ws, st))) return rc;
  return launch_sort(&p, &ws, st);
}
