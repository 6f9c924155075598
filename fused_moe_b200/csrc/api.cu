// C ABI of libb200moe.so (declared in include/b200moe.h): argument checks, workspace carving, stage launches.
#include <string.h>

#include "common.cuh"

namespace b200moe {

static thread_local char g_cuda_err[256] = "";

int record_cuda_error(cudaError_t e) {
  const char* s = cudaGetErrorString(e);
  strncpy(g_cuda_err, s ? s : "unknown CUDA error", sizeof(g_cuda_err) - 1);
  g_cuda_err[sizeof(g_cuda_err) - 1] = 0;
  return B200MOE_ECUDA;
}

int launch_route(const b200moe_problem*, const b200moe_workspace*, cudaStream_t);
int launch_topk_bits(const b200moe_problem*, const b200moe_workspace*, cudaStream_t);
int launch_route_topk(const float*, const uint16_t*, int, float, int*, float*, cudaStream_t);
int launch_small_prologue(const b200moe_problem*, const b200moe_workspace*, cudaStream_t);
int launch_sort(const b200moe_problem*, const b200moe_workspace*, cudaStream_t);
int launch_gather(const b200moe_problem*, const b200moe_workspace*, int, cudaStream_t);
int launch_gemm1(const b200moe_problem*, const b200moe_workspace*, int, cudaStream_t);
int launch_gemm2(const b200moe_problem*, const b200moe_workspace*, int, cudaStream_t, bool half_out);
int launch_quantize_act(const void*, int, void*, float*, int, cudaStream_t);
int launch_gemm1_skinny(const b200moe_problem*, const b200moe_workspace*, int, cudaStream_t, bool);
int launch_gemm2_skinny(const b200moe_problem*, const b200moe_workspace*, int, cudaStream_t, bool);
int launch_reduce(const b200moe_problem*, const b200moe_workspace*, cudaStream_t, bool half_src);
int launch_gemv1(const b200moe_problem*, const b200moe_workspace*, int, cudaStream_t);
int launch_gemv2(const b200moe_problem*, const b200moe_workspace*, int, cudaStream_t);

struct DeviceInfo {
  int checked = 0;  // 0 unknown, 1 ok, -1 unsupported
  int num_sms = 0;
};

// Per-device facts, looked up once (the current device must be an sm_100 part).
static int device_info(int* num_sms) {
  static DeviceInfo info[64];
  int dev = 0;
  B200MOE_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return B200MOE_EINVAL;
  if (!info[dev].checked) {
    int major = 0, sms = 0;
    B200MOE_CUDA_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
    B200MOE_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    info[dev].num_sms = sms;
    info[dev].checked = (major == 10) ? 1 : -1;
  }
  if (info[dev].checked < 0) return B200MOE_EUNSUPPORTED;
  *num_sms = info[dev].num_sms;
  return B200MOE_OK;
}

static size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

static int r_max_for(int T, int E) {
  long long blocks = (8LL * T) / BLOCK_M + E;
  return static_cast<int>(blocks * BLOCK_M);
}

// Token-minor GEMM tiles: at most R_max / 64 sub-blocks of sorted rows x 28 n-tiles (GEMM2; GEMM1 has 16).
static size_t tile_ctr_count(size_t r_max) { return r_max / 64 * 28; }

// Walks the workspace layout; with base == nullptr only the total is computed.
static size_t layout(uint8_t* base, int T, int E, b200moe_workspace* w) {
  const size_t R = static_cast<size_t>(r_max_for(T, E));
  const size_t n_chunks = (static_cast<size_t>(T) + 31) / 32;
  size_t off = 0;
  auto take = [&](size_t bytes) -> uint8_t* {
    uint8_t* p = base ? base + off : nullptr;
    off = align_up(off + bytes, 256);
    return p;
  };
  uint8_t* topk_idx = take(sizeof(int32_t) * 8 * T);
  uint8_t* topk_w = take(sizeof(float) * 8 * T);
  uint8_t* chunk_bits = take(sizeof(uint32_t) * n_chunks * E);
  uint8_t* chunk_base = take(sizeof(int32_t) * n_chunks * E);
  uint8_t* counts = take(sizeof(int32_t) * E);
  uint8_t* block_offsets = take(sizeof(int32_t) * (E + 1));
  uint8_t* total_blocks = take(sizeof(int32_t));
  uint8_t* status = take(sizeof(int32_t) * 4);
  uint8_t* sorted_token_ids = take(sizeof(int32_t) * R);
  uint8_t* sorted_weights = take(sizeof(float) * R);
  uint8_t* scatter_map = take(sizeof(int32_t) * 8 * T);
  uint8_t* a_sorted = take(R * H);
  uint8_t* a_scale_sorted = take(sizeof(float) * H_BLOCKS * R);
  uint8_t* inter_q = take(2 * R * I);
  uint8_t* inter_scale = take(sizeof(float) * I_BLOCKS * R);
  uint8_t* expert_out = take(sizeof(float) * R * H);
  uint8_t* gemm_tile_ctr = take(sizeof(int32_t) * tile_ctr_count(R));
  uint8_t* gemm_partial = take(sizeof(float) * B200MOE_GEMM_MAX_CTAS * 2 * (2 * 64 * 128));
  if (w) {
    w->T = T;
    w->E_local = E;
    w->R_max = static_cast<int32_t>(R);
    w->n_chunks = static_cast<int32_t>(n_chunks);
    w->topk_idx = reinterpret_cast<int32_t*>(topk_idx);
    w->topk_w = reinterpret_cast<float*>(topk_w);
    w->chunk_bits = reinterpret_cast<uint32_t*>(chunk_bits);
    w->chunk_base = reinterpret_cast<int32_t*>(chunk_base);
    w->counts = reinterpret_cast<int32_t*>(counts);
    w->block_offsets = reinterpret_cast<int32_t*>(block_offsets);
    w->total_blocks = reinterpret_cast<int32_t*>(total_blocks);
    w->status = reinterpret_cast<int32_t*>(status);
    w->sorted_token_ids = reinterpret_cast<int32_t*>(sorted_token_ids);
    w->sorted_weights = reinterpret_cast<float*>(sorted_weights);
    w->scatter_map = reinterpret_cast<int32_t*>(scatter_map);
    w->a_sorted = a_sorted;
    w->a_scale_sorted = reinterpret_cast<float*>(a_scale_sorted);
    w->inter_q = inter_q;
    w->inter_scale = reinterpret_cast<float*>(inter_scale);
    w->expert_out = reinterpret_cast<float*>(expert_out);
    w->gemm_tile_ctr = reinterpret_cast<int32_t*>(gemm_tile_ctr);
    w->gemm_partial = reinterpret_cast<float*>(gemm_partial);
    w->status_mirror = nullptr;
  }
  return off;
}

static int check_dims(int T, int E) {
  if (T < 0 || T > (1 << 24)) return B200MOE_EINVAL;
  if (E < 1 || E > E_GLOBAL) return B200MOE_EINVAL;
  return B200MOE_OK;
}

static int check_problem(const b200moe_problem* p, const b200moe_workspace* ws) {
  if (!p || !ws) return B200MOE_EINVAL;
  int rc = check_dims(p->T, p->E_local);
  if (rc) return rc;
  if (ws->T != p->T || ws->E_local != p->E_local || !ws->status) return B200MOE_EWORKSPACE;
  if (p->local_expert_offset < 0 || p->local_expert_offset + p->E_local > E_GLOBAL) return B200MOE_EINVAL;
  return B200MOE_OK;
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace b200moe

using namespace b200moe;

extern "C" {

int b200moe_version(void) { return 100; }

const char* b200moe_strerror(int code) {
  switch (code) {
    case B200MOE_OK: return "ok";
    case B200MOE_EINVAL: return "invalid argument";
    case B200MOE_EWORKSPACE: return "workspace too small, misaligned or carved for other sizes";
    case B200MOE_ECUDA: return "CUDA call failed";
    case B200MOE_EDEVICE: return "device status word reports a failed kernel";
    case B200MOE_EUNSUPPORTED: return "current device is not an sm_100 GPU";
    case B200MOE_ETOOLARGE: return "problem exceeds the fixed scratch capacity of this entry point";
    default: return "unknown error";
  }
}

const char* b200moe_last_cuda_error(void) { return g_cuda_err; }

int b200moe_workspace_bytes(int32_t T, int32_t E_local, size_t* bytes) {
  if (!bytes) return B200MOE_EINVAL;
  int rc = check_dims(T, E_local);
  if (rc) return rc;
  *bytes = layout(nullptr, T, E_local, nullptr);
  return B200MOE_OK;
}

int b200moe_workspace_carve(void* base, size_t bytes, int32_t T, int32_t E_local, b200moe_workspace* out) {
  if (!base || !out) return B200MOE_EINVAL;
  int rc = check_dims(T, E_local);
  if (rc) return rc;
  if (reinterpret_cast<uintptr_t>(base) & 255u) return B200MOE_EWORKSPACE;
  if (layout(nullptr, T, E_local, nullptr) > bytes) return B200MOE_EWORKSPACE;
  layout(static_cast<uint8_t*>(base), T, E_local, out);
  return B200MOE_OK;
}

int b200moe_workspace_init(const b200moe_workspace* ws, void* stream) {
  if (!ws || !ws->status) return B200MOE_EINVAL;
  B200MOE_CUDA_TRY(cudaMemsetAsync(ws->status, 0, sizeof(int32_t) * 4, static_cast<cudaStream_t>(stream)));
  if (ws->gemm_tile_ctr)
    B200MOE_CUDA_TRY(cudaMemsetAsync(ws->gemm_tile_ctr, 0, sizeof(int32_t) * tile_ctr_count(ws->R_max),
                                     static_cast<cudaStream_t>(stream)));
  return B200MOE_OK;
}

int b200moe_quantize_act(const void* x_bf16, int32_t T, void* q_out, float* scale_out, void* stream) {
  if (T < 0 || T > (1 << 24)) return B200MOE_EINVAL;
  if (T > 0 && (!x_bf16 || !q_out || !scale_out)) return B200MOE_EINVAL;
  if (T > 0 && ((reinterpret_cast<uintptr_t>(x_bf16) & 15u) || (reinterpret_cast<uintptr_t>(q_out) & 7u)))
    return B200MOE_EINVAL;
  int sms, rc;
  if ((rc = device_info(&sms))) return rc;
  return launch_quantize_act(x_bf16, T, q_out, scale_out, sms, static_cast<cudaStream_t>(stream));
}

int b200moe_route(const b200moe_problem* p, const b200moe_workspace* ws, void* stream) {
  int rc = check_problem(p, ws);
  if (rc) return rc;
  if (p->T > 0 && (!p->routing_logits || !p->routing_bias)) return B200MOE_EINVAL;
  int sms;
  if ((rc = device_info(&sms))) return rc;
  return launch_route(p, ws, static_cast<cudaStream_t>(stream));
}

int b200moe_route_topk(const float* routing_logits, const uint16_t* routing_bias, int32_t T,
                       float routed_scaling_factor, int32_t* topk_idx, float* topk_w, void* stream) {
  if (T < 0 || T > (1 << 24)) return B200MOE_EINVAL;
  if (T > 0 && (!routing_logits || !routing_bias || !topk_idx || !topk_w)) return B200MOE_EINVAL;
  int sms, rc;
  if ((rc = device_info(&sms))) return rc;
  return launch_route_topk(routing_logits, routing_bias, T, routed_scaling_factor, topk_idx, topk_w,
                           static_cast<cudaStream_t>(stream));
}

int b200moe_topk_bits(const b200moe_problem* p, const b200moe_workspace* ws, void* stream) {
  int rc = check_problem(p, ws);
  if (rc) return rc;
  int sms;
  if ((rc = device_info(&sms))) return rc;
  return launch_topk_bits(p, ws, static_cast<cudaStream_t>(stream));
}

int b200moe_sort(const b200moe_problem* p, const b200moe_workspace* ws, void* stream) {
  int rc = check_problem(p, ws);
  if (rc) return rc;
  if (p->T > 0 && !p->routing_logits && (!p->topk_idx_in || !p->topk_w_in)) return B200MOE_EINVAL;
  int sms;
  if ((rc = device_info(&sms))) return rc;
  return launch_sort(p, ws, static_cast<cudaStream_t>(stream));
}

int b200moe_gather(const b200moe_problem* p, const b200moe_workspace* ws, void* stream) {
  int rc = check_problem(p, ws);
  if (rc) return rc;
  if (p->T > 0 && (!p->hidden_states || !p->hidden_states_scale || !aligned16(p->hidden_states)))
    return B200MOE_EINVAL;
  int sms;
  if ((rc = device_info(&sms))) return rc;
  return launch_gather(p, ws, sms, static_cast<cudaStream_t>(stream));
}

int b200moe_prologue_small(const b200moe_problem* p, const b200moe_workspace* ws, void* stream) {
  int rc = check_problem(p, ws);
  if (rc) return rc;
  if (p->T > B200MOE_PROLOGUE_MAX_T) return B200MOE_ETOOLARGE;
  if (p->hidden_row_stride || p->scale_token_stride || p->scale_block_stride) return B200MOE_EINVAL;
  if (p->T > 0 && (!p->routing_logits || !p->routing_bias || !p->hidden_states || !p->hidden_states_scale ||
                   !aligned16(p->hidden_states)))
    return B200MOE_EINVAL;
  return launch_small_prologue(p, ws, static_cast<cudaStream_t>(stream));
}

int b200moe_gemm1(const b200moe_problem* p, const b200moe_workspace* ws, void* stream) {
  int rc = check_problem(p, ws);
  if (rc) return rc;
  if (p->T > 0 && (!p->gemm1_weights || !p->gemm1_weights_scale || !aligned16(p->gemm1_weights)))
    return B200MOE_EINVAL;
  int sms;
  if ((rc = device_info(&sms))) return rc;
  return launch_gemm1(p, ws, sms, static_cast<cudaStream_t>(stream));
}

static int gemm2_stage(const b200moe_problem* p, const b200moe_workspace* ws, void* stream, bool half_out) {
  int rc = check_problem(p, ws);
  if (rc) return rc;
  if (p->T > 0 && (!p->gemm2_weights || !p->gemm2_weights_scale || !aligned16(p->gemm2_weights)))
    return B200MOE_EINVAL;
  int sms;
  if ((rc = device_info(&sms))) return rc;
  return launch_gemm2(p, ws, sms, static_cast<cudaStream_t>(stream), half_out);
}
int b200moe_gemm2(const b200moe_problem* p, const b200moe_workspace* ws, void* stream) {
  return gemm2_stage(p, ws, stream, false);
}
int b200moe_gemm2_half(const b200moe_problem* p, const b200moe_workspace* ws, void* stream) {
  return gemm2_stage(p, ws, stream, true);
}

int b200moe_gemm1_skinny(const b200moe_problem* p, const b200moe_workspace* ws, void* stream) {
  int rc = check_problem(p, ws);
  if (rc) return rc;
  if (p->T > 0 && (!p->gemm1_weights || !p->gemm1_weights_scale || !aligned16(p->gemm1_weights)))
    return B200MOE_EINVAL;
  int sms;
  if ((rc = device_info(&sms))) return rc;
  return launch_gemm1_skinny(p, ws, sms, static_cast<cudaStream_t>(stream), false);
}

int b200moe_gemm2_skinny(const b200moe_problem* p, const b200moe_workspace* ws, void* stream) {
  int rc = check_problem(p, ws);
  if (rc) return rc;
  if (p->T > 0 && (!p->gemm2_weights || !p->gemm2_weights_scale || !aligned16(p->gemm2_weights)))
    return B200MOE_EINVAL;
  int sms;
  if ((rc = device_info(&sms))) return rc;
  return launch_gemm2_skinny(p, ws, sms, static_cast<cudaStream_t>(stream), false);
}

int b200moe_gemv1(const b200moe_problem* p, const b200moe_workspace* ws, void* stream) {
  int rc = check_problem(p, ws);
  if (rc) return rc;
  if (p->T > B200MOE_DECODE_MAX_T) return B200MOE_EINVAL;
  if (p->T > 0 && (!p->hidden_states || !p->hidden_states_scale || !p->gemm1_weights || !p->gemm1_weights_scale ||
                   !aligned16(p->hidden_states) || !aligned16(p->gemm1_weights)))
    return B200MOE_EINVAL;
  int sms;
  if ((rc = device_info(&sms))) return rc;
  return launch_gemv1(p, ws, sms, static_cast<cudaStream_t>(stream));
}

int b200moe_gemv2(const b200moe_problem* p, const b200moe_workspace* ws, void* stream) {
  int rc = check_problem(p, ws);
  if (rc) return rc;
  if (p->T > B200MOE_DECODE_MAX_T) return B200MOE_EINVAL;
  if (p->T > 0 && (!p->gemm2_weights || !p->gemm2_weights_scale || !aligned16(p->gemm2_weights) ||
                   (!p->output && !p->output_f32)))
    return B200MOE_EINVAL;
  int sms;
  if ((rc = device_info(&sms))) return rc;
  return launch_gemv2(p, ws, sms, static_cast<cudaStream_t>(stream));
}

static int reduce_stage(const b200moe_problem* p, const b200moe_workspace* ws, void* stream, bool half_src) {
  int rc = check_problem(p, ws);
  if (rc) return rc;
  if (p->T > 0 && p->out_seg_count == 0 && !p->plan &&
      ((!p->output && !p->output_f32) || !aligned16(p->output) || !aligned16(p->output_f32)))
    return B200MOE_EINVAL;
  if (p->out_seg_count < 0 || p->out_seg_count > 8) return B200MOE_EINVAL;
  if (p->partial_format != B200MOE_PARTIAL_F32 && p->partial_format != B200MOE_PARTIAL_HALF) return B200MOE_EINVAL;
  int sms;
  if ((rc = device_info(&sms))) return rc;
  return launch_reduce(p, ws, static_cast<cudaStream_t>(stream), half_src);
}

int b200moe_reduce(const b200moe_problem* p, const b200moe_workspace* ws, void* stream) {
  return reduce_stage(p, ws, stream, false);
}
int b200moe_reduce_half(const b200moe_problem* p, const b200moe_workspace* ws, void* stream) {
  return reduce_stage(p, ws, stream, true);
}

int b200moe_forward(const b200moe_problem* p, const b200moe_workspace* ws, void* stream) {
  int rc = check_problem(p, ws);
  if (rc) return rc;
  if (p->T == 0) return B200MOE_OK;
  if (!p->hidden_states || !p->hidden_states_scale || !p->gemm1_weights || !p->gemm1_weights_scale ||
      !p->gemm2_weights || !p->gemm2_weights_scale ||
      (!p->output && !p->output_f32 && p->out_seg_count == 0 && !p->plan))
    return B200MOE_EINVAL;
  if (p->plan && p->routing_logits) return B200MOE_EINVAL;  // a device-side plan describes received records only
  if (!aligned16(p->hidden_states) || !aligned16(p->gemm1_weights) || !aligned16(p->gemm2_weights) ||
      !aligned16(p->output) || !aligned16(p->output_f32))
    return B200MOE_EINVAL;
  if (p->routing_logits) {
    if (!p->routing_bias) return B200MOE_EINVAL;
  } else if (!p->topk_idx_in || !p->topk_w_in) {
    return B200MOE_EINVAL;
  }
  if (p->out_seg_count < 0 || p->out_seg_count > 8) return B200MOE_EINVAL;
  if (p->partial_format != B200MOE_PARTIAL_F32 && p->partial_format != B200MOE_PARTIAL_HALF) return B200MOE_EINVAL;
  for (int i = 0; i < p->out_seg_count; ++i)
    if (!p->out_seg_base[i] || !aligned16(p->out_seg_base[i]) || p->out_seg_start[i] > p->out_seg_start[i + 1])
      return B200MOE_EINVAL;
  int sms;
  if ((rc = device_info(&sms))) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (p->routing_logits && p->T <= B200MOE_DECODE_MAX_T && p->T * p->E_local <= B200MOE_DECODE_MAX_WORK &&
      p->out_seg_count == 0 && !p->hidden_row_stride &&
      !p->scale_token_stride && !p->scale_block_stride) {
    // decode: a few tokens, one or two rows per expert — stream the weights through matrix-vector kernels
    if ((rc = launch_route(p, ws, st))) return rc;
    if ((rc = launch_gemv1(p, ws, sms, st))) return rc;
    return launch_gemv2(p, ws, sms, st);
  }
  bool after_gather = false;   // GEMM1 directly follows k_gather (whose release tells it the sort is complete)
  if (p->routing_logits && p->T <= B200MOE_PROLOGUE_MAX_T && !p->hidden_row_stride && !p->scale_token_stride && !p->scale_block_stride) {
    // small batch: routing, ranking, layout, scatter and gather in one single-CTA kernel (same results)
    if ((rc = launch_small_prologue(p, ws, st))) return rc;
  } else {
    after_gather = true;
    if (p->routing_logits) {
      if ((rc = launch_route(p, ws, st))) return rc;
    } else {
      if ((rc = launch_topk_bits(p, ws, st))) return rc;
    }
    if ((rc = launch_sort(p, ws, st))) return rc;
    if ((rc = launch_gather(p, ws, sms, st))) return rc;
  }
  // Few rows per expert (8 T / 256 per expert on average): token-minor tiles, bound by streaming the weights; else
  // 128-token tiles.  Both kernels are correct for every batch; the choice is about speed only.
  if (p->T <= B200MOE_SKINNY_MAX_T) {
    if ((rc = launch_gemm1_skinny(p, ws, sms, st, after_gather))) return rc;
    if ((rc = launch_gemm2_skinny(p, ws, sms, st, true))) return rc;
    return launch_reduce(p, ws, st, false);
  }
  if ((rc = launch_gemm1(p, ws, sms, st))) return rc;
  // Between the tile GEMM2 and the reduce of one call the per-expert rows live in the half form (eight float16 per
  // power-of-two scale byte): the two kernels are bound by writing and reading them.  (The stage entry points
  // b200moe_gemm2 / b200moe_reduce keep float32 rows.)
  if ((rc = launch_gemm2(p, ws, sms, st, true))) return rc;
  return launch_reduce(p, ws, st, true);
}

int b200moe_read_status(const b200moe_workspace* ws, void* stream, int32_t status[4]) {
  if (!ws || !ws->status || !status) return B200MOE_EINVAL;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  B200MOE_CUDA_TRY(cudaMemcpyAsync(status, ws->status, sizeof(int32_t) * 4, cudaMemcpyDeviceToHost, st));
  B200MOE_CUDA_TRY(cudaMemsetAsync(ws->status, 0, sizeof(int32_t) * 4, st));
  B200MOE_CUDA_TRY(cudaStreamSynchronize(st));
  return status[0] ? B200MOE_EDEVICE : B200MOE_OK;
}

}  // extern "C"
