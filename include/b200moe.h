/*
 * b200moe.h — C ABI of libb200moe.so: the DeepSeek-V3 FP8 block-scale fused MoE layer for NVIDIA B200 (sm_100a).
 *
 * The library replaces the device side of the reference operator
 *     kernel(routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights, gemm1_weights_scale,
 *            gemm2_weights, gemm2_weights_scale, local_expert_offset, routed_scaling_factor, output)
 * (reference: solution/python/kernel.py:71-83, host orchestration solution/python/pure_triton_impl.py:2125-2403).
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless its comment says "host";
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream);
 *   - every function returns 0 (B200MOE_OK) or a negative B200MOE_E* code; nothing throws, exits or prints;
 *   - no function synchronises the stream except b200moe_read_status();
 *   - no function allocates device memory: the caller owns a workspace sized by b200moe_workspace_bytes().
 *
 * Fixed operator geometry (reference: solution/python/pure_triton_impl.py:23-57, solution/cuda/binding.py:24-31):
 *   hidden H = 7168, intermediate I = 2048, 256 global experts in 8 groups of 32, top-4 groups, top-8 experts,
 *   quantisation block 128.  The number of local experts E_local is a run-time argument (1..256); the reference
 *   hard-codes 32.
 */
#ifndef B200MOE_H_
#define B200MOE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200MOE_HIDDEN 7168
#define B200MOE_INTER 2048
#define B200MOE_NUM_EXPERTS 256
#define B200MOE_TOP_K 8
#define B200MOE_N_GROUP 8
#define B200MOE_TOPK_GROUP 4
#define B200MOE_QBLOCK 128
#define B200MOE_BLOCK_M 128 /* rows per expert tile; every expert segment is padded to a multiple of this */
#define B200MOE_GEMM_MAX_CTAS 160  /* CTAs of a token-minor GEMM launch (one per SM, at most this many) */
#ifndef B200MOE_SKINNY_MAX_T
#define B200MOE_SKINNY_MAX_T 112   /* b200moe_forward uses the token-minor GEMM kernels up to this batch size */
#endif
#define B200MOE_PROLOGUE_MAX_T 32  /* largest batch of b200moe_prologue_small */
#define B200MOE_DECODE_MAX_T 8 /* the matrix-vector (decode) stages take at most this many tokens; b200moe_forward
                                  uses them while T * E_local <= B200MOE_DECODE_MAX_WORK */
#define B200MOE_DECODE_MAX_WORK 128 /* = 4 expected (token, local expert) pairs: T * 8 * E_local / 256 */

enum {
  B200MOE_OK = 0,
  B200MOE_EINVAL = -1,    /* bad argument (null pointer, T < 0, E_local out of range, misaligned pointer) */
  B200MOE_EWORKSPACE = -2,/* workspace too small or misaligned */
  B200MOE_ECUDA = -3,     /* a CUDA runtime / driver call failed; see b200moe_last_cuda_error() */
  B200MOE_EDEVICE = -4,   /* a kernel recorded a failure in the device status word (bounded wait ran out) */
  B200MOE_EUNSUPPORTED = -5,/* the current device is not sm_100 */
  B200MOE_ETOOLARGE = -6    /* the problem exceeds the fixed capacity of an entry point that allocates nothing */
};

/* Inputs and output of one layer call.  Tensor layouts are exactly those of the reference operator
 * (solution/python/pure_triton_impl.py:2127-2137):
 *   routing_logits        [T, 256]            float32, row-major
 *   routing_bias          [256]               bfloat16
 *   hidden_states         [T, 7168]           float8 e4m3fn
 *   hidden_states_scale   [56, T]             float32 (k-block major: the 56 scales of one token are strided by T)
 *   gemm1_weights         [E_local, 4096, 7168] e4m3fn  (rows 0..2047 = W1 "up", rows 2048..4095 = W3 "gate")
 *   gemm1_weights_scale   [E_local, 32, 56]   float32
 *   gemm2_weights         [E_local, 7168, 2048] e4m3fn
 *   gemm2_weights_scale   [E_local, 56, 16]   float32
 *   output                [T, 7168]           bfloat16; every row is written (zeros for tokens with no local expert)
 *   output_f32            [T, 7168]           float32, optional: the same sums before the bfloat16 rounding (partial
 *                                             results of an expert-parallel shard travel in this form)
 *
 * If routing_logits is NULL the routing stage is skipped and (topk_idx_in, topk_w_in) — [T,8] int32 global expert
 * ids and [T,8] float32 final weights — are used instead.  This is the path the expert-parallel receiver takes for
 * tokens routed on another rank; the reference has no counterpart (it only has `local_expert_offset`,
 * solution/python/pure_triton_impl.py:2141). */
struct b200moe_ep_plan;
typedef struct b200moe_problem {
  int32_t T;
  int32_t E_local;
  int32_t local_expert_offset;
  float routed_scaling_factor;
  const float* routing_logits;
  const uint16_t* routing_bias;
  const uint8_t* hidden_states;
  const float* hidden_states_scale;
  const uint8_t* gemm1_weights;
  const float* gemm1_weights_scale;
  const uint8_t* gemm2_weights;
  const float* gemm2_weights_scale;
  uint16_t* output;
  const int32_t* topk_idx_in;
  const float* topk_w_in;
  float* output_f32; /* optional [T,7168] float32: if non-NULL the un-rounded sums go here and `output` may be NULL */
  /* Optional strides, 0 = the dense layouts above.  They let the layer read token rows in place from an
   * expert-parallel receive buffer (b200moe_ep_dispatch row format) instead of from four separate tensors. */
  int64_t hidden_row_stride;  /* bytes between token rows of hidden_states (0 = 7168) */
  int64_t scale_token_stride; /* floats between tokens in hidden_states_scale (0 = 1) */
  int64_t scale_block_stride; /* floats between 128-column blocks in hidden_states_scale (0 = T) */
  int64_t topk_row_stride;    /* elements between tokens in topk_idx_in / topk_w_in (0 = 8) */
  /* Optional segmented float32 output (expert-parallel receiver writing straight into its peers' memory): rows
   * [out_seg_start[i], out_seg_start[i+1]) of the result go to out_seg_base[i] + (row - out_seg_start[i]) * 7168.
   * out_seg_count = 0 disables it; when set, `output` and `output_f32` are ignored.  The bases may be peer-GPU
   * addresses (plain stores over NVLink; no TMA and no multicast touch them). */
  int32_t out_seg_count;
  int32_t out_seg_start[9];
  float* out_seg_base[8];
  /* Optional DEVICE pointer (expert-parallel receiver, see b200moe_ep_exchange_counts): when set, the number of valid
   * rows and the placement of the float32 result rows are read on the device from *plan instead of from the host —
   * only the first plan->n_recv of the T rows exist (T is then a capacity: the rest is skipped by every stage), and row
   * r of segment s goes to plan->seg_base[s] + (r - plan->seg_start[s]) * 7168.  `output`, `output_f32` and out_seg_*
   * are ignored.  This is what lets a rank launch the layer on received records without reading their count back to
   * the host. */
  const struct b200moe_ep_plan* plan;
  /* Form of the un-rounded result rows (`output_f32`, out_seg_base[], plan->seg_base[]; `output` is always bfloat16):
   *   B200MOE_PARTIAL_F32  (0)  7168 float32 per row, 28672 bytes;
   *   B200MOE_PARTIAL_HALF (1)  15232 bytes per row: 896 groups of eight consecutive columns as eight float16 that
   *     share one power-of-two scale (14336 bytes), then the 896 scale bytes.  Group g, scale byte b: column 8g + j =
   *     half[8g + j] * 2^(b - 141); b is the biased float32 exponent of the group's largest magnitude (at least 14),
   *     so that magnitude lands in [2^14, 2^15) and every value keeps 11 significant bits relative to it.
   * In the second form the float* bases above are byte addresses of rows with a 15232-byte pitch.  It halves what an
   * expert-parallel shard returns over NVLink; the sum of up to eight such rows per token (b200moe_ep_combine_half)
   * stays within the bfloat16 rounding of the result.  The reference has no counterpart. */
  int32_t partial_format;
} b200moe_problem;
#define B200MOE_PARTIAL_F32 0
#define B200MOE_PARTIAL_HALF 1
#define B200MOE_HALF_ROW_BYTES 15232

/* Typed view of the caller-owned workspace.  R_max = (8*T/128 + E_local) * 128 rows bounds the padded sorted rows.
 * Integer metadata follows the reference's sort kernel (solution/python/pure_triton_impl.py:474-551):
 *   sorted_token_ids[r] = token of sorted row r, or T for a pad row;  sorted_weights[r] = routing weight or 0;
 *   scatter_map[t*8+k]  = sorted row of pair (t,k), or -1 when expert k of token t is not local;
 *   block_offsets[e]    = first 128-row block of local expert e, block_offsets[E_local] = total blocks.
 * Within an expert, rows are in ascending token order (the order of a stable sort of the flat pair list by expert,
 * as in solution/cuda/binding.py:147); the reference's Triton sort is atomic-ordered and not deterministic. */
typedef struct b200moe_workspace {
  int32_t T;
  int32_t E_local;
  int32_t R_max;
  int32_t n_chunks;          /* ceil(T/32): tokens are ranked in chunks of one warp */
  int32_t* topk_idx;         /* [T,8]   global expert ids, descending biased score, ties to the lower id */
  float* topk_w;             /* [T,8]   s_k / (sum_k s_k + 1e-20) * routed_scaling_factor */
  uint32_t* chunk_bits;      /* [n_chunks, E_local] bit j set: token 32*chunk+j selected local expert e */
  int32_t* chunk_base;       /* [n_chunks, E_local] pairs of expert e in earlier chunks (scratch between the scan and
                                the scatter; not written when n_chunks <= 32, where the scatter scans by itself) */
  int32_t* counts;           /* [E_local] */
  int32_t* block_offsets;    /* [E_local+1] */
  int32_t* total_blocks;     /* [1] */
  int32_t* status;           /* [4] device status word: 0 = ok */
  int32_t* sorted_token_ids; /* [R_max] */
  float* sorted_weights;     /* [R_max] */
  int32_t* scatter_map;      /* [T*8] */
  uint8_t* a_sorted;         /* [R_max, 7168] e4m3 activations gathered in sorted order */
  float* a_scale_sorted;     /* [56, R_max]   their scales, k-block major */
  uint8_t* inter_q;          /* [2, R_max, 2048] e4m3: SwiGLU output as value term + residual term, shared scale */
  float* inter_scale;        /* [16, R_max]   per row per 128 columns */
  float* expert_out;         /* [R_max, 7168] float32 GEMM2 result per sorted row (unweighted) */
  int32_t* gemm_tile_ctr;    /* [(R_max / 64) * 28] tickets of GEMM tiles shared by several CTAs; zero between launches
                                (b200moe_workspace_init clears it, the kernels return it to zero) */
  float* gemm_partial;       /* [B200MOE_GEMM_MAX_CTAS, 2, 2 * 64 * 128] float32 partial sums of shared tiles */
  int32_t* status_mirror;    /* optional, set by the caller after carving (carve leaves it NULL): device-accessible
                                address of 4 ints in MAPPED HOST memory.  The last kernel of b200moe_forward copies a
                                non-zero status word there, so the host can notice a failed call by reading its own
                                memory, without synchronising the stream.  Never written while status is 0. */
} b200moe_workspace;

/* Library / build identification.  No reference counterpart. */
int b200moe_version(void);
const char* b200moe_strerror(int code);
/* Text of the last CUDA error seen by this thread ("" if none).  No reference counterpart. */
const char* b200moe_last_cuda_error(void);

/* Bytes of workspace needed for up to T tokens and E_local local experts.
 * Replaces the reference's per-T module-level buffer caches (solution/python/pure_triton_impl.py:1945-1950,
 * :2162-2205; MAX_PADDED = 8*T + 32*BLOCK_M at :2171). */
int b200moe_workspace_bytes(int32_t T, int32_t E_local, size_t* bytes /* host */);

/* Carve `base` (256-byte aligned, `bytes` long) into the typed view for exactly (T, E_local). */
int b200moe_workspace_carve(void* base, size_t bytes, int32_t T, int32_t E_local, b200moe_workspace* out /* host */);

/* Clears the device status word of a freshly carved workspace (asynchronous on `stream`); call once before the first
 * launch that uses the workspace.  No reference counterpart. */
int b200moe_workspace_init(const b200moe_workspace* ws /* host */, void* stream);

/* Whole layer: route -> rank -> scatter -> gather -> GEMM1+SwiGLU -> GEMM2 -> weighted reduce, all on `stream`,
 * no host synchronisation.  With routing_logits given, T <= B200MOE_DECODE_MAX_T and T * E_local <=
 * B200MOE_DECODE_MAX_WORK it runs route -> GEMV1+SwiGLU -> GEMV2+reduce instead (b200moe_gemv1 / b200moe_gemv2 below): no sort, no gather, fp32 intermediate.  Replaces solution/python/pure_triton_impl.py:2125-2403 (kernel), :2025-2123 (_kernel_t1),
 * solution/python/triton_impl.py:346-566 and solution/python/triton_impl_t901.py:40-185. */
int b200moe_forward(const b200moe_problem* p /* host */, const b200moe_workspace* ws /* host */, void* stream);

/* Upstream of the layer: bf16 activations [T, 7168] -> e4m3 [T, 7168] and float32 scales [56, T], one scale per token
 * per 128 columns: s = max(amax * (1/448), 1e-12), q = e4m3(x * (1/s)), every operation rounded to float32 (round to
 * nearest even, conversion saturating at +-448).  Produces the `hidden_states` / `hidden_states_scale` pair that
 * kernel() takes (the reference has no kernel for it; its profiling script builds the pair with torch by multiplying
 * with 448 / amax, scripts/yjl_ncu.py:413-416).  x_bf16 16-byte aligned, q_out 8-byte aligned; needs no workspace. */
int b200moe_quantize_act(const void* x_bf16, int32_t T, void* q_out, float* scale_out, void* stream);

/* Stage entry points (unit tests, profiling).  Each runs one stage of b200moe_forward on the same buffers. */

/* No-aux routing: sigmoid, +bias, group score = two largest of each 32-expert group, top-4 groups, top-8 experts,
 * normalise, scale; also records which local experts each 32-token chunk selected (chunk_bits).
 * Replaces triton_ds_routing_kernel / _fused_routing_histogram_kernel (solution/python/pure_triton_impl.py:96-265). */
int b200moe_route(const b200moe_problem* p, const b200moe_workspace* ws, void* stream);
/* The same routing into caller-owned arrays topk_idx / topk_w [T,8], without a workspace and without the selection
 * bits: an expert-parallel rank routes its own tokens this way before dispatch.  Same reference kernels as above. */
int b200moe_route_topk(const float* routing_logits, const uint16_t* routing_bias, int32_t T,
                       float routed_scaling_factor, int32_t* topk_idx, float* topk_w, void* stream);
/* chunk_bits from an existing topk_idx (used when routing ran elsewhere).  No reference counterpart. */
int b200moe_topk_bits(const b200moe_problem* p, const b200moe_workspace* ws, void* stream);
/* Per-expert prefix over chunks (chunk_base, counts), then the padded layout and the stable scatter
 * (block_offsets, total_blocks, sorted_token_ids, sorted_weights, scatter_map).
 * Replaces triton_sort_and_scatter_kernel and token_sort_and_scatter
 * (solution/python/pure_triton_impl.py:474-551, :832-879). */
int b200moe_sort(const b200moe_problem* p, const b200moe_workspace* ws, void* stream);
/* a_sorted / a_scale_sorted from hidden_states / hidden_states_scale via sorted_token_ids.
 * Replaces the in-kernel row gather of the reference GEMM1 (solution/python/pure_triton_impl.py:986-994) and
 * _dequantize_gemm1_sorted_a_kernel (solution/python/triton_impl.py:67-110), without the dequantisation. */
int b200moe_gather(const b200moe_problem* p, const b200moe_workspace* ws, void* stream);
/* b200moe_route + b200moe_sort + b200moe_gather in ONE launch for batches of at most B200MOE_PROLOGUE_MAX_T tokens with
 * dense inputs (all strides 0, routing_logits given); B200MOE_ETOOLARGE above that size, B200MOE_EINVAL for strided
 * inputs.  Leaves exactly the same workspace contents as the three stages.  b200moe_forward uses it for such batches.
 * Replaces, for such batches, the reference's routing + sort sequence (solution/python/pure_triton_impl.py:2207-2273). */
int b200moe_prologue_small(const b200moe_problem* p, const b200moe_workspace* ws, void* stream);
/* Grouped FP8 GEMM1 with fp32 block-scale promotion every 128 K, SwiGLU, two-term e4m3 re-quantisation.
 * Replaces _fused_moe_gemm1_swiglu_kernel (solution/python/pure_triton_impl.py:886-1046) and the CuTe GEMM1 chain
 * (solution/python/cute_gemm1_mma.py:247-289, solution/python/triton_impl.py:113-150). */
int b200moe_gemm1(const b200moe_problem* p, const b200moe_workspace* ws, void* stream);
/* Grouped FP8 GEMM2 over the two-term intermediate, float32 rows out.
 * Replaces _fused_moe_gemm2_kernel (solution/python/pure_triton_impl.py:1056-1196) and the CuTe GEMM2
 * (solution/python/cute_gemm2_mma.py:250-304). */
int b200moe_gemm2(const b200moe_problem* p, const b200moe_workspace* ws, void* stream);
/* The same two GEMMs with the operands swapped (weight rows on the M side of the MMA, at most 64 tokens on the N side):
 * same inputs, outputs and results as b200moe_gemm1 / b200moe_gemm2, faster when experts see few tokens because a tile
 * then costs what streaming its weights costs.  b200moe_forward picks them for T <= B200MOE_SKINNY_MAX_T.
 * They replace the reference's small-batch GEMM buckets (_small_medium_fused_moe_gemm1_swiglu_kernel /
 * _small_medium_fused_moe_gemm2_kernel, solution/python/pure_triton_impl.py:1278-1466). */
int b200moe_gemm1_skinny(const b200moe_problem* p, const b200moe_workspace* ws, void* stream);
int b200moe_gemm2_skinny(const b200moe_problem* p, const b200moe_workspace* ws, void* stream);
/* Decode path stages (need topk_idx / topk_w of b200moe_route in the workspace; the fp32 intermediate [T*8, 2048] is
 * kept in the workspace's expert_out array): one warp per output element streams the weight rows from HBM.
 * Replaces the reference's T = 1 path: GEMM1 with BLOCK_M = 16 (solution/python/pure_triton_impl.py:1824-1940) and
 * _t1_fused_gemm2_reduce_kernel (solution/python/pure_triton_impl.py:1676-1750). */
int b200moe_gemv1(const b200moe_problem* p, const b200moe_workspace* ws, void* stream);
int b200moe_gemv2(const b200moe_problem* p, const b200moe_workspace* ws, void* stream);
/* out[t] = sum_k topk_w[t,k] * expert_out[scatter_map[t,k]], fp32 accumulate, bf16 (and/or fp32) store, no atomics.
 * Replaces _token_reduce_kernel (solution/python/pure_triton_impl.py:1758-1821) and
 * _token_reduce_weighted_kernel (solution/python/triton_impl.py:163-207). */
int b200moe_reduce(const b200moe_problem* p, const b200moe_workspace* ws, void* stream);
/* The pair b200moe_forward runs for batches above B200MOE_SKINNY_MAX_T: b200moe_gemm2 with its rows left in the
 * workspace's expert_out array in the half form (see partial_format: 15232-byte pitch), and b200moe_reduce reading that
 * form.  Both kernels are bound by those rows' bytes, which this halves; a value keeps 11 significant bits, the sum of
 * eight is rounded to bfloat16.  Same reference kernels as the float32 pair above. */
int b200moe_gemm2_half(const b200moe_problem* p, const b200moe_workspace* ws, void* stream);
int b200moe_reduce_half(const b200moe_problem* p, const b200moe_workspace* ws, void* stream);

/* Token sort for callers that cannot allocate device memory (a process that gave all of HBM to its own pool, a plugin
 * with a memory budget fixed at start-up, a region where allocation is forbidden).  Same results as b200moe_topk_bits
 * + b200moe_sort — counts[E_local], block_offsets[E_local+1], total_blocks[1], sorted_token_ids / sorted_weights
 * [(8*T/128 + E_local)*128], scatter_map[T*8] (16-byte aligned), all caller-owned device buffers — computed from
 * topk_idx / topk_w [T,8].  The two scratch tables live in a fixed array inside the library, so the call uses no
 * allocator of any kind.  Limits and rules:
 *   - ceil(T/32) * E_local <= B200MOE_SORT_STATIC_MAX_ENTRIES, else B200MOE_ETOOLARGE (e.g. T <= 32768 at 32 local
 *     experts, T <= 4096 at 256);
 *   - every GPU that loads the library holds the array (256 KB) until the process exits;
 *   - all calls on one GPU share the array: calls whose kernels overlap on the device race; serialise them;
 *   - the first call on each GPU looks up the array's device address (with that GPU current); make that first call
 *     before any stream capture begins.
 * This entry point has no counterpart in the reference. */
#define B200MOE_SORT_STATIC_MAX_ENTRIES 32768
int b200moe_sort_static(const int32_t* topk_idx, const float* topk_w, int32_t T, int32_t E_local,
                        int32_t local_expert_offset, int32_t* counts, int32_t* block_offsets, int32_t* total_blocks,
                        int32_t* sorted_token_ids, float* sorted_weights, int32_t* scatter_map, void* stream);

/* ---- Expert parallelism (no reference counterpart: the reference is single-GPU) -------------------------------------
 * A token row travels once to every rank that owns at least one of its eight experts, as one 7456-byte record:
 *   [0,7168) e4m3 activations | [7168,7392) 56 float32 scales | [7392,7424) 8 int32 expert ids | [7424,7456) 8 float32
 *   weights.
 * b200moe_ep_dispatch ranks the (token, destination) pairs (stable: by destination rank, then token id), writes the
 * records into `send_rows` in that order, the number of records per destination into `send_counts[world]` and, for
 * each of the token's eight experts, the record index its destination uses into `slot_map[T,8]` (-1 for an expert whose
 * rank already got the token through an earlier expert).  The receiver runs b200moe_forward on the records in place
 * (routing_logits = NULL, the four strides of b200moe_problem set by b200moe_ep_record_layout) and returns float32 rows
 * in the same order; b200moe_ep_combine adds the rows of each token and writes bfloat16.
 * `scratch` needs b200moe_ep_scratch_bytes(T, world) bytes; send_rows holds up to T * min(8, world) records. */
#define B200MOE_EP_RECORD_BYTES 7456
int b200moe_ep_scratch_bytes(int32_t T, int32_t world, size_t* bytes /* host */);
int b200moe_ep_dispatch(const int32_t* topk_idx, const float* topk_w, const uint8_t* hidden_states,
                        const float* hidden_states_scale, int32_t T, int32_t world, void* scratch, size_t scratch_bytes,
                        uint8_t* send_rows, int32_t* send_counts, int32_t* slot_map, void* stream);
/* Fills the pointer and stride fields of `p` for `n` records at `records` (p->T is set to n). */
int b200moe_ep_record_layout(const uint8_t* records, int32_t n, b200moe_problem* p /* host */);
/* Peer-memory variant for up to 8 GPUs of one node (buffers mapped into every rank, e.g. torch symmetric memory):
 * b200moe_ep_rank does the ranking only (send_counts, slot_map, and the record order kept in `scratch`);
 * b200moe_ep_pack_peers then writes each record directly into its destination's receive buffer —
 * record j of the segment for rank d goes to recv_records[d] + (dst_row0[d] + j) * 7456 — so dispatch needs no
 * collective for the payload.  b200moe_ep_barrier is a bounded all-rank barrier on a small flag array in the same
 * mapped memory: every rank stores `epoch` into flags[rank] of every peer and waits (about 2 s at most) until its own
 * copy shows `epoch` from everybody; on a timeout it records B200MOE status code 2 in `status` and returns. */
typedef struct b200moe_ep_peers {
  int32_t world;
  int32_t rank;
  uint8_t* recv_records[8];
  int32_t* flags[8];
  /* used by b200moe_ep_exchange_counts only (may stay NULL / 0 otherwise): */
  int32_t* counts[8];    /* rank r's copy of the count matrix, int32 [8][8]: counts[r][s*8+d] = records s sends to d */
  float* back_rows[8];   /* rank r's buffer for the partial rows returning to it: cap_back rows of back_row_bytes */
  int32_t cap_recv;      /* records every receive buffer holds */
  int32_t cap_back;      /* rows every return buffer holds */
  int32_t back_row_bytes; /* pitch of the return buffers' rows: 0 or 28672 = float32 rows, 15232 = half rows
                             (b200moe_problem.partial_format of the layer call that writes them must match) */
} b200moe_ep_peers;
/* What one rank needs to know about a step's traffic, computed ON THE DEVICE by b200moe_ep_exchange_counts and read
 * there by the kernels that follow (pack, the layer on the received records, the return of partial rows), so that no
 * count ever travels to the host.  ok = 0 (and every count 0) if a barrier wait ran out or the counts would overflow a
 * buffer; the status word then holds code 2 or 3. */
typedef struct b200moe_ep_plan {
  int32_t ok;
  int32_t n_recv;        /* records this rank receives = valid leading rows of its receive buffer */
  int32_t n_send;        /* records this rank sends */
  int32_t seg_count;     /* = world */
  int32_t seg_start[9];  /* received rows [seg_start[s], seg_start[s+1]) come from rank s */
  int32_t dst_row0[8];   /* this rank's records for rank d start at row dst_row0[d] of d's receive buffer */
  int32_t rank;          /* this rank: kernels that store into peers start with the NEXT rank's segment and wrap
                            around, so that at any moment the ranks write to different peers instead of all to one */
  float* seg_base[8];    /* where the partial rows of segment s go: inside rank s's return buffer */
  int32_t matrix[64];    /* the count matrix, matrix[s*8+d] */
} b200moe_ep_plan;
int b200moe_ep_rank(const int32_t* topk_idx, int32_t T, int32_t world, void* scratch, size_t scratch_bytes,
                    int32_t* send_counts, int32_t* slot_map, void* stream);
int b200moe_ep_pack_peers(const int32_t* topk_idx, const float* topk_w, const uint8_t* hidden_states,
                          const float* hidden_states_scale, int32_t T, const b200moe_ep_peers* peers /* host */,
                          const int32_t* dst_row0 /* host, [world] */, void* scratch, size_t scratch_bytes,
                          void* stream);
int b200moe_ep_barrier(const b200moe_ep_peers* peers /* host */, int32_t epoch, int32_t* status, void* stream);
/* Count exchange without the host: every rank stores its `send_counts[world]` (device, from b200moe_ep_rank) into row
 * `rank` of every peer's count matrix, passes the same bounded flag barrier as b200moe_ep_barrier, and then derives
 * *plan (device memory of this rank) from its own, now complete, copy of the matrix.  Replaces an all-gather of the
 * counts plus a device-to-host read.  b200moe_ep_pack_peers_planned is b200moe_ep_pack_peers with the destination rows
 * taken from the plan on the device (a destination that is misaligned or lies past cap_recv is not stored: status code
 * 4); b200moe_forward with b200moe_problem.plan set is the receiver. */
int b200moe_ep_exchange_counts(const b200moe_ep_peers* peers /* host */, const int32_t* send_counts, int32_t epoch,
                               b200moe_ep_plan* plan, int32_t* status, void* stream);
int b200moe_ep_pack_peers_planned(const int32_t* topk_idx, const float* topk_w, const uint8_t* hidden_states,
                                  const float* hidden_states_scale, int32_t T, const b200moe_ep_peers* peers /* host */,
                                  const b200moe_ep_plan* plan, void* scratch, size_t scratch_bytes, int32_t* status,
                                  void* stream);
/* Upper bound, in SM clock cycles, of the waits inside b200moe_ep_barrier and b200moe_ep_exchange_counts for launches
 * made after this call (process-wide; 0 restores the default of about 2 s).  Tests use it to make a wait run out
 * quickly; a deployment can use it to bound how long a lost peer stalls a step. */
int b200moe_set_wait_limit_cycles(int64_t cycles);
int b200moe_ep_combine(const float* returned_rows, const int32_t* slot_map, int32_t T, uint16_t* output, void* stream);
/* The same sum over returned rows in the B200MOE_PARTIAL_HALF form (15232-byte pitch): rows are decoded to float32,
 * added in slot order and rounded to bfloat16 once. */
int b200moe_ep_combine_half(const void* returned_rows, const int32_t* slot_map, int32_t T, uint16_t* output,
                            void* stream);

/* Synchronises `stream`, copies the device status word to *status (host) and clears it.
 * Returns B200MOE_EDEVICE if it was non-zero.  No reference counterpart (the reference has no device-side waits). */
int b200moe_read_status(const b200moe_workspace* ws, void* stream, int32_t status[4] /* host */);

#ifdef __cplusplus
}
#endif
#endif /* B200MOE_H_ */
