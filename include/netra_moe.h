/* C ABI of the sm_100a routed-MoE layer (libnetra_sm100.so).
 *
 * Two groups of entry points:
 *
 * 1. Per-kernel bridges with the names, argument order and return convention of the
 *    reference's bridges (0 = ok, -1 = see last_error, otherwise a raw runtime error code;
 *    thread-local last_error string; load() idempotent; launch() does not allocate,
 *    synchronise or touch module state and is stream-capture safe):
 *      runtime/gfx950/routing/verify/qwen36_router_bf16_bridge.h:10-21
 *      runtime/gfx950/routing/decode/qwen36_shared_gate_append_bridge.h:10-23
 *      runtime/gfx950/fp8/moe/qwen36_moe_silu_mul_quant_bridge.h:14-64
 *      runtime/gfx950/fp8/moe/moe_prefill_m768_bridge.h:10-23
 *    Differences: hipStream_t -> cudaStream_t; the kernels are linked into the library, so
 *    load(path) ignores its argument (NULL is accepted) and only performs one-time set-up;
 *    `rows` may be any positive count (the reference kernels take 1..16).
 *
 * 2. The fused layer: router logits -> softmax/top-8/renormalise (+ shared slot) -> stable
 *    expert sort -> per-token FP8 quantisation -> grouped gate_up with SiLU*up requantising
 *    epilogue -> grouped down -> slot-ordered weighted combine.  The reference has no single
 *    entry point for this sequence: it spans the engine launch of
 *    runtime/gfx950/engine/netra_engine.h:84-86 plus third-party top-k / sort / quantisation
 *    (SGLang fused_topk, AITER moe_sorting, per_token_group_quant_fp8).  All buffers are
 *    caller-owned device memory; the library allocates no device memory (the one exception is
 *    netra_ep_window_create in the expert-parallel group below, which says so).
 */
#pragma once

#include <cuda_runtime_api.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------ reference bridges */
int netra_qwen36_router_bf16_load(const char* unused_path);
int netra_qwen36_router_bf16_launch(void* output_logits_bf16, const void* hidden_bf16,
                                    const void* router_weight_bf16, uint32_t rows, cudaStream_t stream);
int netra_qwen36_router_bf16_unload(void);
const char* netra_qwen36_router_bf16_last_error(void);

int netra_qwen36_shared_gate_append_load(const char* unused_path);
int netra_qwen36_shared_gate_append_launch(void* output_ids_i32, void* output_weights_f32,
                                           const void* hidden_bf16, const void* shared_gate_weight_bf16,
                                           const void* routed_ids_i32, const void* routed_weights_f32,
                                           uint32_t rows, cudaStream_t stream);
int netra_qwen36_shared_gate_append_unload(void);
const char* netra_qwen36_shared_gate_append_last_error(void);

int netra_qwen36_moe_gate_up_load(const char* unused_path);
int netra_qwen36_moe_gate_up_launch(const void* hidden_fp8, const float* hidden_scale_f32,
                                    const void* w13_fp8, const float* w13_scale_f32,
                                    const int32_t* topk_ids_i32, float* output_f32, int rows,
                                    cudaStream_t stream);
int netra_qwen36_moe_gate_up_unload(void);
const char* netra_qwen36_moe_gate_up_last_error(void);

int netra_qwen36_moe_silu_mul_quant_load(const char* unused_path);
int netra_qwen36_moe_silu_mul_quant_launch(const float* input_f32, void* output_fp8,
                                           float* output_scale_f32, int rows, cudaStream_t stream);
int netra_qwen36_moe_silu_mul_quant_unload(void);
const char* netra_qwen36_moe_silu_mul_quant_last_error(void);

int netra_qwen36_moe_down_reduce_load(const char* unused_path);
int netra_qwen36_moe_down_reduce_launch(const void* activation_fp8, const float* activation_scale_f32,
                                        const void* w2_fp8, const float* w2_scale_f32,
                                        const float* topk_weights_f32, const int32_t* topk_ids_i32,
                                        void* output_bf16, int rows, cudaStream_t stream);
int netra_qwen36_moe_down_reduce_unload(void);
const char* netra_qwen36_moe_down_reduce_last_error(void);

/* Residual add + RMSNorm + per-128 FP8 quantisation (runtime/gfx950/group_quant/verify/group_quant_assembly_bridge.h:21-31,
 * netra_add_rmsnorm_group_quant_n5120_launch, there at width 5120; here at this model's width 2048, same argument list):
 *   x = f32(input) + f32(residual); residual_out = bf16(x); y = bf16(x * rsqrt(mean(x^2) + epsilon) * weight);
 *   output_bf16 = y; per 128 columns scale = max(amax |y|, 1e-10) * fl(1/448), code = e4m3_rne_sat(y / scale).
 * Differences: scales are row-major [rows, 16] (the reference stores them group-major), the mean of squares is
 * defined exactly (FP64 sum, one rounding) so that the result does not depend on the reduction order, rows may be
 * any count up to 2^20.  load() ignores its six paths. */
int netra_group_quant_assembly_load(const char* unused0, const char* unused1, const char* unused2, const char* unused3,
                                    const char* unused4, const char* unused5);
int netra_group_quant_assembly_unload(void);
int netra_add_rmsnorm_group_quant_n2048_launch(const void* input_bf16, const void* residual_bf16, const void* weight_f32,
                                               void* output_bf16, void* residual_out_bf16, void* output_fp8,
                                               void* output_scale_f32, uint32_t rows, float epsilon, cudaStream_t stream);
const char* netra_group_quant_assembly_last_error(void);

/* The 768-row prefill call (runtime/gfx950/fp8/moe/moe_prefill_m768_bridge.h:10-23): quantised token rows
 * [768, 2048] + scales [768, 16], the expert slabs in the checkpoint's row-major layout ([257, 1024, 2048] /
 * [257, 2048, 512], slab 256 = shared expert), and the routing in the sorted-id format of the reference's fused
 * producer (kernels/gfx950/templates/moe/prefill/fused_splitk2/entry_routing.inc:67-111): sorted_token_ids [23360]
 * words token | slot << 24 in 64-entry blocks of one expert each (padding words have token >= 768),
 * sorted_expert_ids [365] per block, num_valid_ids [1], topk_weights [768, 9] in slot order with slot 8 = the
 * shared expert (id 256, what netra_qwen36_shared_gate_append produces).  Output BF16 [768, 2048].
 * load(): both paths are ignored; allocates the bridge's scratch (about 90 MB) on the current device.  launch():
 * allocates nothing; its first call with a given set of slab pointers encodes their descriptors (host work and one
 * small memset: make it outside stream capture).  sorted_weights_f32, route_scale_workspace_f32 and partials_f16
 * are accepted for signature compatibility and not used: at 768 rows the rows between down and combine stay FP32.
 * status(): no counterpart in the reference; word 3 counts routing entries that name the shared expert in a routed
 * slot or a routed expert in slot 8 (such a call's output is invalid). */
int netra_moe_prefill_m768_load(const char* unused_producer_path, const char* unused_reducer_path);
int netra_moe_prefill_m768_launch(const void* hidden_fp8, const float* hidden_scale_f32,
                                  const void* w13_fp8, const float* w13_scale_f32,
                                  const void* w2_fp8, const float* w2_scale_f32,
                                  const int32_t* sorted_token_ids_i32, const float* sorted_weights_f32,
                                  const int32_t* sorted_expert_ids_i32, const int32_t* num_valid_ids_i32,
                                  const float* topk_weights_f32, float* route_scale_workspace_f32,
                                  void* partials_f16, void* output_bf16, cudaStream_t stream);
int netra_moe_prefill_m768_status(uint32_t status_out[4]);
int netra_moe_prefill_m768_unload(void);
const char* netra_moe_prefill_m768_last_error(void);

/* ------------------------------------------------------------------ fused layer */
typedef struct netra_moe_layer netra_moe_layer_t;

/* Byte offsets of every intermediate inside the caller-owned workspace for a capacity of
 * `tokens` rows (P = tokens * 8 routed pairs).  Row spaces: rows [0, P) of a_fp8 / a_scale /
 * h_fp8 / h_scale / down_f32 are in expert-sorted order, rows [P, P + tokens) are in token
 * order and belong to the shared expert. */
typedef struct netra_moe_workspace_layout {
  uint32_t struct_size;
  uint32_t tokens;
  uint64_t total_bytes;
  uint64_t logits_bf16;   /* [tokens, 256] bf16 */
  uint64_t topk_ids;      /* [tokens, 9] i32, slot 8 = 256 (shared) */
  uint64_t topk_weights;  /* [tokens, 9] f32 */
  uint64_t perm;          /* [P] i32: sorted position -> pair index t*8+slot */
  uint64_t inv_perm;      /* [P] i32: pair index -> sorted position */
  uint64_t counts;        /* [256] i32 */
  uint64_t offsets;       /* [258] i32: exclusive prefix; [256] = P, [257] = P + tokens */
  uint64_t seg_hist;      /* sort scratch */
  uint64_t a_fp8;         /* [P + tokens, 2048] e4m3 */
  uint64_t a_scale;       /* [P + tokens, 16] f32 */
  uint64_t h_fp8;         /* [P + tokens, 512] e4m3 */
  uint64_t h_scale;       /* [P + tokens, 4] f32 */
  uint64_t down_f32;      /* [P + tokens, 2048] f32 */
  uint64_t status;        /* [4] u32 device status words (0 = ok): 0 gate_up, 1 down, 2 tensor-core router */
  uint64_t logits_f32;    /* [tokens, 256] f32: tensor-core router output before the exact rounding (calls above 1024 rows) */
  uint64_t wnorm;         /* [256] f32: Euclidean norms of the router rows (upper bounds) */
  uint64_t router_stats;  /* [4] u32: word 0 counts the logits recomputed in FP64 since the layer was created */
  uint64_t gemm_ready;    /* [1024] u32: per-unit arrival counters of the launch that runs both projections (decode sizes) */
  uint64_t front_counters; /* [128] u32: arrival counters of the one-launch routing front end; zero between launches */
} netra_moe_workspace_layout_t;

int netra_moe_workspace_layout_query(uint32_t tokens, netra_moe_workspace_layout_t* output);

typedef struct netra_moe_layer_desc {
  uint32_t struct_size;
  uint32_t max_tokens;                /* capacity the workspace was sized for */
  const void* router_weight_bf16;     /* [256, 2048] */
  const float* router_bias_f32;       /* [256] or NULL */
  const void* w13_fp8;                /* [257, 1024, 2048], slab 256 = shared expert */
  const float* w13_scale_f32;         /* [257, 8, 16] */
  const void* w2_fp8;                 /* [257, 2048, 512] */
  const float* w2_scale_f32;          /* [257, 16, 4] */
  void* workspace;                    /* device, 1024-byte aligned */
  uint64_t workspace_bytes;
  uint32_t weights_tiled;             /* 0: w13/w2 are the row-major slabs above; 1: they were rewritten by
                                         netra_moe_repack_tiles_launch (same bytes, tile order); 2: the experts are
                                         MXFP4 - w13_fp8/w2_fp8 are the code blocks and w13_scale_f32/w2_scale_f32 the
                                         scale atoms (bytes) written by netra_moe_mxfp4_pack_launch */
  uint32_t num_expert_slabs;          /* slabs behind w13/w2; 0 means 257.  Fewer is only meaningful for callers that
                                         use the routing stages (0-5, 8) and run the experts elsewhere */
} netra_moe_layer_desc_t;

/* Load-time weight layout step (the role of the reference's repack plan,
 * compiler/netra_compiler/layouts.py:109-164): rewrites row-major byte rows [total_rows, k_bytes]
 * into consecutive tiles of 128 rows x 128 bytes ordered (row tile, K-block), so that every TMA
 * box of the grouped GEMMs is one contiguous 16 KiB read.  dst and src must not alias; total_rows
 * and k_bytes are multiples of 128.  Call once per weight tensor: (257*1024, 2048) for W13 and
 * (257*2048, 512) for W2.  Scales are not touched. */
int netra_moe_repack_tiles_launch(void* dst, const void* src, uint64_t total_rows, uint32_t k_bytes,
                                  cudaStream_t stream);

/* The scale half of the same plan (compiler/netra_compiler/layouts.py:166-206, "widen_bf16_to_fp32_exact"): checkpoints
 * that store weight_scale_inv as BF16 are widened to the FP32 scales the kernels read; the order of the scales
 * ([group, N/128, K/128]) is unchanged. */
int netra_moe_widen_scales_bf16_launch(float* dst_f32, const void* src_bf16, uint64_t count, cudaStream_t stream);

/* MXFP4 expert weights (E2M1 codes, one E8M0 scale per 32 K-elements; encoding of the reference's
 * tools/checkpoint/quantize_qwen36_lm_head_mxfp4.py:58-67 and tests/gfx1151/test_netra_mxfp4_sgl_decode.py:23-31):
 * load-time expansion into the layer's operand format - E4M3 codes [total_rows, k] and one power-of-two FP32
 * scale per 128 x 128 tile [total_rows/128, k/128] - after which the MXFP4 checkpoint runs on the FP8 tensor-core
 * kernels with exactly the MXFP4 products.  packed is [total_rows, k/2] (low nibble = even k, K contiguous per
 * row), scales_e8m0 is [total_rows, k/32].  The expansion is exact while the scales inside a tile span at most
 * 15 binades; elements below that are rounded to nearest and counted in *inexact (device word, caller-zeroed).
 * The 4-bit codes are not streamed by the GEMMs: the weight traffic is that of FP8. */
int netra_moe_mxfp4_expand_launch(void* dst_fp8, float* dst_scale_f32, uint32_t* inexact_u32, const void* packed_e2m1,
                                  const void* scales_e8m0, uint64_t total_rows, uint32_t k, cudaStream_t stream);

/* The native MXFP4 path (the role of kernels/gfx1151/mxfp4/decode/mxfp4_decode_gate_gfx1151.s:1-15 and
 * mxfp4_decode_down_gfx1151.s:1-14 in the call sequence of runtime/gfx1151/mxfp4/decode/runtime.h:10-47): the expert
 * weights stay four-bit in memory and are multiplied by tcgen05.mma.kind::mxf8f6f4.block_scale, the E8M0 scales reaching
 * the tensor core through TMEM.  This load-time step rewrites the same packed slabs (packed_e2m1 [total_rows, k/2],
 * scales_e8m0 [total_rows, k/32]) into the operand layout of those kernels, same sizes: dst_codes holds one contiguous
 * 8 KiB block per (128-row tile, 128-element K-block) and dst_scale_atoms one 512-byte atom per block with row r's
 * four scale bytes at 16 * (r % 32) + 4 * (r / 32).  The kernels fetch two blocks per copy (boxes of 256 four-bit
 * rows are what reaches the HBM rate) - the two weight tiles one MMA stage consumes - so the block order matters.  The
 * rows come in groups of 2 * paired_half_rows rows whose two halves are consumed together; blocks are ordered (group,
 * tile within the half, K-block, half).  W2: paired_half_rows = 128 (tiles 2p and 2p + 1 side by side).  W13:
 * paired_half_rows = 512, its slabs of 1024 rows being 512 gate rows followed by 512 up rows: a gate tile next to
 * its up tile.  A layer created with weights_tiled = 2 on these buffers streams 0.53 bytes per weight instead of 1.0.
 * Code pointers must be 32-byte aligned for the layer, total_rows and k multiples of 128, at most 65,535 row tiles per
 * call. */
int netra_moe_mxfp4_pack_launch(void* dst_codes, void* dst_scale_atoms, const void* packed_e2m1, const void* scales_e8m0,
                                uint64_t total_rows, uint32_t k, uint32_t paired_half_rows, cudaStream_t stream);

/* Control plane (serialised by the caller): encodes the tensor maps of the persistent buffers
 * and clears the status words.  No device memory is allocated. */
int netra_moe_layer_create(const netra_moe_layer_desc_t* desc, netra_moe_layer_t** output);

/* Enqueues one layer call on the caller's stream: no allocation, no synchronisation, no host
 * read-back, so the call may be captured into a CUDA graph.  shared_weight_f32 may be NULL
 * (the shared expert is then always on with weight 1). */
int netra_moe_layer_launch(netra_moe_layer_t* layer, const void* hidden_bf16,
                           const float* shared_weight_f32, void* output_bf16, uint32_t tokens,
                           cudaStream_t stream);

/* The layer call with the upstream fusion: residual add + RMSNorm + input quantisation in one kernel (see
 * netra_add_rmsnorm_group_quant_n2048_launch) that writes the layer's quantised token rows directly, so that the
 * routing stage no longer reads the hidden row a second time to quantise it.  hidden_out_bf16 [tokens, 2048] receives
 * the normalised rows (the router reads them), residual_out_bf16 the updated residual.  The result equals
 * netra_moe_layer_launch on hidden_out_bf16 bit for bit. */
int netra_moe_layer_launch_with_norm(netra_moe_layer_t* layer, const void* input_bf16, const void* residual_bf16,
                                     const float* norm_weight_f32, float epsilon, void* hidden_out_bf16,
                                     void* residual_out_bf16, const float* shared_weight_f32, void* output_bf16,
                                     uint32_t tokens, cudaStream_t stream);

/* The same layer call with a top-k computed by the caller (a serving stack that keeps its own fused top-k:
 * the reference's position, scripts/rocm/integrations/sglang/sglang-gfx1151-bf16-router.patch:64, and its
 * apply(layer, hidden, topk_weights, topk_ids) entry, scripts/rocm/integrations/sglang/netra_gfx1151_sglang.py:1297-1311).
 * topk_ids i32 [tokens, 8] (global expert ids 0..255; out-of-range ids are clamped), topk_weights f32 [tokens, 8]
 * already normalised by the caller.  The router and top-k stages are skipped; everything from the input
 * quantisation on is the fused sequence. */
int netra_moe_layer_launch_with_topk(netra_moe_layer_t* layer, const void* hidden_bf16, const int32_t* topk_ids_i32,
                                     const float* topk_weights_f32, const float* shared_weight_f32, void* out_bf16,
                                     uint32_t tokens, cudaStream_t stream);

/* Launches ONE stage of the same sequence (0 router logits, 1 top-k + input quantisation,
 * 2-4 sort (stage 2 alone sorts up to 1024 rows; 3 and 4 then launch nothing), 5 row gather, 6 grouped gate_up, 7 grouped down, 8 combine), for callers that
 * migrate one boundary at a time and for per-kernel timing; same rules as the call above.
 * Counterpart: netra_engine_launch_operation, runtime/gfx950/engine/netra_engine.h:90-92. */
int netra_moe_layer_launch_stage(netra_moe_layer_t* layer, uint32_t stage, const void* hidden_bf16,
                                 const float* shared_weight_f32, void* output_bf16, uint32_t tokens,
                                 cudaStream_t stream);

/* ------------------------------------------------------------------ expert parallelism
 * No counterpart in the reference (its multi-GPU mode is independent replicas).  An expert block
 * runs the grouped gate_up and down kernels over `num_groups` expert slabs held by this GPU on a
 * caller-provided row space: rows of group g are [offsets[g], offsets[g+1]); the last group is
 * scheduled first (by convention the shared expert).  a_scale / h_scale need 64 spare rows after
 * max_rows.  status_u32 points at two device words (0 = ok). */
typedef struct netra_moe_expert_block netra_moe_expert_block_t;
typedef struct netra_moe_expert_block_desc {
  uint32_t struct_size;
  uint32_t num_groups;
  uint32_t max_rows;
  uint32_t weights_tiled;
  const void* w13_fp8;          /* [num_groups, 1024, 2048] (or its tile order) */
  const float* w13_scale_f32;   /* [num_groups, 8, 16] */
  const void* w2_fp8;           /* [num_groups, 2048, 512] */
  const float* w2_scale_f32;    /* [num_groups, 16, 4] */
  const void* a_fp8;            /* in  [max_rows, 2048] e4m3, rows grouped by slab */
  const float* a_scale_f32;     /* in  [max_rows + 64, 16] */
  void* h_fp8;                  /* scratch [max_rows, 512] */
  float* h_scale_f32;           /* scratch [max_rows + 64, 4] */
  float* down_f32;              /* out [max_rows, 2048] */
  const int32_t* offsets_i32;   /* device, [num_groups + 1] */
  uint32_t* status_u32;         /* device, [2] */
} netra_moe_expert_block_desc_t;
int netra_moe_expert_block_create(const netra_moe_expert_block_desc_t* desc, netra_moe_expert_block_t** output);
int netra_moe_expert_block_launch(netra_moe_expert_block_t* block, cudaStream_t stream);
int netra_moe_expert_block_destroy(netra_moe_expert_block_t* block);

/* Rows received source-rank-major (source ascending, local expert ascending inside a source) ->
 * expert-major positions.  counts is [sources, experts] on the device.  Writes src_base / dst_base
 * [sources*experts], offsets [experts + 2] and index[i] for i < index_rows (-1 for an unused slot
 * row).  slot_rows == 0: the rows are compact; slot_rows > 0: source s owns rows
 * [s*slot_rows, (s+1)*slot_rows) (fixed-capacity exchange, index_rows = sources*slot_rows).
 * shared_first == 0: offsets = prefix over local experts, then total, then total + extra_rows;
 * shared_first == 1: group 0 is the extra (shared-expert) rows at [0, extra_rows), routed groups follow. */
int netra_ep_regroup_launch(int32_t* src_base, int32_t* dst_base, int32_t* offsets, int32_t* index,
                            const int32_t* counts, uint32_t sources, uint32_t experts, uint32_t extra_rows,
                            uint32_t index_rows, uint32_t slot_rows, uint32_t shared_first, cudaStream_t stream);
/* scatter == 0: dst row r <- src row index[r];  scatter == 1: dst row index[r] <- src row r;  r < rows,
 * rows with index[r] < 0 are skipped.  copy_bytes at column offsets dst_col / src_col of rows with
 * pitches dst_pitch / src_pitch (all multiples of 16). */
int netra_moe_move_rows_launch(void* dst, const void* src, const int32_t* index, uint32_t rows, uint32_t copy_bytes,
                               uint32_t dst_pitch, uint32_t src_pitch, uint32_t dst_col, uint32_t src_col,
                               uint32_t scatter, cudaStream_t stream);
/* Fixed-capacity exchange.  pack: this rank's sorted FP8 rows and scales for rank g -> slot rows
 * [g*slot_rows, ...) of send_slots (2112 bytes per row: 2048 codes + 16 FP32 scales); a destination
 * that needs more than slot_rows rows records its count in *overflow (device word, 0 = fits).
 * unpack: returned FP32 rows, slot row (g, i) -> sorted row offsets[g*experts_per_rank] + i of down. */
int netra_ep_pack_rows_launch(void* send_slots, const void* a_fp8, const float* a_scale_f32, const int32_t* offsets_i32,
                              uint32_t ranks, uint32_t experts_per_rank, uint32_t slot_rows, uint32_t* overflow,
                              cudaStream_t stream);
int netra_ep_unpack_rows_launch(float* down_f32, const float* back_slots_f32, const int32_t* offsets_i32, uint32_t ranks,
                                uint32_t experts_per_rank, uint32_t slot_rows, cudaStream_t stream);

/* ---- Expert parallelism over peer memory (no counterpart in the reference, whose 8-GPU mode is
 * eight replicas: manifests/gfx950/models/qwen36-moe-m1-golden.json:11-12).
 * Rank r owns routed experts [r*256/world, (r+1)*256/world) and a copy of the shared expert; its
 * weight arrays hold the shared slab FIRST, then its routed slabs.  Every exchange (pair counts,
 * FP8 rows to the owners' expert-major blocks, FP32 rows back to the senders' sorted order) is done
 * by this library's kernels with stores into the peers' windows and epoch flags; every wait is
 * bounded by wait_timeout_ns and reports through the status words instead of hanging.  One call is
 * netra_ep_layer_launch_count() launches (eight up to 1024 tokens, ten above), no host read-back, so a
 * caller may capture it into a CUDA graph.  All ranks must make the same sequence of calls.
 *
 * A window is device memory that the peers can write: netra_ep_window_create allocates one
 * (cudaMalloc, zero-filled) and exports a 64-byte CUDA IPC handle that another PROCESS on the same
 * node opens with netra_ep_window_open; ranks inside one process pass each other's pointers
 * directly.  All ranks must have created (zeroed) their windows before any rank's first call. */
int netra_ep_sizes_query(uint32_t world, uint32_t max_tokens, uint32_t row_capacity, uint64_t* workspace_bytes,
                         uint64_t* window_bytes);
int netra_ep_window_create(uint64_t bytes, void** window, void* ipc_handle_64);
int netra_ep_window_open(const void* ipc_handle_64, void** window);
int netra_ep_window_close(void* window);     /* a window obtained from netra_ep_window_open */
int netra_ep_window_destroy(void* window);   /* a window obtained from netra_ep_window_create */

typedef struct netra_ep_layer netra_ep_layer_t;
typedef struct netra_ep_layer_desc {
  uint32_t struct_size;
  uint32_t world;               /* ranks; divides 256, at most 16 */
  uint32_t rank;
  uint32_t max_tokens;          /* this rank's tokens per call, at most */
  uint32_t row_capacity;        /* rows one rank's expert block can hold (its own tokens + routed rows from all
                                   ranks); the same on every rank.  A call that needs more reports the needed
                                   count in status word 2 and its result is invalid. */
  uint32_t weights_tiled;
  uint64_t wait_timeout_ns;     /* bound of every flag wait */
  const void* router_weight_bf16;
  const float* router_bias_f32; /* may be NULL */
  const void* w13_fp8;          /* [1 + 256/world, 1024, 2048] (or its tile order), shared slab first */
  const float* w13_scale_f32;
  const void* w2_fp8;           /* [1 + 256/world, 2048, 512] */
  const float* w2_scale_f32;
  void* workspace;              /* local device scratch, 1024-byte aligned, netra_ep_sizes_query bytes */
  uint64_t workspace_bytes;
  void* const* windows;         /* host array of `world` device pointers; windows[rank] is this rank's own */
  uint64_t window_bytes;
} netra_ep_layer_desc_t;
int netra_ep_layer_create(const netra_ep_layer_desc_t* desc, netra_ep_layer_t** output);
/* hidden BF16 [tokens, 2048], out BF16 [tokens, 2048], shared_weight FP32 [tokens] or NULL (1.0). */
int netra_ep_layer_launch(netra_ep_layer_t* layer, const void* hidden_bf16, const float* shared_weight_f32, void* out_bf16,
                          uint32_t tokens, cudaStream_t stream);
/* One stage of the call (0 router, 1 top-8 + quantise, 2 sort, 3 publish counts, 4 plan, 5 push rows + return table,
 * 6 gate_up (waits for the pushed rows first), 7 down with the return fused in, 8 combine (waits for the returned rows
 * first)): for per-stage timing, and for running several ranks' calls interleaved stage by stage on one stream of one
 * GPU, where every wait finds its flags already raised.  netra_ep_layer_launch runs stages 3 and 4 as one launch, which
 * is only possible when every rank has a GPU of its own. */
int netra_ep_layer_launch_stage(netra_ep_layer_t* layer, uint32_t stage, const void* hidden_bf16, const float* shared_weight_f32,
                                void* out_bf16, uint32_t tokens, cudaStream_t stream);
uint32_t netra_ep_layer_stage_count(void);
uint32_t netra_ep_layer_launch_count(const netra_ep_layer_t* layer, uint32_t tokens);
/* format 1: calls served by the token-major GEMMs (an average of 32 rows per routed expert over all ranks, or more) use
 * the prefill contract of netra_moe_layer_set_partial_format: the token-major down projection rounds its rows to FP16
 * partials and its epilogue sends every run of rows that one source sent to one expert home as one bulk copy over NVLink
 * (half the bytes of the FP32 return), and the reducer widens them (f32(p) * w, slot ascending, one BF16 rounding).  Results equal the one-GPU layer
 * with the same setting bit for bit.  Every rank of a world must use the same format.  format 0 (default): FP32 rows
 * stored by the down projection's epilogue. */
int netra_ep_layer_set_partial_format(netra_ep_layer_t* layer, uint32_t format);
/* Status words (synchronises): 0 gate_up wait expired, 1 down wait expired, 2 rows needed when that
 * exceeds row_capacity, 3 bit (8*phase + min(rank,7)) set when the flag of that phase and rank timed out. */
int netra_ep_layer_status(netra_ep_layer_t* layer, uint32_t status_out[4]);
int netra_ep_layer_destroy(netra_ep_layer_t* layer);

/* Block size and dynamic shared memory of the tensor-core kernels (which: 0 gate_up, 1 down, 2 and 3 their
 * token-major forms, 4 token-major down with FP16 rows, 5 tensor-core router, 6 and 7 gate_up and down on MXFP4 weights,
 * 8 and 9 their token-major forms, 10 gate_up and down in one launch), so
 * that an engine manifest written ahead of time can be checked against the built library. */
int netra_moe_kernel_launch_info(uint32_t which, uint32_t* block_threads, uint32_t* dynamic_smem_bytes);

/* The two grouped GEMMs exist in two forms: swap-AB (weights are the MMA M dimension; decode sizes) and
 * token-major (128 token rows x 256 weight rows per MMA; from an average of 32 rows per routed expert).
 * mode 0 (default) picks by the token count of the call, mode 1 always uses the swap-AB kernels.  Both
 * forms produce identical results.  mode 2 = swap-AB with the two projections in one launch for calls of up to 1,024
 * tokens on E4M3 weights (netra_moe_gate_up_down_umma_sm100: the down half starts on an expert chunk's rows as soon as
 * the gate_up half has written them): the same results, one launch fewer, measured 4 us slower per 256-token call
 * than two launches - a recorded tactic. */
int netra_moe_layer_set_gemm_mode(netra_moe_layer_t* layer, uint32_t mode);

/* mode 1: calls of up to 1,024 tokens run router logits, softmax / top-8 + quantisation and the expert sort in one launch
 * (netra_moe_route_front_sm100: blocks hand over by last-arriver counters, nothing waits): stage 0 is then the whole
 * routing front end and stages 1 and 2 launch nothing.  Same results as the three launches of mode 0 (default), two
 * launches fewer, measured 4 us slower per 256-token call: a recorded tactic. */
int netra_moe_layer_set_front_mode(netra_moe_layer_t* layer, uint32_t mode);

/* Where gate_up (E4M3 weights) takes its token rows from.  in_gemm 0 (default): an expert-sorted copy of the quantised
 * rows written by the row-gather stage.  in_gemm 1: no copy; the GEMM's producer fetches the rows from token order with
 * four-row TMA gathers (cp.async.bulk.tensor tile::gather4).  Same results, one launch fewer; measured 2.5 times slower
 * at 8,192 tokens (token-major form: 32 gather instructions per 128-row tile and K-block) and 9 us slower per 256-token
 * call (swap-AB form: eight per 32-row tile and K-block), kept as a recorded tactic. */
int netra_moe_layer_set_row_gather(netra_moe_layer_t* layer, uint32_t in_gemm);

/* Router of calls above 1024 rows.  mode 0 (default): BF16 tensor-core pass with FP32 accumulation, then an FP64
 * recomputation of those logits that can reach the top 8 and whose BF16 rounding the FP32 value cannot decide:
 * the selected ids, their logits and the routing weights are those of the exactly rounded dot products; logits
 * of experts that cannot be selected keep the rounded tensor-core value (within 2^-18 |h| |w| plus one BF16
 * spacing of the exact rounding).  mode 2: the same with every undecided
 * logit recomputed, so that the whole logits array is the exactly rounded one (several times slower).  mode 1:
 * every logit on the FP64 tensor cores (the form used up to 1024 rows). */
int netra_moe_layer_set_router_mode(netra_moe_layer_t* layer, uint32_t mode);
/* Copies the router statistics words (see netra_moe_workspace_layout_t.router_stats) to the host (synchronises). */
int netra_moe_layer_router_stats(netra_moe_layer_t* layer, uint32_t stats_out[4]);

/* Format of the down projection's rows between the grouped GEMM and the combine, for calls served by the
 * token-major kernels.  format 0 (default): FP32 rows (the decode contract,
 * kernels/gfx950/templates/moe/decode/down_reduce_mfma_2wave.inc:73-217).  format 1: FP16 partial rows, half the
 * bytes, the reference's prefill contract (kernels/gfx950/templates/moe/prefill/fused_splitk2/down_partial.inc:435-458,
 * route_reduce_splitk2_f16.inc:107-118: f32(partial) * weight, slot ascending, one BF16 rounding).  Calls served
 * by the swap-AB kernels keep FP32 rows under either setting. */
int netra_moe_layer_set_partial_format(netra_moe_layer_t* layer, uint32_t format);

/* Copies the four device status words to the host (synchronises the device). */
int netra_moe_layer_status(netra_moe_layer_t* layer, uint32_t status_out[4]);
/* Kernels launched by one netra_moe_layer_launch call with `tokens` rows (the sort is one launch
 * up to 1024 rows and three above). */
uint32_t netra_moe_layer_launch_count(const netra_moe_layer_t* layer, uint32_t tokens);
int netra_moe_layer_destroy(netra_moe_layer_t* layer);
const char* netra_moe_last_error(void);

/* No counterpart in the reference.  Stable expert-major sort of the rows*8 routed pairs for
 * callers that cannot allocate device memory (a process whose memory belongs to one framework
 * allocator, a plugin barred from driver allocations after start-up, a step inside stream
 * capture): the scratch table lives in a fixed 128 KiB device array inside the library, so only
 * inputs and outputs are passed.  topk_ids_i32 is [rows, 9] (slot 8 ignored; ids outside 0..255
 * are treated as the nearest valid expert, 0 or 255, so that no id can index out of range); outputs
 * are perm [rows*8], inv_perm [rows*8], counts [256], offsets [258], identical to the fused layer's.
 * rows must be 1..16384 (larger is refused).  The first call on a device resolves the array's
 * address and should be made outside stream capture.  All calls on a device share the array:
 * calls that overlap on the GPU race and must be serialised by the caller. */
int netra_moe_sort_static_scratch_launch(const int32_t* topk_ids_i32, int32_t* perm_i32,
                                         int32_t* inv_perm_i32, int32_t* counts_i32,
                                         int32_t* offsets_i32, uint32_t rows, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
