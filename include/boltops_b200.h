/*
 * boltops_b200 -- C ABI of the B200 (sm_100a) fused-MoE hot path.
 *
 * Every entry point takes raw device pointers, sizes and a CUDA stream handle
 * (cudaStream_t passed as void*), launches asynchronously on that stream, never
 * synchronises the host, and returns a bolt_status.  No torch types appear in
 * any signature.  Unless stated otherwise an entry point allocates nothing: the
 * caller owns inputs, outputs and workspaces.
 *
 * The reference project exposes this path through Python only; the closest
 * native interface it has is the pybind entry moe_sorting_fwd
 * (boltops/fused_moe/triton/moe_sorting_hipc/csrc/moe_sorting_binding.cu:73-88).
 * Each declaration below names the reference function it replaces
 * (paths relative to the reference project root).
 */
#ifndef BOLTOPS_B200_H_
#define BOLTOPS_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BOLT_ABI_VERSION 3

enum bolt_status {
  BOLT_OK = 0,
  BOLT_ERR_INVALID = 1,      /* argument contract violated                      */
  BOLT_ERR_CUDA = 2,         /* a CUDA runtime/driver call failed               */
  BOLT_ERR_UNSUPPORTED = 3,  /* valid request, not built for this variant       */
  BOLT_ERR_DEVICE = 4        /* a kernel reported a bounded-wait expiry         */
};

enum bolt_dtype {
  BOLT_BF16 = 0,
  BOLT_F16 = 1,
  BOLT_F32 = 2,
  BOLT_FP8_E4M3 = 3,
  BOLT_INT8 = 4
};

/* activation kinds of bolt_moe_activation (names follow the reference registry,
 * boltops/fused_moe/triton/moe_activation.py:1065-1116) */
enum bolt_activation {
  BOLT_ACT_SILU = 0,
  BOLT_ACT_GELU = 1,
  BOLT_ACT_GELU_TANH = 2,
  BOLT_ACT_RELU2 = 3,
  BOLT_ACT_SWIGLU_OAI = 4,   /* gate'*sigmoid(alpha*gate')*(up'+1), chunked layout */
  BOLT_ACT_SWIGLU_STEP = 5,  /* min(silu(gate),limit)*clamp(up,+-limit)            */
  BOLT_ACT_SILU_CLAMP = 6,   /* silu(min(gate,limit))*clamp(up,+-limit)            */
  BOLT_ACT_SWIGLU_OAI_INTERLEAVED = 7, /* as SWIGLU_OAI on the [g0,u0,g1,u1,...] layout   */
  BOLT_ACT_SITU = 8          /* beta*tanh(gate/beta)*sigmoid(gate) * up', with alpha = beta and
                                up' = limit*tanh(up/limit) when limit > 0, else up  */
};

/* grouped-GEMM operand kinds */
enum bolt_gemm_kind {
  BOLT_GEMM_BF16 = 0,         /* bf16 x bf16 -> fp32                                    */
  BOLT_GEMM_F16 = 1,          /* fp16 x fp16 -> fp32                                    */
  BOLT_GEMM_FP8_BLOCK = 2,    /* e4m3, [128,128] weight blocks, 1x128 activation groups */
  BOLT_GEMM_INT8_CHANNEL = 3, /* int8, per-row activation / per-output-channel weight   */
  BOLT_GEMM_FP8_CHANNEL = 4,  /* e4m3, per-row activation / per-output-channel weight   */
  BOLT_GEMM_INT8_BLOCK = 5,   /* int8, [128,128] weight blocks, 1x128 activation groups */
  BOLT_GEMM_MXFP8 = 6,        /* e4m3 with one E8M0 byte per 32 K elements on both operands,
                                 applied by the tensor core; a_scale / b_scale carry BYTE
                                 arrays in the tiled layout of bolt_mx_sf_layout; plain
                                 epilogue or the gated activation + MX re-quantisation
                                 (BOLT_EPI_SILU_MUL_QUANT); k a multiple of 128            */
  BOLT_GEMM_MXFP4 = 7         /* e4m3 rows x PACKED e2m1 weights ([E, n, k/2] bytes, low nibble
                                 first, 32-byte aligned), one E8M0 byte per 32 K elements on
                                 both operands in the same tiled layout as BOLT_GEMM_MXFP8;
                                 plain epilogue, k a multiple of 128                        */
};

/* grouped-GEMM schedules */
enum bolt_gemm_schedule {
  BOLT_GEMM_SCHEDULE_ROW_TILES = 0,  /* one CTA per 128-row x 256-column tile                      */
  BOLT_GEMM_SCHEDULE_TILE_PAIRS = 1  /* two CTAs of a cluster share the weight tile of two row
                                        tiles of one expert (tcgen05 cta_group::2, 256 x 256 per
                                        pair): for experts with several row tiles.  Needs the
                                        segment list of bolt_moe_sort_ck with segment_rows =
                                        BOLT_PAIR_SEGMENT_ROWS; not for the MX kind.               */
};
#define BOLT_PAIR_SEGMENT_ROWS 256

enum bolt_gemm_epilogue {
  BOLT_EPI_STORE = 0,        /* C = dequant(A.B^T)                                      */
  BOLT_EPI_SILU_MUL = 1,     /* C = silu(gate)*up, B rows [0,N/2) gate, [N/2,N) up       */
  BOLT_EPI_SILU_MUL_QUANT = 2/* as above, then 1x128-group quantisation to e4m3/int8    */
};

/* Message of the last non-OK status returned on the calling thread. */
const char* bolt_last_error(void);
int bolt_abi_version(void);

/* ---------------------------------------------------------------------------
 * Token-to-expert sort, CK format.
 * Replaces moe_sorting_fwd (moe_sorting_hipc/csrc/moe_sorting_binding.cu:15-71,
 * moe_sorting_api.cu:118-180) as driven by moe_sorting_ck
 * (boltops/fused_moe/triton/fused_moe.py:441-485).
 *   sorted_ids[i]   = token | slot << 24, ascending route order inside an expert,
 *                     every expert padded to unit_size with id num_tokens|topk<<24
 *                     and weight 0; experts without routes get no block; with a
 *                     mask, masked experts get no block and expert ids are the
 *                     count of enabled experts before them.
 *   capacity        = num_tokens*topk + num_experts*unit_size - topk entries
 *   sorted_expert_ids: ceil(capacity/unit_size) entries
 *   tokens_positions_per_expert: [0,E) route counts, [E,2E) padded start offsets
 *                     (-1 for masked experts)
 *   num_valid_ids[0] = padded total
 *   route_pos (optional, may be NULL): [num_tokens*topk] position of every route in the
 *                     sorted order, -1 for routes to masked or out-of-range experts (an
 *                     addition of this library: the inverse permutation the combine uses)
 *   segments / num_segments (optional, may be NULL; another addition): every enabled expert's
 *                     live rows cut into runs of at most segment_rows rows, in sorted order:
 *                     segments[4*s..] = {expert id as in sorted_expert_ids, first sorted row,
 *                     rows, 0}; at most min(E, routes) + routes/segment_rows entries;
 *                     num_segments[0] = their number.  Consumed by the tile-pair schedule
 *                     of bolt_grouped_gemm (segment_rows = 2 * unit_size = 256).
 *   moe_buf (optional, may be NULL): zero-filled, moe_buf_bytes long.
 *   workspace: bolt_moe_sort_workspace_bytes() bytes, 16-byte aligned; contents
 *   are scratch and need no initialisation.
 */
size_t bolt_moe_sort_workspace_bytes(int num_tokens, int topk, int num_experts);
int bolt_moe_sort_ck(const int32_t* topk_ids, const float* topk_weights,
                     const int32_t* local_expert_mask, int num_tokens, int topk,
                     int num_experts, int unit_size, int32_t* sorted_ids,
                     float* sorted_weights, int32_t* sorted_expert_ids,
                     int32_t* tokens_positions_per_expert, int32_t* num_valid_ids,
                     int32_t* route_pos, int32_t* segments, int32_t* num_segments,
                     int segment_rows, void* moe_buf, size_t moe_buf_bytes, void* workspace,
                     size_t workspace_bytes, void* stream);

/* Allocation-free CK-format sort.  Same outputs as bolt_moe_sort_ck, but the scratch
 * memory of the multi-block path is a fixed 1 MiB array inside the library image
 * (bolt_moe_sort_static_scratch_bytes()), so the caller passes inputs and outputs
 * only and no device memory is allocated by anyone.
 *
 * Written for callers that cannot allocate on the device when they reach this call:
 * a serving engine that gave the whole device heap to its own pools at start-up (a
 * late cudaMalloc there fails or stalls the device), or a host-language binding that
 * owns no device allocator at all and can only hand over the buffers it was given.
 *
 * It has no counterpart in the reference, whose sorter always receives a workspace
 * tensor from torch.
 *
 * Limits and rules:
 *  - Requests whose scratch need (bolt_moe_sort_workspace_bytes) exceeds the array are
 *    refused with BOLT_ERR_INVALID and a message; use bolt_moe_sort_ck then.
 *  - The first call on each device resolves the array's device address (a
 *    cudaGetSymbolAddress look-up, with that device current).  Make that first call
 *    during start-up, before any stream capture.
 *  - All calls on a device share the one array and it keeps the previous call's
 *    contents.  Nothing in it has to be cleared between calls (every entry is written
 *    before it is read), but two calls that overlap on the GPU -- different streams,
 *    or different host threads -- race on it; keep calls on one device in stream order.
 *  - Every GPU that loads the library holds the 1 MiB until the process exits.
 *  - moe_buf zeroing is not offered here.
 */
size_t bolt_moe_sort_static_scratch_bytes(void);
int bolt_moe_sort_ck_static(const int32_t* topk_ids, const float* topk_weights,
                            const int32_t* local_expert_mask, int num_tokens, int topk,
                            int num_experts, int unit_size, int32_t* sorted_ids,
                            float* sorted_weights, int32_t* sorted_expert_ids,
                            int32_t* tokens_positions_per_expert, int32_t* num_valid_ids,
                            void* stream);

/* Token-to-expert sort, vLLM format.
 * Replaces moe_align_block_size (boltops/fused_moe/triton/fused_moe.py:330-439,
 * stages :194-327): sorted_ids = flat route index, whole capacity
 * numel + E*(block_size-1) pre-filled with numel; expert_ids zero-filled over
 * ceil(capacity/block_size) entries, then mapped through expert_map if given.
 */
int bolt_moe_align_block_size(const int32_t* topk_ids, int numel, int num_experts,
                              int block_size, const int32_t* expert_map,
                              int32_t* sorted_ids, int32_t* expert_ids,
                              int32_t* num_tokens_post_pad, void* workspace,
                              size_t workspace_bytes, void* stream);

/* ---------------------------------------------------------------------------
 * Router front-end (the step right before the sort).  Replaces fused_topk
 * (boltops/tools/fused_moe_triton_tune/routing.py:10-35): scores = softmax (or sigmoid)
 * of the fp32 logits, top-k, optional renormalisation; fp32 weights, int32 ids.
 * gating [num_tokens, num_experts] bf16/f16/f32, num_experts <= 1024, topk <= 32.
 */
int bolt_fused_topk(const void* gating, int dtype, int64_t num_tokens, int num_experts, int topk,
                    int renormalize, int is_softmax, float* topk_weights, int32_t* topk_ids,
                    void* stream);

/* Grouped gate with optional fused shared expert.  Replaces moe_fused_gate
 * (boltops/tools/fused_moe_triton_tune/routing.py:38-79): sigmoid scores, + bias for the
 * choice, group score = sum of the two best choices of a group, topk_group groups kept, top-k
 * experts inside them, weights = unbiased scores renormalised; with one fused shared expert
 * the last slot is expert id num_experts with weight sum(others)/routed_scaling_factor.
 */
int bolt_moe_fused_gate(const void* gating, int dtype, const float* bias, int64_t num_tokens,
                        int num_experts, int num_expert_group, int topk_group, int topk,
                        int num_fused_shared_experts, float routed_scaling_factor,
                        float* topk_weights, int32_t* topk_ids, void* stream);

/* Expert-parallel dispatch helper (no reference counterpart: the reference leaves expert
 * parallelism to the serving engine and only takes its expert_map,
 * boltops/fused_moe/__init__.py:127-133).  routes[t][r] = r when one of token t's experts
 * lives on rank r (experts sharded contiguously, experts_per_rank each), else -1; ids outside
 * [0, num_experts) hit no rank.  Sorting these routes with bolt_moe_sort_ck (ranks as experts,
 * unit 1) yields the send order, the per-rank counts and the inverse permutation.  With
 * chunk_tokens > 0 the value is (t / chunk_tokens) * world + r, so the same sort orders the
 * rows by (token chunk, rank, token) for a dispatch that is pipelined chunk by chunk.
 */
int bolt_ep_dest_ranks(const int32_t* topk_ids, int64_t num_tokens, int topk, int num_experts,
                       int experts_per_rank, int world, int64_t chunk_tokens, int32_t* routes,
                       void* stream);

/* Expert-parallel wire format (no reference counterpart).  One row per (token, destination
 * rank): [row data | fp32 scales of the row | top-k ids | top-k weights], each part padded to a
 * multiple of 16 bytes; bolt_ep_wire_row_bytes gives the row size.  bolt_ep_pack_rows fills
 * rows [0, rows) of `out` from the tokens send_ids[first + i] & 0xFFFFFF (send_ids = the sorted
 * ids of the dispatch sort), so the whole send buffer of a chunk is written by one kernel and
 * travels in one all-to-all.  The receiver reads the parts in place (bolt_gather_rows takes a
 * source row stride).  data: [tokens, row_bytes] (quantised codes or 16-bit rows), scales:
 * [tokens, groups] or NULL with groups = 0.
 */
int64_t bolt_ep_wire_row_bytes(int row_bytes, int groups, int topk);
int bolt_ep_pack_rows(const void* data, int row_bytes, const float* scales, int groups,
                      const int32_t* topk_ids, const float* topk_weights, int topk,
                      const int32_t* send_ids, int64_t first, int64_t rows, void* out,
                      int64_t out_stride, void* stream);

/* ---------------------------------------------------------------------------
 * Dynamic activation quantisation.
 * Replaces per_token_quant_triton / dynamic_per_token_quant_fp8_i8
 * (boltops/fused_moe/triton/moe_compat.py:55-106, quant.py:145-368) and, with
 * power2 != 0, dynamic_per_group_quant_fp8_power2 (quant.py:636-661).
 *   x [rows, cols] (bf16/f16/f32, contiguous); group = cols (per token) or a
 *   divisor of cols (1 x group); q [rows, cols] e4m3 or int8; scales fp32
 *   [rows, cols/group] (scales_ld == 0) or group-major [cols/group, scales_ld] with
 *   scales_ld >= rows (the layout bolt_grouped_gemm reads its a_scale in).
 */
int bolt_quant_rows(const void* x, int x_dtype, int64_t rows, int cols, int group,
                    int q_dtype, int power2, void* q, float* scales, int64_t scales_ld,
                    void* stream);

/* Row gather into the expert-sorted padded layout used by the grouped GEMMs.
 *   dst[i, :] = src[sorted_ids[i] & 0xFFFFFF, :] for i < num_valid_ids[0]
 *   (zero rows for pad ids); row_bytes must be a multiple of 16.
 *   If src_scale != NULL, scales are gathered too:
 *     groups > 1 : dst_scale[g * dst_scale_ld + i] = src_scale[token*groups + g]
 *     groups == 1: dst_scale[i] = src_scale[token]
 *   src_stride_bytes / src_scale_stride: distance between source rows in bytes / in floats
 *   (0 = dense rows), so rows and scales can be read in place from a wider record.
 * No counterpart in the reference (its GEMM gathers rows through pointer
 * arithmetic, boltops/fused_moe/triton/moe_op.py:1479,1611-1615).
 */
int bolt_gather_rows(const void* src, int num_tokens, int row_bytes, int64_t src_stride_bytes,
                     const float* src_scale, int64_t src_scale_stride, int groups,
                     const int32_t* sorted_ids, const int32_t* num_valid_ids, int capacity,
                     void* dst, float* dst_scale, int64_t dst_scale_ld, void* stream);

/* bolt_quant_rows and bolt_gather_rows in one pass for 1 x group quantisation (group a
 * multiple of the 16-byte input vector, at most 256 vectors: 128-wide blocks as well as whole
 * rows up to 2048 bf16 / 1024 fp32 elements): every token is quantised once and its codes
 * and scales are written to the sorted rows route_pos[token][k] >= 0 (route_pos as produced by
 * bolt_moe_sort_ck, [num_tokens, slots]); rows below num_valid_ids[0] that hold no token are
 * zero-filled.  dst [capacity, cols] 8-bit, dst_scale [cols/group, dst_scale_ld] fp32 (one
 * group per row: a plain [capacity] vector).
 * codes_in_token_order != 0: for a GEMM that gathers its rows itself (bolt_gemm_args.a_gather).
 * dst is then [num_tokens, cols]: every token's codes once, in token order; the scales still go
 * to the sorted positions (zeros for the padding positions).
 * Same arithmetic and the same reference functions as bolt_quant_rows.
 */
int bolt_quant_scatter_rows(const void* x, int x_dtype, int64_t num_tokens, int cols, int group,
                            int q_dtype, int power2, const int32_t* route_pos, int slots,
                            const int32_t* sorted_ids, const int32_t* num_valid_ids,
                            int capacity, void* dst, float* dst_scale, int64_t dst_scale_ld,
                            int codes_in_token_order, void* stream);

/* MX (microscaling) e4m3 quantisation with 1 x 32 groups and E8M0 exponent bytes.  Replaces
 * mxfp8_e4m3_quantize (boltops/fused_moe/triton/mxfp8.py:122-175): byte =
 * clamp(ceil(log2(amax/448)) + 127, 0, 254), q = e4m3(v * 2^(127-byte)); with gated != 0 the
 * input is [rows, 2*cols] = [gate | up] and v = min(g,L) * sigmoid(alpha*g) * (clamp(u,+-L) + beta)
 * in fp32 (L only when has_limit).  Outputs, each optional: q [rows, cols] e4m3, scales
 * [rows, cols/32] bytes, deq [rows, cols] = q * 2^(byte-127) in deq_dtype (exact).
 */
int bolt_mx_quant_rows(const void* x, int x_dtype, int64_t rows, int cols, int gated, float alpha,
                       float beta, int has_limit, float limit, void* q, uint8_t* scales, void* deq,
                       int deq_dtype, void* stream);

/* q [rows, cols] e4m3 with exponent bytes [rows, cols/32] -> out [rows, cols] in out_dtype
 * (w * 2^(byte-127); the decoding of MX checkpoint weights,
 * boltops/fused_moe/triton/moe_compat.py `_upcast_e8m0_to_fp32` applied per group).
 */
int bolt_mx_dequant_rows(const void* q, const uint8_t* scales, int64_t rows, int cols, void* out,
                         int out_dtype, void* stream);

/* E8M0 bytes [src_rows, sf_cols] (sf_cols = K/32, a multiple of 4) -> the tiled layout that
 * BOLT_GEMM_MXFP8 reads: [dst_rows/128][sf_cols/4][512] bytes, byte (r%32)*16 + (r/32)*4 + g for
 * row r of a 128-row tile and K group g of a 128-wide K block.  row_ids (optional) gathers rows
 * as the expert-sorted layout does (token in the low 24 bits, rows at or beyond
 * num_valid_ids[0] and padding ids get byte 0).  No reference counterpart: the reference's
 * Triton kernel reads the plain [rows, K/32] array (boltops/fused_moe/triton/mxfp8.py).
 */
int bolt_mx_sf_layout(const uint8_t* src, int64_t src_rows, int sf_cols, const int32_t* row_ids,
                      const int32_t* num_valid_ids, int64_t dst_rows, uint8_t* dst, void* stream);

/* ---------------------------------------------------------------------------
 * Activations.  Replaces _apply_activation / moe_activation
 * (boltops/fused_moe/triton/moe_activation.py:1382-1525; kernels :70-128 etc.).
 * gated: in [rows, 2*n_out] = [gate | up], out [rows, n_out]; else in [rows, n_out].
 * fp32 math, result stored in `dtype`.  alpha/limit as gemm1_alpha/gemm1_limit.
 * rows_dev (optional): device int32 row count that further bounds `rows`.
 */
int bolt_moe_activation(const void* in, void* out, int dtype, int64_t rows, int n_out,
                        int activation, int gated, float alpha, float limit,
                        const int32_t* rows_dev, void* stream);

/* Fused activation + per-token quantisation.  Replaces triton_activation_quant
 * (boltops/fused_moe/triton/moe_activation.py:290-421,1239-1332): activation,
 * rounding to `dtype`, per-row absmax quantisation, optional scale *= row
 * multiplier (router-weight folding).
 */
int bolt_act_quant(const void* in, int dtype, int64_t rows, int n_out, int activation,
                   int gated, int q_dtype, const float* row_multiplier, void* q,
                   float* scales, const int32_t* rows_dev, void* stream);

/* ---------------------------------------------------------------------------
 * Top-k combine.  Replaces triton_moe_sum / moe_sum_kernel
 * (boltops/fused_moe/triton/fused_moe.py:72-188):
 *   out[m, :] = cast(scale * sum_k f32(in[m, k, :]) [* weights[m, k]]).
 */
int bolt_moe_sum(const void* in, int in_dtype, void* out, int out_dtype, int64_t num_tokens,
                 int topk, int n, float scale, const float* weights, void* stream);

/* Expert-parallel combine on the source rank:
 *   out[m, :] = cast(scale * sum over j in [0, slots) with pos[m, j] >= 0 of f32(src[pos[m, j], :]))
 * (j ascending, fp32 accumulator).  `src` holds the partial layer outputs that came back
 * from the ranks owning a token's experts, `pos` [num_tokens, slots] their row numbers.
 * With pos = route_pos of bolt_moe_sort_ck and src = the down-GEMM output in sorted row
 * order this is the layer's top-k combine (same summation order as bolt_moe_sum, without the
 * [M, topk, H] intermediate).  No counterpart in the reference, which scatters to [M, topk, H]
 * and leaves the cross-rank reduction to its caller
 * (boltops/fused_moe/triton/fused_moe.py:1374-1377 documents the partial-sum contract).
 */
int bolt_moe_gather_sum(const void* src, int dtype, const int32_t* pos, void* out, int out_dtype,
                        int64_t num_tokens, int slots, int n, float scale, void* stream);

/* ---------------------------------------------------------------------------
 * Direct expert-parallel exchange over peer memory (no reference counterpart: the reference
 * leaves expert parallelism to the serving engine, boltops/fused_moe/__init__.py:127-133).
 * Every rank owns one exchange buffer of the same layout that all ranks can address (`peers`: a
 * device array of the `world` base addresses, in rank order):
 *   hdr_off  : int32 [world][2]  = {rows sent by rank s, first row of s's return region for me}
 *   flag_off : int32 [world + 1] = epochs of bolt_ep_barrier: flag of every rank, then this rank's
 *                                  own epoch counter (all zero before the first call)
 *   recv_off : world segments of seg_rows wire rows (layout of bolt_ep_pack_rows), segment s
 *              written by rank s
 *   return region (its address goes into seg_ptrs): partial output rows, in the owner's send order
 * bolt_ep_dispatch_rows: rank `me` writes its wire rows (send order = sorted ids of the dispatch
 *   sort, counts [world] = its per-rank counts, both in device memory: no host round trip) into
 *   segment `me` of every destination's receive region and {count, first row} into its header;
 *   max_rows bounds the grid.  Counts above seg_rows are clamped and flagged in *status (21).
 * bolt_ep_unpack_routes: the receiver's dense top-k ids (-1 for rows a segment does not hold) and
 *   weights for all world * seg_rows rows, which the masked local layer then takes as its batch;
 *   optionally (src_tokens != NULL) every row's token index on the rank it came from, which
 *   bolt_ep_dispatch_rows leaves at byte bolt_ep_wire_row_bytes(...) of a wire row that is at
 *   least 16 bytes longer than that (src_off = that byte offset).
 * bolt_moe_gather_sum_to_peers: bolt_moe_gather_sum whose output row m (m = first_row + i) goes to
 *   row hdr[2 s + 1] + q of the region seg_ptrs[s], s = m / seg_rows, q = m % seg_rows, and is
 *   skipped when q >= hdr[2 s]: the top-k combine of the local layer writes every partial row
 *   straight into the return region of the rank the token came from.
 * bolt_ep_barrier: all ranks meet (flags in peer memory; the kernel advances its rank's epoch
 *   counter itself, so every rank must call it the same number of times and a step holds no
 *   host-side state); every wait is bounded (~1 s), on expiry *status is set to 20 and the
 *   kernel returns.
 * One process per GPU; the kernels use plain loads and stores on peer addresses only.
 */
int bolt_ep_dispatch_rows(const void* data, int row_bytes, const float* scales, int groups,
                          const int32_t* topk_ids, const float* topk_weights, int topk,
                          const int32_t* send_ids, const int32_t* counts, int world, int me,
                          int64_t max_rows, int64_t seg_rows, const int64_t* peers, int64_t hdr_off,
                          int64_t recv_off, int64_t wire_bytes, int32_t* status, void* stream);
int bolt_ep_unpack_routes(const void* recv, int64_t wire_bytes, int64_t ids_off, int64_t wts_off,
                          int topk, int64_t seg_rows, int nseg, const int32_t* hdr,
                          int32_t* topk_ids, float* topk_weights, int64_t src_off,
                          int32_t* src_tokens, void* stream);
int bolt_moe_gather_sum_to_peers(const void* src, int dtype, const int32_t* pos, int64_t num_tokens,
                                 int slots, int n, float scale, int64_t seg_rows,
                                 const int64_t* seg_ptrs, const int32_t* hdr, int64_t first_row,
                                 void* stream);
int bolt_ep_barrier(const int64_t* peers, int world, int me, int64_t flag_off, int32_t* status,
                    void* stream);

/* ---------------------------------------------------------------------------
 * MXFP4 (w4a8) experts.  Replace the element-wise parts of fused_experts_mxfp_impl with
 * use_mxfp4_w4a8 (boltops/fused_moe/triton/fused_moe.py:923-1197): weight decoding
 * (boltops/fused_moe/triton/mxfp4.py:61-157 reads packed e2m1 nibbles, low nibble first, with
 * one E8M0 byte per 32 K elements), the activation quantisers
 * (per_token_group_quant_fp8_mxfp4 and silu_mul_quant_fp8_packed_triton,
 * boltops/fused_moe/triton/mxfp4_quant.py:38-80,206-317; static_per_tensor_quant_fp8_i8,
 * boltops/fused_moe/triton/quant.py:33-82) and the fused epilogues of the static recipe
 * (moe_gemm_mxfp4 with fuse_swiglu / quant_scale / bias, mxfp4.py:194-286).  The contractions
 * themselves run through bolt_grouped_gemm on decoded operands (exact, see csrc/mxfp4.cu).
 *
 * bolt_mxfp4_decode: packed [rows, cols/2] + scales [rows, cols/32] -> out [rows, cols].
 * bolt_mx4_act_quant: x [rows, cols] (or [rows, 2*cols] = [gate | up] with gated != 0: SiLU(gate)
 *   * up, optional clamp, rounded through bf16) -> e4m3 per 1 x 128 group with the power-of-two
 *   scale at or above max(amax, 1e-10)/448 (mode 0) or with *static_scale (mode 1; e4m3 input is
 *   taken as already quantised); deq (decoded values), codes, scales [rows, cols/128] and sf32
 *   (the scale's E8M0 byte repeated per 32 elements, [rows, cols/32]) optional.
 * bolt_fp8_group_decode: codes [rows, cols] * scales [rows, cols/group] -> out.
 * bolt_mx4_swiglu_static: g1 fp32 [capacity, 2*inter] in sorted rows -> decoded e4m3 of
 *   swigluoai(g1 * a1_scale + bias[expert]) [* row_weight] / a2_scale, [capacity, inter].
 * bolt_mx4_affine_rows: out = cast((g2 * scale + bias[expert]) [* row_weight]) for the live
 *   rows; scatter != 0 writes row i to token * topk + slot.
 */
int bolt_mxfp4_decode(const uint8_t* packed, const uint8_t* scales, int64_t rows, int cols,
                      void* out, int out_dtype, void* stream);
int bolt_mx4_act_quant(const void* x, int x_dtype, int64_t rows, int cols, int gated,
                       int has_limit, float limit, int mode, const float* static_scale, void* deq,
                       int deq_dtype, uint8_t* codes, float* scales, uint8_t* sf32, void* stream);
int bolt_fp8_group_decode(const uint8_t* codes, const float* scales, int64_t rows, int cols,
                          int group, void* out, int out_dtype, void* stream);
int bolt_mx4_swiglu_static(const float* g1, const int32_t* sorted_expert_ids,
                           const int32_t* num_valid_ids, int capacity, int inter, int num_experts,
                           const float* a1_scale, const float* bias, float alpha, float limit,
                           const float* row_weight, const float* a2_scale, void* out,
                           int out_dtype, void* stream);
int bolt_mx4_affine_rows(const float* g2, const int32_t* sorted_expert_ids,
                         const int32_t* sorted_ids, const int32_t* num_valid_ids, int capacity,
                         int cols, int num_experts, int num_tokens, int topk, const float* scale,
                         const float* bias, const float* row_weight, int scatter, void* out,
                         int out_dtype, void* stream);

/* ---------------------------------------------------------------------------
 * Grouped expert GEMM (tcgen05 / TMEM / TMA, persistent).
 * Replaces moe_op.fused_moe + fused_moe_kernel
 * (boltops/fused_moe/triton/moe_op.py:2846-3417, 1294-1914) for the bf16/f16,
 * fp8/int8 block-scaled and fp8/int8 per-channel variants.
 *
 * A rows are in the expert-sorted padded layout produced by bolt_moe_sort_ck with
 * unit_size 128 (+ bolt_gather_rows for GEMM1): row tile t belongs to expert
 * sorted_expert_ids[t]; only tiles below num_valid_ids[0] are computed.
 */
typedef struct bolt_gemm_args {
  int kind;                 /* enum bolt_gemm_kind                               */
  int epilogue;             /* enum bolt_gemm_epilogue                           */
  int capacity;             /* rows of A (multiple of 128)                       */
  int n;                    /* rows of B per expert                              */
  int k;                    /* reduction length                                  */
  int num_experts;          /* experts in B                                      */
  const void* a;            /* [capacity, k] row-major                           */
  const void* b;            /* [num_experts, n, k] row-major                     */
  const float* a_scale;     /* block: [k/128, a_scale_ld]; channel: [capacity]   */
  int64_t a_scale_ld;
  const float* b_scale;     /* block: [E, n/128, k/128]; channel: [E, n]         */
  const void* bias;         /* optional [E, n] in c_dtype-compatible float type  */
  int bias_dtype;
  void* c;                  /* output                                            */
  int c_dtype;              /* BOLT_BF16/F16/F32, or FP8/INT8 for SILU_MUL_QUANT */
  int mid_dtype;            /* gated epilogues: dtype the GEMM result and the
                               activation are rounded through (the reference's
                               intermediate cache dtype); BOLT_F32 = no rounding */
  int64_t c_ld;             /* elements between output rows                      */
  float* c_scale;           /* SILU_MUL_QUANT: [n/2/128, c_scale_ld]             */
  int64_t c_scale_ld;
  int scatter;              /* 0: row i -> c[i]; 1: row i -> c[token*topk+slot]  */
  int num_tokens;           /* for pad detection: token >= num_tokens is a pad   */
  int topk;
  int mul_routed_weight;    /* multiply by sorted_weights[i] before the cast     */
  const int32_t* sorted_ids;
  const float* sorted_weights;
  const int32_t* sorted_expert_ids;
  const int32_t* num_valid_ids;
  int32_t* status;          /* optional device int32: set non-zero if a bounded
                               device-side wait expired                          */
  int sm_count;             /* 0 = all SMs of the current device                 */
  /* BOLT_GEMM_MXFP8 with BOLT_EPI_SILU_MUL_QUANT only: split gated activation
     min(g,L) * sigmoid(alpha g) * (clamp(u,+-L) + beta) on the mid_dtype-rounded
     GEMM result, then 1 x 32 MX quantisation: c = e4m3 codes [capacity, n/2],
     c_scale = BYTES [capacity, c_scale_ld] (c_scale_ld >= n/2/32).               */
  float act_alpha;
  float act_beta;
  float act_limit;
  int act_has_limit;
  /* schedule (enum bolt_gemm_schedule).  The tile-pair schedule takes its work from the expert
     segments instead of sorted_expert_ids: segments [max_segments][4] int32 = {expert, first
     row, live rows, 0}, num_segments [1], both written by bolt_moe_sort_ck.  The reference's
     nearest notion is its choice between kernel variants by token count
     (boltops/fused_moe/triton/fused_moe.py:801-821).                                          */
  int schedule;
  int max_segments;
  const int32_t* segments;
  const int32_t* num_segments;
  /* Gathered row operand (plain kinds, single-tile schedule).  With a_gather != 0, `a` is NOT in
     sorted order: it is the token-order matrix [a_rows >= num_tokens, k] (a_row_bytes between
     rows, a multiple of 16; 0 = dense), and sorted position p reads row sorted_ids[p] & 0xFFFFFF,
     or zeros where that id is not a token (id >= num_tokens: tile padding).  a_scale stays in
     sorted order.  The reference gathers the same way, by pointer arithmetic inside its kernel
     (boltops/fused_moe/triton/moe_op.py:1479,1611-1615).                                      */
  int a_gather;
  int a_rows;
  int64_t a_row_bytes;
  /* Scattered output with per-segment bases (scatter != 0, plain kinds): the row of token t goes
     to row scatter_src[t] * topk + slot of the region that begins scatter_seg_off[t /
     scatter_seg_rows] ELEMENTS behind c.  In the expert-parallel exchange over peer memory the
     tokens of segment s came from rank s, scatter_src is their index there and the region is
     rank s's [tokens, topk, n] return buffer: the down projection writes every route's row
     straight to the rank that owns the token.  16-bit rows of the block-scaled kinds leave as
     whole 256-byte segments.                                                                  */
  const int32_t* scatter_src;
  const int64_t* scatter_seg_off;
  int scatter_seg_rows;
} bolt_gemm_args;

int bolt_grouped_gemm(const bolt_gemm_args* args, void* stream);

/* ---------------------------------------------------------------------------
 * One whole layer in one call.  Replaces fused_experts_impl
 * (boltops/fused_moe/triton/fused_moe.py:1200-1777) for its common variant: gated SiLU,
 * combined [num_tokens, model_dim] output, unquantised bf16 / f16 hidden_states, experts in
 * bf16 / f16, fp8 / int8 with [128,128] blocks or fp8 / int8 per channel; optional biases,
 * expert mask (expert parallelism) and router weight applied on the input.  Same kernels and
 * the same arithmetic as driving bolt_moe_sort_ck, bolt_quant_scatter_rows / bolt_gather_rows,
 * bolt_grouped_gemm (twice) and bolt_moe_gather_sum one by one; the point is the host cost of
 * a decode-sized layer: one foreign call and one workspace instead of one of each per kernel.
 * The workspace (bolt_moe_layer_workspace_bytes(), 256-byte aligned) is scratch: nothing in it
 * has to be initialised and nothing survives the call.  out may alias hidden_states.
 */
typedef struct bolt_layer_args {
  int kind;                    /* enum bolt_gemm_kind, BF16 .. INT8_BLOCK                    */
  int x_dtype;                 /* BOLT_BF16 / BOLT_F16                                        */
  int out_dtype;               /* output and intermediate dtype (BF16 / F16 / F32)            */
  int num_tokens, topk;
  int hidden, inter, model_dim;        /* w1 [E, 2*inter, hidden], w2 [E, model_dim, inter]   */
  int num_experts;             /* experts in w1 / w2 (local experts under a mask)             */
  int global_num_experts;      /* range of topk_ids                                           */
  const void* hidden_states;   /* [num_tokens, hidden]                                        */
  const void* w1;
  const void* w2;
  const float* w1_scale;       /* block: [E, 2*inter/128, hidden/128]; channel: [E, 2*inter]  */
  const float* w2_scale;
  const void* b1;              /* optional [E, 2*inter]                                       */
  const void* b2;              /* optional [E, model_dim]                                     */
  int bias_dtype;
  int apply_router_weight_on_input;
  const float* topk_weights;   /* [num_tokens, topk] fp32                                     */
  const int32_t* topk_ids;     /* [num_tokens, topk]                                          */
  const int32_t* expert_mask;  /* optional [global_num_experts]: 1 = expert is local          */
  float routed_scaling_factor;
  void* out;                   /* [num_tokens, model_dim] in out_dtype                        */
  void* workspace;
  size_t workspace_bytes;
  int32_t* status;             /* optional, as in bolt_gemm_args                              */
} bolt_layer_args;

/* kernels one bolt_moe_layer call with these arguments launches (-1: invalid arguments) */
int bolt_moe_layer_kernel_count(const bolt_layer_args* args);
size_t bolt_moe_layer_workspace_bytes(const bolt_layer_args* args);
int bolt_moe_layer(const bolt_layer_args* args, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* BOLTOPS_B200_H_ */
