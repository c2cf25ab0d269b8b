/*
 * libdlblas_b200 -- C ABI of the B200 (sm_100a) kernels behind the dlBLAS hot-path ops.
 *
 * Conventions
 *   - plain pointers and sizes only; every pointer is a DEVICE pointer unless stated,
 *     owned by the caller; the library never allocates, frees or retains device memory;
 *   - strides are in ELEMENTS; the innermost dimension is contiguous;
 *   - `stream` is a cudaStream_t passed as void*; the call only enqueues work;
 *   - return value: 0 ok, < 0 argument/support error (text in dlb_last_error()),
 *     > 0 a cudaError_t from the launch;
 *   - `status` (optional, may be NULL) is a device int32[4] the tensor-core kernels
 *     write if one of their bounded waits gives up:
 *     {code (0 = none, 1 = wait timed out), wait site, block index, tile}.
 *
 * Paths below are relative to the reference project root (DeepLink-org/DLCompiler).
 */
#ifndef DLBLAS_B200_H
#define DLBLAS_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DLB_DTYPE_F16 0
#define DLB_DTYPE_BF16 1
#define DLB_DTYPE_F32 2

#define DLB_SCORE_SIGMOID 0
#define DLB_SCORE_SOFTMAX 1

#define DLB_GEMM_FUSE_SILU 1 /* B = [gate; up] halves, store silu(gate) * up */
#define DLB_GEMM_WEIGHT 2    /* scale each row by its routing weight (fp32) before the cast */
#define DLB_GEMM_SCATTER 4   /* write row p to row sorted_token_ids[p] of the output */

/* Library version (major * 100 + minor). */
int dlb_version(void);
/* Text of the last error raised on the calling thread. */
const char* dlb_last_error(void);
/* Wall-clock limit, in milliseconds (1..60000, default 2000), of every wait on a flag that ANOTHER GPU
 * raises (expert-parallel kernels).  A wait that runs out writes `status` and the kernel goes on; it
 * never hangs.  Process-wide; applies to launches made after the call. */
int dlb_set_wait_budget_ms(int64_t ms);

/* silu_and_mul: out[t, i] = silu(x[t, i]) * x[t, n + i], fp32 math, one rounding.
 * Replaces python/dlBLAS/dlblas/kernels/activation.py:88-130 (wrapper) and :17-85 (kernels). */
int dlb_silu_and_mul(const void* gate_up, void* out, int64_t rows, int64_t n, int64_t gate_up_row_stride,
                     int64_t out_row_stride, int dtype, void* stream);

/* Router.  scoring = sigmoid/softmax over `experts` fp32 logits per token; optional per-expert
 * selection bias; optional group-limited selection (n_group groups, score = sum of the group's two
 * largest biased scores, keep topk_group groups); top_k experts by biased score (ties: lower index,
 * output in descending order); weights = un-biased scores, optionally renormalised, times `scale`.
 * The reference computes its routers in torch (python/dlBLAS/tests/kernels/test_fused_moe.py:207-218,
 * softmax -> topk) or with the capacity-based topk_gating family
 * (python/dlBLAS/dlblas/kernels/topk_gating.py:259-290); the group-limited sigmoid form has no
 * counterpart in the reference. */
int dlb_grouped_topk_gating(const float* logits, const float* bias, int32_t* ids, float* weights, int64_t tokens,
                            int experts, int64_t logits_row_stride, int n_group, int topk_group, int top_k,
                            int scoring, int renormalize, float scale, void* stream);

/* GShard-style top-k gating with capacity (forward + backward of the auxiliary loss), the reference's
 * `topk_gating` op: python/dlBLAS/dlblas/kernels/topk_gating.py:259-290 (autograd function),
 * topk_gating_fwd_part1.py:24-81, topk_gating_fwd_part2.py:11-66, topk_gating_fwd_part3.py:11-62,135-169,
 * topk_gating_bwd.py:20-85; torch statement python/dlBLAS/benchmarks/topk_gating.py:132-206.
 *   dlb_gshard_gate     gates = softmax(logits) [tokens, experts] fp32 and the k largest experts per token
 *                       (ids [tokens, top_k], descending, ties to the lower index).
 *   dlb_gshard_assign   from the choice-major id list [top_k * tokens] and its stable sort by expert
 *                       (dlb_moe_align_block_size with block 1): queue position of every choice (loc),
 *                       me / ce / l_aux = mean(me * ce) * E^2, kept choices (position < capacity),
 *                       weights = kept gate / max(sum of the token's kept gates, fp32 eps),
 *                       ec_idx = expert * capacity + position (0 when dropped),
 *                       expert_select_token_idx [experts * capacity] int64 = tokens of each expert's queue
 *                       in arrival order, unfilled capacity padded with unrelated zero-weight tokens.
 *                       colsum_scratch: fp32 [colsum_blocks * experts].
 *   dlb_gshard_gate_bwd grad_logits = softmax backward of grad_l_aux * ce * E / tokens. */
int dlb_gshard_gate(const float* logits, int64_t tokens, int experts, int top_k, float* gates, int32_t* ids,
                    float* scratch_weights, void* stream);
int dlb_gshard_assign(const float* gates, const int32_t* ids_choice_major, const int32_t* sorted_slots,
                      const int32_t* expert_prefix, int64_t tokens, int experts, int top_k, int64_t capacity,
                      float* colsum_scratch, int64_t colsum_blocks, int32_t* loc, float* me, float* ce, float* l_aux,
                      int32_t* ec_idx, float* weights, int64_t* expert_select_token_idx, void* stream);
int dlb_gshard_gate_bwd(const float* gates, const float* ce, const float* grad_l_aux, float* grad_logits,
                        int64_t tokens, int experts, void* stream);
/* Backward of topk_gating's `higher_precision` mode (python/dlBLAS/dlblas/kernels/topk_gating.py:145-256,
 * 286-294): the gradient of the routing weights (grad_weights, fp32 [top_k * tokens], choice-major) flows
 * through weights = kept gate / max(sum of kept gates, fp32 eps) back to the gates, the auxiliary-loss
 * term is added, and the sum goes through the softmax backward.  ids_choice_major / loc as produced by
 * dlb_gshard_gate / dlb_gshard_assign. */
int dlb_gshard_gate_bwd_weights(const float* gates, const float* ce, const float* grad_l_aux,
                                const int32_t* ids_choice_major, const int32_t* loc, const float* grad_weights,
                                float* grad_logits, int64_t tokens, int experts, int top_k, int64_t capacity,
                                void* stream);

/* moe_align_block_size: stable counting sort of the numel (token, k) slots by expert id, each expert
 * segment padded to a multiple of `block` with the sentinel `numel`.  Block-padded form of the
 * reference's argsort + [start, end) ranges
 * (python/dlBLAS/dlblas/kernels/fused_moe.py:314-320, :267-293, kernel :238-264).
 *   sorted_token_ids  int32[sorted_capacity],  sorted_capacity  >= numel + experts * (block - 1)
 *   expert_ids        int32[expert_ids_capacity], >= ceil(sorted_capacity / block); unused = -1
 *   num_tokens_post_padded int32[1]
 *   block_start       int32[experts + 1], first block of each expert (prefix sum of blocks) */
int dlb_moe_align_block_size(const void* topk_ids, int ids_are_int64, int64_t numel, int num_experts, int block,
                             int32_t* sorted_token_ids, int64_t sorted_capacity, int32_t* expert_ids,
                             int64_t expert_ids_capacity, int32_t* num_tokens_post_padded, int32_t* block_start,
                             void* stream);

/* Per-expert [start, end) ranges inside the ascending sort of the flattened ids: start = number of ids
 * below the expert's (negative ids included), end = start + count, both 0 for an expert without slots.
 * Outputs int32 or int64 [num_experts].  Replaces get_start_end / _start_end_kernel,
 * python/dlBLAS/dlblas/kernels/fused_moe.py:267-293, :238-264. */
int dlb_moe_start_end(const void* topk_ids, int ids_are_int64, int64_t numel, int num_experts, void* exp_start,
                      void* exp_end, int out_is_int64, void* stream);

/* dst[p, :] = src[sorted_token_ids[p] / top_k, :] for p < num_tokens_post_padded (zeros for sentinel
 * rows).  The gather the reference does inside its GEMM by pointer arithmetic (reindex_a,
 * python/dlBLAS/dlblas/kernels/fused_moe.py:136-140), as a separate pass so the GEMM can use TMA. */
int dlb_moe_permute_rows(const void* src, void* dst, const int32_t* sorted_token_ids,
                         const int32_t* num_tokens_post_padded, int64_t numel, int top_k, int64_t hidden,
                         int64_t src_row_stride, int64_t sorted_capacity, int elem_size, void* stream);

/* Grouped GEMM over the block-padded row list: for every 128-row block b,
 * out[rows of b] = A[rows of b] @ B[expert of b]^T (fp32 accumulate), with the epilogue chosen by
 * `flags` (DLB_GEMM_*).  A is [a_rows, k] with a_rows a multiple of 128, B is
 * [num_experts * rows_per_expert, k].  Replaces fused_moe_kernel and its launcher,
 * python/dlBLAS/dlblas/kernels/fused_moe.py:77-175 and :178-235. */
int dlb_moe_grouped_gemm(const void* a, int64_t a_rows, int64_t a_row_stride, const void* b, int num_experts,
                         int64_t rows_per_expert, int64_t k, int64_t b_row_stride, void* out,
                         int64_t out_row_stride, int64_t n_out, const int32_t* sorted_token_ids,
                         const int32_t* block_start, const float* topk_weights, int64_t numel, int flags,
                         int dtype, int32_t* status, void* stream);

/* dlb_moe_grouped_gemm with the pieces expert parallelism needs (no counterpart in the reference, which
 * keeps tokens replicated: python/dlBLAS/dlblas/kernels/fused_moe.py:113-114, 329-332):
 *   - flags may add DLB_GEMM_PEER (8, with DLB_GEMM_WEIGHT): row p is stored straight into the result
 *     buffer of the rank that sent it, peer_out[row_meta[p] >> 24] + (row_meta[p] & 0xffffff) *
 *     out_row_stride, with plain stores into peer memory over NVLink (fuses the down projection of
 *     fused_moe.py:359-373 with the combine exchange);
 *   - wait_flags (device int32[sync_world], may be NULL): before its first load the kernel waits until
 *     wait_flags[r] >= sync_epoch for every rank r (A's rows are stored by other GPUs);
 *   - signal_flags (HOST array of sync_world device pointers, may be NULL) + done_counter (device int32,
 *     zero): after its last store the last CTA writes sync_epoch to *signal_flags[r] for every rank r.
 * Waits are bounded; a timeout is reported in `status` and the kernel proceeds. */
#define DLB_GEMM_PEER 8
int dlb_moe_grouped_gemm_sync(const void* a, int64_t a_rows, int64_t a_row_stride, const void* b, int num_experts,
                              int64_t rows_per_expert, int64_t k, int64_t b_row_stride, void* out,
                              void* const* peer_out, int num_peers, int64_t out_row_stride, int64_t n_out,
                              const int32_t* sorted_token_ids, const int32_t* block_start, const float* row_weights,
                              const int32_t* row_meta, int64_t numel, int flags, int dtype,
                              const int32_t* wait_flags, void* const* signal_flags, int32_t* done_counter,
                              int sync_world, int sync_epoch, int32_t* status, void* stream);

/* Expert-parallel exchange over peer memory (one process per GPU; `*_sym` arguments are HOST arrays of
 * `world` device pointers, one per rank, to buffers of identical size on every rank).  No counterpart
 * in the reference.  flags_sym: int32 [8][16] zero-initialised; slot s, source rank r at [s * 16 + r];
 * `epoch` must grow by one per step.
 *   dlb_ep_route    counts this rank's slots per GLOBAL expert, publishes the counts into every rank's
 *                   count matrix (counts_sym: int32 [world][experts]), synchronises the ranks (flag slot
 *                   0), derives the receive layout (block_start[experts/world + 1], num_post_padded[1],
 *                   row_map[cap]: p for rows that will hold a token, cap otherwise) and the row every
 *                   local slot will occupy in its owner's buffer (dest_pos[numel], stable inside an
 *                   expert, -1 for ids out of range).
 *   dlb_ep_send     stores every slot's hidden row, routing weight and (rank << 24 | slot) into the owner
 *                   rank's rows_sym [cap][hidden], w_sym [cap], meta_sym [cap]; the last CTA raises flag
 *                   slot 1 on every rank (done_counter: device int32, zero).
 *   dlb_ep_combine  dlb_moe_combine that first waits until wait_flags[r] >= epoch for every rank r; with
 *                   dest_pos (may be NULL) slots whose dest_pos is negative add nothing (they were sent
 *                   to no rank, so their row of `partial` is stale).
 *   dlb_ep_combine_pull  the same wait, then out[t] = sum over k of row dest_pos[t * top_k + k] of the
 *                   down-projection output y_sym [cap][hidden] of the rank that owns expert
 *                   topk_ids[t * top_k + k], read over NVLink with coalesced peer loads (slots whose
 *                   dest_pos is outside [0, cap) contribute nothing).  The expert side then runs
 *                   dlb_moe_grouped_gemm_sync with DLB_GEMM_WEIGHT alone, writing y locally.
 *   dlb_ep_barrier  stand-alone cross-GPU barrier on a flag slot (bounded wait; timeout -> status). */
int dlb_ep_route(const void* topk_ids, int ids_are_int64, int64_t numel, void* const* counts_sym,
                 void* const* flags_sym, int32_t* dest_pos, int32_t* block_start, int32_t* num_post_padded,
                 int32_t* row_map, int rank, int world, int experts, int64_t cap, int epoch, int32_t* status,
                 void* stream);
int dlb_ep_send(const void* hidden, int64_t hidden_row_stride, int64_t hidden_cols, int elem_size,
                const void* topk_ids, int ids_are_int64, const float* topk_weights, const int32_t* dest_pos,
                void* const* rows_sym, void* const* w_sym, void* const* meta_sym, void* const* flags_sym,
                int32_t* done_counter, int64_t numel, int top_k, int rank, int world, int experts, int64_t cap,
                int epoch, void* stream);
int dlb_ep_combine(const void* partial, void* out, int64_t tokens, int top_k, int64_t hidden,
                   int64_t out_row_stride, int dtype, const int32_t* wait_flags, int world, int epoch,
                   const int32_t* dest_pos, int32_t* status, void* stream);
int dlb_ep_combine_pull(void* const* y_sym, int64_t y_row_stride, const void* topk_ids, int ids_are_int64,
                        const int32_t* dest_pos, void* out, int64_t tokens, int top_k, int64_t hidden,
                        int64_t out_row_stride, int dtype, const int32_t* wait_flags, int world, int experts,
                        int64_t cap, int epoch, int32_t* status, void* stream);
int dlb_ep_barrier(void* const* flags_sym, int slot, int rank, int world, int epoch, int32_t* status, void* stream);

/* out[t, :] = sum over k of partial[t * top_k + k, :] (fp32 accumulate, one rounding): the
 * `intermediate_cache2.sum(dim=1)` of python/dlBLAS/dlblas/kernels/fused_moe.py:375.  With topk_ids
 * (may be NULL: every slot counts) a slot whose id is outside [id_lo, id_hi) adds nothing; its row of
 * `partial` was written by no kernel (the reference zero-fills the buffer instead, :329-332, 355-358). */
int dlb_moe_combine(const void* partial, void* out, int64_t tokens, int top_k, int64_t hidden,
                    int64_t out_row_stride, int dtype, const void* topk_ids, int ids_are_int64, int64_t id_lo,
                    int64_t id_hi, void* stream);

/* Varlen causal GQA flash-attention prefill.  q [total, hq, head_dim], k [total, hkv, head_dim],
 * v [total, hkv, head_dim_v], out [total, hq, head_dim_v] (head sizes: multiples of 8 up to 128),
 * lse (optional, may be NULL) fp32 [hq, total] = m * sm_scale + log(sum) in natural log.
 * q_cos / q_sin (optional, both or neither; [total, head_dim] in q's dtype, head_dim a multiple of 16): the
 * rotate-half rotary embedding is applied to every Q tile inside the kernel, in the 16-bit type, bit-identical
 * to dlb_apply_rotary; K must arrive rotated.  This is the query half of the reference's fused rotary +
 * attention kernel (python/dlBLAS/dlblas/kernels/fused_rotary_and_fa.py:132-133); the key half (:177-178,
 * every K tile rotated inside the loop) is done once per token by dlb_fill_kv_cache or dlb_apply_rotary.
 * Replaces context_attention_fwd, python/dlBLAS/dlblas/kernels/prefill_attention.py:155-181
 * (kernel :28-152); LSE convention of python/dlBLAS/dlblas/kernels/flash_attention.py:152-155. */
int dlb_flash_prefill_varlen(const void* q, const void* k, const void* v, void* out, float* lse,
                             const int32_t* b_start_loc, const int32_t* b_seq_len, int64_t batch,
                             int64_t total_tokens, int64_t max_seq_len, int64_t hq, int64_t hkv, int64_t head_dim,
                             int64_t head_dim_v, int64_t q_stride_t, int64_t q_stride_h, int64_t k_stride_t, int64_t k_stride_h,
                             int64_t v_stride_t, int64_t v_stride_h, int64_t o_stride_t, int64_t o_stride_h,
                             float sm_scale, int causal, const void* q_cos, const void* q_sin, int dtype,
                             int32_t* status, void* stream);

/* Prefill over a paged cache that already holds the earlier tokens of each sequence (chunked prefill,
 * prefix reuse): q [total_q, hq, d] packed by sequence (q_start_loc, q_seq_len), caches
 * [num_pages, page_size, hkv, d], block_table [batch, max_pages] (int32 or int64), kv_seq_len [batch] =
 * history + q_seq_len; query i of a sequence sees keys 0 .. history + i (with window > 0 only the last
 * window + 1 of them; with softcap > 0 scores become softcap * tanh(score * sm_scale / softcap)).  Same
 * kernel as dlb_flash_prefill_varlen with K/V tiles fetched page by page; head_dim / head_dim_v as there
 * (the reference test runs 48 / 32 and 32 / 32 over 16-token pages); q_cos / q_sin as there, indexed by
 * the rows of q.  Replaces the prefill branch of
 * paged_attention_fwd, python/dlBLAS/dlblas/kernels/paged_attention.py:617-671 (kernel :311-489). */
int dlb_flash_prefill_paged(const void* q, const void* k_cache, const void* v_cache, void* out, float* lse,
                            const void* block_table, const int32_t* q_start_loc, const int32_t* q_seq_len,
                            const int32_t* kv_seq_len, int64_t batch, int64_t total_q_tokens, int64_t max_q_len,
                            int64_t hq, int64_t hkv, int64_t head_dim, int64_t head_dim_v, int64_t page_size,
                            int64_t num_pages, int64_t max_pages, int64_t q_stride_t, int64_t q_stride_h,
                            int64_t k_stride_page, int64_t k_stride_slot, int64_t k_stride_head,
                            int64_t v_stride_page, int64_t v_stride_slot, int64_t v_stride_head, int64_t o_stride_t,
                            int64_t o_stride_h, int64_t bt_stride, int table_is_int64, int64_t window, float sm_scale,
                            float softcap, int causal, const void* q_cos, const void* q_sin, int dtype,
                            int32_t* status, void* stream);

/* Number of fp32 elements of the split-KV workspace dlb_paged_decode needs (0 when max_splits == 1);
 * head_dim = the larger of the q/k and the v head size. */
int64_t dlb_paged_decode_workspace_floats(int64_t batch, int64_t hq, int64_t head_dim, int64_t max_splits);

/* Paged flash-decode (one query token per sequence), split over the KV length in `chunk`-token
 * pieces with a log-sum-exp merge.  Caches are [num_pages, page_size, hkv, d]; block_table is
 * [batch, max_pages] (int32 or int64).  head_dim is the q / k head size, head_dim_v the v / out head
 * size: multiples of 8 up to 128, not necessarily equal (the reference handles any head size by a power
 * of two plus a remainder, and a v size of its own: paged_attention.py:526-539).  page_size is a power of
 * two; pages of 1, 2 or 4 tokens (page size 1 = the token-granular cache of decode_attention_fwd,
 * decode_attention.py:559-620) are gathered row by row when the caches are 16-byte aligned with page and slot
 * strides below 4 GiB, and fall back to one tensor-map box per page otherwise (slower, same result).
 * Replaces the decode branch of paged_attention_fwd, python/dlBLAS/dlblas/kernels/paged_attention.py:492-671 (kernels :40-285). */
int dlb_paged_decode(const void* q, const void* k_cache, const void* v_cache, void* out, const void* block_table,
                     const void* kv_seqlens, float* partial, int64_t batch, int64_t hq, int64_t hkv,
                     int64_t head_dim, int64_t head_dim_v, int64_t page_size, int64_t num_pages, int64_t max_pages,
                     int64_t q_stride_b, int64_t q_stride_h, int64_t o_stride_b, int64_t o_stride_h,
                     int64_t k_stride_page, int64_t k_stride_slot, int64_t k_stride_head, int64_t v_stride_page,
                     int64_t v_stride_slot, int64_t v_stride_head, int64_t bt_stride, int table_is_int64,
                     int lens_is_int64, int64_t chunk, int64_t max_splits, int64_t window, float sm_scale,
                     float softcap, int dtype, int32_t* status, void* stream);

/* rms_norm with optional residual add.  new_x = x + residual in the storage dtype (written to
 * out_residual when given); out = w * (new_x * rsqrt(mean(new_x^2) + eps)).  weight_after_cast = 0
 * multiplies in fp32 and rounds once (python/dlBLAS/dlblas/kernels/rms_norm.py:8-132);
 * weight_after_cast = 1 rounds the normalised value first and multiplies in the storage dtype
 * (python/dlBLAS/dlblas/kernels/add_rms_norm.py:11-80).  out_residual uses residual_row_stride. */
int dlb_rms_norm(const void* x, const void* weight, const void* residual, void* out, void* out_residual,
                 int64_t rows, int64_t n, int64_t x_row_stride, int64_t residual_row_stride, int64_t out_row_stride,
                 float eps, int weight_after_cast, int dtype, void* stream);

/* Rotary position embedding, rotate-half convention, arithmetic in the tensors' dtype; cos/sin are
 * [tokens, dim] in that dtype; outputs may alias the inputs.
 * Replaces python/dlBLAS/dlblas/kernels/apply_rotary_pos_emb.py:8-164. */
int dlb_apply_rotary(const void* q, const void* k, const void* cos, const void* sin, void* q_out, void* k_out,
                     int64_t tokens, int hq, int hk, int dim, int64_t q_stride_t, int64_t q_stride_h,
                     int64_t k_stride_t, int64_t k_stride_h, int64_t qo_stride_t, int64_t qo_stride_h,
                     int64_t ko_stride_t, int64_t ko_stride_h, int dtype, void* stream);

/* Scatter the new tokens' key/value states into the paged caches [pages, page_size, heads, d]:
 * token i of sequence b lands in slot (history + i) % page_size of page
 * block_offsets[b, (history + i) / page_size], history = kv_seq_length[b] - q_seq_length[b].
 * Bit-exact copy.  Replaces python/dlBLAS/dlblas/kernels/fill_kv_cache.py:24-185.
 * k_cos / k_sin (optional, both or neither; [total new tokens, dim_k] in the states' dtype, fp16/bf16, dim_k a
 * multiple of 16, `dtype` = DLB_DTYPE_*): K is rotated (rotate-half rotary embedding, bit-identical to
 * dlb_apply_rotary) while it is written, so the cache holds rotated keys and no pass over K precedes the
 * attention; this takes the place of the per-tile K rotation of
 * python/dlBLAS/dlblas/kernels/fused_rotary_and_fa.py:177-178.  `dtype` is ignored without them. */
int dlb_fill_kv_cache(const void* k_states, const void* v_states, void* k_caches, void* v_caches,
                      const void* q_start_loc, const void* q_seq_length, const void* kv_seq_length,
                      const void* block_offsets, int64_t batch, int64_t max_q_seq_length, int64_t page_size,
                      int64_t heads, int64_t dim_k, int64_t dim_v, int64_t num_pages, int64_t max_pages,
                      int64_t ks_stride_t, int64_t ks_stride_h, int64_t vs_stride_t, int64_t vs_stride_h,
                      int64_t kc_stride_page, int64_t kc_stride_slot, int64_t kc_stride_head, int64_t vc_stride_page,
                      int64_t vc_stride_slot, int64_t vc_stride_head, int64_t table_stride, int start_is_int64,
                      int qlen_is_int64, int kvlen_is_int64, int table_is_int64, int elem_size, const void* k_cos,
                      const void* k_sin, int dtype, void* stream);

/* Capacity, in fp32 elements (32 MiB), of the fixed device array used by dlb_paged_decode_static. */
#define DLB_DECODE_STATIC_FLOATS (8ll * 1024 * 1024)

/* dlb_paged_decode without a caller-provided workspace: no counterpart in the reference (its
 * wrapper allocates the split workspace with torch on every call, paged_attention.py:606).
 * For callers that cannot allocate device memory around a decode step (a serving engine whose
 * pool was handed out completely to the KV cache at start-up, or a latency-critical token loop
 * that must stay out of the allocator because an allocation can synchronise the device or fail).
 * The split-KV partials live in a device array that is part of the library image: every GPU that
 * loads the library holds its 32 MiB until the process exits.  The call allocates nothing.
 *   - needs dlb_paged_decode_workspace_floats(batch, hq, head_dim, max_splits) <=
 *     DLB_DECODE_STATIC_FLOATS, otherwise it returns an error (status -5) and launches nothing;
 *     `status` may be NULL (a caller that must not allocate may not have a status word yet);
 *   - the first call on a device looks up the array's device address; make that call before any
 *     stream capture on that device;
 *   - all calls on a device share the array (it keeps the last call's contents; no part of it
 *     needs clearing between calls), so calls whose kernels may overlap on the GPU must be
 *     serialised by the caller.
 * All other arguments are those of dlb_paged_decode, with one head size for q/k and v (head_dim). */
int dlb_paged_decode_static(const void* q, const void* k_cache, const void* v_cache, void* out,
                            const void* block_table, const void* kv_seqlens, int64_t batch, int64_t hq, int64_t hkv,
                            int64_t head_dim, int64_t page_size, int64_t num_pages, int64_t max_pages,
                            int64_t q_stride_b, int64_t q_stride_h, int64_t o_stride_b, int64_t o_stride_h,
                            int64_t k_stride_page, int64_t k_stride_slot, int64_t k_stride_head,
                            int64_t v_stride_page, int64_t v_stride_slot, int64_t v_stride_head, int64_t bt_stride,
                            int table_is_int64, int lens_is_int64, int64_t chunk, int64_t max_splits, int64_t window,
                            float sm_scale, float softcap, int dtype, int32_t* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* DLBLAS_B200_H */
