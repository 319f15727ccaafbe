/* C ABI of the VSA2 part of libechosparse_sm100.so (B200, sm_100a): the stages behind `echosparse.vsa`.
 *
 * Conventions (all entry points):
 *   - plain device pointers and sizes; the caller allocates every buffer (the reference's extension allocates its outputs
 *     with torch::empty; here the Python layer above this ABI does); `stream` is a cudaStream_t; nothing synchronises;
 *   - return 0 on success, a negative code on a rejected call or a failed launch; es_last_error() gives the text;
 *   - token tensors are [BH, L, D] contiguous, L = NB * 64, D = 64 or 128, dtype 0 = bf16, 1 = fp16;
 *     blk_cnt [NB] int32 = valid tokens per 64-token block (1..64, valid tokens first); padded slots output 0;
 *   - CSR block lists: ptr [BH * (NB + 1)] int32 absolute offsets into idx, ids ascending per row;
 *   - lse [BH, L] fp32 is the natural-log LSE over the selected keys, -inf for rows without a key and for padded rows.
 * Each declaration names the launcher / binding of the reference (shaoshitong/self_trainable_or_free_attn) it replaces.
 */
#ifndef ECHOSPARSE_VSA_SM100_H
#define ECHOSPARSE_VSA_SM100_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Group means of the R-token router groups (qr, kr, optionally vr: [BH, Lr_pad, D], row = block * (64 / R) + group) and
 * block means (qc, kc, vc: [BH, NBc_pad, D]) over the valid tokens, rounded once to the element type; padding rows zero.
 * Any output pointer may be NULL. Replaces `pool_fwd` (csrc/vsa/vsa2_api.cpp:904, launch_pool csrc/vsa/vsa2_kernels.h:193). */
int es_vsa_pool(const void* q, const void* k, const void* v, void* qr, void* kr, void* vr, void* qc, void* kc, void* vc,
                const int32_t* blk_cnt, int32_t BH, int32_t L, int32_t D, int32_t R, int32_t Lr_pad, int32_t NBc_pad,
                int32_t dtype, void* stream);

/* log2-domain LSE of every pooled query row over all valid pooled keys: lse2 [BH, Lr_pad].
 * Replaces `router_lse` (launch_router_lse, csrc/vsa/vsa2_kernels.h:208). */
int es_vsa_router_lse(const void* qr, const void* kr, float* lse2, const int32_t* blk_cnt, int32_t BH, int32_t NB, int32_t D,
                      int32_t R, int32_t Lr_pad, int32_t dtype, void* stream);

/* Block scores [bh_count, NB, NB] fp32 of the heads bh0 .. bh0 + bh_count - 1: the pooled softmax summed over the group
 * pairs of a block pair; row_norm 1 divides by (64 / R)^2, 0 by the query block's number of valid groups.
 * Replaces `router_scores` (launch_router_scores, csrc/vsa/vsa2_kernels.h:209). */
int es_vsa_router_scores(const void* qr, const void* kr, const float* lse2, float* scores, const int32_t* blk_cnt, int32_t BH,
                         int32_t NB, int32_t D, int32_t R, int32_t Lr_pad, int32_t bh0, int32_t bh_count, int32_t row_norm,
                         int32_t dtype, void* stream);

/* Bytes of scratch es_vsa_global_topk needs. Replaces topk_workspace_bytes (csrc/vsa/vsa2_kernels.h:222). */
long long es_vsa_topk_workspace_bytes(int32_t bh_count, int32_t NB);

/* Exact global selection: the `budget` largest scores of every (b, h) in the order (score descending, flat index
 * ascending), as q -> kv lists and their inverse. ptr arrays [BH * (NB + 1)] (rows of heads bh0 .. are written), idx arrays
 * [BH * budget]; head bh owns idx[bh * budget, (bh + 1) * budget). Replaces `global_topk_into` / `route`
 * (launch_global_topk, csrc/vsa/vsa2_kernels.h:238). */
int es_vsa_global_topk(const float* scores, int32_t NB, int32_t bh0, int32_t bh_count, long long budget, int32_t* q2k_ptr,
                       int32_t* q2k_idx, int32_t* k2q_ptr, int32_t* k2q_idx, void* workspace, void* stream);

/* Byte offset, inside the workspace of es_vsa_global_topk, of the selection bitmap it leaves behind: [bh_count, NB,
 * ceil(NB / 32)] uint32, bit j of row i set when (i, j) is selected (the `bits_a` / `bits_ab` of the tier router,
 * experiments/vsa2_representative/csrc/rep/rep_api.cpp:90-170 `route_tiers`, which runs the same top-k at two budgets). */
long long es_vsa_topk_bits_offset(int32_t bh_count, int32_t NB);

/* Original-VSA router, stage 1: whole-block scores [bh_count, NB, NB] in the element type, S = rnd(rnd(qc . kc) * (1 / sqrt(D))),
 * rnd = round to the element type (what Torch's bf16 / fp16 `(q_c @ k_c^T) / sqrt(D)` computes).
 * Replaces `block_scores` (launch_block_scores, csrc/vsa/vsa2_kernels.h:253). */
int es_vsa_block_scores(const void* qc, const void* kc, void* scores, int32_t BH, int32_t NB, int32_t D, int32_t NBc_pad,
                        int32_t bh0, int32_t bh_count, int32_t dtype, void* stream);

/* Original-VSA router, stage 2: exactly K = min(topk, NB) kv blocks per query row, larger score first, ties to the smaller kv
 * index, -0 == +0; q -> kv lists (row r of head bh owns idx[(bh * NB + r) * K ..)) and their inverse. The workspace is
 * es_vsa_topk_workspace_bytes(bh_count, NB) bytes. Replaces `row_topk_into` / `route_rows` (launch_row_topk,
 * csrc/vsa/vsa2_kernels.h:270). */
int es_vsa_row_topk(const void* scores, int32_t NB, int32_t bh0, int32_t bh_count, int32_t topk, int32_t* q2k_ptr,
                    int32_t* q2k_idx, int32_t* k2q_ptr, int32_t* k2q_idx, void* workspace, int32_t dtype, void* stream);

/* Attention of every 64-row query block over the valid tokens of its listed kv blocks (online softmax): o [BH, L, D],
 * lse [BH, L]. Also the coarse branch (block means as a sequence, 64-row tiles with their own counts, dense lists).
 * Replaces `attn_fwd` (launch_attn_fwd, csrc/vsa/vsa2_kernels.h:146). */
int es_vsa_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, const int32_t* q2k_ptr,
                    const int32_t* q2k_idx, const int32_t* blk_cnt, int32_t BH, int32_t L, int32_t D, int32_t dtype,
                    void* stream);

/* dK, dV of the same attention from the kv -> q lists, one owner per kv block (no atomics). Outputs in the element type
 * (dk, dv) or fp32 (dk_f32, dv_f32, used instead when not NULL); add_dk / add_dv [BH, add_nb, D] fp32 are optional per-block
 * gradients added as add / count to every valid token (the unpooling of the coarse branch). delta [BH, L] = rowsum(dO * O).
 * Replaces the dK / dV part of `attn_bwd` (launch_attn_bwd, csrc/vsa/vsa2_kernels.h:151). */
int es_vsa_attn_bwd_kv(const void* q, const void* k, const void* v, const void* dout, const float* lse, const float* delta,
                       void* dk, void* dv, float* dk_f32, float* dv_f32, const float* add_dk, const float* add_dv,
                       int32_t add_nb, const int32_t* k2q_ptr, const int32_t* k2q_idx, const int32_t* blk_cnt, int32_t BH,
                       int32_t L, int32_t D, int32_t dtype, void* stream);

/* dQ from the q -> kv lists, one owner per query block (no atomics); same output and add conventions.
 * Replaces `attn_bwd_q` (launch_attn_bwd_q, csrc/vsa/vsa2_kernels.h:177). */
int es_vsa_attn_bwd_q(const void* q, const void* k, const void* v, const void* dout, const float* lse, const float* delta,
                      void* dq, float* dq_f32, const float* add_dq, int32_t add_nb, const int32_t* q2k_ptr,
                      const int32_t* q2k_idx, const int32_t* blk_cnt, int32_t BH, int32_t L, int32_t D, int32_t dtype,
                      void* stream);

/* o = valid ? o_f + w * o_c[block] : 0 with w = act(gate); gate_mode 0 none (w = 1), 1 per token [BH, L], 2 per element
 * [BH, L, D]; gate_act 0 tanh, 1 identity. Replaces `fuse_fwd` (launch_fuse_fwd, csrc/vsa/vsa2_kernels.h:279). */
int es_vsa_fuse_fwd(const void* of, const void* oc, const void* gate, void* o, const int32_t* blk_cnt, int32_t BH, int32_t L,
                    int32_t D, int32_t NBc_pad, int32_t gate_mode, int32_t gate_act, int32_t dtype, void* stream);

/* Backward of the fusion: dout_f (dO on valid rows, 0 elsewhere; may be NULL), delta_f [BH, L] = rowsum(dO * o_f),
 * dout_c [BH, NBc_pad, D] = sum over the block's valid rows of w * dO (rows >= NB are left to the caller),
 * delta_c [BH, NBc_pad] = rowsum(dout_c * o_c), dgate like gate. Replaces `fuse_bwd` (csrc/vsa/vsa2_kernels.h:295). */
int es_vsa_fuse_bwd(const void* dout, const void* of, const void* oc, const void* gate, void* dout_f, float* delta_f,
                    void* dout_c, float* delta_c, void* dgate, const int32_t* blk_cnt, int32_t BH, int32_t L, int32_t D,
                    int32_t NBc_pad, int32_t gate_mode, int32_t gate_act, int32_t dtype, void* stream);

/* out = valid ? acc + add[block] / count : 0 in the element type (acc [BH, L, D] fp32 and add [BH, add_nb, D] fp32 may each
 * be NULL). Replaces `finalize` (launch_finalize, csrc/vsa/vsa2_kernels.h:306). */
int es_vsa_finalize(const float* acc, const float* add, void* out, const int32_t* blk_cnt, int32_t BH, int32_t L, int32_t D,
                    int32_t add_nb, int32_t dtype, void* stream);

/* ---- 64 / RM / 1 representative tiers (one softmax over: tokens of the tier-A blocks of the CSR list; the RM group means of
 * the blocks in bits_ab & ~bits_a, each + log2(tokens in the group); the block means of the blocks in ~bits_ab, + log2(count)).
 * Tables: k_mid, v_mid [BH, mid_stride, D] (row = block * RM + group) and k_tail, v_tail [BH, tail_stride, D] in the element
 * type, strides padded to multiples of 64 rows: the pooled means of es_vsa_pool with R = 64 / RM. bits [BH, NB, ceil(NB/32)].
 * phases: mask of 1 (A), 2 (B), 4 (C). mid_reps RM in {2, 4, 8, 16}. ---- */

/* Forward of the three-tier fine branch. Replaces `rep_attn_fwd` (experiments/vsa2_representative/csrc/rep/rep_api.cpp:200-290). */
int es_vsa_tier_attn_fwd(const void* q, const void* k, const void* v, const void* k_mid, const void* v_mid, const void* k_tail,
                         const void* v_tail, void* o, float* lse, const int32_t* q2k_ptr, const int32_t* q2k_idx,
                         const int32_t* bits_a, const int32_t* bits_ab, const int32_t* blk_cnt, int32_t BH, int32_t L, int32_t D,
                         int32_t mid_reps, int32_t mid_stride, int32_t tail_stride, int32_t phases, int32_t dtype, void* stream);

/* dQ over all three tiers, one owner per query block; add_dq as in es_vsa_attn_bwd_q.
 * Replaces the dQ part of `rep_attn_bwd_q` (rep_api.cpp:292-400). */
int es_vsa_tier_attn_bwd_q(const void* q, const void* k, const void* v, const void* k_mid, const void* v_mid,
                           const void* k_tail, const void* v_tail, const void* dout, const float* lse, const float* delta,
                           void* dq, const float* add_dq, int32_t add_nb, const int32_t* q2k_ptr, const int32_t* q2k_idx,
                           const int32_t* bits_a, const int32_t* bits_ab, const int32_t* blk_cnt, int32_t BH, int32_t L,
                           int32_t D, int32_t mid_reps, int32_t mid_stride, int32_t tail_stride, int32_t phases, int32_t dtype,
                           void* stream);

/* Gradients of the representative tables, fp32, shaped like the tables (zero-filled by the caller): one owner per table row, no
 * atomics. Replaces the table accumulation of `rep_attn_bwd_q` (dk_mid, dv_mid, dk_tail, dv_tail; rep_api.cpp:292-400).
 * Tier-A token gradients come from es_vsa_attn_bwd_kv on the tier-A kv -> q lists (`tier_a_bwd_kv`, rep_api.cpp:402-450). */
int es_vsa_tier_rep_bwd(const void* q, const void* k_mid, const void* v_mid, const void* k_tail, const void* v_tail,
                        const void* dout, const float* lse, const float* delta, float* dk_mid, float* dv_mid, float* dk_tail,
                        float* dv_tail, const int32_t* bits_a, const int32_t* bits_ab, const int32_t* blk_cnt, int32_t BH,
                        int32_t L, int32_t D, int32_t mid_reps, int32_t mid_stride, int32_t tail_stride, int32_t phases,
                        int32_t dtype, void* stream);

/* Token gradient from its three sources: out = valid ? tok + mid[group] / tokens in the group + (tail[block] + add[block]) /
 * tokens in the block : 0; every fp32 source may be NULL. Replaces `rep_unpool` (rep_api.cpp:452-505). */
int es_vsa_tier_unpool(const float* tok, const float* mid, const float* tail, const float* add, int32_t add_nb, void* out,
                       const int32_t* blk_cnt, int32_t BH, int32_t L, int32_t D, int32_t mid_reps, int32_t mid_stride,
                       int32_t tail_stride, int32_t dtype, void* stream);

/* ---- split-KV scheduling (balanced chunk tasks for long lists) ----
 * Plan of one CSR list ptr [BH * (NB + 1)] (q -> kv for the forward and the dQ pass, kv -> q for the dK / dV pass). A row of n
 * blocks is eligible when n >= max(min_len, ceil(tail_frac * W / resident), ceil(rel_mean * edges of its (b, h) / NB)) (W = all
 * edges; min_len >= chunk + 1; rel_mean = tail_frac = 0 switch those terms off); eligible rows have ceil(n / chunk) balanced
 * chunks; nothing splits when more than `budget` rows are eligible; rows split while the running chunk count of the eligible
 * rows stays <= max_slots. tasks [(BH * NB + max_slots), 4] = {row, first edge, end edge, slot} (split chunks first, slot =
 * task index, then one direct task with slot -1 per other row); merges [max(1, min(BH * NB, max_slots / 2)), 4] = {row, first
 * slot, chunks, 0}; info [8] = tasks, split rows, split slots, rows, eligible rows, eligible <= budget, threshold without the
 * per-head term, W. All counts stay on the device. Replaces `split_plan` (csrc/vsa/vsa2_api.cpp:464-520, csrc/vsa/split.cu:33-110). */
long long es_vsa_split_plan_workspace_bytes(int32_t BH, int32_t NB);
int es_vsa_split_plan(const int32_t* ptr, int32_t BH, int32_t NB, int32_t chunk, int32_t max_slots, int32_t min_len,
                      double rel_mean, double tail_frac, int32_t resident, int32_t budget, int32_t* tasks, int32_t* merges,
                      int32_t* info, void* workspace, void* stream);

/* es_vsa_attn_fwd over a task list (grid of n_tasks_cap CTAs; those past info[0] exit): direct tasks write o / lse, chunk
 * tasks write fp32 normalised partials part_o [slots, 64, D] and their log2-domain lse part_lse [slots, 64].
 * Replaces `attn_fwd_tasks` (csrc/vsa/vsa2_api.cpp:522-570). */
int es_vsa_attn_fwd_tasks(const void* q, const void* k, const void* v, void* o, float* lse, const int32_t* q2k_idx,
                          const int32_t* blk_cnt, const int32_t* tasks, const int32_t* task_info, int32_t n_tasks_cap,
                          float* part_o, float* part_lse, int32_t BH, int32_t L, int32_t D, int32_t dtype, void* stream);

/* Merge of the split rows of the forward: o = sum_i 2^(lse_i - M) o_i / sum_i 2^(lse_i - M), lse natural; with mask_rows the
 * padded query rows get 0 and -inf. Grid of n_merge_cap CTAs. Replaces `split_merge_fwd` (csrc/vsa/split.cu:133-175). */
int es_vsa_split_merge_fwd(const float* part_o, const float* part_lse, const int32_t* merges, const int32_t* info,
                           int32_t n_merge_cap, const int32_t* blk_cnt, void* o, float* lse, int32_t L, int32_t D,
                           int32_t mask_rows, int32_t dtype, void* stream);

/* es_vsa_attn_bwd_kv / es_vsa_attn_bwd_q over a task list: chunk tasks write fp32 partial gradients part [slots, 64, D]
 * without the per-block add. Replace `attn_bwd_tasks` and `attn_bwd_q_tasks` (csrc/vsa/vsa2_api.cpp:600-730). */
int es_vsa_attn_bwd_kv_tasks(const void* q, const void* k, const void* v, const void* dout, const float* lse,
                             const float* delta, void* dk, void* dv, float* dk_f32, float* dv_f32, const float* add_dk,
                             const float* add_dv, int32_t add_nb, const int32_t* k2q_idx, const int32_t* blk_cnt,
                             const int32_t* tasks, const int32_t* task_info, int32_t n_tasks_cap, float* part_dk,
                             float* part_dv, int32_t BH, int32_t L, int32_t D, int32_t dtype, void* stream);
int es_vsa_attn_bwd_q_tasks(const void* q, const void* k, const void* v, const void* dout, const float* lse,
                            const float* delta, void* dq, float* dq_f32, const float* add_dq, int32_t add_nb,
                            const int32_t* q2k_idx, const int32_t* blk_cnt, const int32_t* tasks, const int32_t* task_info,
                            int32_t n_tasks_cap, float* part_dq, int32_t BH, int32_t L, int32_t D, int32_t dtype,
                            void* stream);

/* Merge of split rows of a backward pass, in chunk order: out = valid ? sum_i part_i + add[block] / count : 0, in the element
 * type (out) or fp32 (out_f32). Replaces `split_merge_sum` (csrc/vsa/split.cu:177-228). */
int es_vsa_split_merge_sum(const float* part, const int32_t* merges, const int32_t* info, int32_t n_merge_cap,
                           const float* add, int32_t add_nb, const int32_t* blk_cnt, void* out, float* out_f32, int32_t L,
                           int32_t D, int32_t dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif
