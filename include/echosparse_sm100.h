/* C ABI of libechosparse_sm100.so: the EchoSparse kernel set for B200 (sm_100a).
 *
 * Conventions (all entry points):
 *   - plain device pointers and sizes; the caller owns and allocates every buffer, outputs are written in place;
 *   - `stream` is a cudaStream_t (NULL = the default stream); nothing here synchronises or allocates, except
 *     es_device_status (synchronises) and the one-time function-attribute set-up of a kernel's first launch;
 *   - return 0 on success, a negative code on a rejected call or a failed launch; es_last_error() gives the text;
 *   - q / k / v / out are (L, H, 128) bf16, contiguous; query tiles have 128 rows (nq = ceil(L/128)), kv blocks have
 *     64 tokens (nb = ceil(L/64)); offsets and LSEs are log2 values, (nq*128, H) fp32, rows >= L hold 1e30.
 * Each declaration names the function of the reference (shaoshitong/self_trainable_or_free_attn) that it replaces.
 */
#ifndef ECHOSPARSE_SM100_H
#define ECHOSPARSE_SM100_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Text of the last error returned on this thread. */
const char* es_last_error(void);
/* Version of this ABI (1). */
int es_abi_version(void);
/* Kernels launched by this library in this process so far. */
long long es_launch_count(void);
/* Synchronises the current device, reads its status word into *status_out and clears it. 0 = fine; any other value is
 * (code of the bounded in-kernel wait that gave up) + 1000 * (its CTA index): that kernel returned early, its outputs are
 * invalid, and attention kernels launched before the word is read return at once. */
int es_device_status(int32_t* status_out);
/* Self test of that mechanism (no counterpart in the reference): launches one warp that waits on a barrier nobody arrives
 * on, with a limit of limit_us microseconds (1 .. 100000). The wait gives up the way a wait of the attention kernels does:
 * the kernel returns and the status word receives code 777. Nothing faults or hangs; read the word with es_device_status
 * afterwards, or the attention kernels of this device stay switched off. */
int es_selftest_wait_timeout(int32_t limit_us, void* stream);

/* Sequence <-> head exchange of a sequence-sharded caller, one kernel per rank: for every peer p < peers, `rows` rows of
 * `row_bytes` bytes are read from src + p * src_slab_stride + i * src_row_stride and stored at
 * dst_ptrs[p] + dst_offset + i * dst_row_stride, where dst_ptrs[p] is rank p's receive buffer as mapped on this GPU (a peer
 * mapping; this rank's own entry is an ordinary pointer). dst_ptrs is a HOST array of `peers` pointers (1 .. 16). All
 * pointers, strides, offsets and row_bytes are multiples of 16. The kernel waits on nobody: the caller orders it against the
 * peers' use of the buffers with a collective on the same stream before the data is read and before a buffer is written
 * again. Replaces the pair of layout copies and the torch.distributed.all_to_all_single of the reference's sequence-parallel
 * recipe around its processor (no single reference function; README, multi-GPU section). */
int es_exchange_rows(const void* src, int64_t src_slab_stride, int64_t src_row_stride, void* const* dst_ptrs,
                     int64_t dst_offset, int64_t dst_row_stride, int32_t peers, int64_t rows, int32_t row_bytes,
                     void* stream);

/* Exact attention over a list of 64-token blocks at a fixed softmax offset, with per-block masses.
 * Replaces echosparse/kernels/block_attention.py:327 `block_attention(q, k, v, out, counts, blocks, offset, lse, flags,
 * mass, threshold)`. counts (nq, H) int32; blocks (nq, H, nk) int32 ascending; flags (nq, H) int32 out;
 * mass (H, nq, nb) fp32 or NULL: entries of listed blocks are overwritten (not added to). */
int es_block_attention(const void* q, const void* k, const void* v, void* out, const int32_t* counts,
                       const int32_t* blocks, int32_t nk, const float* offset, float* lse, int32_t* flags, float* mass,
                       int32_t L, int32_t H, float threshold, void* stream);

/* The fused sparse step: listed blocks exactly, every block whose skip bit is clear through its mean key / value, the
 * refine list through four representatives each, one softmax at the fixed offset.
 * Replaces echosparse/kernels/sparse_attention.py:603 `sparse_attention(q, k, v, k_mean, v_mean, skip_bits, out, counts,
 * blocks, offset, lse, flags, refine, k_rep, v_rep, log_counts, mass, threshold)`.
 * k_mean, v_mean (nb, H, 128) bf16; skip_bits (H, nq, nw) int32 with nw >= 4*ceil(nb/128); refine (nq, H, rw) int32
 * padded with nb, rw a multiple of 32 (0 allowed); k_rep, v_rep (H, (nb+1)*4, 128) bf16; log_counts (H, (nb+1)*4) fp32. */
int es_sparse_attention(const void* q, const void* k, const void* v, const void* k_mean, const void* v_mean,
                        const int32_t* skip_bits, int32_t nw, void* out, const int32_t* counts, const int32_t* blocks,
                        int32_t nk, const float* offset, float* lse, int32_t* flags, const int32_t* refine, int32_t rw,
                        const void* k_rep, const void* v_rep, const float* log_counts, float* mass, int32_t L, int32_t H,
                        float threshold, void* stream);

/* Online-softmax attention over the block list for the tiles whose flag is set; writes out and lse of those tiles.
 * Replaces echosparse/kernels/triton_ops.py:237 `exact_fallback(q, k, v, out, counts, blocks, lse, flags)`.
 * tile_scratch: device scratch of ceil(L / 128) * H + 1 int32, or NULL. With it the flagged tiles are first listed (one
 * small kernel) and one CTA per SM walks the list; without it one CTA per tile is launched and tests its own flag, which
 * costs more than the work when a fraction of a percent of the tiles is flagged. The results are the same. */
int es_exact_fallback(const void* q, const void* k, const void* v, void* out, const int32_t* counts,
                      const int32_t* blocks, int32_t nk, float* lse, const int32_t* flags, int32_t L, int32_t H,
                      int32_t* tile_scratch, void* stream);

/* Block-mean compensation of the blocks not kept, for flagged tiles, in place on out and lse.
 * Replaces echosparse/kernels/triton_ops.py:285 `compensate_fallback(q, k_mean, v_mean, keep, lse, out, flags)`.
 * keep (H, nq, nb) uint8. tile_scratch: as for es_exact_fallback. */
int es_compensate_fallback(const void* q, const void* k_mean, const void* v_mean, const uint8_t* keep, float* lse,
                           void* out, const int32_t* flags, int32_t L, int32_t H, int32_t* tile_scratch, void* stream);

/* Mean key and value of every 64-token block. Replaces echosparse/kernels/triton_ops.py:37 `block_means`. */
int es_block_means(const void* k, const void* v, void* k_mean, void* v_mean, int32_t L, int32_t H, void* stream);

/* Top-k blocks of every (tile, head) by scaled mass plus the forced ones; sorted list, keep mask, refine list (top-r
 * skipped blocks by raw mass, padded with nb to width rw), skip bit mask.
 * Replaces echosparse/kernels/triton_ops.py:108 `select_blocks(mass, keep_prev, scale_exact, scale_skip, keep, counts,
 * blocks, flags, skip_bits, refine, k, r, L, sink)`. blocks is (nq, H, nb). */
int es_select_blocks(const float* mass, const uint8_t* keep_prev, const float* scale_exact, const float* scale_skip,
                     uint8_t* keep, int32_t* counts, int32_t* blocks, const int32_t* flags, int32_t* skip_bits,
                     int32_t nw, int32_t* refine, int32_t rw, int32_t k, int32_t r, int32_t L, int32_t H, int32_t sink,
                     void* stream);

/* Mass estimates of the skipped blocks and the per-tile scales.
 * Replaces echosparse/kernels/triton_ops.py:170 `estimate_skipped(q, k_mean, keep, offset, lse, mass, scale_exact,
 * scale_skip)`. */
int es_estimate_skipped(const void* q, const void* k_mean, const uint8_t* keep, const float* offset, const float* lse,
                        float* mass, float* scale_exact, float* scale_skip, int32_t L, int32_t H, void* stream);

/* Scales after a step that computed every block; resets the padding rows of lse to 1e30.
 * Replaces echosparse/kernels/triton_ops.py:196 `full_step_scales(offset, lse, scale_exact, scale_skip, L)`. */
int es_full_step_scales(const float* offset, float* lse, float* scale_exact, float* scale_skip, int32_t L, int32_t H,
                        void* stream);

/* keep (H, nq, nb) uint8 -> exact_bits (H, nq, nw) int32. Replaces echosparse/kernels/sm120.py:268 `pack_plan`. */
int es_pack_plan(const uint8_t* keep, int32_t* exact_bits, int32_t nw, int32_t H, int32_t nq, int32_t nb, void* stream);

/* The two bit masks of a plan -> keep mask, sorted block list, refine list (padded with nb), mean list, with counts.
 * Replaces echosparse/kernels/sm120.py:299 `rebuild_plan`. blocks and means are (nq, H, nb). means and mean_counts may
 * both be NULL: the fused kernel of this library reads the block-mean columns from skip_bits, not from a list. */
int es_rebuild_plan(const int32_t* exact_bits, const int32_t* skip_bits, int32_t nw, uint8_t* keep, int32_t* counts,
                    int32_t* blocks, int32_t* refine, int32_t rw, int32_t* refine_counts, int32_t* means,
                    int32_t* mean_counts, int32_t H, int32_t nq, int32_t nb, void* stream);

/* Number of Gram partial sums es_reps_metric needs for a sequence of L tokens. */
int es_reps_gram_splits(int32_t L);

/* Query metric and probes of every head. Replaces echosparse/kernels/representatives.py:156 `_metric_and_probes`.
 * gram_parts: scratch, es_reps_gram_splits(L) * H * 128 * 128 floats; gram (H, 128, 128) fp32 gets the regularised Gram
 * matrix when not NULL; metric (H, 128, 128) bf16; probes (H, 64, 128) bf16. */
int es_reps_metric(const void* q, float* gram_parts, float* gram, void* metric, void* probes, int32_t L, int32_t H,
                   void* stream);

/* The same as es_reps_metric for callers that cannot provide scratch memory (no counterpart in the reference).
 * Some hosts of this library may not allocate device memory at the point where they call it: a plugin running inside
 * another framework's memory pool, a caller inside a region where allocation is forbidden or would synchronise. This
 * entry point takes no scratch pointer and calls no allocator: the partial Gram sums go to a 16 MiB array that is part
 * of the library image on every GPU that loads it. Limits and rules:
 *   - H <= es_reps_metric_static_max_heads() (256); more heads are rejected with an error;
 *   - the first call on a device looks up the array's device address; make that call outside any stream capture;
 *   - all calls share the one array: calls that may overlap on the GPU (different streams) race and must be serialised
 *     by the caller. Nothing in the array has to start at zero: every call overwrites what it reads.
 * Results match es_reps_metric within rounding (the rows are split into fewer partial sums when H is large). */
int es_reps_metric_static(const void* q, float* gram, void* metric, void* probes, int32_t L, int32_t H, void* stream);
int es_reps_metric_static_max_heads(void);

/* Representatives of every kv block. Replaces the k-means launch of echosparse/kernels/representatives.py:147 `build`.
 * k_rep, v_rep (H, (nb+1)*4, 128) bf16 and log_counts (H, (nb+1)*4) fp32; block nb of the tables is not written.
 * k_mean, v_mean (nb, H, 128) bf16 are also written when both are given (NULL, NULL otherwise). */
int es_reps_kmeans(const void* k, const void* v, const void* metric, const void* probes, void* k_rep, void* v_rep,
                   float* log_counts, void* k_mean, void* v_mean, int32_t L, int32_t H, int32_t iters, void* stream);

#ifdef __cplusplus
}
#endif
#endif
