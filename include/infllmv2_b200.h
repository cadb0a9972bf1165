/*
 * infllmv2_b200 -- C ABI of the B200 (sm_100a) kernels for InfLLM-V2 two-stage sparse attention.
 *
 * Conventions (all entry points):
 *   - plain pointers and sizes only; every pointer is DEVICE memory of the current CUDA device
 *     unless stated otherwise; the caller allocates every output and every workspace;
 *   - `stream` is a cudaStream_t passed as void*; work is enqueued, never synchronised;
 *   - return value: 0 on success, a negative IFV2_ERR_* for a rejected argument (nothing was
 *     launched), or a positive cudaError_t reported by the launch;
 *   - ifv2_last_error() returns a thread-local, human-readable message for the last non-zero
 *     return on the calling thread.
 *
 * Each declaration names the interface of the reference (OpenBMB/infllmv2_cuda_impl) that it
 * replaces, by file:line inside that project.
 */
#ifndef INFLLMV2_B200_H_
#define INFLLMV2_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define IFV2_OK                 0
#define IFV2_ERR_INVALID_ARG   -1   /* null pointer, negative size, bad flag             */
#define IFV2_ERR_UNSUPPORTED   -2   /* feature the reference compiles out / d != 128 ... */
#define IFV2_ERR_TOO_LARGE     -3   /* size beyond a documented limit                    */
#define IFV2_ERR_DRIVER        -4   /* a driver entry point (tensor-map encode) failed   */
#define IFV2_ERR_DEVICE_STATUS -5   /* a kernel reported a bounded wait that ran out     */

const char* ifv2_last_error(void);
/* Library version, for loaders that want to check what they bound. */
int ifv2_version(void);

/* The status block of the tensor-core kernels (stage 1, stage-2 forward and backward): int32[4]
 * device words owned by the caller, zero-initialised once.  Every wait inside those kernels is
 * bounded (about 0.3 s); a wait that runs out stores its site code in
 *   word 0: the flag of the RUNNING launch.  Each entry point clears it on the stream before it
 *           launches; thread blocks that start after a failure see it and return at once, so a
 *           failed launch ends quickly and leaves its outputs undefined;
 *   word 1: sticky.  It keeps the first failing site of any launch until ifv2_check_status.
 * A failed launch therefore never disables later launches, and it cannot go unnoticed by a caller
 * that checks: ifv2_check_status is the ONE entry point that synchronises -- it waits for
 * `stream`, reads the block, clears it, and returns IFV2_ERR_DEVICE_STATUS (site code in
 * ifv2_last_error) if any launch since the last check abandoned a wait, else 0.  Call it where
 * the host synchronises anyway (end of a step, before results are consumed).  No counterpart in
 * the reference, whose kernels have no waits that can run out. */
int ifv2_check_status(int32_t* status, void* stream);

/* ---------------------------------------------------------------- bitmask kernels ---------- */

/* Rows of block indices -> rows of 64-bit words (bit idx%64 of word idx/64; indices outside
 * [0, 64*words) are skipped).  Writes every output word.
 * Replaces C.topk_to_uint64: csrc/entry.cu:79-97, kernel csrc/topk_to_uint64.cuh:10-76. */
int ifv2_topk_to_uint64(const int32_t* topk_idx, int64_t* out_words, int64_t rows, int k,
                        int k_blocks, int words, void* stream);

/* Bool rows (1 byte per element) -> 64-bit words, element 64w+b = bit b of word w, tail bits 0.
 * Replaces C.blockmask_to_uint64: csrc/entry.cu:61-77, kernel csrc/blockmask_to_uint64.cuh:10-74. */
int ifv2_blockmask_to_uint64(const uint8_t* mask, int64_t* out_words, int64_t rows,
                             int64_t last_dim, int64_t words, void* stream);

/* Inverse of the above, restricted to the first last_dim bits of each row.
 * Replaces C.uint64_to_bool: csrc/entry.cu:99-115, kernel csrc/uint64_to_bool.cuh:10-66. */
int ifv2_uint64_to_bool(const int64_t* in_words, uint8_t* out_mask, int64_t rows,
                        int64_t last_dim, int64_t words, void* stream);

/* Row mask (heads, tokens, ceil(k_blocks/64)) -> column mask (heads, k_blocks, ceil(tokens/64)):
 * out[h, blk, t/64] bit t%64 = in[h, t, blk/64] bit blk%64.  One kernel in place of the
 * reference's unpack -> transpose(1,2).contiguous() -> synchronize -> pack sequence,
 * infllm_v2/infllmv2_sparse_attention.py:343-350. */
int ifv2_transpose_blockmask(const int64_t* fwd_words, int64_t* bwd_words, int heads,
                             int64_t tokens, int k_blocks, void* stream);

/* ---------------------------------------------------------------- selection kernels -------- */

/* Key compression in front of the stage-1 scorer: compressed key j of a sequence = mean of the keys
 * of tokens [stride*j, stride*j + kernel) (full windows only), per KV head and feature, fp32
 * accumulation, bf16 result.  k: (total_k, heads_k, 128) bf16; kc: (total_c, heads_k, 128) bf16.
 * cu_seqlens_k / cu_seqlens_c: (batch+1) int32 device tables of keys / compressed keys per
 * sequence (cu_c[b+1]-cu_c[b] = (len_b - kernel)/stride + 1, or 0 when len_b < kernel); both null =
 * one sequence.  The reference keeps this step in its caller and tests
 * (tests/test_stage1_compressed_lse.py:11-99, compress_tensor / calc_chunks_with_stride). */
int ifv2_compress_keys(const void* k, void* kc, const int32_t* cu_seqlens_k,
                       const int32_t* cu_seqlens_c, int batch, int64_t total_k, int64_t total_c,
                       int heads_k, int head_dim, int kernel_size, int kernel_stride, void* stream);

/* Decode-time update of a compressed-key cache after one token was appended to every sequence:
 * a sequence whose new length L satisfies L >= kernel and (L - kernel) % stride == 0 has completed
 * window j = (L - kernel)/stride, and kc_cache[b, j] is written; other sequences are untouched.
 * k_cache: (batch, cache_capacity, heads_k, 128); kc_cache: (batch, compressed_capacity, heads_k, 128);
 * cache_seqlens: (batch) int32 lengths after the append.  No counterpart in the reference (its
 * caller recompresses). */
int ifv2_compress_keys_append(const void* k_cache, void* kc_cache, const int32_t* cache_seqlens,
                              int batch, int64_t cache_capacity, int64_t compressed_capacity,
                              int heads_k, int head_dim, int kernel_size, int kernel_stride,
                              void* stream);

/* Prefill -> cache: copies the packed rows of every sequence (src: (total, heads_k, 128) bf16,
 * cu_seqlens: (batch+1)) to rows [0, len_b) of its cache slot (cache: (batch, capacity, heads_k,
 * 128)); rows past the capacity are dropped.  seqlens_out (may be null): min(len_b, capacity).
 * Used for keys, values and both compressed-key tensors.  The reference leaves this to its caller
 * (the k_cache / v_cache tensors of infllm_v2/infllmv2_sparse_attention.py:609-630 arrive filled). */
int ifv2_cache_fill(const void* src, void* cache, const int32_t* cu_seqlens, int32_t* seqlens_out,
                    int batch, int64_t total, int64_t capacity, int heads_k, int head_dim,
                    void* stream);

/* One decode step of cache bookkeeping in one launch: k_new / v_new (batch, heads_k, 128) go to
 * position cache_seqlens[b] of k_cache / v_cache (batch, capacity, heads_k, 128); a sequence whose
 * new length L completes a compression window (L >= kernel, (L - kernel) % stride == 0) gets the
 * mean of its last `kernel` keys written to kc_cache[b, (L - kernel)/stride] (and likewise to
 * kc2_cache with kernel2 / stride2: the coarse keys of the compressed-LSE mode); either compressed
 * cache may be null.  cache_seqlens is updated IN PLACE to L; positions[b] (may be null, must not
 * alias) receives the old length, i.e. the position of the new token -- the cache_lens of the
 * pool and top-k kernels; n_comp[b] / n_comp2[b] (may be null) = compressed keys now valid, the
 * seqused_k of the stage-1 scorer.  All pointers keep their values from step to step, so a decode
 * step can be replayed from a CUDA graph.  A sequence whose cache is full is left untouched.
 * Stands in for the in-kernel append of mha_fwd_kvcache (csrc/flash_attn/flash_api.cpp:1549-1843,
 * knew / vnew) plus the caller-side recompression the reference has no kernel for. */
int ifv2_decode_append(const void* k_new, const void* v_new, void* k_cache, void* v_cache,
                       void* kc_cache, void* kc2_cache, int32_t* cache_seqlens, int32_t* positions,
                       int32_t* n_comp, int32_t* n_comp2, int batch, int64_t capacity,
                       int64_t c_capacity, int64_t c2_capacity, int heads_k, int head_dim,
                       int kernel_size, int kernel_stride, int kernel2_size, int kernel2_stride,
                       void* stream);

/* 1-D max-pool of stage-1 scores to block scores with +inf on the init and causal-local blocks.
 * in: (heads, q_len, k_len) with `in_row_stride` elements between rows (>= k_len);
 * out: (heads, q_len, out_len) contiguous.  dtype: is_bf16 ? bf16 : fp16.
 * Replaces C.max_pooling_1d: csrc/entry.cu:117-152, kernel csrc/max_pooling_1d.cuh:106-160. */
int ifv2_max_pooling_1d(const void* in, void* out, int is_bf16, int heads, int q_len, int k_len,
                        int64_t in_row_stride, int out_len, int cache_len, int kernel_size,
                        int stride, int padding, int block_size, int local_blocks,
                        int init_blocks, void* stream);

/* Packed-sequence variant: rows are global query tokens, the key length and cache length are
 * per sequence.  total_q is taken from the caller (no device->host read).
 * Replaces C.max_pooling_1d_varlen: csrc/entry.cu:154-195, kernel csrc/max_pooling_1d.cuh:11-103. */
int ifv2_max_pooling_1d_varlen(const void* in, void* out, const int32_t* cu_seqlens_q,
                               const int32_t* cu_seqlens_k, const int32_t* cache_lens,
                               int is_bf16, int batch, int heads, int64_t total_q,
                               int max_seqlen_k, int64_t in_row_stride, int out_len,
                               int kernel_size, int stride, int padding, int block_size,
                               int local_blocks, int init_blocks, void* stream);

/* Per-row top-k of block scores: the k entries first in (value descending, index ascending)
 * order, written ascending as int32 with -1 in the unused tail; indices greater than the
 * row's own query block ((local token + cache_len) / block_size) become -1.
 * score: (heads, total_q, n_blocks), `row_stride` elements between rows.
 * cu_seqlens_q / cache_lens may be null (single sequence, scalar cache_len).
 * The reference has no public op for this step (README.md:40-42); the ordering is that of its
 * bitonic top-k, csrc/topk.cuh:6-42.  n_blocks <= 8192. */
int ifv2_topk_select(const void* score, int32_t* out_idx, int is_bf16, int heads, int64_t total_q,
                     int n_blocks, int64_t row_stride, int k, const int32_t* cu_seqlens_q,
                     const int32_t* cache_lens, int batch, int cache_len, int block_size,
                     void* stream);

/* ifv2_topk_select with the block mask packed in the same pass: row_mask (heads, total_q,
 * ceil(k_blocks/64)) receives exactly the words ifv2_topk_to_uint64 would build from the selected
 * list (bit b of a row = block b selected and not after the row's own block; every word is
 * written), so the int32 list never has to travel through memory; out_idx may be null.
 * col_mask (may be null): the column mask (heads, k_blocks, ceil(total_q/64)) of the backward, as
 * ifv2_transpose_blockmask gives it, produced by that kernel in a second launch of this call.
 * Stands for the caller-side top-k (README.md:40-42) followed by C.topk_to_uint64
 * (csrc/topk_to_uint64.cuh:10-52) and the unpack / transpose / pack sequence of
 * infllm_v2/infllmv2_sparse_attention.py:343-350.  n_blocks, k_blocks <= 8192. */
int ifv2_topk_select_mask(const void* score, int32_t* out_idx, int64_t* row_mask, int64_t* col_mask,
                          int is_bf16, int heads, int64_t total_q, int n_blocks, int64_t row_stride,
                          int k, int k_blocks, const int32_t* cu_seqlens_q,
                          const int32_t* cache_lens, int batch, int cache_len, int block_size,
                          void* stream);

/* Block selection of a decode step in one launch: for every (sequence, KV head) row of stage-1
 * scores (score: (heads, batch, row_stride), one query token per sequence) the 64-token max-pool
 * (window block_size/stride + 1, stride block_size/stride, padding 1, +inf on the init and
 * causal-local blocks), the top-k of the n_blocks block scores and the packed block mask
 * mask[b, h, :] (batch, heads, mask_words) that ifv2_decode / ifv2_decode_paged read.
 * seqused_c: (batch) number of compressed keys of each sequence (null = max_seqlen_c);
 * positions: (batch) position of the query token in its sequence (its block is position /
 * block_size); topk_idx (may be null): (batch, heads, k) int32, ascending, -1 tail.  Results are
 * identical to ifv2_max_pooling_1d_varlen -> ifv2_topk_select -> ifv2_topk_to_uint64 on the same
 * row (csrc/max_pooling_1d.cuh:11-103, the tie rule of csrc/topk.cuh:6-42,
 * csrc/topk_to_uint64.cuh:10-76); the reference runs these (and a torch.topk) as separate
 * launches.  dense_len (0 = off): a sequence whose query sits at a position below dense_len gets
 * every block up to its own instead of a selection (short sequences attend densely; decided per
 * sequence on the device, so a captured step and an eager one agree); its topk_idx row then names
 * the first k of those blocks. */
int ifv2_decode_select(const void* score, int is_bf16, int64_t row_stride, const int32_t* seqused_c,
                       const int32_t* positions, int64_t* mask, int32_t* topk_idx, int batch,
                       int heads, int max_seqlen_c, int n_blocks, int mask_words, int k,
                       int local_blocks, int init_blocks, int block_size, int stride, int dense_len,
                       void* stream);

/* ---------------------------------------------------------------- stage 1 ------------------ */

/* Stage-1 scorer: out[h, t, j] = sum over the 16 query heads of KV head h of
 * softmax_j(scale * q[t, 16h+g] . kc[j, h]) over the compressed keys visible to token t.
 * q: (total_q, heads_q, 128) bf16, kc: (total_c, heads_k, 128) bf16, both dense row-major.
 * out: (heads_k, total_q, out_row_stride) bf16; columns [0, max_seqlen_k) of every row are
 * written (0 where invisible).  lse_keys / cu_seqlens_v / total_v: the keys the row maxima and
 * sums are taken over (the reference's `v` argument): null / null / 0 = the same keys as kc; a
 * sequence whose count differs from its kc count is treated as the coarse compression (kernel
 * 128, stride 64) whose log-sum-exp normalises the scores, as flash_fwd_kernel.h:1236-1240 does.
 * seqused_k: optional (batch) int32, the number of keys of each sequence actually in use (the
 * reference's seqused_k, flash_api.cpp:792, 906-911; block_info.h:24); cu_seqlens_k then only
 * gives where a sequence's keys start, e.g. b * capacity for a per-sequence cache of compressed
 * keys.  seqused_v: the same for lse_keys / cu_seqlens_v.
 * status: the int32[4] status block described at ifv2_check_status.
 * Replaces C.varlen_fwd_stage1: csrc/entry.cu:209-214 -> mha_varlen_fwd_stage1,
 * csrc/flash_attn/flash_api.cpp:784-1049 (+ the GQA transpose, slice and NaN scrub of
 * infllm_v2/infllmv2_sparse_attention.py:554-589). */
int ifv2_stage1_scores(const void* q, const void* kc, const void* lse_keys, void* out,
                       const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                       const int32_t* cu_seqlens_v, int64_t total_v, const int32_t* seqused_k,
                       const int32_t* seqused_v, int batch, int64_t total_q, int64_t total_c, int heads_q, int heads_k,
                       int head_dim, int max_seqlen_q, int max_seqlen_k, int64_t out_row_stride,
                       float softmax_scale, int causal, int32_t* status, void* stream);

/* Stage-1 scorer for decode: exactly ONE query token per sequence (q: (batch, heads_q, 128)), same
 * output layout and values as ifv2_stage1_scores called with cu_seqlens_q = 0, 1, 2, ...; the
 * keys of a sequence are split over CTAs so that the launch is bandwidth-bound instead of being
 * serialised per sequence.  workspace: ifv2_stage1_decode_workspace_bytes(...) bytes, 16-byte
 * aligned; it holds the per-chunk softmax statistics and the unnormalised bf16 exponentials
 * (32 bytes per key and KV head) between the two kernels, so the keys are read once.
 * Same reference path as ifv2_stage1_scores (mha_varlen_fwd_stage1 with seqlen_q = 1 per
 * sequence, as the decode caller of infllm_v2/infllmv2_sparse_attention.py:483-606 uses it). */
int64_t ifv2_stage1_decode_workspace_bytes(int batch, int heads_k, int max_seqlen_k);
int ifv2_stage1_decode_scores(const void* q, const void* kc, void* out, const int32_t* cu_seqlens_k,
                              const int32_t* seqused_k /* may be null */, int batch,
                              int64_t total_c, int heads_q, int heads_k, int head_dim,
                              int max_seqlen_k, int64_t out_row_stride, float softmax_scale,
                              int causal, void* workspace, int64_t workspace_bytes, void* stream);

/* Decode selection straight from the compressed keys, two launches: the first kernel of
 * ifv2_stage1_decode_scores, then one kernel that forms each (sequence, KV head) score row in
 * shared memory and runs ifv2_decode_select's pool / top-k / mask pack on it -- the score row
 * never reaches HBM.  Arguments as in those two entries (positions, mask, topk_idx, n_blocks,
 * mask_words, k, local_blocks, init_blocks, block_size, stride as in ifv2_decode_select; the rest
 * as in ifv2_stage1_decode_scores, same workspace size; dense_len as in ifv2_decode_select);
 * max_seqlen_k <= 32768.  Results are identical to ifv2_stage1_decode_scores followed by
 * ifv2_decode_select. */
int ifv2_stage1_decode_select(const void* q, const void* kc, const int32_t* cu_seqlens_k,
                              const int32_t* seqused_k, const int32_t* positions, int64_t* mask,
                              int32_t* topk_idx, int batch, int64_t total_c, int heads_q,
                              int heads_k, int head_dim, int max_seqlen_k, int n_blocks,
                              int mask_words, int k, int local_blocks, int init_blocks,
                              int block_size, int stride, int dense_len, float softmax_scale,
                              int causal, void* workspace, int64_t workspace_bytes, void* stream);

/* Stage-1 scorer with the 64-token max-pool fused in: writes block scores
 * (heads_k, total_q, n_blocks) bf16 that are bit-identical to ifv2_max_pooling_1d[_varlen]
 * (kernel 5, stride 4, padding 1, block 64) applied to the output of ifv2_stage1_scores, without
 * the score tensor ever reaching HBM.  scores_or_null: optional (heads_k, total_q,
 * scores_row_stride) score output as in ifv2_stage1_scores.  cache_lens: per-sequence cache
 * length (may be null -> scalar cache_len); n_blocks = ceil((max_seqlen_q + max cache) / 64).
 * Fuses mha_varlen_fwd_stage1 (csrc/flash_attn/flash_api.cpp:784-1049) with
 * max_pooling_1d_varlen_kernel (csrc/max_pooling_1d.cuh:11-103); the reference runs them as two
 * launches with a (heads_k, total_q, max_seqlen_k) tensor in between. */
int ifv2_stage1_block_scores(const void* q, const void* kc, const void* lse_keys,
                             void* scores_or_null, void* block_scores,
                             const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                             const int32_t* cu_seqlens_v, int64_t total_v,
                             const int32_t* seqused_k /* may be null */,
                             const int32_t* seqused_v /* may be null */,
                             const int32_t* cache_lens, int batch, int64_t total_q,
                             int64_t total_c, int heads_q, int heads_k, int head_dim,
                             int max_seqlen_q, int max_seqlen_k, int64_t scores_row_stride,
                             int n_blocks, int cache_len, int local_blocks, int init_blocks,
                             float softmax_scale, int causal, int32_t* status, void* stream);

/* Stage-1 scorer over a PAGED or left-padded cache of compressed keys, the addressing options of
 * mha_varlen_fwd_stage1 (csrc/flash_attn/flash_api.cpp:906-911, 1001-1008; src/block_info.h:22-24):
 * kc is (num_pages * page_size, heads_k, 128) rows with block_table (batch, block_table_stride)
 * naming the page of every page_size compressed keys of a sequence (page_size a multiple of 128;
 * the reference wants 256), or a packed tensor whose sequences start leftpad_k[b] rows into their
 * cu_seqlens_k extent.  Writes the scores (scores_or_null, layout of ifv2_stage1_scores) and / or
 * the block scores (block_scores_or_null, as ifv2_stage1_block_scores); the row sums run over the
 * scored keys.  Other arguments as in those two entries. */
int ifv2_stage1_paged(const void* q, const void* kc, void* scores_or_null, void* block_scores_or_null,
                      const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                      const int32_t* seqused_k, const int32_t* leftpad_k, const int32_t* block_table,
                      int block_table_stride, int page_size, const int32_t* cache_lens, int batch,
                      int64_t total_q, int64_t total_c, int heads_q, int heads_k, int head_dim,
                      int max_seqlen_q, int max_seqlen_k, int64_t scores_row_stride, int n_blocks,
                      int cache_len, int local_blocks, int init_blocks, float softmax_scale,
                      int causal, int32_t* status, void* stream);

/* ---------------------------------------------------------------- stage 2 ------------------ */

/* Block-sparse varlen attention forward.  q/out: (total_q, heads_q, 128) bf16; k, v:
 * (total_k, heads_k, 128) bf16; fwd_mask: (heads_k, total_q, mask_words) 64-bit words from
 * ifv2_topk_to_uint64, or null for dense attention; lse: (heads_k, total_q*16) fp32 with row
 * token*16 + head-in-group.  Rows that see no key get out = 0 and lse = +inf.
 * Replaces C.varlen_fwd: csrc/entry.cu:209-214 -> mha_varlen_fwd,
 * csrc/flash_attn/flash_api.cpp:519-782 (+ the GQA transposes of
 * infllm_v2/infllmv2_sparse_attention.py:81-90, 123-130). */
int ifv2_sparse_attn_fwd(const void* q, const void* k, const void* v, void* out, float* lse,
                         const int64_t* fwd_mask, int mask_words, const int32_t* cu_seqlens_q,
                         const int32_t* cu_seqlens_k, int batch, int64_t total_q, int64_t total_k,
                         int heads_q, int heads_k, int head_dim, int max_seqlen_q,
                         int max_seqlen_k, float softmax_scale, int causal, int32_t* status,
                         void* stream);

/* ifv2_sparse_attn_fwd with the key addressing options of the reference's varlen forward
 * (csrc/flash_attn/flash_api.cpp:592-596, 717-742; src/block_info.h:22-24, 40):
 *  seqused_k (batch) int32 or null: keys of each sequence actually in use;
 *  leftpad_k (batch) int32 or null: the keys of sequence b start leftpad_k[b] rows into its
 *    cu_seqlens_k extent (and there are that many fewer); block indices count from the first key;
 *  block_table (batch, block_table_stride) int32 or null: paged K / V, k and v are then
 *    (num_pages * page_size, heads_k, 128) rows (total_k = num_pages * page_size) and key position
 *    p of sequence b lives in page block_table[b][p / page_size]; page_size a multiple of 64 (the
 *    reference wants 256); cu_seqlens_k (or seqused_k) still gives the key count per sequence.
 * As in the reference a paged cache takes no leftpad_k, and there is no paged backward. */
int ifv2_sparse_attn_fwd_paged(const void* q, const void* k, const void* v, void* out, float* lse,
                               const int64_t* fwd_mask, int mask_words, const int32_t* cu_seqlens_q,
                               const int32_t* cu_seqlens_k, const int32_t* seqused_k,
                               const int32_t* leftpad_k, const int32_t* block_table,
                               int block_table_stride, int page_size, int batch, int64_t total_q,
                               int64_t total_k, int heads_q, int heads_k, int head_dim,
                               int max_seqlen_q, int max_seqlen_k, float softmax_scale, int causal,
                               int32_t* status, void* stream);

/* Bytes of scratch ifv2_sparse_attn_bwd needs (D = rowsum(dO * O), one fp32 per query row). */
int64_t ifv2_sparse_attn_bwd_workspace_bytes(int64_t total_q, int heads_q, int head_dim);

/* Backward of the above: dq (total_q, heads_q, 128), dk/dv (total_k, heads_k, 128) bf16; every
 * element of dq, dk and dv is written.  Needs BOTH mask layouts or neither (dense):
 * fwd_mask (heads_k, total_q, fwd_mask_words) as given to the forward, and bwd_mask
 * (heads_k, ceil(max_seqlen_k/64), bwd_mask_words = ceil(total_q/64)) from
 * ifv2_transpose_blockmask.  workspace: caller-allocated, 16-byte aligned scratch of at least
 * ifv2_sparse_attn_bwd_workspace_bytes bytes (contents on entry are ignored).  Deterministic:
 * no atomics are used.
 * Replaces C.varlen_bwd: csrc/entry.cu:209-214 -> mha_varlen_bwd,
 * csrc/flash_attn/flash_api.cpp:1278-1547 (+ the transposes, the Python loop and the
 * synchronisations of infllm_v2/infllmv2_sparse_attention.py:174-263, 343-350). */
int ifv2_sparse_attn_bwd(const void* dout, const void* q, const void* k, const void* v,
                         const void* out, const float* lse, void* dq, void* dk, void* dv,
                         const int64_t* fwd_mask, int fwd_mask_words, const int64_t* bwd_mask,
                         int64_t bwd_mask_words, const int32_t* cu_seqlens_q,
                         const int32_t* cu_seqlens_k, int batch, int64_t total_q, int64_t total_k,
                         int heads_q, int heads_k, int head_dim, int max_seqlen_q,
                         int max_seqlen_k, float softmax_scale, int causal, void* workspace,
                         int64_t workspace_bytes, int32_t* status, void* stream);

/* Backward without any allocation, for hosts that bind this C ABI directly and cannot hand over
 * a workspace: a serving engine that reserved all of HBM for its own pools at start-up has no
 * memory left for cudaMalloc at request time, and cudaMalloc/cudaFree also serialise the whole
 * device, which a latency-bound decode or training loop cannot afford.  Same arguments and
 * results as ifv2_sparse_attn_bwd minus (workspace, workspace_bytes): the scratch (one fp32 per
 * query row) is a 16 MiB array built into the library and resident on every GPU that loads it.
 * Limit: total_q * heads_q <= 4194304 rows; larger calls return IFV2_ERR_TOO_LARGE.
 * The first call on each device looks the array's device address up (with that device
 * current); make that first call before any stream capture begins.  With CUDA's lazy module
 * loading the 16 MiB are only reserved when the library's device code is first loaded on a GPU
 * (its first kernel launch there, or this look-up), so also make that first call -- or any launch
 * from this library under CUDA_MODULE_LOADING=EAGER -- BEFORE the host engine reserves the rest
 * of the device memory; afterwards it can fail with an out-of-memory error.  All calls on a device share
 * the array: two calls whose kernels overlap on the GPU (different streams) race on it.  Nothing
 * in it needs clearing between calls.  No cudaMalloc, cudaFree or allocating library routine
 * is called.  This entry point has no counterpart in the reference. */
int ifv2_sparse_attn_bwd_noalloc(const void* dout, const void* q, const void* k, const void* v,
                                 const void* out, const float* lse, void* dq, void* dk, void* dv,
                                 const int64_t* fwd_mask, int fwd_mask_words,
                                 const int64_t* bwd_mask, int64_t bwd_mask_words,
                                 const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                                 int batch, int64_t total_q, int64_t total_k, int heads_q,
                                 int heads_k, int head_dim, int max_seqlen_q, int max_seqlen_k,
                                 float softmax_scale, int causal, int32_t* status, void* stream);

/* Bytes of scratch ifv2_decode needs for its split partials. */
int64_t ifv2_decode_workspace_bytes(int batch, int heads_q, int head_dim, int max_blocks);

/* Sparse decode over a KV cache: one query token per sequence.
 * q/out: (batch, heads_q, 128) bf16; k_cache, v_cache: (batch_cache, cache_capacity, heads_k,
 * 128) bf16 with `cache_batch_stride` elements between sequences; k_new/v_new (batch, heads_k,
 * 128) or null are first written in place at position cache_seqlens[b]; mask: (batch, heads_k,
 * mask_words) words or null; lse: (batch, heads_q) fp32 or null.
 * A sequence attends positions [0, min(cache_seqlens[b] + new, cache_capacity)): when
 * cache_seqlens[b] >= cache_capacity the new token has no room, is NOT appended and is not
 * attended, and a length beyond the capacity reads only the positions that exist (the host cannot
 * reject this without a device synchronisation, so the kernels define it instead).
 * Replaces C.fwd_kvcache: csrc/entry.cu:209-214 -> mha_fwd_kvcache,
 * csrc/flash_attn/flash_api.cpp:1549-1843. */
int ifv2_decode(const void* q, void* k_cache, void* v_cache, const void* k_new, const void* v_new,
                void* out, float* lse, const int64_t* mask, int mask_words,
                const int32_t* cache_seqlens, int batch, int heads_q, int heads_k, int head_dim,
                int64_t cache_capacity, int64_t cache_batch_stride, float softmax_scale,
                void* workspace, int64_t workspace_bytes, void* stream);

/* Rotary embedding for a decode step with an append: rotates q (batch, heads_q, 128) and k_new
 * (batch, heads_k, 128) at position cache_seqlens[b] into q_out / k_out (same shapes, may not
 * alias the inputs); rotary_cos / rotary_sin: (seqlen_ro, rotary_dim / 2) bf16; interleaved != 0
 * pairs features (2i, 2i+1), otherwise (i, i + rotary_dim / 2).  The rotated tensors are then
 * passed to ifv2_decode[_paged] as q and k_new.  Replaces the rotary-on-append branch of
 * mha_fwd_kvcache (csrc/flash_attn/flash_api.cpp:1773-1797, src/rotary.h). */
int ifv2_decode_rotary(const void* q, const void* k_new, void* q_out, void* k_out,
                       const void* rotary_cos, const void* rotary_sin, const int32_t* cache_seqlens,
                       int batch, int heads_q, int heads_k, int head_dim, int rotary_dim,
                       int seqlen_ro, int interleaved, void* stream);

/* ifv2_decode with the cache addressing options of the reference's fwd_kvcache
 * (csrc/flash_attn/flash_api.cpp:1590-1640, 1773-1797):
 *  block_table (batch, block_table_stride) int32 or null: paged cache, k_cache / v_cache are then
 *    (num_pages, page_size, heads_k, 128) and position p of sequence b lives in page
 *    block_table[b][p / page_size]; page_size a multiple of 64; cache_capacity = the largest
 *    position + 1 any sequence may use (<= block_table_stride * page_size);
 *  cache_batch_idx (batch) int32 or null: sequence b uses row cache_batch_idx[b] of the caches;
 *  cache_leftpad (batch) int32 or null: the keys of sequence b are positions
 *    [cache_leftpad[b], cache_seqlens[b]); block indices of the mask count from the first key.
 * As in the reference, a paged cache takes neither of the last two. */
int ifv2_decode_paged(const void* q, void* k_cache, void* v_cache, const void* k_new,
                      const void* v_new, void* out, float* lse, const int64_t* mask, int mask_words,
                      const int32_t* cache_seqlens, int batch, int heads_q, int heads_k,
                      int head_dim, int64_t cache_capacity, int64_t cache_batch_stride,
                      const int32_t* block_table, int block_table_stride, int page_size,
                      const int32_t* cache_batch_idx, const int32_t* cache_leftpad,
                      float softmax_scale, void* workspace, int64_t workspace_bytes, void* stream);

/* ---------------------------------------------------------------- self-tests -------------- */
/* Test infrastructure shipped in the library so that a deployment can check the tensor-core
 * building blocks on its own GPU; not part of the attention path.  No counterpart in the
 * reference.
 * ifv2_selftest_umma: one tile product through TMA + tcgen05 in the operand arrangement `mode`
 *   (0: Q.K^T shape, 1/2: P.V with P in shared memory / TMEM, 3: MN-major x MN-major,
 *   4/5: thread-written K-major tiles without / with the 32-byte swizzle); d receives fp32.
 * ifv2_selftest_wait_timeout: makes a bounded wait run out on purpose, safely: a kernel waits at
 *   most limit_cycles (<= 2^24) SM clocks on a barrier that nothing arms, stores `site` in the
 *   status block, frees its tensor memory and returns; result: int32[3] = {abort flag seen by
 *   the block, kernel reached its end, the wait returned "gave up"}. */
int ifv2_selftest_umma(int mode, const void* a, const void* b, float* d, int32_t* status,
                       void* stream);
int ifv2_selftest_wait_timeout(int32_t* status, int64_t limit_cycles, int site, int32_t* result,
                               void* stream);

#ifdef __cplusplus
}
#endif
#endif /* INFLLMV2_B200_H_ */
