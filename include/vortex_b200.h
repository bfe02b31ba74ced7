/*
 * vortex_b200 — C ABI of the B200-native (sm_100a) kernels behind the Vortex
 * vFlow sparse-attention decode path.
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer owned by the caller unless said otherwise.
 *   - No entry point allocates, synchronises the host, or throws.  Every entry
 *     point enqueues its work on `stream` (a cudaStream_t passed as void*) and
 *     returns a status: VTX_OK or one of the VTX_ERR_* codes below.
 *   - `dtype` selects the element type of q / caches / scores: VTX_BF16 or VTX_F32.
 *   - "segment" = one (request, KV head) pair, numbered request * num_kv_heads + head.
 *   - Citations name the interface of the reference project that each entry point
 *     replaces (path:line inside that project).
 */
#ifndef VORTEX_B200_H
#define VORTEX_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define VTX_OK 0
#define VTX_ERR_INVALID_ARGUMENT 1 /* null pointer, negative size, bad enum */
#define VTX_ERR_UNSUPPORTED 2      /* shape outside what the kernels are built for */
#define VTX_ERR_CUDA 3             /* the CUDA runtime reported an error at launch */
#define VTX_ERR_SCRATCH_LIMIT 4    /* the call needs more scratch than the library's built-in buffer holds */

#define VTX_BF16 0
#define VTX_F32 1

/* Library version, major * 10000 + minor * 100 + patch. */
int vtx_version(void);

/* Static, NUL-terminated description of a status code. */
const char* vtx_status_string(int status);

/* Text of the last CUDA runtime error seen by this thread's most recent failing call. */
const char* vtx_last_cuda_error(void);

/*
 * Programmatic dependent launch for every later launch of this library in the process.
 *   0  off (the default): plain stream order.
 *   non-zero  each kernel is launched with the programmatic stream-serialization attribute and waits for
 *      the complete preceding launch before it touches memory: results unchanged, launch latency overlaps.
 * A single launch may go further and start reading before that wait: see VTX_LAYER_EARLY_PROLOGUE, which is
 * a per-call flag of vtx_sparse_layer, not part of this process-wide switch.
 * No counterpart in the reference (it launches every kernel with plain stream order).
 */
int vtx_set_programmatic_launch(int enable);

/*
 * Sticky device status word.  A kernel that meets a condition it cannot report through a return code (its
 * launch has already succeeded) sets one of the bits below with an atomic OR and carries on with a well
 * defined result; the word keeps its bits until cleared.  vtx_device_status_word returns its device address
 * on the current device (or NULL); vtx_device_status_read copies it to *host_bits with a synchronous
 * cudaMemcpy (it waits for the device) and, with clear != 0, zeroes it afterwards.
 *   VTX_STATUS_CANDIDATE_OVERFLOW  a segment had more candidate pages than the call's
 *       max_num_pages_per_request allows for (that argument sizes shared memory and the grid).  The
 *       selection written for that segment is its first topk_val candidates, not its best ones.
 *       Precondition of every entry point that takes max_num_pages_per_request:
 *       ceil(cached_seq_len / page_size) <= max_num_pages_per_request for every request of the batch.
 *   VTX_STATUS_BAD_ROW  (checked builds only) a row id or cache slot outside the range the caller gave.
 * No counterpart in the reference (it aborts with TORCH_CHECK above 4096 pages, csrc/topk.cu:200).
 */
#define VTX_STATUS_CANDIDATE_OVERFLOW 1u
#define VTX_STATUS_BAD_ROW 2u
void* vtx_device_status_word(void);
int vtx_device_status_read(uint32_t* host_bits, int clear);

/*
 * Checked build.  The library built with -DVTX_CHECKED (``build.py --checked``, a second file
 * ``libvortex_b200_checked.so`` with the same entry points) compares every index that a kernel reads from a
 * caller's array and then uses as an address with the limits given here: rows of the K/V caches
 * (kv_rows = pages x KV heads), rows of a page-summary cache (summary_rows), token slots of ``loc`` and of the
 * request-to-token table (loc_tokens = pages x page_size), rows of the request-to-token table (req_rows).
 * A negative limit leaves that kind unchecked.  An index outside [0, limit) raises VTX_STATUS_BAD_ROW and is
 * replaced by 0: the kernel touches only valid memory and finishes.  The limits are set by a one-thread kernel
 * on ``stream`` (ordered with the launches that follow, legal inside a stream capture) and hold until set again.
 * vtx_checked_build returns 1 in that library and 0 in the normal one, where vtx_checked_set_limits and
 * vtx_checked_get_limits return VTX_ERR_UNSUPPORTED and the kernels carry no checks.  The reference has no counterpart (its device-side
 * guards are the TORCH_CHECKs of its launchers, e.g. csrc/utils_sglang.cu:322-340, csrc/topk.cu:190-204).
 */
int vtx_checked_build(void);
int vtx_checked_set_limits(int64_t kv_rows, int64_t summary_rows, int64_t loc_tokens, int64_t req_rows,
                           void* stream);
/* The limits in force on the device, in the argument order above, into host_limits[4]; waits for the device. */
int vtx_checked_get_limits(int64_t* host_limits);

/*
 * Block-table builder for one decode step.
 * Replaces `sglang_plan_decode` (csrc/register.h:15-36, csrc/utils_sglang.cu:313-460;
 * kernels :123-184, :188-254, :257-309) and, when the four trailing table pointers
 * are non-null, `sglang_plan_decode_fa3` (csrc/register.h, csrc/utils_sglang.cu:949-1239).
 *
 *   cached_seq_lens [bs] i32, req_to_token [pool, req_to_token_stride] i32,
 *   req_indices [bs] i64.
 *   dense/sparse_kv_indptr [bs*H + 1], dense/sparse_kv_indices (packed),
 *   kv_last_page_len [bs*H], winfo_* workload arrays and two device scalars.
 *   dense/sparse_page_table [bs*H, page_table_stride] and dense/sparse_cache_seqlens
 *   [bs*H] are written only when all four are non-null; in that form kv_last_page_len
 *   may be null (the reference's block-table planner has no such output).
 * One kernel launch; no limit on bs (the reference stops at 1024).
 */
int vtx_plan_decode(const int32_t* cached_seq_lens, const int32_t* req_to_token,
                    int64_t req_to_token_stride, const int64_t* req_indices,
                    int32_t* dense_kv_indptr, int32_t* dense_kv_indices,
                    int32_t* sparse_kv_indptr, int32_t* sparse_kv_indices,
                    int32_t* kv_last_page_len, int32_t* winfo_q_indices,
                    int32_t* winfo_kv_offsets, int32_t* winfo_kv_lens,
                    int32_t* winfo_num_workloads, int32_t* winfo_chunk_size,
                    int32_t* dense_page_table, int32_t* dense_cache_seqlens,
                    int32_t* sparse_page_table, int32_t* sparse_cache_seqlens,
                    int64_t page_table_stride, int batch_size, int page_size,
                    int num_kv_heads, int topk_val, int page_reserved_bos,
                    int page_reserved_eos, int max_chunk_size, int min_chunk_size,
                    void* stream);

/*
 * Scatter new tokens into the paged K and V caches.
 * Replaces `set_kv_buffer_launcher` (cache/triton_kernels/set_kv.py:5-62).
 * Cache layout [num_pages, H, page_size, D]; new_k/new_v [nnz, H, D]; loc [nnz] i64.
 */
int vtx_set_kv(void* k_cache, void* v_cache, const void* new_k, const void* new_v,
               const int64_t* loc, int64_t nnz, int num_kv_heads, int head_dim,
               int page_size, int dtype, void* stream);

/*
 * Page-completion mean over the token axis: the cache-side `Mean(dim=1)` op.
 * Replaces `reduce_pp` with ReduceType.Mean, DIM=1 (cache/triton_kernels/reduce_impl.py:7-89).
 * x [num_pages*H, rows, cols]; out [num_pages*H, 1, cols]; loc [nnz] i64.  A slot t does
 * work only when (t + 1) % page_size == 0.  fp32 accumulation in row order, one rounding.
 */
int vtx_cmean(const void* x, void* out, const int64_t* loc, int64_t nnz, int num_kv_heads,
              int rows, int cols, int page_size, int dtype, void* stream);

/*
 * Page-completion reduction over the token axis with a choice of operator: op 0 mean (= vtx_cmean),
 * 1 maximum, 2 minimum - the cache-side `Mean/Max/Min(dim=1)` ops.  Replaces `reduce_pp` with
 * REDUCE_TYPE 0/1/2, DIM=1 (cache/triton_kernels/reduce_impl.py:7-89).  Arguments as vtx_cmean.
 */
int vtx_creduce(const void* x, void* out, const int64_t* loc, int64_t nnz, int num_kv_heads,
                int rows, int cols, int page_size, int op, int dtype, void* stream);

/*
 * KV write together with the page-completion mean of K: same results as vtx_set_kv followed by
 * vtx_cmean(k_cache -> centroids) on the same loc, in one call - one launch up to 16384 (token, head) items (a
 * decode step), the streaming copy and the page reduction as two launches above that (a prefill), whichever
 * was measured faster.  Replaces the pair set_kv_buffer_launcher (cache/triton_kernels/set_kv.py:39-62) +
 * reduce_pp Mean (cache/triton_kernels/reduce_impl.py:7-89) that the runtime issues back to back
 * for flows whose forward_cache is `CMean(dim=1)(cache["k"], cache["centroids"])`
 * (flow/algorithms.py:172-205).  centroids [num_pages*H, 1, D].
 * Decode (one new token per page) and prefill (many rows of a page in one call) alike, on one condition:
 * the rows of one page that a call writes are consecutive entries of loc in ascending slot order, which is
 * what a prefill produces (each page id appears once, flow/algorithms.py:15).  Rows of the page written by
 * earlier calls are read from the cache.  For any other order of loc use vtx_set_kv then vtx_cmean.
 */
int vtx_set_kv_cmean(void* k_cache, void* v_cache, const void* new_k, const void* new_v,
                     void* centroids, const int64_t* loc, int64_t nnz, int num_kv_heads,
                     int head_dim, int page_size, int dtype, void* stream);

/*
 * Centroid GeMV: score of every non-reserved candidate page of every segment that has
 * more than topk_val candidates, stored at the candidate's packed dense position.
 * Replaces `mv_bpr` (indexer/triton_kernels/mv_impl.py:6-81).
 * q_mean [eff_bs, 1, D]; centroids [num_pages*H, 1, D]; scores [>= dense_indptr[eff_bs]].
 */
int vtx_gemv(const void* q_mean, const void* centroids, void* scores,
             const int32_t* dense_kv_indptr, const int32_t* dense_kv_indices, int eff_batch_size,
             int head_dim, int topk_val, int page_reserved_bos, int page_reserved_eos,
             int dtype, void* stream);

/*
 * Top-k page selection from packed scores into the sparse page list.
 * Replaces `topk_output` (csrc/topk.cu:117-203; kernel :56-113).  Order: score descending,
 * ties by ascending candidate position; output = that sorted prefix of dense row ids.
 * max_num_pages_per_request bounds the candidates of one segment (sizes shared memory).
 */
int vtx_topk(const void* scores, const int32_t* dense_kv_indptr, const int32_t* sparse_kv_indptr,
             const int32_t* dense_kv_indices, int32_t* sparse_kv_indices, int eff_batch_size,
             int topk_val, int page_reserved_bos, int page_reserved_eos,
             int max_num_pages_per_request, int dtype, void* stream);

/*
 * Fused indexer: grouped-query mean + centroid GeMV + top-k, one CTA per segment, scores
 * never leave the SM.  Same results as mean -> vtx_gemv -> vtx_topk.
 * Replaces the chain flow/algorithms.py:168-170 (torch mean, mv_bpr, topk_output).
 * q [eff_bs, group, D].  sparse_page_table (optional, may be null) receives the same ids at
 * [segment, bos + j] for block-table consumers.
 */
int vtx_indexer_fused(const void* q, const void* centroids, const int32_t* dense_kv_indptr,
                      const int32_t* sparse_kv_indptr, const int32_t* dense_kv_indices,
                      int32_t* sparse_kv_indices, int32_t* sparse_page_table,
                      int64_t page_table_stride, int eff_batch_size, int group_size, int head_dim,
                      int topk_val, int page_reserved_bos, int page_reserved_eos,
                      int max_num_pages_per_request, int dtype, void* stream);

/*
 * Fused indexer of the gqa_block_sparse_attention flow (flow/algorithms.py:238-352): per query head the
 * dot of q with each candidate page's centroid (GeMM: fp32 products and sum, bf16 result,
 * indexer/triton_kernels/matmul_impl.py:6-113), a softmax of softmax_scale * score over the segment's
 * candidates (softmax_impl.py:6-105, bf16 result), the maximum over the group's heads
 * (reduce_impl.py:58-75) and the top-k selection (csrc/topk.cu), one CTA per segment, nothing but the
 * selection leaves the SM.  q [eff_bs, group, D]; other arguments as vtx_indexer_fused.  bf16 only.
 */
int vtx_indexer_gqa_softmax_fused(const void* q, const void* centroids, const int32_t* dense_kv_indptr,
                                  const int32_t* sparse_kv_indptr, const int32_t* dense_kv_indices,
                                  int32_t* sparse_kv_indices, int32_t* sparse_page_table,
                                  int64_t page_table_stride, int eff_batch_size, int group_size,
                                  int head_dim, int topk_val, int page_reserved_bos,
                                  int page_reserved_eos, int max_num_pages_per_request,
                                  float softmax_scale, int dtype, void* stream);

/*
 * Fused indexer of the gqa_quest_sparse_attention flow (flow/algorithms.py:356-496): per query head
 * sum over the head dim of max(q*page_max, q*page_min) with bf16 products (Multiply x2 and Maximum,
 * indexer/triton_kernels/elementwise_binary_impl.py:167-307; Sum(dim=2) and Max(dim=1),
 * reduce_impl.py:8-120), then the top-k selection, one CTA per segment.
 * cache_max, cache_min [num_pages*H, 1, D]; other arguments as vtx_indexer_fused.  bf16 only.
 */
int vtx_indexer_quest_fused(const void* q, const void* cache_max, const void* cache_min,
                            const int32_t* dense_kv_indptr, const int32_t* sparse_kv_indptr,
                            const int32_t* dense_kv_indices, int32_t* sparse_kv_indices,
                            int32_t* sparse_page_table, int64_t page_table_stride, int eff_batch_size,
                            int group_size, int head_dim, int topk_val, int page_reserved_bos,
                            int page_reserved_eos, int max_num_pages_per_request, int dtype,
                            void* stream);

/*
 * One launch for a sparse layer: [vtx_set_kv_cmean,] vtx_indexer_fused and vtx_decode_gqa on the sparse
 * lists, run by the same CTA per segment (new-token write, selection, then attention over the selected
 * pages; the selection is also written to sparse_kv_indices).  Same results as the separate calls.
 * Replaces, per layer, set_kv_buffer_launcher + CMean (flow/algorithms.py:172-205), the indexer chain
 * (flow/algorithms.py:168-170) and the paged-decode call the SGLang fork makes afterwards.
 * new_k, new_v [bs, num_kv_heads, D] and loc [bs] are all null (no write) or all set; with them set,
 * k_cache, v_cache and centroids are written and page_reserved_eos must be >= 1.  bf16 only.
 */
int vtx_sparse_layer_fused(const void* q, const void* centroids, const void* k_cache, const void* v_cache,
                           void* out, const void* new_k, const void* new_v, const int64_t* loc,
                           int num_kv_heads, const int32_t* dense_kv_indptr, const int32_t* sparse_kv_indptr,
                           const int32_t* dense_kv_indices, int32_t* sparse_kv_indices,
                           const int32_t* kv_last_page_len, int eff_batch_size, int group_size,
                           int head_dim, int page_size, int topk_val, int page_reserved_bos,
                           int page_reserved_eos, int max_num_pages_per_request, float sm_scale,
                           int dtype, void* stream);

/*
 * General form of the one-launch sparse layer (the three entry points around it are this call with a fixed
 * score_mode, no workspace and no flags).
 *   score_mode  VTX_SCORE_MEAN_DOT: group mean . centroid (block_sparse_attention, flow/algorithms.py:168-170),
 *               VTX_SCORE_GQA_SOFTMAX: GeMM -> Softmax(softmax_scale) -> Max (flow/algorithms.py:281-309),
 *               VTX_SCORE_QUEST: envelope bound from summary (page maximum) and summary2 (page minimum)
 *               (flow/algorithms.py:411-451).
 *   workspace   optional caller-owned device scratch of vtx_sparse_layer_workspace_bytes(...) bytes, ZEROED
 *               ONCE by the caller after allocation (every call leaves it zeroed where that matters).  With
 *               it, a segment with more than 512 candidate pages (768 in batches of at most 384 segments) is
 *               scanned by several CTAs whose best keys the last of them to arrive merges; selections are the
 *               same bits as without it.  Without it
 *               (or for VTX_SCORE_GQA_SOFTMAX, whose softmax spans the whole segment) one CTA scans a
 *               segment.  Calls that share a workspace must not overlap on the GPU.
 *   flags       VTX_LAYER_EARLY_PROLOGUE: when programmatic launch is on, the kernel stages its row ids and
 *               starts its first summary-row gathers BEFORE it waits for the preceding launch.  Those reads
 *               touch only vtx_plan_decode's outputs and summary rows of non-reserved pages, so the caller
 *               must guarantee that the plan launch of the step has completed when this kernel starts:
 *               set the flag only for a launch that follows, on the same stream, at least one launch of
 *               this library that was issued after vtx_plan_decode and that itself waits for its
 *               predecessor before it lets its successor start (every kernel of this library does, except
 *               the tcgen05 form of vtx_decode_mla / vtx_mla_sparse_layer and a vtx_sparse_layer launch that
 *               carries this flag).
 * No counterpart in the reference for workspace and flags (its Triton indexer kernels split work through
 * the planner's workload list instead, csrc/utils_sglang.cu:188-254).
 */
#define VTX_SCORE_MEAN_DOT 0
#define VTX_SCORE_GQA_SOFTMAX 2
#define VTX_SCORE_QUEST 3
#define VTX_LAYER_EARLY_PROLOGUE 1
typedef struct vtx_sparse_layer_params {
    const void* q;        /* [eff_bs, group, D] */
    const void* summary;  /* centroids, or the page-maximum cache for VTX_SCORE_QUEST */
    const void* summary2; /* page-minimum cache (VTX_SCORE_QUEST), else NULL */
    const void* k_cache;
    const void* v_cache;
    void* out;            /* [eff_bs, group, D] */
    const void* new_k;    /* [bs, num_kv_heads, D] or NULL */
    const void* new_v;
    const int64_t* loc;   /* [bs] or NULL */
    const int32_t* dense_kv_indptr;
    const int32_t* sparse_kv_indptr;
    const int32_t* dense_kv_indices;
    int32_t* sparse_kv_indices;
    const int32_t* kv_last_page_len;
    void* workspace;
    int64_t workspace_bytes;
    int32_t eff_batch_size, group_size, head_dim, page_size, num_kv_heads;
    int32_t topk_val, page_reserved_bos, page_reserved_eos, max_num_pages_per_request;
    int32_t score_mode, flags, dtype;
    float sm_scale, softmax_scale;
} vtx_sparse_layer_params;
int64_t vtx_sparse_layer_workspace_bytes(int eff_batch_size, int max_num_pages_per_request, int topk_val,
                                         int page_reserved_bos, int page_reserved_eos);
int vtx_sparse_layer(const vtx_sparse_layer_params* params, void* stream);

/*
 * The same single launch for the gqa_block_sparse_attention flow: page scores are those of
 * vtx_indexer_gqa_softmax_fused (GeMM -> Softmax(scale = softmax_scale) -> Max over the group's heads,
 * flow/algorithms.py:281-309) on the same centroid cache; token write and attention as above.
 */
int vtx_sparse_layer_fused_gqa_softmax(const void* q, const void* centroids, const void* k_cache,
                                       const void* v_cache, void* out, const void* new_k, const void* new_v,
                                       const int64_t* loc, int num_kv_heads, const int32_t* dense_kv_indptr,
                                       const int32_t* sparse_kv_indptr, const int32_t* dense_kv_indices,
                                       int32_t* sparse_kv_indices, const int32_t* kv_last_page_len,
                                       int eff_batch_size, int group_size, int head_dim, int page_size,
                                       int topk_val, int page_reserved_bos, int page_reserved_eos,
                                       int max_num_pages_per_request, float sm_scale, float softmax_scale,
                                       int dtype, void* stream);

/*
 * The same single launch for the gqa_quest_sparse_attention flow: page scores are those of
 * vtx_indexer_quest_fused from the per-page maximum and minimum caches (flow/algorithms.py:411-451); with
 * new_k / new_v / loc set, the launch writes the new token and, for a page it closes, that page's row of
 * both caches (what the flow's cache Max and Min operators compute, flow/algorithms.py:453-496).
 */
int vtx_sparse_layer_fused_quest(const void* q, const void* cache_max, const void* cache_min, const void* k_cache,
                                 const void* v_cache, void* out, const void* new_k, const void* new_v,
                                 const int64_t* loc, int num_kv_heads, const int32_t* dense_kv_indptr,
                                 const int32_t* sparse_kv_indptr, const int32_t* dense_kv_indices,
                                 int32_t* sparse_kv_indices, const int32_t* kv_last_page_len, int eff_batch_size,
                                 int group_size, int head_dim, int page_size, int topk_val, int page_reserved_bos,
                                 int page_reserved_eos, int max_num_pages_per_request, float sm_scale, int dtype,
                                 void* stream);

/*
 * Paged grouped-query decode attention over each segment's page list (sparse or dense).
 * Takes the place of the flashinfer paged-decode call the SGLang fork makes on
 * sparse_kv_indptr / sparse_kv_indices / kv_last_page_len (data contract:
 * indexer/context.py:117-121, csrc/utils_sglang.cu:148-151).
 * q, out [eff_bs, group, D]; k_cache, v_cache [num_pages*H, page_size, D].
 * softmax(q . K^T * sm_scale) . V with fp32 softmax and accumulation.
 */
int vtx_decode_gqa(const void* q, const void* k_cache, const void* v_cache, void* out,
                   const int32_t* kv_indptr, const int32_t* kv_indices,
                   const int32_t* kv_last_page_len, int eff_batch_size, int group_size,
                   int head_dim, int page_size, float sm_scale, int dtype, void* stream);

/*
 * vtx_decode_gqa with the page list of every segment cut into num_splits parts (one CTA per part, a
 * second kernel merges the parts): for batches too small to fill the GPU with one CTA per segment.
 * workspace: caller-owned device scratch of at least vtx_decode_gqa_splitkv_workspace_bytes(...) bytes,
 * fully overwritten by each call.  Same data contract and results (up to fp32 re-association) as
 * vtx_decode_gqa; bf16 only.  The split count plays the role of flashinfer's split-KV planning inside
 * the reference's third-party decode call.
 */
int64_t vtx_decode_gqa_splitkv_workspace_bytes(int eff_batch_size, int group_size, int head_dim,
                                               int num_splits);
int vtx_decode_gqa_splitkv(const void* q, const void* k_cache, const void* v_cache, void* out,
                           const int32_t* kv_indptr, const int32_t* kv_indices,
                           const int32_t* kv_last_page_len, int eff_batch_size, int group_size,
                           int head_dim, int page_size, float sm_scale, int num_splits, void* workspace,
                           int64_t workspace_bytes, int dtype, void* stream);

/*
 * vtx_decode_gqa_splitkv for callers that must not allocate device memory.  (No counterpart in the
 * reference.)  Some hosts of this library cannot call cudaMalloc when they reach the attention step: a
 * serving engine that handed the whole device to its own memory pool at start-up has nothing left to
 * ask the driver for, and a latency-critical decode loop cannot afford the device-wide synchronisation an
 * allocation implies.  This variant takes no workspace: the split states go to a fixed array of
 * VTX_NOALLOC_SCRATCH_BYTES that is part of the library image (each GPU that loads the library holds it
 * until the process exits).  Inputs and outputs are still the caller's.
 *   - A call whose states need more than that - eff_batch_size * num_splits * group_size * (head_dim + 2)
 *     * 4 bytes - is refused with VTX_ERR_SCRATCH_LIMIT; lower num_splits or use vtx_decode_gqa_splitkv.
 *   - The first call on each device looks up the array's device address (with that device current); make
 *     that first call before any stream capture begins.  No call allocates or frees anything.
 *   - All calls on a device share the array.  Every call overwrites all of the states it reads, so
 *     nothing needs clearing between calls, but two calls whose kernels overlap on the GPU (different
 *     streams) would overwrite each other's states: serialise them.
 */
#define VTX_NOALLOC_SCRATCH_BYTES (8 * 1024 * 1024)
int vtx_decode_gqa_splitkv_noalloc(const void* q, const void* k_cache, const void* v_cache, void* out,
                                   const int32_t* kv_indptr, const int32_t* kv_indices,
                                   const int32_t* kv_last_page_len, int eff_batch_size, int group_size,
                                   int head_dim, int page_size, float sm_scale, int num_splits,
                                   int dtype, void* stream);

/*
 * Block-table decode attention over a shared compressed latent (multi-head latent attention):
 * keys are the full latent row, values its first value_dim dims.  No counterpart in the reference
 * (it has no MLA path); the page table and sequence lengths are the block-table form its planner
 * emits (csrc/utils_sglang.cu:949-1083), as written by vtx_plan_decode and vtx_indexer_fused.
 * q [bs, num_heads, latent_dim]; latent_cache [rows, page_size, latent_dim]; out [bs, num_heads, value_dim];
 * page_table [bs, page_table_stride] row ids; cache_seqlens [bs] token counts.
 * num_cache_pages = rows of latent_cache (bounds what the TMA tensor map may address).
 * Built for bf16, 16 heads, latent 576, values 512.  Two forms: tcgen05 tensor cores fed by TMA
 * (page_size a power of two >= 16; the default) and warp-level mma.sync fed by cp.async (page_size a
 * multiple of 16).  vtx_set_mla_path picks: 0 = tcgen05 where the page size allows (default),
 * 1 = always mma.sync.  Returns the previous setting.
 * Every wait inside the tcgen05 kernel is bounded; one that gives up sets a bit in a device word that
 * stays set.  vtx_mla_fault_word returns that word's device address (or NULL); vtx_mla_fault_read
 * copies it to *host_bits with a synchronous cudaMemcpy (so it waits for the device).
 */
int vtx_decode_mla(const void* q, const void* latent_cache, int64_t num_cache_pages, void* out,
                   const int32_t* page_table, int64_t page_table_stride, const int32_t* cache_seqlens,
                   int batch_size, int num_heads, int latent_dim, int value_dim, int page_size,
                   float sm_scale, int dtype, void* stream);

/*
 * One MLA sparse layer in one launch: the page selection of vtx_indexer_fused (query mean over the heads,
 * scores of the candidate pages' summary rows, top-k, written to sparse_kv_indices and to the request's row of
 * sparse_page_table) followed by vtx_decode_mla over that row.  Arguments as in those two entry points
 * (summary [num_cache_pages, 1, latent_dim]; one KV head, so eff_batch_size = batch_size).  The tcgen05 form of
 * the decode runs the selection as its first phase when topk_val <= 64 and the candidates fit its scratch;
 * otherwise, and in the mma.sync form, the call issues the two launches.  Results are those of the two calls,
 * bit for bit.  No counterpart in the reference (it has no MLA path).
 */
int vtx_mla_sparse_layer(const void* q, const void* summary, const void* latent_cache, int64_t num_cache_pages,
                         void* out, const int32_t* dense_kv_indptr, const int32_t* sparse_kv_indptr,
                         const int32_t* dense_kv_indices, int32_t* sparse_kv_indices, int32_t* sparse_page_table,
                         int64_t page_table_stride, const int32_t* sparse_cache_seqlens, int batch_size,
                         int num_heads, int latent_dim, int value_dim, int page_size, int topk_val,
                         int page_reserved_bos, int page_reserved_eos, int max_num_pages_per_request,
                         float sm_scale, int dtype, void* stream);
int vtx_set_mla_path(int path);
void* vtx_mla_fault_word(void);
int vtx_mla_fault_read(uint32_t* host_bits);

/*
 * Unary elementwise operators on a RAGGED indexer tensor (x, out: [max_rows, inner_size] bf16, the first
 * *packed_row_count rows are processed; packed_row_count is a device pointer, normally
 * &dense_kv_indptr[eff_batch_size]).  Replaces elementwise_rr_kernel
 * (indexer/triton_kernels/elementwise_impl.py:8-114) behind Relu / Sigmoid / Silu / Abs / Add_Mul
 * (indexer/elementwise.py:158-297).  op: 0 x >= alpha ? x : beta; 1 1/(1+exp(beta x+alpha));
 * 2 x/(1+exp(beta x+alpha)); 3 |beta x+alpha|; 4 beta x+alpha.  alpha and beta are rounded to bf16 first,
 * every bf16 operation rounds once, the logistic forms use a fixed fp32 exp.  x and out 16-byte aligned.
 */
int vtx_elementwise(const void* x, void* out, const int32_t* packed_row_count, int64_t max_rows,
                    int inner_size, int op, float alpha, float beta, int dtype, void* stream);

/*
 * Binary elementwise operators on two RAGGED indexer tensors x [max_rows, x_c, x_d], y [max_rows, y_c, y_d]
 * (bf16; an inner size of 1 broadcasts), out [max_rows, max(x_c, y_c), max(x_d, y_d)], first
 * *packed_row_count rows.  Replaces elementwise_binary_rrr_kernel
 * (indexer/triton_kernels/elementwise_binary_impl.py:7-100) behind Maximum / Minimum / Add / Multiply on
 * (RAGGED, RAGGED) inputs (indexer/elementwise_binary.py:211-326).  op: 0 max, 1 min,
 * 2 bf16(alpha x) + bf16(beta y), 3 x y; one rounding per bf16 operation.
 */
int vtx_elementwise_binary(const void* x, const void* y, void* out, const int32_t* packed_row_count,
                           int64_t max_rows, int x_c, int x_d, int y_c, int y_d, int op, float alpha,
                           float beta, int dtype, void* stream);

/*
 * Cache-side operators beyond the page mean: every layout of the page-completion reductions, GeMM, unary and
 * binary elementwise.  Like vtx_cmean they act, for every slot t of loc with (t + 1) % page_size == 0 and every
 * KV head h, on one block per operand.  A PAGED operand keeps that block at row (t / page_size) * H + h of a
 * [num_pages * H, ...] cache, a RAGGED one at row i * H + h of a [nnz * H, ...] tensor (i = the slot's index in
 * loc); the *_is_ragged flags say which.  bf16 only, fp32 arithmetic, one rounding per output.
 *
 * vtx_cache_reduce      x block [rows, cols] -> vector of cols (dim 1, reduced over rows) or rows (dim 2) values;
 *                       kind 0 mean, 1 max, 2 min, 3 l2norm.  Replaces reduce_pp / _rp / _pr / _rr
 *                       (cache/triton_kernels/reduce_impl.py:7-508) behind cache Mean / Max / Min / L2Norm
 *                       (cache/reduce.py:354-525).
 * vtx_cache_elementwise the unary family of vtx_elementwise on a block of inner_size values.  Replaces
 *                       elementwise_pp / _pr / _rp / _rr (cache/triton_kernels/elementwise_impl.py) behind cache
 *                       Relu / Silu / Sigmoid / Abs / Add_Mul (cache/elementwise.py).  op 5 writes bf16(alpha) to
 *                       the whole block without reading x (pass x = out): fill_p_kernel
 *                       (cache/triton_kernels/fill_impl.py:6-49) behind cache/fill.py:8-165.
 * vtx_cache_binary      x block [x_c, x_d] with y block [y_c, y_d] (a size of 1 repeats); op 0 max, 1 min,
 *                       2 bf16(alpha x) + bf16(beta y), 3 x y; x and y share a layout.  Replaces
 *                       elementwise_binary_ppp / _ppr / _rrp / _rrr
 *                       (cache/triton_kernels/elementwise_binary_impl.py) behind cache Maximum / Minimum / Add /
 *                       Multiply (cache/elementwise_binary.py).
 * vtx_cache_gemm        out block [y_rows, x_rows] = Y [y_rows, inner_dim] . X [x_rows, inner_dim]^T, fp32 products
 *                       and sum.  Replaces gemm_ppp / _ppr / _rrp / _rrr (cache/triton_kernels/matmul_impl.py)
 *                       behind cache GeMM (cache/matmul.py).
 */
int vtx_cache_reduce(const void* x, void* out, const int64_t* loc, int64_t nnz, int num_kv_heads,
                     int rows, int cols, int page_size, int dim, int kind, int x_is_ragged,
                     int out_is_ragged, int dtype, void* stream);
int vtx_cache_elementwise(const void* x, void* out, const int64_t* loc, int64_t nnz, int num_kv_heads,
                          int inner_size, int page_size, int op, float alpha, float beta, int x_is_ragged,
                          int out_is_ragged, int dtype, void* stream);
int vtx_cache_binary(const void* x, const void* y, void* out, const int64_t* loc, int64_t nnz,
                     int num_kv_heads, int x_c, int x_d, int y_c, int y_d, int page_size, int op, float alpha,
                     float beta, int inputs_are_ragged, int out_is_ragged, int dtype, void* stream);
int vtx_cache_gemm(const void* x, const void* y, void* out, const int64_t* loc, int64_t nnz,
                   int num_kv_heads, int x_rows, int y_rows, int inner_dim, int page_size,
                   int inputs_are_ragged, int out_is_ragged, int dtype, void* stream);

/*
 * Stand-alone forms of the indexer operators that the shipped flows chain.  (The flows themselves run them as
 * links of vtx_indexer_gqa_softmax_fused / vtx_indexer_quest_fused; these entry points serve flows that
 * compose the operators differently or read an intermediate, and return the same bits.)  All work on the
 * candidate window of every segment - packed positions [dense_kv_indptr[s] + bos, dense_kv_indptr[s+1] - eos)
 * of segments with more than topk_val candidates, the rows the reference's workload list covers
 * (csrc/utils_sglang.cu:219-251) - and leave other rows untouched.  bf16 only; one rounding per operator output.
 *
 * vtx_gemm_bpr       out[p, c, g] = table[row_p, c, :] . q[s, g, :] (fp32 products and sum); q [eff_bs, G, D],
 *                    table [rows, C, D], out [N, C, G].  Replaces mm_bpr (indexer/triton_kernels/matmul_impl.py:6-113).
 * vtx_softmax_ragged in place on x [N, inner]: softmax of scale * x over a segment's candidates, per inner
 *                    element.  Replaces softmax_inplace_r (indexer/triton_kernels/softmax_impl.py:6-105).
 * vtx_normalize_ragged  in place: x divided by max(L2 norm over the segment's candidates, eps), per inner
 *                    element.  Replaces normalize_inplace_r (indexer/triton_kernels/normalize_impl.py:6-119).
 * vtx_reduce_ragged  x [N, rows, cols] -> out [N, 1, cols] (dim 1) or [N, rows, 1] (dim 2); kind 0 mean, 1 max,
 *                    2 min, 3 l2norm, 4 sum (the reference's ReduceType values).  Replaces reduce_rr
 *                    (indexer/triton_kernels/reduce_impl.py:8-120).
 * vtx_binary_bpr     out[p] = op(q[s], table[row_p]) with the inner dims broadcast; q [eff_bs, q_c, q_d],
 *                    table [rows, table_c, table_d]; op 0 max, 1 min, 2 bf16(alpha x) + bf16(beta y), 3 x y.
 *                    With x_is_ragged the left operand is the RAGGED row q[p] ([N, q_c, q_d]) instead.
 *                    Replaces elementwise_binary_bpr and _rpr
 *                    (indexer/triton_kernels/elementwise_binary_impl.py:167-307, 348-476).
 * vtx_transpose_ragged  out[p, c, r] = x[p, r, c].  Replaces transpose_rr (indexer/triton_kernels/transpose_impl.py:6-101).
 * vtx_save_load_ragged  save != 0: paged[row_p] = ragged[p]; save == 0: ragged[p] = paged[row_p], inner_size
 *                    elements per row.  Replaces save_rp / load_pr (indexer/triton_kernels/save_load_impl.py:6-229).
 */
int vtx_gemm_bpr(const void* q, const void* table, void* out, const int32_t* dense_kv_indptr,
                 const int32_t* dense_kv_indices, int eff_batch_size, int group_size, int table_rows,
                 int head_dim, int topk_val, int page_reserved_bos, int page_reserved_eos, int dtype,
                 void* stream);
int vtx_softmax_ragged(void* x, const int32_t* dense_kv_indptr, int eff_batch_size, int inner_size,
                       int topk_val, int page_reserved_bos, int page_reserved_eos, float scale, int dtype,
                       void* stream);
int vtx_normalize_ragged(void* x, const int32_t* dense_kv_indptr, int eff_batch_size, int inner_size,
                         int topk_val, int page_reserved_bos, int page_reserved_eos, float eps, int dtype,
                         void* stream);
int vtx_reduce_ragged(const void* x, void* out, const int32_t* dense_kv_indptr, int eff_batch_size,
                      int rows, int cols, int dim, int kind, int topk_val, int page_reserved_bos,
                      int page_reserved_eos, int dtype, void* stream);
int vtx_binary_bpr(const void* q, const void* table, void* out, const int32_t* dense_kv_indptr,
                   const int32_t* dense_kv_indices, int eff_batch_size, int q_c, int q_d, int table_c,
                   int table_d, int op, float alpha, float beta, int x_is_ragged, int topk_val,
                   int page_reserved_bos, int page_reserved_eos, int dtype, void* stream);
int vtx_transpose_ragged(const void* x, void* out, const int32_t* dense_kv_indptr, int eff_batch_size,
                         int rows, int cols, int topk_val, int page_reserved_bos, int page_reserved_eos,
                         int dtype, void* stream);
int vtx_save_load_ragged(void* ragged, void* paged, const int32_t* dense_kv_indptr,
                         const int32_t* dense_kv_indices, int eff_batch_size, int inner_size, int save,
                         int topk_val, int page_reserved_bos, int page_reserved_eos, int dtype, void* stream);

/*
 * Prefill planner.  Replaces `sglang_plan_prefill` (csrc/register.h, csrc/utils_sglang.cu:462-621).
 * cached_seq_lens, input_seq_lens [bs] i32; outputs dense_kv_indptr, qo_indptr_paged [bs*H + 1],
 * qo_indptr_ragged [bs + 1], dense_kv_indices (packed row ids), kv_last_page_len [bs*H],
 * batch_table [sum of input lengths] u16 (token -> request).  One launch, no batch limit up to 65536.
 */
int vtx_plan_prefill(const int32_t* cached_seq_lens, const int32_t* input_seq_lens,
                     const int32_t* req_to_token, int64_t req_to_token_stride,
                     const int64_t* req_indices, int32_t* dense_kv_indptr, int32_t* dense_kv_indices,
                     int32_t* qo_indptr_ragged, int32_t* qo_indptr_paged, int32_t* kv_last_page_len,
                     uint16_t* batch_table, int batch_size, int page_size, int num_kv_heads,
                     void* stream);

/*
 * Prefill planner, block-table form.  Replaces `sglang_plan_prefill_fa3` (csrc/utils_sglang.cu:797-869).
 * cached_seq_lens [bs*H] (per segment), cu_seqlens_q [bs*H + 1]; outputs page_table [bs*H, stride] and
 * batch_table u16.
 */
int vtx_plan_prefill_fa3(const int32_t* cached_seq_lens, const int32_t* cu_seqlens_q,
                         const int32_t* req_to_token, int64_t req_to_token_stride,
                         const int64_t* req_indices, int32_t* page_table, int64_t page_table_stride,
                         uint16_t* batch_table, int batch_size, int page_size, int num_kv_heads,
                         void* stream);

/*
 * Token-major [N, H*G, D] -> per-request head-major [N*H, G, D] shuffle of bf16 rows (q before the
 * prefill attention).  Replaces `Chunkwise_NH2HN_Transpose` (csrc/utils_sglang.cu:623-695); the caller
 * owns x_out.  indptr [bs + 1] token offsets per request, batch_table [N] u16.
 */
int vtx_chunkwise_nh2hn(const void* x, void* x_out, const int32_t* indptr, const uint16_t* batch_table,
                        int64_t num_tokens, int num_kv_heads, int group_size, int head_dim,
                        void* stream);

/*
 * The inverse shuffle for the attention output x (bf16) and, when y / y_out are non-null, the fp32
 * log-sum-exp [N*H, G] -> [N, H*G].  Replaces `Chunkwise_HN2NH_Transpose` (csrc/utils_sglang.cu:698-793)
 * and, with y null, `Chunkwise_HN2NH_Transpose_FA3` (:872-946).
 */
int vtx_chunkwise_hn2nh(const void* x, void* x_out, const float* y, float* y_out, const int32_t* indptr,
                        const uint16_t* batch_table, int64_t num_tokens, int num_kv_heads,
                        int group_size, int head_dim, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* VORTEX_B200_H */
