/* C ABI of libmsa_b200.so: the sm_100a kernels behind the MSA block-sparse
 * attention hot path (proxy max-score pass, top-k page selector, sparse paged
 * attention prefill / FP8 decode).
 *
 * Conventions: every pointer is a DEVICE pointer unless it says "host"; the
 * library never allocates or frees device memory; `stream` is a cudaStream_t
 * passed as void*; calls are asynchronous on that stream.  Return value:
 * 0 = ok, > 0 = cudaError_t, < 0 = MSA_ERR_* below.  Nothing throws.
 *
 * Each entry point names the reference interface it stands in for
 * (paths inside the MiniMax-AI/MSA project).
 */
#ifndef MSA_B200_H_
#define MSA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MSA_OK 0
#define MSA_ERR_INVALID (-1)     /* bad argument */
#define MSA_ERR_UNSUPPORTED (-2) /* shape / dtype combination not built */
#define MSA_ERR_TIMEOUT (-3)     /* a bounded device-side wait ran out (status word) */
#define MSA_ERR_DRIVER (-4)      /* driver entry point or tensor-map encode failed */
#define MSA_ERR_TOO_LARGE (-5)   /* size beyond a stated maximum */
#define MSA_ERR_BOUNDS (-6)      /* a page-table entry outside [0, kv_rows) reached a kernel (status word): the page was
                                    replaced by page 0, so the result is wrong but nothing was read out of bounds --
                                    the role of the reference's FMHA_GMEM_CHECK build (csrc/gmem_bounds_check.h:27-95),
                                    always on here because it costs one compare per page */
/* msa_validate_inputs: the first rule of the index contract that the inputs break */
#define MSA_EVAL_Q_ROWS (-101)            /* q rows != sum(qo_lens) */
#define MSA_EVAL_KV_ROWS (-102)           /* ragged K/V rows != sum(kv_lens) */
#define MSA_EVAL_PAGE_TABLE_LENGTH (-103) /* kv_indices length != sum(ceil(kv_lens / 128)) */
#define MSA_EVAL_PAGE_TABLE_RANGE (-104)  /* a kv_indices entry outside [0, num_pages) */
#define MSA_EVAL_LIST_SHAPE (-105)        /* kv_block_indexes heads not num_kv_heads | num_qo_heads, or topk <= 0 */
#define MSA_EVAL_LIST_NEGATIVE (-106)     /* a page-list entry below -1 */
#define MSA_EVAL_LIST_PADDING (-107)      /* a valid entry after a -1 (padding must be at the tail) */
#define MSA_EVAL_LIST_RANGE (-108)        /* an entry >= the request's page count */
#define MSA_EVAL_LIST_ORDER (-109)        /* entries not strictly ascending */

/* K/V storage formats */
#define MSA_KV_BF16 0
#define MSA_KV_FP8_E4M3 1 /* per-tensor scale folded into qk_scale / v_scale by the caller */
#define MSA_KV_NVFP4 2    /* packed e2m1 + e4m3 scale per 16 values (128x4 tiles) + fp32 global scale */

/* Library version, for the loader to check. */
int msa_abi_version(void);

/* Short text for a negative MSA_ERR_* code (host pointer, static storage). */
const char* msa_error_string(int code);

/* ---------------------------------------------------------------------------
 * Planner (host only: every pointer below is a HOST pointer, nothing is launched).
 * Replaces the TVM-FFI function `plan(...22 args...)` (python/fmha_sm100/csrc/fmha_sm100_plan.cu:18-35) and the
 * Python planner around it (python/fmha_sm100/api.py:510-747): the persistent kernels here take 128-row query
 * tiles round-robin from an ordered list, so the plan is that list (heaviest tile first), the page-table
 * offsets of the requests and, for the decode kernels, each token's (request, last visible key) and the number
 * of KV splits.  The caller copies the arrays it needs to the device and passes them as msa_fmha_args.work /
 * msa_decode_args.{kv_page_indptr, token_request, token_pos, num_splits}.
 */
typedef struct msa_plan_desc {
  int32_t batch;
  const int32_t* qo_lens;   /* [batch] query tokens per request */
  const int32_t* kv_lens;   /* [batch] keys per request */
  const int32_t* qo_offset; /* [batch] causal offset (row i sees key j iff i + offset >= j); NULL = kv_len - qo_len */
  int32_t causal;           /* 0: every key visible */
  int32_t paged;            /* 1: work[6] counts page-table slots; 0: K/V tokens (ragged K/V) */
  int32_t num_qo_heads, num_kv_heads;
  int32_t kv_block_num;     /* page-list length of a sparse call (> 0), else <= 0 */
  int32_t num_kv_splits;    /* > 0 forces the decode split count, else chosen for whole waves of CTAs */
  int32_t num_sms;          /* SMs the decode split choice may assume (usable_SM_count), <= 0 = 148 */
  int32_t tile_rows;        /* query tokens per work entry: 0 or 128; 256 for the score-only pass, whose work items
                               are two query tiles against one stream of K pages (msa_fmha_args.tile_rows); any
                               value up to 256 (256 / hb with msa_fmha_args.score_pack_heads = hb) */
  int32_t dense_kv_splits;  /* > 1: every query tile becomes this many work entries, each over a contiguous range of
                               the tile's visible pages, writing output rows split * total_q + token (merged by
                               msa_fmha_combine); for dense calls whose query tiles alone cannot fill the GPU.
                               0 or 1: one entry per tile */
} msa_plan_desc;

/* Sizes of the arrays msa_plan fills: query tiles, total query tokens, total page-table slots. */
int msa_plan_sizes(const msa_plan_desc* desc, int32_t* n_work, int64_t* total_q, int64_t* total_pages);

/* Fills (each may be NULL to skip it): work int32 [n_work, 8] (layout of msa_fmha_args.work),
 * kv_page_indptr int32 [batch + 1], token_request / token_pos int32 [total_q], *num_splits. */
int msa_plan(const msa_plan_desc* desc, int32_t* work, int32_t* kv_page_indptr, int32_t* token_request,
             int32_t* token_pos, int32_t* num_splits);

/* Host re-check of the index contract before a launch (host pointers; nothing is launched): what the asserts of
 * `_validate_fmha_inputs` (python/fmha_sm100/api.py:128-263) check, on raw arrays.  Returns MSA_OK or the
 * MSA_EVAL_* code of the first broken rule (rules in the order of the defines above); *where (may be NULL)
 * receives the flat index of the first offending element of kv_indices / kv_block_indexes, else -1. */
typedef struct msa_validate_args {
  int32_t batch;
  const int32_t* qo_lens;
  const int32_t* kv_lens;
  int64_t total_q;                 /* rows of q */
  int64_t kv_rows;                 /* num_pages (paged) or rows of ragged K/V */
  int32_t paged;
  const int32_t* kv_indices;       /* [n_kv_indices] or NULL */
  int64_t n_kv_indices;
  const int32_t* kv_block_indexes; /* [total_q, list_heads, topk] or NULL */
  int32_t list_heads, topk;
  int32_t num_qo_heads, num_kv_heads;
} msa_validate_args;
int msa_validate_inputs(const msa_validate_args* args, int64_t* where);

/* ---------------------------------------------------------------------------
 * Stage 2: top-k page selector.
 * Replaces the TVM-FFI function `sparse_topk_select(max_score, out, workspace,
 * topk, num_valid_pages, force_begin, force_end, stream)`
 * (python/fmha_sm100/csrc/sparse_topk_select.cu:17-68) called by
 * `sparse_topk_select` (python/fmha_sm100/api.py:1179-1290).  No workspace.
 *   max_score  float32 [num_heads, max_k_tiles, total_q], contiguous
 *   out        int32   [total_q, num_heads, topk], ascending page ids, -1 tail
 *   topk       16, 32 or 64
 *   num_valid_pages  in (0, max_k_tiles]; tiles >= it are never selected
 *   force_begin / force_end  leading / trailing valid tiles that are always taken
 * Ties go to the lower page id; a pick whose score is -inf is reported as -1.
 */
int msa_topk_select(const float* max_score, int32_t num_heads, int32_t max_k_tiles, int32_t total_q, int32_t topk,
                    int32_t num_valid_pages, int32_t force_begin, int32_t force_end, int32_t* out, void* stream);

/* Max over the tokens of each query block: [H, K, T] -> [H, K, n_blocks].
 * `block_starts` int32 [n_blocks + 1] token offsets.  The reference selects per
 * token (python/fmha_sm100/api.py:398-429); this reducer gives the per-128-query-
 * block granularity when the caller wants one page list per block. */
int msa_block_max(const float* max_score, int32_t num_heads, int32_t max_k_tiles, int32_t total_q,
                  const int32_t* block_starts, int32_t n_blocks, float* out, void* stream);

/* The other end of the per-block granularity: `block_lists` int32 [n_blocks, num_heads, topk] (what
 * msa_topk_select returns on the output of msa_block_max) is written to every token of its block,
 * out int32 [total_q, num_heads, topk] -- the per-token layout `kv_block_indexes` has in the reference
 * (python/fmha_sm100/api.py:1046-1060).  num_heads * topk must be a multiple of 4, both buffers 16-byte aligned. */
int msa_expand_block_lists(const int32_t* block_lists, const int32_t* block_starts, int32_t n_blocks,
                           int32_t num_heads, int32_t topk, int32_t* out, void* stream);

/* ---------------------------------------------------------------------------
 * Stages 1 and 3 (prefill): dense / score-only / block-sparse paged attention.
 * Replaces the TVM-FFI function `run_<variant>(...34 args...)`
 * (python/fmha_sm100/csrc/fmha_sm100_variant_run.cu.jinja:15-205) in its four
 * modes (Off, Full, OnlyScore, Sparse) and, for long-Q sparse calls, the
 * `sparse_atten_func` / `sparse_atten_nvfp4_kv_func` kernels
 * (python/fmha_sm100/cute/interface.py:600-991).
 */
typedef struct msa_fmha_args {
  const void* q;          /* bf16 [total_q, num_qo_heads, 128] */
  const void* k;          /* paged: [num_pages, num_kv_heads, 128, 128] (bf16 | e4m3) or u8 [.., 128, 64] (nvfp4);
                             ragged (paged = 0): [total_kv, num_kv_heads, 128] */
  const void* v;          /* same layout as k */
  void* out;              /* bf16 [total_q, num_qo_heads, 128], or NULL for the score-only pass */
  float* lse;             /* float32 [total_q, num_qo_heads] natural-log LSE, or NULL */
  float* max_score;       /* float32 [num_qo_heads, max_k_tiles, total_q] raw q.k tile maxima, or NULL.
                             Only tiles the kernel visits are written; the caller pre-fills -inf (or, for the
                             score-only pass, sets score_fill_tail). */
  const int32_t* work;    /* int32 [n_work, 8], one entry per 128-row query tile, heaviest first:
                             {request, first token (global), valid rows <= 128 | first page << 10,
                              first token (request-local),
                              kv_len, causal offset (row i sees key j iff i + offset >= j),
                              first page-table slot of the request (paged) | first K/V token (ragged),
                              output row offset}.
                             "first page" and "output row offset" are 0 unless the list was planned with
                             dense_kv_splits > 1: an entry then covers the pages [first page, ceil(kv_len / 128))
                             of a dense request (kv_len cut at the end of the entry's page range) and writes its
                             output / LSE rows at token + output row offset.
                             With page lists (kv_block_indexes != NULL) kv_len is at most 16384 pages
                             (2 097 152 keys); a longer request is skipped (zero output) and the status word
                             receives MSA_ERR_UNSUPPORTED. */
  int32_t n_work;
  const int32_t* kv_indices;         /* flat physical page table (paged) */
  const int32_t* kv_block_indexes;   /* [total_q, list_heads, topk] request-local page ids, ascending, -1 tail;
                                        NULL = dense */
  const uint8_t* k_scale_128x4;      /* nvfp4: e4m3 block scales, row = (page * num_kv_heads + head) * 128 + token */
  const uint8_t* v_scale_128x4;
  int64_t total_q;
  int64_t kv_rows;        /* num_pages (paged) or total_kv (ragged) */
  int32_t num_qo_heads, num_kv_heads;
  int32_t topk, list_heads; /* list_heads = num_kv_heads or num_qo_heads */
  int32_t max_k_tiles;
  int32_t kv_dtype;       /* MSA_KV_* */
  int32_t paged, causal;
  float sm_scale;         /* softmax scale */
  float qk_scale;         /* q_scale * k_scale (* k global scale for nvfp4) */
  float v_scale;          /* v_scale * o_scale (* v global scale for nvfp4) */
  int32_t* status;        /* device int32, zeroed by the caller; receives MSA_ERR_TIMEOUT if a wait ran out,
                             MSA_ERR_UNSUPPORTED for a request beyond the page-list limit above, MSA_ERR_BOUNDS for
                             a page-table entry outside [0, kv_rows) */
  int32_t max_ctas;       /* > 0 caps the persistent grid (the reference's usable_SM_count); 0 = one CTA per SM */
  int32_t qk_dim;         /* 0 or 128: all of the head dimension; 64: the score-only pass (out = NULL) uses only the
                             first 64 elements of q and k (a 64-wide proxy zero-padded to 128 costs half) */
  int32_t tile_rows;      /* 0 or 128: `work` holds 128-row tiles.  256 (score-only pass, out = NULL, only): `work`
                             holds 256-row entries (msa_plan_desc.tile_rows = 256), so that every K page is fetched
                             once for two query tiles; the score-only pass also takes 128-row entries, at half the
                             arithmetic per K byte */
  const uint8_t* tile_uniform;   /* optional, uint8 [n_work, list_heads] from msa_list_uniformity: non-zero where all
                                    rows of a query tile carry the same page list (the tile's page set is then taken
                                    from one row instead of 128); NULL = no tile is assumed uniform */
  int64_t max_score_tile_stride; /* elements between consecutive tiles of max_score; 0 = total_q (contiguous) */
  int64_t max_score_head_stride; /* elements between consecutive heads; 0 = max_k_tiles * tile stride.  The two
                                    strides let a call write its tokens into a slice [.., .., t0:t1] of a larger
                                    score tensor (the decode and prefill halves of a mixed batch) */
  int32_t k_scale_format;        /* score-only pass over packed e2m1 K (kv_dtype MSA_KV_NVFP4, out = NULL): 0 = one
                                    e4m3 scale per 16 values (1024 scale bytes per (page, head), two 128x4 tiles),
                                    1 = one ue8m0 scale per 32 values (MXFP4: 512 bytes, one 128x4 tile; exponents
                                    outside 2^-24 .. 2^15 saturate) */
  int32_t score_pack_heads;      /* score-only pass: 0 or 1 = one query head per 128-row tile; hb > 1 (a power of two
                                    dividing the query heads per KV head) = a tile holds 128 / hb tokens x hb heads,
                                    for requests that bring only a few tokens (decode): `work` then holds entries of up
                                    to 256 / hb tokens (msa_plan_desc.tile_rows = 256 / hb = msa_fmha_args.tile_rows).
                                    An entry may also cover only the pages from `first page` up (work[2] >> 10, as
                                    msa_plan_desc.dense_kv_splits writes it): per-page maxima need no merging */
  int32_t score_fill_tail;       /* score-only pass: non-zero = work entries whose last field (work[7]) is 1 also write
                                    -inf into max_score for the tiles above their own page range, up to max_k_tiles,
                                    so the caller need not pre-fill the tensor.  Flag exactly one entry per (request,
                                    query tile) -- the one that covers the highest pages when the page range is split
                                    -- and keep the pre-fill if some query tile sees no page at all (it has no entry
                                    that runs). */
  int32_t fp8_p_f16;             /* e4m3 K/V attention: 0 = P is rounded to e4m3 and multiplies the V pages as stored
                                    (fastest; max-abs error vs fp32 ~1e-2 on outputs of magnitude 1); non-zero = V is
                                    dequantised to f16 and P stays f16 (P exact to 11 bits, ~13 % slower).  Ignored
                                    for other K/V formats and by the score-only pass */
  int64_t out_rows;              /* rows of out / lse; 0 = total_q.  dense_kv_splits * total_q when the work list
                                    was planned with KV splits: out and lse are then the partial buffers that
                                    msa_fmha_combine merges (lse must be given) */
} msa_fmha_args;

int msa_fmha_fwd(const msa_fmha_args* args, void* stream);

/* Merges the partial results of a call planned with msa_plan_desc.dense_kv_splits = n_splits (the role of the
 * combine step behind num_kv_splits in python/fmha_sm100/api.py:944-1026):
 *   out[t, h, :] = sum_s exp(lse_s[t, h] - lse[t, h]) * partial_out[s, t, h, :],  lse = log sum_s exp(lse_s)
 * partial_out bf16 [n_splits, total_q, num_qo_heads, 128], partial_lse float32 [n_splits, total_q, num_qo_heads]
 * (natural log, -inf where a split saw no key); out bf16 [total_q, num_qo_heads, 128]; lse float32 or NULL. */
int msa_fmha_combine(const void* partial_out, const float* partial_lse, int32_t n_splits, int64_t total_q,
                     int32_t num_qo_heads, void* out, float* lse, void* stream);

/* Optional pre-pass for page-list calls: flags[w * list_heads + h] = 1 iff every row of query tile `w` (an entry of
 * `work`) has the same list for list head `h`.  MSA selects pages per query block, so the per-token lists of the
 * reference API (python/fmha_sm100/api.py:207-238) are usually 128 copies of one row; pass the flags as
 * msa_fmha_args.tile_uniform.  Reads the list tensor once; the reference has no counterpart (its KV-outer kernel
 * consumes the reverse index instead). */
int msa_list_uniformity(const int32_t* work, int32_t n_work, const int32_t* kv_block_indexes, int32_t list_heads,
                        int32_t topk, uint8_t* flags, void* stream);

/* FP4 indexer (fp4_indexer_block_scores, python/fmha_sm100/cute/fp4_indexer_interface.py:745-1056): per-page maxima
 * of Q K^T with Q and K given as packed e2m1 (two values per byte, low nibble = even element) and block scales.
 * The scores come from msa_fmha_fwd in its score-only form (out = NULL) with kv_dtype = MSA_KV_NVFP4, k = the packed
 * pages [pages, num_kv_heads, 128, 64], k_scale_128x4 = the K scales in 128x4-tiled storage (one 1024- or 512-byte
 * block per (page, head)), k_scale_format = the format below, and q = Q dequantised to bf16 by
 * msa_fp4_dequant_rows (exact: e2m1 times a block scale has at most six significant bits).
 *   format        0: NVFP4, one e4m3 scale per 16 values (8 per row); 1: MXFP4, one ue8m0 scale per 32 (4 per row)
 *   scale_layout  0: logical [rows, heads, G]; 1: 128x4-tiled storage with mn = rows, l = heads
 *                 (fp4_indexer_mma_scale_storage_shape, fp4_indexer_interface.py:236-249)
 *   packed uint8 [rows, heads, 64]; out bf16 [rows, heads, 128]. */
#define MSA_FP4_NVFP4 0
#define MSA_FP4_MXFP4 1
int msa_fp4_dequant_rows(const void* packed, const void* scales, int32_t format, int32_t scale_layout, int64_t rows,
                         int32_t heads, void* out, void* stream);

/* Logical scales -> 128x4-tiled storage (Fp4IndexerScaleReorderSm100,
 * python/fmha_sm100/cute/src/sm100/fp4_indexer.py:83-199): element (m, g, l) goes to
 * l * 512 * ceil(mn / 128) * ceil(G / 4) + (m / 128) * 512 * ceil(G / 4) + (g / 4) * 512 + (m % 32) * 16
 * + ((m % 128) / 32) * 4 + g % 4.  k_layout = 1: src is [l_extent, mn, G] (K scales, mn = 128, l = page * heads +
 * head); k_layout = 0: src is [mn, l_extent, G] (Q scales, mn = tokens, l = head).  dst holds
 * l_extent * ceil(mn / 128) * ceil(G / 4) * 512 bytes; bytes of rows beyond mn are left untouched. */
int msa_fp4_reorder_scales(const void* src, int32_t format, int64_t mn, int64_t l_extent, int32_t k_layout, void* dst,
                           void* stream);

/* k2q CSR -> per-query page lists, on the device.  The reference's sparse prefill is KV-outer and consumes the
 * reverse index built by `build_k2q_csr` (python/fmha_sm100/cute/sparse_index_utils.py:331-420,
 * python/fmha_sm100/cute/src/sm100/prepare_k2q_csr.py:54); the kernel here is query-stationary, so the
 * CSR-driven entry points turn it back into kv_block_indexes before msa_fmha_fwd.
 *   row_ptr     int32 [num_kv_heads, n_rows + 1] (row_ptr_stride elements between heads)
 *   q_indices   int32 [num_kv_heads, >= nnz] request-local query ids (q_indices_stride between heads)
 *   row_request / row_block  int32 [n_rows]: request and KV block of each CSR row (block-major packing)
 *   cu_seqlens_q int32 [batch + 1]
 *   counters    int32 [total_q * num_kv_heads] scratch (cleared by the call)
 *   out         int32 [total_q, num_kv_heads, topk] ascending block ids, -1 tail; a query selected by more
 *               than topk rows keeps topk of them.  topk in {4, 8, 16, 32, 64}. */
int msa_k2q_csr_to_lists(const int32_t* row_ptr, const int32_t* q_indices, const int32_t* row_request,
                         const int32_t* row_block, const int32_t* cu_seqlens_q, int32_t num_kv_heads,
                         int32_t n_rows, int64_t row_ptr_stride, int64_t q_indices_stride, int64_t total_q,
                         int32_t topk, int32_t* counters, int32_t* out, void* stream);

/* q2k page lists -> k2q CSR, on the device: what `build_k2q_csr` (python/fmha_sm100/cute/sparse_index_utils.py:331,
 * kernels python/fmha_sm100/cute/src/sm100/build_k2q_csr/build_k2q_csr.cu) produces for callers that feed the
 * CSR-driven entry points.  Rows are packed block-major (block 0 of every request, then block 1, ...); inside a row
 * the batch-local query ids ascend; the unused tail of q_indices is -1.  The small metadata arrays (device int32)
 * describe the batch: queries are cut into chunks of at most 256 that do not cross requests.
 *   q2k                 [num_kv_heads, total_q, topk] request-local block ids, -1 = unused
 *   chunk_request / chunk_first_query / chunk_len   [n_chunks]
 *   cu_seqlens_q        [batch + 1];  request_first_chunk [batch + 1];  request_blocks [batch] (CSR rows per request)
 *   row_of_block        [batch, max_blocks] CSR row of (request, block)
 *   workspace           msa_build_k2q_csr_workspace_bytes(...) bytes (cleared by the call)
 *   row_ptr             [num_kv_heads, total_rows + 1];  q_indices [num_kv_heads, q_indices_stride >= total_q * topk] */
typedef struct msa_csr_build_args {
  const int32_t* q2k;
  const int32_t* chunk_request;
  const int32_t* chunk_first_query;
  const int32_t* chunk_len;
  const int32_t* cu_seqlens_q;
  const int32_t* request_first_chunk;
  const int32_t* request_blocks;
  const int32_t* row_of_block;
  void* workspace;
  size_t workspace_bytes;
  int32_t* row_ptr;
  int32_t* q_indices;
  int64_t total_q, q_indices_stride;
  int32_t num_kv_heads, topk, n_chunks, batch, max_blocks, total_rows;
} msa_csr_build_args;
size_t msa_build_k2q_csr_workspace_bytes(int32_t num_kv_heads, int32_t n_chunks, int32_t max_blocks, int32_t total_rows);
int msa_build_k2q_csr(const msa_csr_build_args* args, void* stream);

/* ---------------------------------------------------------------------------
 * Stage 3 (decode): paged FP8 sparse decode, split-KV + combine.
 * Replaces `run_<variant>` in SparseAttnMode::Sparse for q_len <= 32
 * (python/fmha_sm100/csrc/include/sm100_fmha_load_tma_warpspecialized.hpp:529-568)
 * with its `reduction` step (python/fmha_sm100/csrc/fmha_sm100_reduction.cu:40-89),
 * and the split-KV FP8 decode of `SparseDecodePagedAttentionWrapper.run`
 * (python/fmha_sm100/cute/interface.py:1336-1423).
 */
typedef struct msa_decode_args {
  const void* q;                   /* bf16 [num_tokens, num_qo_heads, 128] */
  const void* k;                   /* e4m3 [num_pages, num_kv_heads, 128, 128] */
  const void* v;
  void* out;                       /* bf16 [num_tokens, num_qo_heads, 128] */
  float* lse;                      /* float32 [num_tokens, num_qo_heads] or NULL */
  const int32_t* kv_indices;       /* flat physical page table */
  const int32_t* kv_page_indptr;   /* [batch + 1] */
  const int32_t* kv_block_indexes; /* [num_tokens, num_kv_heads, topk] request-local page ids, -1 tail */
  const int32_t* token_request;    /* [num_tokens] request of each token */
  const int32_t* token_pos;        /* [num_tokens] last visible key position (min(i + qo_offset, kv_len - 1)) */
  int32_t num_tokens, num_qo_heads, num_kv_heads, topk;
  int32_t num_splits;              /* >= 1, <= topk */
  float sm_scale, qk_scale, v_scale;
  void* workspace;                 /* msa_decode_workspace_bytes(...) bytes when num_splits > 1 */
  size_t workspace_bytes;
  int64_t num_pages;               /* pages in the K/V pool (first dimension of k and v) */
  int32_t* status;                 /* device int32 or NULL; receives MSA_ERR_TIMEOUT if a bounded wait ran out */
} msa_decode_args;

size_t msa_decode_workspace_bytes(int32_t num_tokens, int32_t num_qo_heads, int32_t num_splits);
int msa_decode_fwd(const msa_decode_args* args, void* stream);

/* The same decode with no workspace from the caller and no allocation anywhere: `workspace` and
 * `workspace_bytes` are ignored and the split-KV partials go to a fixed 16 MiB array inside the library
 * (one copy per device).  No counterpart in the reference, whose Python caller always owns a torch workspace;
 * it is for callers that cannot allocate at call time -- a serving loop whose memory pool is frozen once the
 * model is loaded, or a host binding (cgo, JNI, a C plugin) with no device allocator of its own to size a
 * buffer that grows with the batch.
 *   - Limit: msa_decode_workspace_bytes(num_tokens, num_qo_heads, num_splits) <= MSA_DECODE_STATIC_SCRATCH_BYTES
 *     (num_tokens * num_qo_heads * num_splits <= 32263); beyond it the call returns MSA_ERR_TOO_LARGE and
 *     launches nothing.
 *   - The first call on each device, made with that device current, looks up the array's device address
 *     (and, like msa_decode_fwd, sets the kernels' attributes); make it once before any stream capture.
 *   - All calls on a device share the one array.  Nothing in it has to be cleared: a call writes every slot
 *     before reading it.  Two calls that can overlap (different streams, or two host threads) race on it;
 *     keep them on one stream or order them with events. */
#define MSA_DECODE_STATIC_SCRATCH_BYTES ((size_t)16 << 20)
int msa_decode_fwd_static(const msa_decode_args* args, void* stream);

/* ---------------------------------------------------------------------------
 * KV-cache append: quantise new BF16 K/V rows and scatter them into the paged cache.
 * Stands in for the reference's cache-side quantisers, which run as PyTorch / Transformer Engine calls:
 * per-tensor FP8 (python/fmha_sm100/cute/test_sparse_atten.py:1229-1235 quantises with scale = amax / 448)
 * and NVFP4 with 128x4-tiled block scales (python/fmha_sm100/cute/quantize.py:93-142 swizzle, :145-159 global
 * scale, :162-232 quantize_bf16_to_nvfp4_128x4; scale row = (page * Hkv + head) * 128 + token-in-page,
 * python/fmha_sm100/cute/src/sm100/fwd/atten_fwd_nvfp4_kv.py:1329-1336).
 *
 * k_new / v_new: bf16 [num_tokens, num_kv_heads, 128], 16-byte aligned.
 * slots: int32 [num_tokens], physical_page * 128 + position-in-page of each token; a negative or out-of-range
 *        slot skips the token.  Two tokens must not share a slot.
 * MSA_KV_FP8_E4M3: k_cache / v_cache uint8 [num_pages, num_kv_heads, 128, 128]; value = e4m3_rne(x * (1 / scale))
 *               saturating at +-448, with k_scale / v_scale the per-tensor DEQUANT scales (x ~= code * scale).
 * MSA_KV_NVFP4: k_cache / v_cache uint8 [num_pages, num_kv_heads, 128, 64] (low nibble = even element);
 *               k_block_scales / v_block_scales uint8 e4m3 in 128x4 tiles over [num_pages * num_kv_heads * 128, 8];
 *               k_scale / v_scale the float32 global scales g.  Arithmetic (float32, round-to-nearest-even):
 *               s = e4m3(min(amax16 / (6 g), 448)); code = e2m1(x * (1 / (s g))) saturating at 6 (x when s == 0).
 * At most 2^31 - 1 (token, head, 16-element block) units per call, else MSA_ERR_TOO_LARGE.
 * Asynchronous on `stream`; allocates nothing. */
typedef struct msa_kv_append_args {
  uint32_t struct_size; /* sizeof(msa_kv_append_args) */
  int32_t format;       /* MSA_KV_FP8_E4M3 or MSA_KV_NVFP4 */
  const void* k_new;
  const void* v_new;
  void* k_cache;
  void* v_cache;
  void* k_block_scales; /* NVFP4 only */
  void* v_block_scales; /* NVFP4 only */
  const int32_t* slots;
  int32_t num_tokens;
  int32_t num_kv_heads;
  int32_t head_dim; /* 128 */
  int32_t num_pages;
  float k_scale;
  float v_scale;
} msa_kv_append_args;
int msa_kv_append(const msa_kv_append_args* args, void* stream);

/* max |x| over a BF16 tensor of n elements (16-byte aligned), folded into *out (device float32, set to 0 by the
 * caller) -- the amax from which the per-tensor FP8 scale (amax / 448) and the NVFP4 global scale
 * (amax / (448 * 6), python/fmha_sm100/cute/quantize.py:145-159) are taken. */
int msa_absmax_bf16(const void* x, int64_t n, float* out, void* stream);

/* ---------------------------------------------------------------------------
 * Tensor-core plumbing self-test: S = Q K^T and O = P V on one 128x128x128 tile
 * each through the same TMA / tcgen05 / TMEM path the attention kernel uses.
 * q, k, v, p: bf16 [128, 128] row-major; s_out, o_out: float32 [128, 128].
 * No counterpart in the reference (diagnostic only). */
int msa_umma_selftest(const void* q, const void* k, const void* v, const void* p, float* s_out, float* o_out,
                      int32_t* status, void* stream);

/* The same kernel with its operand loads withheld, so that its first bounded wait runs out after `wait_cycles`
 * GPU clock cycles (<= 0 or above the library's limit: the library's limit): every later step is skipped, TMEM
 * is released, the kernel returns normally and *status reads MSA_ERR_TIMEOUT.  This is how the timeout path
 * every kernel of the library shares (bounded mbarrier wait -> CTA-wide abort flag -> teardown -> status word)
 * is exercised without faulting or hanging anything; the outputs are left untouched.  No counterpart in the
 * reference, whose waits are unbounded. */
int msa_umma_selftest_timeout(const void* q, const void* k, const void* v, const void* p, float* s_out,
                              float* o_out, int32_t* status, int64_t wait_cycles, void* stream);

/* Role cycle accounting for the attention kernel: int64 [n_ctas, 16] device buffer, or NULL to stop.
 * Only libraries built with -DMSA_ROLE_TIMING write to it (the default build ignores it).  Stands in for the
 * reference's GPU_TRACE / SM_TIMING builds (python/fmha_sm100/csrc/include/gpu_trace.h). */
void msa_debug_set_timing_buffer(void* buffer);

#ifdef __cplusplus
}
#endif
#endif /* MSA_B200_H_ */
