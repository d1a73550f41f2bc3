// extern "C" surface of libmsa_b200.so (declared in include/msa_b200.h).
#include "msa_internal.h"

extern "C" {

int msa_abi_version(void) { return 4; }

const char* msa_error_string(int code) {
  switch (code) {
    case MSA_OK: return "ok";
    case MSA_ERR_INVALID: return "invalid argument";
    case MSA_ERR_UNSUPPORTED: return "unsupported shape or dtype";
    case MSA_ERR_TIMEOUT: return "device-side wait timed out";
    case MSA_ERR_DRIVER: return "CUDA driver entry point or tensor map encode failed";
    case MSA_ERR_TOO_LARGE: return "size beyond the supported maximum";
    case MSA_ERR_BOUNDS: return "a page-table entry outside the K/V page pool reached a kernel";
    case MSA_EVAL_Q_ROWS: return "sum(qo_segment_lens) != q.shape[0]";
    case MSA_EVAL_KV_ROWS: return "sum(kv_segment_lens) != k.shape[0]";
    case MSA_EVAL_PAGE_TABLE_LENGTH: return "kv_indices length != sum(ceil(kv_segment_lens / page_size))";
    case MSA_EVAL_PAGE_TABLE_RANGE: return "kv_indices has values outside the page pool";
    case MSA_EVAL_LIST_SHAPE: return "kv_block_indexes must be [total_q, num_kv_heads | num_qo_heads, topk]";
    case MSA_EVAL_LIST_NEGATIVE: return "kv_block_indexes must contain only non-negative indices or -1";
    case MSA_EVAL_LIST_PADDING: return "kv_block_indexes: -1 padding must be at the end";
    case MSA_EVAL_LIST_RANGE: return "kv_block_indexes: index out of range for batch page count";
    case MSA_EVAL_LIST_ORDER: return "kv_block_indexes: must be strictly ascending";
    default: return code > 0 ? "CUDA runtime error" : "unknown error";
  }
}

int msa_plan_sizes(const msa_plan_desc* desc, int32_t* n_work, int64_t* total_q, int64_t* total_pages) {
  return msa::plan_sizes(desc, n_work, total_q, total_pages);
}

int msa_plan(const msa_plan_desc* desc, int32_t* work, int32_t* kv_page_indptr, int32_t* token_request,
             int32_t* token_pos, int32_t* num_splits) {
  return msa::plan(desc, work, kv_page_indptr, token_request, token_pos, num_splits);
}

int msa_validate_inputs(const msa_validate_args* args, int64_t* where) { return msa::validate_inputs(args, where); }

int msa_k2q_csr_to_lists(const int32_t* row_ptr, const int32_t* q_indices, const int32_t* row_request,
                         const int32_t* row_block, const int32_t* cu_seqlens_q, int32_t num_kv_heads,
                         int32_t n_rows, int64_t row_ptr_stride, int64_t q_indices_stride, int64_t total_q,
                         int32_t topk, int32_t* counters, int32_t* out, void* stream) {
  return msa::k2q_csr_to_lists(row_ptr, q_indices, row_request, row_block, cu_seqlens_q, num_kv_heads, n_rows,
                               row_ptr_stride, q_indices_stride, total_q, topk, counters, out,
                               static_cast<cudaStream_t>(stream));
}

size_t msa_build_k2q_csr_workspace_bytes(int32_t num_kv_heads, int32_t n_chunks, int32_t max_blocks,
                                         int32_t total_rows) {
  return msa::build_k2q_csr_workspace_bytes(num_kv_heads, n_chunks, max_blocks, total_rows);
}

int msa_build_k2q_csr(const msa_csr_build_args* args, void* stream) {
  return msa::build_k2q_csr(args, static_cast<cudaStream_t>(stream));
}

int msa_topk_select(const float* max_score, int32_t num_heads, int32_t max_k_tiles, int32_t total_q, int32_t topk,
                    int32_t num_valid_pages, int32_t force_begin, int32_t force_end, int32_t* out, void* stream) {
  return msa::topk_select(max_score, num_heads, max_k_tiles, total_q, topk, num_valid_pages, force_begin, force_end,
                          out, static_cast<cudaStream_t>(stream));
}

int msa_block_max(const float* max_score, int32_t num_heads, int32_t max_k_tiles, int32_t total_q,
                  const int32_t* block_starts, int32_t n_blocks, float* out, void* stream) {
  return msa::block_max(max_score, num_heads, max_k_tiles, total_q, block_starts, n_blocks, out,
                        static_cast<cudaStream_t>(stream));
}

int msa_expand_block_lists(const int32_t* block_lists, const int32_t* block_starts, int32_t n_blocks,
                           int32_t num_heads, int32_t topk, int32_t* out, void* stream) {
  return msa::expand_block_lists(block_lists, block_starts, n_blocks, num_heads, topk, out,
                                 static_cast<cudaStream_t>(stream));
}

int msa_fp4_dequant_rows(const void* packed, const void* scales, int32_t format, int32_t scale_layout, int64_t rows,
                         int32_t heads, void* out, void* stream) {
  return msa::fp4_dequant_rows(packed, scales, format, scale_layout, rows, heads, out,
                               static_cast<cudaStream_t>(stream));
}

int msa_fp4_reorder_scales(const void* src, int32_t format, int64_t mn, int64_t l_extent, int32_t k_layout, void* dst,
                           void* stream) {
  return msa::fp4_reorder_scales(src, format, mn, l_extent, k_layout, dst, static_cast<cudaStream_t>(stream));
}

int msa_list_uniformity(const int32_t* work, int32_t n_work, const int32_t* kv_block_indexes, int32_t list_heads,
                        int32_t topk, uint8_t* flags, void* stream) {
  return msa::list_uniformity(work, n_work, kv_block_indexes, list_heads, topk, flags,
                              static_cast<cudaStream_t>(stream));
}

int msa_fmha_fwd(const msa_fmha_args* args, void* stream) {
  return msa::fmha_fwd(args, static_cast<cudaStream_t>(stream));
}

int msa_fmha_combine(const void* partial_out, const float* partial_lse, int32_t n_splits, int64_t total_q,
                     int32_t num_qo_heads, void* out, float* lse, void* stream) {
  return msa::fmha_combine(partial_out, partial_lse, n_splits, total_q, num_qo_heads, out, lse,
                           static_cast<cudaStream_t>(stream));
}

size_t msa_decode_workspace_bytes(int32_t num_tokens, int32_t num_qo_heads, int32_t num_splits) {
  return msa::decode_workspace_bytes(num_tokens, num_qo_heads, num_splits);
}

int msa_decode_fwd(const msa_decode_args* args, void* stream) {
  return msa::decode_fwd(args, static_cast<cudaStream_t>(stream));
}

int msa_decode_fwd_static(const msa_decode_args* args, void* stream) {
  return msa::decode_fwd_static(args, static_cast<cudaStream_t>(stream));
}

int msa_kv_append(const msa_kv_append_args* args, void* stream) {
  return msa::kv_append(args, static_cast<cudaStream_t>(stream));
}

int msa_absmax_bf16(const void* x, int64_t n, float* out, void* stream) {
  return msa::absmax_bf16(x, n, out, static_cast<cudaStream_t>(stream));
}

void msa_debug_set_timing_buffer(void* buffer) { msa::set_timing_buffer(buffer); }

int msa_umma_selftest(const void* q, const void* k, const void* v, const void* p, float* s_out, float* o_out,
                      int32_t* status, void* stream) {
  return msa::umma_selftest(q, k, v, p, s_out, o_out, status, 0, 0, static_cast<cudaStream_t>(stream));
}

int msa_umma_selftest_timeout(const void* q, const void* k, const void* v, const void* p, float* s_out,
                              float* o_out, int32_t* status, int64_t wait_cycles, void* stream) {
  return msa::umma_selftest(q, k, v, p, s_out, o_out, status, 1, wait_cycles, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
