// Internal C++ entry points behind the C ABI (include/msa_b200.h).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

#include "../../include/msa_b200.h"

namespace msa {

// One-time set-up that belongs to a device, not to the process: function attributes
// (cudaFuncSetAttribute applies to the current device only) and the SM count.  Keyed by the ordinal
// of the device that is current at the call, so a process that drives several GPUs, or several host
// threads on one GPU, gets each device configured exactly once.
class DeviceSetup {
 public:
  static constexpr int kMaxDevices = 64;
  // Runs configure() -> int (MSA_OK or an error code) the first time the current device is seen by this
  // object and stores the device's SM count in *num_sms (if not null).
  template <class F>
  int ensure(int* num_sms, F&& configure) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (dev < 0 || dev >= kMaxDevices) return MSA_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> guard(mu_);
    if (!done_[dev]) {
      const int rc = configure();
      if (rc != MSA_OK) return rc;
      e = cudaDeviceGetAttribute(&sms_[dev], cudaDevAttrMultiProcessorCount, dev);
      if (e != cudaSuccess) return static_cast<int>(e);
      done_[dev] = true;
    }
    if (num_sms != nullptr) *num_sms = sms_[dev];
    return MSA_OK;
  }

 private:
  std::mutex mu_;
  bool done_[kMaxDevices] = {};
  int sms_[kMaxDevices] = {};
};

int topk_select(const float* ms, int H, int K, int T, int topk, int nvp, int fb, int fe, int* out, cudaStream_t st);
int block_max(const float* ms, int H, int K, int T, const int* block_starts, int n_blocks, float* out,
              cudaStream_t st);
int expand_block_lists(const int* lists, const int* block_starts, int n_blocks, int H, int topk, int* out,
                       cudaStream_t st);
int fmha_fwd(const msa_fmha_args* a, cudaStream_t st);
void set_timing_buffer(void* ptr);
int fmha_combine(const void* partial_out, const float* partial_lse, int n_splits, int64_t total_q, int num_qo_heads,
                 void* out, float* lse, cudaStream_t st);
int fp4_dequant_rows(const void* packed, const void* scales, int format, int scale_layout, int64_t rows, int heads,
                     void* out, cudaStream_t st);
int fp4_reorder_scales(const void* src, int format, int64_t mn, int64_t l_extent, int k_layout, void* dst,
                       cudaStream_t st);
int list_uniformity(const int32_t* work, int n_work, const int32_t* lists, int list_heads, int topk, uint8_t* flags,
                    cudaStream_t st);
// 4-D TMA map over paged e4m3 K or V [pages, Hkv, 128, 128]: one 128x128-byte box per (page, head), 128-byte swizzle
int make_paged_e4m3_map(void* tensor_map, const void* kv, int64_t pages, int hkv);
// 3-D TMA map over a float32 score tensor [H, K, T] (T innermost): boxes of box_k pages x box_t tokens
int make_score_map(void* tensor_map, const float* ms, int H, int K, int T, int box_t, int box_k);
int umma_selftest(const void* q, const void* k, const void* v, const void* p, float* s_out, float* o_out,
                  int* status, int skip_loads, long long wait_cycles, cudaStream_t st);
int decode_fwd(const msa_decode_args* a, cudaStream_t st);
size_t decode_workspace_bytes(int n_tokens, int num_qo_heads, int num_splits);
int decode_fwd_static(const msa_decode_args* a, cudaStream_t st);
int kv_append(const msa_kv_append_args* a, cudaStream_t st);
int absmax_bf16(const void* x, int64_t n, float* out, cudaStream_t st);
int plan_sizes(const msa_plan_desc* d, int32_t* n_work, int64_t* total_q, int64_t* total_pages);
int plan(const msa_plan_desc* d, int32_t* work, int32_t* kv_page_indptr, int32_t* token_request, int32_t* token_pos,
         int32_t* num_splits);
int validate_inputs(const msa_validate_args* a, int64_t* where);
size_t build_k2q_csr_workspace_bytes(int num_kv_heads, int n_chunks, int max_blocks, int total_rows);
int build_k2q_csr(const msa_csr_build_args* a, cudaStream_t st);
int k2q_csr_to_lists(const int* row_ptr, const int* q_indices, const int* row_request, const int* row_block,
                     const int* cu_seqlens_q, int num_kv_heads, int n_rows, int64_t row_ptr_stride,
                     int64_t q_indices_stride, int64_t total_q, int topk, int* counters, int* out, cudaStream_t st);

}  // namespace msa
