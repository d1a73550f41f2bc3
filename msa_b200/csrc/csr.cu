// k2q CSR -> per-query page lists.
//
// The reference executes its sparse prefill KV-outer and therefore takes the reverse index: for every
// (KV head, KV block row) the ascending list of queries that selected it (build_k2q_csr,
// python/fmha_sm100/cute/sparse_index_utils.py:331; rows packed block-major, :176-192).  The attention
// kernel of this library is query-stationary and walks each query's own ascending page list, so the
// CSR-driven entry points (sparse_atten_func, python/fmha_sm100/cute/interface.py:600) turn the CSR back
// into kv_block_indexes[total_q, Hkv, topk] first, on the device:
//   1. one warp per CSR row appends the row's block id to the list of every query in the row (slot from
//      an atomic counter per (query, head));
//   2. one thread per (query, head) sorts its <= topk entries ascending and pads the tail with -1, which
//      makes the result independent of the order the atomics happened in.
#include "msa_internal.h"

namespace msa {

__global__ void __launch_bounds__(256) csr_scatter_kernel(const int* __restrict__ row_ptr, const int* __restrict__ q_idx,
                                                         const int* __restrict__ row_request,
                                                         const int* __restrict__ row_block,
                                                         const int* __restrict__ cu_seqlens_q, int n_rows,
                                                         long long row_ptr_stride, long long q_idx_stride, int H,
                                                         int topk, int* __restrict__ counters, int* __restrict__ out) {
  const int h = blockIdx.y;
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= n_rows) return;
  const int* rp = row_ptr + h * row_ptr_stride;
  const int e0 = __ldg(rp + row), e1 = __ldg(rp + row + 1);
  const int q0 = __ldg(cu_seqlens_q + __ldg(row_request + row));
  const int blk = __ldg(row_block + row);
  const int* qi = q_idx + h * q_idx_stride;
  for (int e = e0 + lane; e < e1; e += 32) {
    const int ql = __ldg(qi + e);
    if (ql < 0) continue;
    const long long qh = static_cast<long long>(q0 + ql) * H + h;
    const int slot = atomicAdd(counters + qh, 1);
    if (slot < topk) out[qh * topk + slot] = blk;
  }
}

template <int TOPK>
__global__ void __launch_bounds__(256) csr_finish_kernel(const int* __restrict__ counters, long long n_lists,
                                                        int* __restrict__ out) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n_lists) return;
  const int n = min(__ldg(counters + i), TOPK);
  int* l = out + i * TOPK;
  int v[TOPK];
#pragma unroll
  for (int e = 0; e < TOPK; ++e) v[e] = e < n ? l[e] : 0x7fffffff;
  // odd-even transposition sort: fixed register indices, TOPK rounds
#pragma unroll
  for (int r = 0; r < TOPK; ++r) {
#pragma unroll
    for (int e = r & 1; e + 1 < TOPK; e += 2) {
      const int a = v[e], b = v[e + 1];
      v[e] = min(a, b);
      v[e + 1] = max(a, b);
    }
  }
#pragma unroll
  for (int e = 0; e < TOPK; ++e) l[e] = e < n ? v[e] : -1;
}

int k2q_csr_to_lists(const int* row_ptr, const int* q_indices, const int* row_request, const int* row_block,
                     const int* cu_seqlens_q, int num_kv_heads, int n_rows, int64_t row_ptr_stride,
                     int64_t q_indices_stride, int64_t total_q, int topk, int* counters, int* out, cudaStream_t st) {
  if (row_ptr == nullptr || q_indices == nullptr || row_request == nullptr || row_block == nullptr ||
      cu_seqlens_q == nullptr || counters == nullptr || out == nullptr)
    return MSA_ERR_INVALID;
  if (num_kv_heads <= 0 || num_kv_heads > 65535 || n_rows < 0 || total_q < 0) return MSA_ERR_INVALID;
  if (topk != 4 && topk != 8 && topk != 16 && topk != 32 && topk != 64) return MSA_ERR_UNSUPPORTED;
  const long long n_lists = static_cast<long long>(total_q) * num_kv_heads;
  if (n_lists == 0) return MSA_OK;
  if (n_lists > 0x7fffffffLL * 64) return MSA_ERR_TOO_LARGE;
  cudaError_t e = cudaMemsetAsync(counters, 0, static_cast<size_t>(n_lists) * sizeof(int), st);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (n_rows > 0) {
    dim3 grid((n_rows + 7) / 8, num_kv_heads);
    csr_scatter_kernel<<<grid, 256, 0, st>>>(row_ptr, q_indices, row_request, row_block, cu_seqlens_q, n_rows,
                                             row_ptr_stride, q_indices_stride, num_kv_heads, topk, counters, out);
    e = cudaGetLastError();
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  const unsigned blocks = static_cast<unsigned>((n_lists + 255) / 256);
  switch (topk) {
    case 4: csr_finish_kernel<4><<<blocks, 256, 0, st>>>(counters, n_lists, out); break;
    case 8: csr_finish_kernel<8><<<blocks, 256, 0, st>>>(counters, n_lists, out); break;
    case 16: csr_finish_kernel<16><<<blocks, 256, 0, st>>>(counters, n_lists, out); break;
    case 32: csr_finish_kernel<32><<<blocks, 256, 0, st>>>(counters, n_lists, out); break;
    default: csr_finish_kernel<64><<<blocks, 256, 0, st>>>(counters, n_lists, out); break;
  }
  return static_cast<int>(cudaGetLastError());
}

}  // namespace msa
