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

// ---------------------------------------------------------------------------------------------------
// q2k lists -> k2q CSR on the device (build_k2q_csr, python/fmha_sm100/cute/sparse_index_utils.py:331;
// the reference's five-kernel pipeline is python/fmha_sm100/cute/src/sm100/build_k2q_csr/build_k2q_csr.cu).
// Output contract: for every (KV head, CSR row) the batch-local queries that selected the row's block, in
// ASCENDING order, rows packed block-major; unused tail of q_indices = -1.
//
// The ascending order comes from the traversal, not from a sort.  Queries are cut into chunks of 256 that do not
// cross requests; one warp owns a (chunk, head) pair in both passes and walks its entries in (query, slot) order:
//   1. count:   cnt[h][chunk][block] += 1 per entry;
//   2. offsets: per (head, request, block) an exclusive scan over the request's chunks turns the counts into each
//               chunk's first position inside the row, and yields the row length;
//   3. row_ptr: exclusive scan of the row lengths (one CTA per head);
//   4. scatter: the warp re-walks its entries; entries of one step that hit the same block are ranked with
//               match_any (a query names a block at most once, so equal blocks mean different queries, and lane
//               order is query order), the block's running offset is read and advanced by the group's leader.
// ---------------------------------------------------------------------------------------------------
namespace msa {

constexpr int kCsrChunk = 256;

struct CsrBuildParams {
  const int* q2k;            // [H, total_q, topk]
  const int* chunk_request;  // [n_chunks]
  const int* chunk_q0;       // [n_chunks] first global query of the chunk
  const int* chunk_len;      // [n_chunks]
  const int* cu_q;           // [B + 1]
  const int* req_chunk0;     // [B + 1] first chunk of each request
  const int* req_blocks;     // [B] KV blocks (CSR rows) of each request
  const int* row_lut;        // [B, max_blocks] CSR row of (request, block), -1 where the request has no such block
  int* cnt;                  // [H, n_chunks, max_blocks] workspace
  int* row_len;              // [H, total_rows + 1] workspace
  int* row_ptr;              // [H, total_rows + 1]
  int* q_indices;            // [H, q_stride]
  long long total_q, q_stride;
  int H, topk, n_chunks, batch, max_blocks, total_rows;
};

// pass 1 (SCATTER = false) and pass 4 (SCATTER = true): one warp per (chunk, head)
template <bool SCATTER>
__global__ void __launch_bounds__(128) csr_walk_kernel(const CsrBuildParams p) {
  const int c = blockIdx.x * 4 + (threadIdx.x >> 5);
  const int h = blockIdx.y, lane = threadIdx.x & 31;
  if (c >= p.n_chunks) return;
  const int req = __ldg(p.chunk_request + c), q0 = __ldg(p.chunk_q0 + c), len = __ldg(p.chunk_len + c);
  const int nblk = __ldg(p.req_blocks + req);
  const int qbase = __ldg(p.cu_q + req);
  int* cnt = p.cnt + (static_cast<size_t>(h) * p.n_chunks + c) * p.max_blocks;
  const int* src = p.q2k + (static_cast<size_t>(h) * p.total_q + q0) * p.topk;
  const int n_entries = len * p.topk;
  for (int e0 = 0; e0 < n_entries; e0 += 32) {
    const int e = e0 + lane;
    int blk = -1;
    if (e < n_entries) blk = __ldg(src + e);
    const bool valid = blk >= 0 && blk < nblk;
    if (!SCATTER) {
      if (valid) atomicAdd(cnt + blk, 1);
    } else {
      // entries of this step that name the same block: lane order = query order
      const uint32_t active = __ballot_sync(0xffffffffu, valid);
      if (valid) {
        const uint32_t peers = __match_any_sync(active, blk);
        const int rank = __popc(peers & ((1u << lane) - 1u));
        const int first = *(volatile int*)(cnt + blk);             // offset inside the row, so far
        const int row = __ldg(p.row_lut + static_cast<size_t>(req) * p.max_blocks + blk);
        const int pos = __ldg(p.row_ptr + static_cast<size_t>(h) * (p.total_rows + 1) + row) + first + rank;
        p.q_indices[static_cast<size_t>(h) * p.q_stride + pos] = q0 + e / p.topk - qbase;
        __syncwarp(active);                                         // every peer has read the offset
        if (rank == 0) *(volatile int*)(cnt + blk) = first + __popc(peers);
      }
      __syncwarp();
    }
  }
}

// pass 2: thread per (head, request, block), block fastest (coalesced over the block axis of cnt)
__global__ void __launch_bounds__(256) csr_offsets_kernel(const CsrBuildParams p) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long per_head = static_cast<long long>(p.batch) * p.max_blocks;
  if (i >= per_head * p.H) return;
  const int h = static_cast<int>(i / per_head);
  const int req = static_cast<int>((i % per_head) / p.max_blocks), blk = static_cast<int>(i % p.max_blocks);
  if (blk >= __ldg(p.req_blocks + req)) return;
  const int c0 = __ldg(p.req_chunk0 + req), c1 = __ldg(p.req_chunk0 + req + 1);
  int run = 0;
  for (int c = c0; c < c1; ++c) {
    int* slot = p.cnt + (static_cast<size_t>(h) * p.n_chunks + c) * p.max_blocks + blk;
    const int n = *slot;
    *slot = run;
    run += n;
  }
  const int row = __ldg(p.row_lut + static_cast<size_t>(req) * p.max_blocks + blk);
  p.row_len[static_cast<size_t>(h) * (p.total_rows + 1) + row] = run;
}

// pass 3: exclusive scan of the row lengths of one head, 1024 threads, in tiles of 1024 rows
__global__ void __launch_bounds__(1024) csr_row_ptr_kernel(const CsrBuildParams p) {
  __shared__ int warp_sum[32];
  __shared__ int carry;
  const int h = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int* len = p.row_len + static_cast<size_t>(h) * (p.total_rows + 1);
  int* out = p.row_ptr + static_cast<size_t>(h) * (p.total_rows + 1);
  if (tid == 0) carry = 0;
  __syncthreads();
  for (int base = 0; base < p.total_rows; base += 1024) {
    const int r = base + tid;
    const int v = r < p.total_rows ? len[r] : 0;
    int x = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int y = __shfl_up_sync(0xffffffffu, x, o);
      if (lane >= o) x += y;
    }
    if (lane == 31) warp_sum[warp] = x;
    __syncthreads();
    if (warp == 0) {
      int w = warp_sum[lane];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int y = __shfl_up_sync(0xffffffffu, w, o);
        if (lane >= o) w += y;
      }
      warp_sum[lane] = w;
    }
    __syncthreads();
    const int before = carry + (warp > 0 ? warp_sum[warp - 1] : 0) + x - v;
    if (r < p.total_rows) out[r] = before;
    __syncthreads();
    if (tid == 1023) carry = before + v;
    __syncthreads();
  }
  if (tid == 0) out[p.total_rows] = carry;
}

size_t build_k2q_csr_workspace_bytes(int num_kv_heads, int n_chunks, int max_blocks, int total_rows) {
  return (static_cast<size_t>(num_kv_heads) * n_chunks * max_blocks + static_cast<size_t>(num_kv_heads) * (total_rows + 1)) *
         sizeof(int);
}

int build_k2q_csr(const msa_csr_build_args* a, cudaStream_t st) {
  if (a == nullptr || a->q2k == nullptr || a->row_ptr == nullptr || a->q_indices == nullptr || a->workspace == nullptr)
    return MSA_ERR_INVALID;
  if (a->num_kv_heads <= 0 || a->num_kv_heads > 65535 || a->topk <= 0 || a->total_q < 0 || a->n_chunks < 0 ||
      a->batch <= 0 || a->max_blocks <= 0 || a->total_rows < 0)
    return MSA_ERR_INVALID;
  if (a->q_indices_stride < a->total_q * a->topk) return MSA_ERR_INVALID;
  const size_t need = build_k2q_csr_workspace_bytes(a->num_kv_heads, a->n_chunks, a->max_blocks, a->total_rows);
  if (a->workspace_bytes < need) return MSA_ERR_INVALID;
  CsrBuildParams p;
  p.q2k = a->q2k;
  p.chunk_request = a->chunk_request;
  p.chunk_q0 = a->chunk_first_query;
  p.chunk_len = a->chunk_len;
  p.cu_q = a->cu_seqlens_q;
  p.req_chunk0 = a->request_first_chunk;
  p.req_blocks = a->request_blocks;
  p.row_lut = a->row_of_block;
  p.cnt = static_cast<int*>(a->workspace);
  p.row_len = p.cnt + static_cast<size_t>(a->num_kv_heads) * a->n_chunks * a->max_blocks;
  p.row_ptr = a->row_ptr;
  p.q_indices = a->q_indices;
  p.total_q = a->total_q;
  p.q_stride = a->q_indices_stride;
  p.H = a->num_kv_heads;
  p.topk = a->topk;
  p.n_chunks = a->n_chunks;
  p.batch = a->batch;
  p.max_blocks = a->max_blocks;
  p.total_rows = a->total_rows;
  cudaError_t e = cudaMemsetAsync(a->workspace, 0, need, st);
  if (e == cudaSuccess)
    e = cudaMemsetAsync(a->q_indices, 0xff, static_cast<size_t>(a->num_kv_heads) * a->q_indices_stride * sizeof(int), st);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (a->n_chunks > 0 && a->total_rows > 0) {
    dim3 grid((a->n_chunks + 3) / 4, a->num_kv_heads);
    csr_walk_kernel<false><<<grid, 128, 0, st>>>(p);
    const long long n = static_cast<long long>(a->num_kv_heads) * a->batch * a->max_blocks;
    csr_offsets_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, st>>>(p);
    csr_row_ptr_kernel<<<a->num_kv_heads, 1024, 0, st>>>(p);
    csr_walk_kernel<true><<<grid, 128, 0, st>>>(p);
  } else {
    e = cudaMemsetAsync(a->row_ptr, 0, static_cast<size_t>(a->num_kv_heads) * (a->total_rows + 1) * sizeof(int), st);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  return static_cast<int>(cudaGetLastError());
}

}  // namespace msa
