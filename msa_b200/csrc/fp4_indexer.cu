// FP4 indexer helpers: what surrounds the score-only kernel when Q and K arrive as packed e2m1 with block scales
// (the contract of fp4_indexer_block_scores, python/fmha_sm100/cute/fp4_indexer_interface.py:745-1056).
//
//   * fp4_dequant_rows: Q [rows, heads, 64 bytes] + block scales -> bf16 [rows, heads, 128].  e2m1 x e4m3 and
//     e2m1 x 2^n are exact in bf16 (at most six significant bits), so the score kernel sees exactly the values
//     the reference's block-scaled MMA multiplies; Q is tiny next to K (one pass, HBM-bound).
//   * fp4_reorder_scales: logical ("public") scale tensors -> the 128x4-tiled storage the MMA-side code reads,
//     the job of Fp4IndexerScaleReorderSm100 (python/fmha_sm100/cute/src/sm100/fp4_indexer.py:83-199): element
//     (row m, group g, batch l) at  l * 512 * restM * restG + (m / 128) * 512 * restG + (g / 4) * 512
//                                   + (m % 32) * 16 + ((m % 128) / 32) * 4 + g % 4.
// K itself is dequantised inside the score kernel (score_kernel.cuh), page by page.
#include <cuda_bf16.h>

#include "msa_internal.h"

namespace msa {
namespace {

__device__ __forceinline__ float e2m1_value(uint32_t code) {
  // sign | 2-bit exponent | 1-bit mantissa: 0, 0.5, 1, 1.5, 2, 3, 4, 6
  const uint32_t mag = code & 7u;
  const float v = mag < 2u ? 0.5f * static_cast<float>(mag)
                           : __uint_as_float(((126u + (mag >> 1)) << 23) | ((mag & 1u) << 22));
  return (code & 8u) ? -v : v;
}

__device__ __forceinline__ float e4m3_value(uint32_t b) {
  const uint32_t e = (b >> 3) & 15u, m = b & 7u;
  float v;
  if (e == 0u) v = static_cast<float>(m) * 0.001953125f;              // subnormal: m * 2^-9
  else if (e == 15u && m == 7u) v = __uint_as_float(0x7fc00000u);     // NaN
  else v = __uint_as_float(((e + 120u) << 23) | (m << 20));
  return (b & 0x80u) ? -v : v;
}

__device__ __forceinline__ float ue8m0_value(uint32_t b) {
  if (b == 255u) return __uint_as_float(0x7fc00000u);
  return b == 0u ? __uint_as_float(0x00400000u) /* 2^-127 */ : __uint_as_float(b << 23);
}

__device__ __forceinline__ int64_t mma_scale_offset(int64_t m, int g, int64_t l, int64_t rest_m, int rest_g) {
  return l * 512 * rest_m * rest_g + (m >> 7) * 512 * rest_g + static_cast<int64_t>(g >> 2) * 512 + (m & 31) * 16 +
         ((m & 127) >> 5) * 4 + (g & 3);
}

// one thread per 16-value block: 8 packed bytes in, 16 bf16 (32 bytes) out
__global__ void __launch_bounds__(256) fp4_dequant_rows_kernel(const uint2* __restrict__ packed,
                                                              const uint8_t* __restrict__ scales, int mx, int mma_layout,
                                                              int64_t rows, int heads, uint4* __restrict__ out) {
  const int64_t blk = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;   // (row, head, block of 16)
  const int64_t n_blk = rows * heads * 8;
  if (blk >= n_blk) return;
  const int b16 = static_cast<int>(blk & 7);
  const int64_t rh = blk >> 3;
  const int head = static_cast<int>(rh % heads);
  const int64_t row = rh / heads;
  const int groups = mx ? 4 : 8, g = mx ? b16 >> 1 : b16;
  const int64_t so = mma_layout ? mma_scale_offset(row, g, head, (rows + 127) >> 7, (groups + 3) >> 2)
                                : rh * groups + g;
  const uint32_t sb = __ldg(scales + so);
  const float s = mx ? ue8m0_value(sb) : e4m3_value(sb);
  const uint2 x = __ldg(packed + blk);
  const uint32_t w[2] = {x.x, x.y};
  uint32_t o[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint32_t byte = (w[i >> 2] >> ((i & 3) * 8)) & 0xffu;
    const __nv_bfloat162 v = __floats2bfloat162_rn(e2m1_value(byte & 15u) * s, e2m1_value(byte >> 4) * s);
    o[i] = *reinterpret_cast<const uint32_t*>(&v);
  }
  out[blk * 2] = make_uint4(o[0], o[1], o[2], o[3]);
  out[blk * 2 + 1] = make_uint4(o[4], o[5], o[6], o[7]);
}

// one thread per scale byte.  k_layout: source [l, m (= 128), G] (K: l = page * heads + head); else [m, l, G] (Q)
__global__ void __launch_bounds__(256) fp4_reorder_scales_kernel(const uint8_t* __restrict__ src, int groups, int64_t mn,
                                                                int64_t l_extent, int k_layout, uint8_t* __restrict__ dst) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= mn * l_extent * groups) return;
  const int g = static_cast<int>(i % groups);
  const int64_t t = i / groups;
  int64_t m, l;
  if (k_layout) {
    m = t % mn;
    l = t / mn;
  } else {
    l = t % l_extent;
    m = t / l_extent;
  }
  dst[mma_scale_offset(m, g, l, (mn + 127) >> 7, (groups + 3) >> 2)] = __ldg(src + i);
}

}  // namespace

int fp4_dequant_rows(const void* packed, const void* scales, int format, int scale_layout, int64_t rows, int heads,
                     void* out, cudaStream_t st) {
  if (packed == nullptr || scales == nullptr || out == nullptr || rows < 0 || heads <= 0) return MSA_ERR_INVALID;
  if ((format != 0 && format != 1) || (scale_layout != 0 && scale_layout != 1)) return MSA_ERR_INVALID;
  const int64_t n_blk = rows * heads * 8;
  if (n_blk == 0) return MSA_OK;
  const int64_t blocks = (n_blk + 255) / 256;
  if (blocks > 0x7fffffffLL) return MSA_ERR_TOO_LARGE;
  fp4_dequant_rows_kernel<<<static_cast<unsigned>(blocks), 256, 0, st>>>(
      static_cast<const uint2*>(packed), static_cast<const uint8_t*>(scales), format, scale_layout, rows, heads,
      static_cast<uint4*>(out));
  return static_cast<int>(cudaGetLastError());
}

int fp4_reorder_scales(const void* src, int format, int64_t mn, int64_t l_extent, int k_layout, void* dst,
                       cudaStream_t st) {
  if (src == nullptr || dst == nullptr || mn < 0 || l_extent < 0 || (format != 0 && format != 1)) return MSA_ERR_INVALID;
  const int groups = format == 1 ? 4 : 8;
  const int64_t n = mn * l_extent * groups;
  if (n == 0) return MSA_OK;
  const int64_t blocks = (n + 255) / 256;
  if (blocks > 0x7fffffffLL) return MSA_ERR_TOO_LARGE;
  fp4_reorder_scales_kernel<<<static_cast<unsigned>(blocks), 256, 0, st>>>(static_cast<const uint8_t*>(src), groups, mn,
                                                                          l_extent, k_layout, static_cast<uint8_t*>(dst));
  return static_cast<int>(cudaGetLastError());
}

}  // namespace msa
