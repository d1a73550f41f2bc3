// Paged FP8 sparse decode: split-KV, HBM-bound.
//
// One CTA = (query token, KV head, split): it walks its share of the pages the
// token selected, every warp owning a 32-key slice of each page and keeping a
// private online-softmax state (flash-decoding inside the CTA), then the four
// warps and, if the row was split, a combine kernel merge (max, sum, O).
//
// K and V pages stay e4m3 all the way into the tensor cores
// (mma.sync m16n8k32 e4m3 x e4m3 -> f32, rows = the query heads of the KV group):
//   * every lane fetches K with 128-bit loads of 16 contiguous head-dim bytes of
//     one key row and feeds the four words straight in as B fragments; the
//     contraction order inside a fragment is free, so Q is laid out to match;
//   * V needs keys along the contraction: lanes fetch 16-byte pieces of four key
//     rows and transpose 4x4 byte blocks with prmt;
//   * Q (bf16) is split into two e4m3 terms per row (q = s * (hi + lo / 16)), which
//     keeps ~7 mantissa bits; P is rounded to e4m3 un-normalised (x256) and the row
//     sum stays fp32, as the reference FP8 kernels do
//     (python/fmha_sm100/cute/test_sparse_atten.py:336-353).
// Causal masking uses original key positions: key page*128+o is visible iff <= pos.
//
// Two memory pipelines.  GQA ratio <= 8 (decode_ring_kernel): persistent CTAs, a producer warp streams whole
// pages through a shared-memory ring with TMA and eight consumer warps take alternate pages.  GQA ratio 9-16
// (decode_kernel): every thread copies the sixteen 16-byte pieces it will consume itself with cp.async into a
// private shared-memory slot, one page ahead of the page being computed, so a warp always has a full 8 KiB
// slice in flight and no thread ever waits on another thread's copy.
#include "common.cuh"
#include "msa_internal.h"

namespace msa {

struct DecodeParams {
  const __nv_bfloat16* q;       // [T, Hq, 128]
  const uint8_t* k;             // [pages, Hkv, 128, 128] e4m3
  const uint8_t* v;
  const int* kv_indices;        // flat page table
  const int* kv_page_indptr;    // [B+1]
  const int* kv_block_indexes;  // [T, Hkv, topk]
  const int* tok_req;           // [T] request of each token
  const int* tok_pos;           // [T] last visible key position of each token
  float* part_o;                // [T, Hq, nsplit, 128]
  float* part_ml;               // [T, Hq, nsplit, 2]  (max in log2 units, sum)
  __nv_bfloat16* out;           // [T, Hq, 128]
  float* lse;                   // [T, Hq] or null
  int T, Hq, Hkv, hr, topk, nsplit, entries_per_split;
  float scale_log2;             // sm_scale * log2(e) * q_scale * k_scale
  float out_scale;              // v_scale * o_scale
};

__device__ __forceinline__ void mma_e4m3(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// same with a zero addend: starts an accumulator chain without first clearing its registers
__device__ __forceinline__ void mma_e4m3_first(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%10, %10, %10, %10};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}
// four floats -> four e4m3 bytes (byte 0 = a)
__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
  uint16_t lo, hi;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(b), "f"(a));
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(d), "f"(c));
  return static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
}
__device__ __forceinline__ float e4m3_to_float(uint32_t byte) {
  uint32_t h2;
  asm("{\n.reg .b16 t;\ncvt.u16.u32 t, %1;\ncvt.rn.f16x2.e4m3x2 %0, t;\n}\n" : "=r"(h2) : "r"(byte));
  return __half2float(__ushort_as_half(static_cast<unsigned short>(h2 & 0xffffu)));
}

template <bool ROWS2>
__global__ void __launch_bounds__(128, ROWS2 ? 2 : 3) decode_kernel(const DecodeParams p) {
  constexpr int NROW = ROWS2 ? 16 : 8;
  __shared__ __align__(16) uint8_t q8[2][16][128];   // [hi/lo][row][d]
  __shared__ float q_rowscale[16];
  __shared__ float red_ml[4][NROW][2];
  // [warp][buffer][piece 0..15][lane] 16-byte slots, 64 KiB; the cross-warp merge reuses it afterwards
  extern __shared__ __align__(16) uint8_t dyn_smem[];
  uint4* stage_buf = reinterpret_cast<uint4*>(dyn_smem);
  float (*red_o)[NROW][128] = reinterpret_cast<float (*)[NROW][128]>(dyn_smem);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int gid = lane >> 2, tig = lane & 3;
  int bid = blockIdx.x;
  const int split = bid % p.nsplit;
  bid /= p.nsplit;
  const int g = bid % p.Hkv;
  const int tok = bid / p.Hkv;
  const int req = p.tok_req[tok];
  const int pos = p.tok_pos[tok];
  const int hr = p.hr;

  // ---- Q: per-row scale, two-term e4m3 split --------------------------------
  for (int row = warp; row < 16; row += 4) {
    float x[4] = {0.f, 0.f, 0.f, 0.f};
    if (row < hr) {
      const uint2 raw = *reinterpret_cast<const uint2*>(p.q + (static_cast<size_t>(tok) * p.Hq + g * hr + row) * 128 +
                                                        lane * 4);
      x[0] = __uint_as_float(raw.x << 16);
      x[1] = __uint_as_float(raw.x & 0xffff0000u);
      x[2] = __uint_as_float(raw.y << 16);
      x[3] = __uint_as_float(raw.y & 0xffff0000u);
    }
    float amax = fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3])));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float qs = amax > 0.f ? amax * (1.0f / 448.0f) : 1.0f;
    const float inv = 1.0f / qs;
    float y[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) y[i] = x[i] * inv;
    const uint32_t hi = pack_e4m3x4(y[0], y[1], y[2], y[3]);
    float rs[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) rs[i] = (y[i] - e4m3_to_float((hi >> (8 * i)) & 0xffu)) * 16.0f;
    const uint32_t lo = pack_e4m3x4(rs[0], rs[1], rs[2], rs[3]);
    *reinterpret_cast<uint32_t*>(&q8[0][row][lane * 4]) = hi;
    *reinterpret_cast<uint32_t*>(&q8[1][row][lane * 4]) = lo;
    if (lane == 0) q_rowscale[row] = qs * p.scale_log2;
  }
  __syncthreads();

  // A fragments: the 16 bytes at d = c2*64 + tig*16 of row gid (and gid+8) feed two k32 steps
  uint4 qa_hi[2], qa_lo[2], qb_hi[2], qb_lo[2];
#pragma unroll
  for (int c2 = 0; c2 < 2; ++c2) {
    qa_hi[c2] = *reinterpret_cast<const uint4*>(&q8[0][gid][c2 * 64 + tig * 16]);
    qa_lo[c2] = *reinterpret_cast<const uint4*>(&q8[1][gid][c2 * 64 + tig * 16]);
    if (ROWS2) {
      qb_hi[c2] = *reinterpret_cast<const uint4*>(&q8[0][gid + 8][c2 * 64 + tig * 16]);
      qb_lo[c2] = *reinterpret_cast<const uint4*>(&q8[1][gid + 8][c2 * 64 + tig * 16]);
    } else {
      qb_hi[c2] = make_uint4(0, 0, 0, 0);
      qb_lo[c2] = make_uint4(0, 0, 0, 0);
    }
  }
  const float rs0 = q_rowscale[gid];
  const float rs1 = ROWS2 ? q_rowscale[gid + 8] : 0.f;

  float o[16][4];
#pragma unroll
  for (int j = 0; j < 16; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

  const int* list = p.kv_block_indexes + (static_cast<size_t>(tok) * p.Hkv + g) * p.topk;
  const int e0 = split * p.entries_per_split;
  const int e1 = min(e0 + p.entries_per_split, p.topk);
  const int page_base = p.kv_page_indptr[req];
  const int n_pages_req = p.kv_page_indptr[req + 1] - page_base;

  // next list entry at or after e whose slice this warp must process, or e1
  auto find_next = [&](int e) {
    for (; e < e1; ++e) {
      const int page = __ldg(list + e);
      if (page < 0) return e1;                               // -1 only at the tail
      if (page >= n_pages_req) continue;
      if (page * 128 + warp * 32 > pos) continue;            // slice fully masked (warp-uniform)
      return e;
    }
    return e1;
  };
  // asynchronous copy of the slice of entry e into buffer b: 8 K pieces then 8 V pieces per thread
  auto issue_copy = [&](int e, int b) {
    const int page = __ldg(list + e);
    const int phys = __ldg(p.kv_indices + page_base + page);
    const size_t tile = (static_cast<size_t>(phys) * p.Hkv + g) * (128 * 128) + static_cast<size_t>(warp) * 32 * 128;
    const uint8_t* kb = p.k + tile;
    const uint8_t* vb = p.v + tile;
    const uint32_t dst = smem_u32(stage_buf + ((warp * 2 + b) * 16) * 32 + lane);
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int c2 = 0; c2 < 2; ++c2) {
        const uint8_t* src = kb + (8 * i + gid) * 128 + c2 * 64 + tig * 16;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + (i * 2 + c2) * 512), "l"(src) : "memory");
      }
#pragma unroll
    for (int sidx = 0; sidx < 8; ++sidx) {
      const int key = (sidx >> 1) * 8 + 2 * tig + (sidx & 1);
      const uint8_t* src = vb + key * 128 + gid * 16;
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + (8 + sidx) * 512), "l"(src) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  int cur = find_next(e0);
  int buf = 0;
  if (cur < e1) issue_copy(cur, 0);
  while (cur < e1) {
    const int nxt = find_next(cur + 1);
    if (nxt < e1) {
      issue_copy(nxt, buf ^ 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    const int key0 = __ldg(list + cur) * 128 + warp * 32;   // first key of my slice
    const uint4* my = stage_buf + ((warp * 2 + buf) * 16) * 32 + lane;
    uint4 kf[4][2], vf[8];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int c2 = 0; c2 < 2; ++c2) kf[i][c2] = my[(i * 2 + c2) * 32];
#pragma unroll
    for (int sidx = 0; sidx < 8; ++sidx) vf[sidx] = my[(8 + sidx) * 32];
    cur = nxt;
    buf ^= 1;

    // ---- S = Q K^T for my 32 keys (4 n-tiles of 8) ---------------------------
    float sc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float ah[4] = {0.f, 0.f, 0.f, 0.f}, al[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c2 = 0; c2 < 2; ++c2) {
        mma_e4m3(ah, qa_hi[c2].x, qb_hi[c2].x, qa_hi[c2].y, qb_hi[c2].y, kf[i][c2].x, kf[i][c2].y);
        mma_e4m3(ah, qa_hi[c2].z, qb_hi[c2].z, qa_hi[c2].w, qb_hi[c2].w, kf[i][c2].z, kf[i][c2].w);
        mma_e4m3(al, qa_lo[c2].x, qb_lo[c2].x, qa_lo[c2].y, qb_lo[c2].y, kf[i][c2].x, kf[i][c2].y);
        mma_e4m3(al, qa_lo[c2].z, qb_lo[c2].z, qa_lo[c2].w, qb_lo[c2].w, kf[i][c2].z, kf[i][c2].w);
      }
      // log2-domain logits; keys 8i+2tig, 8i+2tig+1 of the slice
      const int kpos = key0 + 8 * i + 2 * tig;
      sc[i][0] = (kpos <= pos) ? (ah[0] + al[0] * 0.0625f) * rs0 : -INFINITY;
      sc[i][1] = (kpos + 1 <= pos) ? (ah[1] + al[1] * 0.0625f) * rs0 : -INFINITY;
      sc[i][2] = (ROWS2 && kpos <= pos) ? (ah[2] + al[2] * 0.0625f) * rs1 : -INFINITY;
      sc[i][3] = (ROWS2 && kpos + 1 <= pos) ? (ah[3] + al[3] * 0.0625f) * rs1 : -INFINITY;
    }
    // ---- online softmax (rows gid and gid+8) ----------------------------------
    float t0 = -INFINITY, t1 = -INFINITY;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      t0 = fmaxf(t0, fmaxf(sc[i][0], sc[i][1]));
      t1 = fmaxf(t1, fmaxf(sc[i][2], sc[i][3]));
    }
    t0 = fmaxf(t0, __shfl_xor_sync(0xffffffffu, t0, 1));
    t0 = fmaxf(t0, __shfl_xor_sync(0xffffffffu, t0, 2));
    t1 = fmaxf(t1, __shfl_xor_sync(0xffffffffu, t1, 1));
    t1 = fmaxf(t1, __shfl_xor_sync(0xffffffffu, t1, 2));
    const float n0 = fmaxf(m0, t0), n1 = fmaxf(m1, t1);
    const float b0 = (n0 == -INFINITY) ? 0.f : n0, b1 = (n1 == -INFINITY) ? 0.f : n1;
    const float al0 = fast_exp2(m0 - b0), al1 = fast_exp2(m1 - b1);
    m0 = n0;
    m1 = n1;
    float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      sc[i][0] = fast_exp2(sc[i][0] - b0);
      sc[i][1] = fast_exp2(sc[i][1] - b0);
      sc[i][2] = fast_exp2(sc[i][2] - b1);
      sc[i][3] = fast_exp2(sc[i][3] - b1);
      ps0 += sc[i][0] + sc[i][1];
      ps1 += sc[i][2] + sc[i][3];
    }
    l0 = l0 * al0 + ps0;
    l1 = l1 * al1 + ps1;
    if (__any_sync(0xffffffffu, (al0 != 1.0f) || (ROWS2 && al1 != 1.0f))) {
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        o[j][0] *= al0;
        o[j][1] *= al0;
        o[j][2] *= al1;
        o[j][3] *= al1;
      }
    }
    // P as A fragments (x256 so small probabilities stay normal in e4m3)
    const uint32_t pa0 = pack_e4m3x4(sc[0][0] * 256.f, sc[0][1] * 256.f, sc[1][0] * 256.f, sc[1][1] * 256.f);
    const uint32_t pa2 = pack_e4m3x4(sc[2][0] * 256.f, sc[2][1] * 256.f, sc[3][0] * 256.f, sc[3][1] * 256.f);
    uint32_t pa1 = 0, pa3 = 0;
    if (ROWS2) {
      pa1 = pack_e4m3x4(sc[0][2] * 256.f, sc[0][3] * 256.f, sc[1][2] * 256.f, sc[1][3] * 256.f);
      pa3 = pack_e4m3x4(sc[2][2] * 256.f, sc[2][3] * 256.f, sc[3][2] * 256.f, sc[3][3] * 256.f);
    }
    // ---- O += P V: transpose 4 keys x 4 dims byte blocks into B fragments ------
#pragma unroll
    for (int qd = 0; qd < 4; ++qd) {
      uint32_t w[8];
#pragma unroll
      for (int s = 0; s < 8; ++s) w[s] = qd == 0 ? vf[s].x : qd == 1 ? vf[s].y : qd == 2 ? vf[s].z : vf[s].w;
      const uint32_t a01 = prmt(w[0], w[1], 0x5140), a23 = prmt(w[2], w[3], 0x5140);
      const uint32_t c01 = prmt(w[0], w[1], 0x7362), c23 = prmt(w[2], w[3], 0x7362);
      const uint32_t d01 = prmt(w[4], w[5], 0x5140), d23 = prmt(w[6], w[7], 0x5140);
      const uint32_t f01 = prmt(w[4], w[5], 0x7362), f23 = prmt(w[6], w[7], 0x7362);
      mma_e4m3(o[qd * 4 + 0], pa0, pa1, pa2, pa3, prmt(a01, a23, 0x5410), prmt(d01, d23, 0x5410));
      mma_e4m3(o[qd * 4 + 1], pa0, pa1, pa2, pa3, prmt(a01, a23, 0x7632), prmt(d01, d23, 0x7632));
      mma_e4m3(o[qd * 4 + 2], pa0, pa1, pa2, pa3, prmt(c01, c23, 0x5410), prmt(f01, f23, 0x5410));
      mma_e4m3(o[qd * 4 + 3], pa0, pa1, pa2, pa3, prmt(c01, c23, 0x7632), prmt(f01, f23, 0x7632));
    }
  }

  // ---- merge the four warps ---------------------------------------------------
  __syncthreads();   // the merge buffer aliases the copy slots: every warp must be done reading them
  // row sums live per lane quad: reduce over tig
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  if (tig == 0) {
    red_ml[warp][gid][0] = m0;
    red_ml[warp][gid][1] = l0;
    if (ROWS2) {
      red_ml[warp][gid + 8][0] = m1;
      red_ml[warp][gid + 8][1] = l1;
    }
  }
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    // accumulator column n of n-tile j holds head-dim n*16 + j
    red_o[warp][gid][(2 * tig) * 16 + j] = o[j][0];
    red_o[warp][gid][(2 * tig + 1) * 16 + j] = o[j][1];
    if (ROWS2) {
      red_o[warp][gid + 8][(2 * tig) * 16 + j] = o[j][2];
      red_o[warp][gid + 8][(2 * tig + 1) * 16 + j] = o[j][3];
    }
  }
  __syncthreads();
  const int d = tid;
  for (int row = 0; row < hr; ++row) {
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, red_ml[w][row][0]);
    const float Mb = (M == -INFINITY) ? 0.f : M;
    float L = 0.f, O = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float f = fast_exp2(red_ml[w][row][0] - Mb);
      L += red_ml[w][row][1] * f;
      O += red_o[w][row][d] * f;
    }
    O *= (1.0f / 256.0f);
    const int h = g * hr + row;
    if (p.nsplit == 1) {
      const float inv = L > 0.f ? p.out_scale / L : 0.f;
      p.out[(static_cast<size_t>(tok) * p.Hq + h) * 128 + d] = __float2bfloat16(O * inv);
      if (p.lse != nullptr && d == 0)
        p.lse[static_cast<size_t>(tok) * p.Hq + h] = L > 0.f ? (M + log2f(L)) * 0.6931471805599453f : -INFINITY;
    } else {
      const size_t slot = (static_cast<size_t>(tok) * p.Hq + h) * p.nsplit + split;
      p.part_o[slot * 128 + d] = O;
      if (d == 0) {
        p.part_ml[slot * 2 + 0] = M;
        p.part_ml[slot * 2 + 1] = L;
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------------
// Persistent ring variant (GQA ratio <= 8): one CTA per SM; a producer warp streams the selected K and V
// pages of the CTA's work items through a 5-stage shared-memory ring with TMA (32 KiB per stage, 160 KiB
// in flight per SM -- what the HBM system needs queued to run at full rate), eight consumer warps in two
// groups take alternate pages.  The tiles land in the 128-byte-swizzle image, which makes both fragment
// read patterns (K: 8 rows x 64 B, V: 4 rows x 128 B per warp instruction) bank-conflict free.
// ---------------------------------------------------------------------------------------------------
constexpr int kRingStages = 5;
// Merge buffer column of head-dim d of query row `row`: the 16-byte chunk index is XORed with bits 1-2 of the
// row, which makes the accumulator stores (a lane quad writes four rows at the same head-dims, 16 bytes each)
// and the column-wise reads bank-conflict free.
__device__ __forceinline__ int ring_red_index(int d, int row) { return (((d >> 2) ^ ((row >> 1) & 3)) << 2) | (d & 3); }
struct __align__(1024) DecodeRingSmem {
  uint8_t ring[kRingStages][2][16384];
  float red_o[8][8][128];       // chunk-swizzled: see ring_red_index
  float red_ml[8][8][2];
  uint8_t q8[2][8][128];
  float q_rowscale[8];
  // full[g][s]: stage s holds a page of consumer group g.  One barrier per (group, stage): a group skips the
  // other group's pages, and a parity wait is only sound for a waiter that observes every phase of its barrier
  uint64_t full[2][kRingStages], empty[kRingStages];
  int abort;
};

// 384 threads: warps 0-7 consume, warp 8 produces, warps 9-11 only take part in the register hand-over
// (setmaxnreg works on whole warpgroups): 256 * 216 + 128 * 72 = 384 * 168 registers.
constexpr int kRingThreads = 384, kRingRegsLaunch = 168, kRingRegsConsumer = 216, kRingRegsHelper = 72;
static_assert(256 * kRingRegsConsumer + 128 * kRingRegsHelper == kRingThreads * kRingRegsLaunch, "register budget");

__global__ void __launch_bounds__(kRingThreads, 1)
decode_ring_kernel(const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                   const DecodeParams p, int n_items, int* status) {
  extern __shared__ uint8_t dyn_raw[];
  DecodeRingSmem& sm =
      *reinterpret_cast<DecodeRingSmem*>((reinterpret_cast<uintptr_t>(dyn_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int gid = lane >> 2, tig = lane & 3;
  volatile int* abort_flag = &sm.abort;
  if (tid == 0) {
    for (int s = 0; s < kRingStages; ++s) {
      mbar_init(&sm.full[0][s], 1);
      mbar_init(&sm.full[1][s], 1);
      mbar_init(&sm.empty[s], 4);
    }
    sm.abort = 0;
    mbar_fence_init();
  }
  __syncthreads();
  const int hr = p.hr;

  // the pages of item it that are streamed: list entries of its split that exist and start at or before pos
  auto item_coords = [&](int it, int& tok, int& g, int& split) {
    split = it % p.nsplit;
    it /= p.nsplit;
    g = it % p.Hkv;
    tok = it / p.Hkv;
  };

  // The list entries of one item, 64 at a time (one per lane and round; a split of more than 64 entries is
  // walked in several such chunks): logical page, or -1 when the entry is padding, out of range or entirely
  // beyond the causal position; and its physical page.  Loaded with all lanes at once so that no index load
  // sits in front of a page copy or a softmax step.
  struct ItemPages {
    int page[2], phys[2];
    int tok, g, split, pos;
  };
  const int n_chunks = (p.entries_per_split + 63) >> 6;
  auto load_item_pages = [&](int it, int chunk, bool want_phys) {
    ItemPages ip;
    item_coords(it, ip.tok, ip.g, ip.split);
    const int req = __ldg(p.tok_req + ip.tok);
    ip.pos = __ldg(p.tok_pos + ip.tok);
    const int* list = p.kv_block_indexes + (static_cast<size_t>(ip.tok) * p.Hkv + ip.g) * p.topk;
    const int e0 = ip.split * p.entries_per_split, e1 = min(e0 + p.entries_per_split, p.topk);
    const int page_base = __ldg(p.kv_page_indptr + req);
    const int n_pages_req = __ldg(p.kv_page_indptr + req + 1) - page_base;
#pragma unroll
    for (int rnd = 0; rnd < 2; ++rnd) {
      const int e = e0 + chunk * 64 + rnd * 32 + lane;
      int pg = (e < e1) ? __ldg(list + e) : -1;
      if (pg >= n_pages_req || pg * 128 > ip.pos) pg = -1;
      ip.page[rnd] = pg;
      ip.phys[rnd] = (want_phys && pg >= 0) ? __ldg(p.kv_indices + page_base + pg) : 0;
    }
    return ip;
  };

  if (warp >= 8) {
    setmaxnreg_dec<kRingRegsHelper>();
    if (warp == 8) {
    // ================================ producer ==================================
    if (lane == 0) {
      tma_prefetch_desc(&tmap_k);
      tma_prefetch_desc(&tmap_v);
    }
    uint32_t seq = 0;
    bool ok = true;
    ItemPages nxt;
    if (blockIdx.x < n_items) nxt = load_item_pages(blockIdx.x, 0, true);
    for (int it = blockIdx.x; it < n_items && ok; it += gridDim.x) {
      ItemPages cur = nxt;
      if (it + gridDim.x < n_items) nxt = load_item_pages(it + gridDim.x, 0, true);   // in flight while this item streams
      int n = 0;   // valid pages of the item so far: they go to the consumer groups alternately
      for (int chunk = 0; chunk < n_chunks && ok; ++chunk) {
      if (chunk > 0) cur = load_item_pages(it, chunk, true);
#pragma unroll
      for (int rnd = 0; rnd < 2; ++rnd) {
        uint32_t mask = __ballot_sync(0xffffffffu, cur.page[rnd] >= 0);
        while (mask && ok) {
          const int src = __ffs(mask) - 1;
          mask &= mask - 1;
          const int phys = __shfl_sync(0xffffffffu, cur.phys[rnd], src);
          const int s = seq % kRingStages;
          uint64_t* fullbar = &sm.full[n & 1][s];
          ++n;
          if (lane == 0) {
            ok = mbar_wait(&sm.empty[s], ((seq / kRingStages) & 1) ^ 1, abort_flag);
            if (ok) {
              mbar_expect_tx(fullbar, 32768);
              tma_load_4d(sm.ring[s][0], &tmap_k, fullbar, 0, 0, cur.g, phys);
              tma_load_4d(sm.ring[s][1], &tmap_v, fullbar, 0, 0, cur.g, phys);
            }
          }
          ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
          ++seq;
        }
      }
      }
    }
    if (!ok && lane == 0) {
      const long long t0 = clock64();
      while (clock64() - t0 < (1LL << 22)) {
      }
    }
    }
  } else {
    // ================================ consumers =================================
    setmaxnreg_inc<kRingRegsConsumer>();
    const int grp = warp >> 2, w4 = warp & 3;
    uint32_t seq = 0;
    uint32_t my_phase = 0;   // bit s: parity of my group's next page in stage s
    bool ok = true;
    // my Q row (warp = row) of an item: 4 bf16 per lane
    auto load_q_row = [&](const ItemPages& ip) {
      uint2 raw = make_uint2(0u, 0u);
      if (warp < hr)
        raw = __ldg(reinterpret_cast<const uint2*>(p.q + (static_cast<size_t>(ip.tok) * p.Hq + ip.g * hr + warp) * 128 +
                                                   lane * 4));
      return raw;
    };
    // the page list and the Q row of the next item are fetched while the current item streams
    ItemPages nxt_ip;
    uint2 nxt_q = make_uint2(0u, 0u);
    if (blockIdx.x < n_items) {
      nxt_ip = load_item_pages(blockIdx.x, 0, false);
      nxt_q = load_q_row(nxt_ip);
    }
    for (int it = blockIdx.x; it < n_items; it += gridDim.x) {
      ItemPages ip = nxt_ip;
      const uint2 raw = nxt_q;
      if (it + gridDim.x < n_items) {
        nxt_ip = load_item_pages(it + gridDim.x, 0, false);
        nxt_q = load_q_row(nxt_ip);
      }
      const int tok = ip.tok, g = ip.g, split = ip.split, pos = ip.pos;
      asm volatile("bar.sync 1, 256;" ::: "memory");   // the previous item's merge has finished with q8 / red
      // leave together: a timed-out wait raised the flag before the barrier, so every warp reads the same value
      if (*abort_flag) break;
      ok = true;
      // ---- Q: one row per warp, per-row scale, two-term e4m3 split ------------------
      {
        const int row = warp;
        float x[4];   // rows beyond the group's heads are zero
        x[0] = __uint_as_float(raw.x << 16);
        x[1] = __uint_as_float(raw.x & 0xffff0000u);
        x[2] = __uint_as_float(raw.y << 16);
        x[3] = __uint_as_float(raw.y & 0xffff0000u);
        float amax = fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3])));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        const float qs = amax > 0.f ? amax * (1.0f / 448.0f) : 1.0f;
        const float inv = 1.0f / qs;
        float y[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) y[i] = x[i] * inv;
        const uint32_t hi = pack_e4m3x4(y[0], y[1], y[2], y[3]);
        float rs[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) rs[i] = (y[i] - e4m3_to_float((hi >> (8 * i)) & 0xffu)) * 16.0f;
        const uint32_t lo = pack_e4m3x4(rs[0], rs[1], rs[2], rs[3]);
        *reinterpret_cast<uint32_t*>(&sm.q8[0][row][lane * 4]) = hi;
        *reinterpret_cast<uint32_t*>(&sm.q8[1][row][lane * 4]) = lo;
        if (lane == 0) sm.q_rowscale[row] = qs * p.scale_log2;
      }
      asm volatile("bar.sync 1, 256;" ::: "memory");
      uint4 qa_hi[2], qa_lo[2];
#pragma unroll
      for (int c2 = 0; c2 < 2; ++c2) {
        qa_hi[c2] = *reinterpret_cast<const uint4*>(&sm.q8[0][gid][c2 * 64 + tig * 16]);
        qa_lo[c2] = *reinterpret_cast<const uint4*>(&sm.q8[1][gid][c2 * 64 + tig * 16]);
      }
      const float rs0 = sm.q_rowscale[gid];
      // O^T accumulators: tile m holds head-dims gid * 16 + 2 m (+1) of query rows 2 tig, 2 tig + 1
      float oT[8][4];
#pragma unroll
      for (int j = 0; j < 8; ++j) oT[j][0] = oT[j][1] = oT[j][2] = oT[j][3] = 0.f;
      float m0 = -INFINITY, l0 = 0.f;

      int n = 0;
      for (int chunk = 0; chunk < n_chunks && ok; ++chunk) {
      if (chunk > 0) ip = load_item_pages(it, chunk, false);
#pragma unroll
      for (int rnd = 0; rnd < 2; ++rnd) {
       uint32_t mask = __ballot_sync(0xffffffffu, ip.page[rnd] >= 0);
       while (mask && ok) {
        const int src = __ffs(mask) - 1;
        mask &= mask - 1;
        const int page = __shfl_sync(0xffffffffu, ip.page[rnd], src);
        const uint32_t my_seq = seq++;
        if ((n++ & 1) != grp) continue;                 // the other group's page
        const int s = my_seq % kRingStages;
        ok = mbar_wait(&sm.full[grp][s], (my_phase >> s) & 1u, abort_flag);
        my_phase ^= 1u << s;
        if (!ok) continue;
        // fragments out of the swizzled tiles: chunk c of row r sits at chunk (c ^ (r & 7))
        const uint8_t* kt = sm.ring[s][0] + (w4 * 32) * 128;
        const uint8_t* vt = sm.ring[s][1] + (w4 * 32) * 128;
        const int key0 = page * 128 + w4 * 32;
        if (key0 > pos) {                               // my slice is fully masked (warp-uniform)
          if (lane == 0) mbar_arrive(&sm.empty[s]);
          continue;
        }
        uint4 kf[4][2];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int c2 = 0; c2 < 2; ++c2)
            kf[i][c2] = *reinterpret_cast<const uint4*>(kt + (8 * i + gid) * 128 + (((c2 * 4 + tig) ^ gid) << 4));

        float sc[4][2];
        {
          // The MMA is 16 rows tall and the group has at most 8 query heads: rows 0-7 carry the hi term of Q,
          // rows 8-15 the lo term, so one instruction yields both partial products (c0, c1 = hi, c2, c3 = lo
          // of the same row and keys).  Four independent accumulator chains.
          float acc[4][4];
#pragma unroll
          for (int c2 = 0; c2 < 2; ++c2) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              if (c2 == 0)
                mma_e4m3_first(acc[i], qa_hi[c2].x, qa_lo[c2].x, qa_hi[c2].y, qa_lo[c2].y, kf[i][c2].x, kf[i][c2].y);
              else
                mma_e4m3(acc[i], qa_hi[c2].x, qa_lo[c2].x, qa_hi[c2].y, qa_lo[c2].y, kf[i][c2].x, kf[i][c2].y);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
              mma_e4m3(acc[i], qa_hi[c2].z, qa_lo[c2].z, qa_hi[c2].w, qa_lo[c2].w, kf[i][c2].z, kf[i][c2].w);
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int kpos = key0 + 8 * i + 2 * tig;
            sc[i][0] = (kpos <= pos) ? (acc[i][0] + acc[i][2] * 0.0625f) * rs0 : -INFINITY;
            sc[i][1] = (kpos + 1 <= pos) ? (acc[i][1] + acc[i][3] * 0.0625f) * rs0 : -INFINITY;
          }
        }
        // V fragments only now, when the K fragments are dead: both sets at once do not fit the register budget
        uint4 vf[8];
#pragma unroll
        for (int sidx = 0; sidx < 8; ++sidx) {
          const int key = (sidx >> 1) * 8 + 2 * tig + (sidx & 1);
          vf[sidx] = *reinterpret_cast<const uint4*>(vt + key * 128 + ((gid ^ (key & 7)) << 4));
        }
        float t0 = -INFINITY;
#pragma unroll
        for (int i = 0; i < 4; ++i) t0 = fmaxf(t0, fmaxf(sc[i][0], sc[i][1]));
        t0 = fmaxf(t0, __shfl_xor_sync(0xffffffffu, t0, 1));
        t0 = fmaxf(t0, __shfl_xor_sync(0xffffffffu, t0, 2));
        const float n0 = fmaxf(m0, t0);
        const float b0 = (n0 == -INFINITY) ? 0.f : n0;
        const float al0 = fast_exp2(m0 - b0);
        m0 = n0;
        float ps0 = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          sc[i][0] = fast_exp2(sc[i][0] - b0);
          sc[i][1] = fast_exp2(sc[i][1] - b0);
          ps0 += sc[i][0] + sc[i][1];
        }
        l0 = l0 * al0 + ps0;
        if (__any_sync(0xffffffffu, al0 != 1.0f)) {
          // my accumulators belong to query rows 2 tig and 2 tig + 1, whose factors live in other lanes
          const float fa = __shfl_sync(0xffffffffu, al0, (2 * tig) * 4);
          const float fb = __shfl_sync(0xffffffffu, al0, (2 * tig + 1) * 4);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            oT[j][0] *= fa;
            oT[j][1] *= fb;
            oT[j][2] *= fa;
            oT[j][3] *= fb;
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm.empty[s]);       // registers hold my slice: the stage may be refilled
        const uint32_t pa0 = pack_e4m3x4(sc[0][0] * 256.f, sc[0][1] * 256.f, sc[1][0] * 256.f, sc[1][1] * 256.f);
        const uint32_t pa2 = pack_e4m3x4(sc[2][0] * 256.f, sc[2][1] * 256.f, sc[3][0] * 256.f, sc[3][1] * 256.f);
#pragma unroll
        for (int qd = 0; qd < 4; ++qd) {
          uint32_t w[8];
#pragma unroll
          for (int s2 = 0; s2 < 8; ++s2) w[s2] = qd == 0 ? vf[s2].x : qd == 1 ? vf[s2].y : qd == 2 ? vf[s2].z : vf[s2].w;
          const uint32_t a01 = prmt(w[0], w[1], 0x5140), a23 = prmt(w[2], w[3], 0x5140);
          const uint32_t c01 = prmt(w[0], w[1], 0x7362), c23 = prmt(w[2], w[3], 0x7362);
          const uint32_t d01 = prmt(w[4], w[5], 0x5140), d23 = prmt(w[6], w[7], 0x5140);
          const uint32_t f01 = prmt(w[4], w[5], 0x7362), f23 = prmt(w[6], w[7], 0x7362);
          // O^T += V^T P^T: the 16 rows of a tile are two head-dims per lane group (no padding rows), the 8
          // columns the query rows; the transposed V bytes are the A operand, P of my row and keys the B operand
          mma_e4m3(oT[qd * 2 + 0], prmt(a01, a23, 0x5410), prmt(a01, a23, 0x7632), prmt(d01, d23, 0x5410),
                   prmt(d01, d23, 0x7632), pa0, pa2);
          mma_e4m3(oT[qd * 2 + 1], prmt(c01, c23, 0x5410), prmt(c01, c23, 0x7632), prmt(f01, f23, 0x5410),
                   prmt(f01, f23, 0x7632), pa0, pa2);
        }
       }
      }
      }
      // ---- merge the eight consumer warps --------------------------------------------
      l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
      l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
      if (tig == 0) {
        sm.red_ml[warp][gid][0] = m0;
        sm.red_ml[warp][gid][1] = l0;
      }
#pragma unroll
      for (int e = 0; e < 2; ++e)                                  // query row 2 tig + e, head-dims gid * 16 + [0, 16)
#pragma unroll
        for (int j4 = 0; j4 < 4; ++j4)
          *reinterpret_cast<float4*>(&sm.red_o[warp][2 * tig + e][ring_red_index(gid * 16 + j4 * 4, 2 * tig + e)]) =
              make_float4(oT[2 * j4][e], oT[2 * j4][2 + e], oT[2 * j4 + 1][e], oT[2 * j4 + 1][2 + e]);
      asm volatile("bar.sync 1, 256;" ::: "memory");
      const int d = tid & 127;
      for (int row = tid >> 7; row < hr; row += 2) {
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < 8; ++w) M = fmaxf(M, sm.red_ml[w][row][0]);
        const float Mb = (M == -INFINITY) ? 0.f : M;
        float L = 0.f, O = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) {
          const float f = fast_exp2(sm.red_ml[w][row][0] - Mb);
          L += sm.red_ml[w][row][1] * f;
          O += sm.red_o[w][row][ring_red_index(d, row)] * f;
        }
        O *= (1.0f / 256.0f);
        const int h = g * hr + row;
        if (p.nsplit == 1) {
          const float inv = L > 0.f ? p.out_scale / L : 0.f;
          p.out[(static_cast<size_t>(tok) * p.Hq + h) * 128 + d] = __float2bfloat16(O * inv);
          if (p.lse != nullptr && d == 0)
            p.lse[static_cast<size_t>(tok) * p.Hq + h] = L > 0.f ? (M + log2f(L)) * 0.6931471805599453f : -INFINITY;
        } else {
          const size_t slot = (static_cast<size_t>(tok) * p.Hq + h) * p.nsplit + split;
          p.part_o[slot * 128 + d] = O;
          if (d == 0) {
            p.part_ml[slot * 2 + 0] = M;
            p.part_ml[slot * 2 + 1] = L;
          }
        }
      }
    }
  }
  __syncthreads();
  if (tid == 0 && sm.abort && status != nullptr) atomicExch(status, MSA_ERR_TIMEOUT);
}

// merge the splits of one (token, head): grid = T * Hq, block = 128 (one thread per head-dim)
__global__ void __launch_bounds__(128) decode_combine_kernel(const float* __restrict__ part_o,
                                                            const float* __restrict__ part_ml, int nsplit,
                                                            float out_scale, __nv_bfloat16* __restrict__ out,
                                                            float* __restrict__ lse) {
  const size_t row = blockIdx.x;
  const int d = threadIdx.x;
  float M = -INFINITY;
  for (int s = 0; s < nsplit; ++s) M = fmaxf(M, part_ml[(row * nsplit + s) * 2]);
  const float Mb = (M == -INFINITY) ? 0.f : M;
  float L = 0.f, O = 0.f;
  for (int s = 0; s < nsplit; ++s) {
    const float f = fast_exp2(part_ml[(row * nsplit + s) * 2] - Mb);
    L += part_ml[(row * nsplit + s) * 2 + 1] * f;
    O += part_o[(row * nsplit + s) * 128 + d] * f;
  }
  const float inv = L > 0.f ? out_scale / L : 0.f;
  out[row * 128 + d] = __float2bfloat16(O * inv);
  if (lse != nullptr && d == 0) lse[row] = L > 0.f ? (M + log2f(L)) * 0.6931471805599453f : -INFINITY;
}

size_t decode_workspace_bytes(int n_tokens, int num_qo_heads, int num_splits) {
  if (num_splits <= 1) return 0;
  return static_cast<size_t>(n_tokens) * num_qo_heads * num_splits * (128 + 2) * sizeof(float);
}

int decode_launch(const msa_decode_args* a, float* part_o, float* part_ml, cudaStream_t st) {
  DecodeParams p;
  p.q = static_cast<const __nv_bfloat16*>(a->q);
  p.k = static_cast<const uint8_t*>(a->k);
  p.v = static_cast<const uint8_t*>(a->v);
  p.kv_indices = a->kv_indices;
  p.kv_page_indptr = a->kv_page_indptr;
  p.kv_block_indexes = a->kv_block_indexes;
  p.tok_req = a->token_request;
  p.tok_pos = a->token_pos;
  p.part_o = part_o;
  p.part_ml = part_ml;
  p.out = static_cast<__nv_bfloat16*>(a->out);
  p.lse = a->lse;
  p.T = a->num_tokens;
  p.Hq = a->num_qo_heads;
  p.Hkv = a->num_kv_heads;
  p.hr = a->num_qo_heads / a->num_kv_heads;
  p.topk = a->topk;
  p.nsplit = a->num_splits;
  p.entries_per_split = (a->topk + a->num_splits - 1) / a->num_splits;
  p.scale_log2 = a->sm_scale * 1.4426950408889634f * a->qk_scale;
  p.out_scale = a->v_scale;
  const long long ctas = static_cast<long long>(p.T) * p.Hkv * p.nsplit;
  if (ctas > 0x7fffffffLL) return MSA_ERR_TOO_LARGE;
  constexpr int kDynSmem = 4 * 2 * 16 * 32 * 16;   // 64 KiB of copy slots (>= the 32 KiB merge buffer)
  constexpr int kRingSmem = static_cast<int>(sizeof(DecodeRingSmem)) + 1024;
  static DeviceSetup setup;
  int num_sms = 0;
  const int src = setup.ensure(&num_sms, [] {
    cudaError_t e1 = cudaFuncSetAttribute(decode_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kDynSmem);
    if (e1 != cudaSuccess) return static_cast<int>(e1);
    e1 = cudaFuncSetAttribute(decode_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kDynSmem);
    if (e1 != cudaSuccess) return static_cast<int>(e1);
    e1 = cudaFuncSetAttribute(decode_ring_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kRingSmem);
    if (e1 != cudaSuccess) return static_cast<int>(e1);
    // the in-kernel register hand-over only balances if the CTA starts with exactly kRingRegsLaunch per thread
    cudaFuncAttributes fa;
    e1 = cudaFuncGetAttributes(&fa, decode_ring_kernel);
    if (e1 != cudaSuccess) return static_cast<int>(e1);
    if (fa.numRegs != kRingRegsLaunch) return static_cast<int>(MSA_ERR_UNSUPPORTED);
    return static_cast<int>(MSA_OK);
  });
  if (src != MSA_OK) return src;
  if (p.hr <= 8 && a->num_pages > 0) {
    // persistent ring kernel: one CTA per SM over the (token, KV head, split) items
    CUtensorMap mk, mv;
    int rc = make_paged_e4m3_map(&mk, a->k, a->num_pages, p.Hkv);
    if (rc == MSA_OK) rc = make_paged_e4m3_map(&mv, a->v, a->num_pages, p.Hkv);
    if (rc != MSA_OK) return rc;
    const int grid = ctas < num_sms ? static_cast<int>(ctas) : num_sms;
    decode_ring_kernel<<<grid, kRingThreads, kRingSmem, st>>>(mk, mv, p, static_cast<int>(ctas), a->status);
  } else if (p.hr <= 8) {
    decode_kernel<false><<<static_cast<unsigned>(ctas), 128, kDynSmem, st>>>(p);
  } else {
    decode_kernel<true><<<static_cast<unsigned>(ctas), 128, kDynSmem, st>>>(p);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return static_cast<int>(e);
  if (p.nsplit > 1) {
    decode_combine_kernel<<<p.T * p.Hq, 128, 0, st>>>(part_o, part_ml, p.nsplit, p.out_scale, p.out, p.lse);
    e = cudaGetLastError();
  }
  return static_cast<int>(e);
}

static int decode_check(const msa_decode_args* a) {
  if (a == nullptr || a->q == nullptr || a->k == nullptr || a->v == nullptr || a->out == nullptr) return MSA_ERR_INVALID;
  if (a->kv_indices == nullptr || a->kv_page_indptr == nullptr || a->kv_block_indexes == nullptr) return MSA_ERR_INVALID;
  if (a->token_request == nullptr || a->token_pos == nullptr) return MSA_ERR_INVALID;
  if (a->num_tokens < 0 || a->num_kv_heads <= 0 || a->num_qo_heads <= 0 || a->topk <= 0) return MSA_ERR_INVALID;
  if (a->num_qo_heads % a->num_kv_heads != 0) return MSA_ERR_INVALID;
  if (a->num_qo_heads / a->num_kv_heads > 16) return MSA_ERR_UNSUPPORTED;
  if (a->num_splits < 1 || a->num_splits > a->topk) return MSA_ERR_INVALID;
  return MSA_OK;
}

int decode_fwd(const msa_decode_args* a, cudaStream_t st) {
  const int c = decode_check(a);
  if (c != MSA_OK) return c;
  if (a->num_tokens == 0) return MSA_OK;
  float* part_o = nullptr;
  float* part_ml = nullptr;
  if (a->num_splits > 1) {
    const size_t need = decode_workspace_bytes(a->num_tokens, a->num_qo_heads, a->num_splits);
    if (a->workspace == nullptr || a->workspace_bytes < need) return MSA_ERR_INVALID;
    part_o = static_cast<float*>(a->workspace);
    part_ml = part_o + static_cast<size_t>(a->num_tokens) * a->num_qo_heads * a->num_splits * 128;
  }
  return decode_launch(a, part_o, part_ml, st);
}

// ---------------------------------------------------------------------------------------------------
// Decode without a caller-supplied workspace: the split-KV partials live in a fixed array of this module.
// For callers that cannot hand over device memory at call time: a serving loop that runs with its memory
// pool frozen, or a host binding in a language whose runtime has no device allocator to size and own a buffer
// whose length depends on the batch.  The array is shared by every call of the process on a device.
// ---------------------------------------------------------------------------------------------------
constexpr size_t kStaticScratchBytes = MSA_DECODE_STATIC_SCRATCH_BYTES;   // 16 MiB: tokens * heads * splits <= 32263
static __device__ __align__(256) unsigned char g_decode_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
static void* g_scratch_addr[kMaxDevices] = {};   // device address of g_decode_scratch, per device ordinal

int decode_fwd_static(const msa_decode_args* a, cudaStream_t st) {
  const int c = decode_check(a);
  if (c != MSA_OK) return c;
  if (a->num_tokens == 0) return MSA_OK;
  const size_t need = decode_workspace_bytes(a->num_tokens, a->num_qo_heads, a->num_splits);
  if (need > kStaticScratchBytes) return MSA_ERR_TOO_LARGE;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= kMaxDevices) return MSA_ERR_UNSUPPORTED;
  if (g_scratch_addr[dev] == nullptr) {
    // set-up, once per device and with that device current: ask the runtime where this device's copy of the
    // array lives (the array's name is not a device address on the host side)
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_decode_scratch);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (ptr == nullptr) return MSA_ERR_DRIVER;
    g_scratch_addr[dev] = ptr;
  }
  float* part_o = nullptr;
  float* part_ml = nullptr;
  if (a->num_splits > 1) {
    // every slot a call reads was written by the same call first (each split writes its partial, an empty
    // split writes max = -inf, sum = 0), so nothing in the array has to start at zero
    part_o = static_cast<float*>(g_scratch_addr[dev]);
    part_ml = part_o + static_cast<size_t>(a->num_tokens) * a->num_qo_heads * a->num_splits * 128;
  }
  return decode_launch(a, part_o, part_ml, st);
}

}  // namespace msa
