// Score-only pass on sm_100a: per-page maxima of Q K^T (stage 1 of the sparse pipeline, the "proxy" pass), the
// mode OnlyScore of the reference's FMHA kernel
// (csrc/include/sm100_fmha_fwd_mainloop_tma_warpspecialized.hpp:842-1109, reached from
// fmha_sm100(..., output_o=False, output_maxscore=True), python/fmha_sm100/api.py:1028).
//
// A kernel of its own because nothing of the attention kernel's structure fits it: there is no P, no V and no O.
// The pass has little arithmetic per K byte (one 128 x 128 product per 16 KiB page and query tile), so with one query
// tile per CTA the 148 SMs ask the L2 for more than it delivers; and one row maximum per (query row, page) is so
// little work that the hand-over between the MMA-issuing thread and the warps that read S bounds the loop.  Hence:
//
//   work item  256 query rows of one head (two 128-row tiles) against the pages its last row can see: every K
//              page is fetched once for two tiles
//   warp 8     producer: Q tiles of the item (of the NEXT item into the other buffer where shared memory allows
//              two), K pages two at a time into a ring of page PAIRS (the two pages of a pair lie back to back,
//              so they form one 256-row operand)
//   warps 9,10 MMA issuers, one per tile (one thread spends about as long polling barriers and committing as
//              issuing, so with two the pipe stays fed): tile t accumulates page e of a pair into TMEM columns
//              [256 t + 128 e, + 128); tcgen05.commit hands each page's S to the row-max group, and -- one
//              arrival per issuer -- releases the K pair and, after the item's last pair, the Q buffer
//   warps 11-15 (packed e2m1 K only; the CTA then has 16 warps) dequantise raw pages into f16 operand tiles
//   warps 0-3  row-max group of tile 0: thread = query row; S in 64-column chunks, two in flight; the buffer goes
//   warps 4-7  back as soon as the last chunk has landed.  Same for tile 1.  While one tile's S is being read the
//              tensor pipe works on the other tile.
//
// K formats: bf16 (TMA, 128-byte swizzle), e4m3 fed to kind::f8f6f4 as stored against a two-term e4m3 Q
// (q = s (hi + lo), s a power of two per row), packed e2m1 with e4m3 (group 16) or ue8m0 (group 32) block scales
// dequantised exactly into f16.
#pragma once

#include "fmha_kernel.cuh"

namespace msa {

template <int KVMODE>
struct ScoreCfg {
  static constexpr bool kQuant = KVMODE != KV_BF16;
  static constexpr bool kKDirectFp8 = KVMODE == KV_FP8;
  static constexpr bool kKConvert = KVMODE == KV_NVFP4;
  static constexpr int kPageBytes = kKDirectFp8 ? kHalfBytes : kTileBytes;   // one page as an MMA operand
  static constexpr int kPairBytes = 2 * kPageBytes;
  // shared memory: two Q tiles per buffer (64 KiB); e4m3 K leaves room for two Q buffers and three pairs, the
  // 16-bit operand formats for one Q buffer and two pairs (128 KiB)
  static constexpr int kQBufs = kKDirectFp8 ? 2 : 1;
  static constexpr int kPairs = 2;
  // e4m3 K over a 64-element slice takes 8 KiB per page: the ring then holds five pairs in 80 KiB
  static constexpr int kPairsHalf = 5;
  static constexpr int kMaxPairs = kKDirectFp8 ? kPairsHalf : kPairs;
  static constexpr int kRingBytes = kKDirectFp8 ? kPairsHalf * kPairBytes / 2 : kPairs * kPairBytes;
  static constexpr int kRawStages = kKConvert ? 3 : 0;
  static constexpr int kRawBytes = 8192 + 1024;                              // packed e2m1 page + its scales
  // 12 warps; 16 with packed e2m1 K, where warps 11-15 dequantise (two warps kept the tensor pipe 40 % busy)
  static constexpr int kThreads = kKConvert ? 512 : 384;
  static constexpr int kProducerWarp = 8, kMmaWarp = 9, kMmaWarp1 = 10, kCvtWarp0 = 11;
  static constexpr int kCvtWarps = kKConvert ? 5 : 0;
  // One thread spends about as long polling barriers and committing as issuing; with an issuer per tile one of
  // them is always feeding the pipe.
  static constexpr int kIssuers = 2;
  // setmaxnreg.inc waits, unbounded, for registers released inside the CTA's own launch allocation, so the totals
  // must balance exactly: 256 row-max threads + the helper threads = threads x launch count
  static constexpr int kRegsLaunch = kKConvert ? 128 : 168;
  static constexpr int kRegsRowMax = kKConvert ? 176 : 216;
  static constexpr int kRegsHelper = kKConvert ? 80 : 72;
  static_assert(256 * kRegsRowMax + (kThreads - 256) * kRegsHelper == kThreads * kRegsLaunch,
                "setmaxnreg budget must balance");
  static constexpr int kFmt16 = kQuant ? 0 : 1;   // f16 once K is dequantised, bf16 as loaded
};

template <int KVMODE>
struct __align__(1024) ScoreSmem {
  using Cfg = ScoreCfg<KVMODE>;
  uint8_t q[Cfg::kQBufs][2][kTileBytes];
  uint8_t k[Cfg::kRingBytes];
  uint8_t raw[Cfg::kRawStages > 0 ? Cfg::kRawStages : 1][Cfg::kRawStages > 0 ? Cfg::kRawBytes : 16];
  float q_row_scale[Cfg::kQBufs][2][128];   // e4m3 K: power-of-two scale of every rewritten Q row
  uint64_t q_full[Cfg::kQBufs], q_ready[Cfg::kQBufs], q_empty[Cfg::kQBufs];
  uint64_t k_full[Cfg::kMaxPairs], k_empty[Cfg::kMaxPairs];
  uint64_t raw_full[Cfg::kRawStages > 0 ? Cfg::kRawStages : 1], raw_empty[Cfg::kRawStages > 0 ? Cfg::kRawStages : 1];
  uint64_t sc_full[2][2], sc_free[2][2];   // [tile][page of the pair]
  uint32_t tmem_base;
  int abort;
};

template <int KVMODE>
constexpr int score_smem_bytes() {
  return static_cast<int>(sizeof(ScoreSmem<KVMODE>)) + 1024;
}

// Two query tiles of 128 rows that share one stream of K pages.  A tile holds 128 / hb consecutive tokens of hb
// query heads of one KV head (hb = FmhaParams::pack_heads; row r = token r / hb, head r % hb): hb = 1 for prefill,
// hb > 1 packs the heads of a GQA group into the tile when a request brings only a few tokens (decode).  The walk
// covers the pages [page_lo, n_pages) from the top down; page_lo > 0 when the planner split the page range of an
// entry over several work items (the per-page maxima of different pages are independent, so nothing is merged).
struct ScoreItem {
  int tok0, tokens, qloc0, h, g, kv_len, qo_off, kv_base, n_pages, n_walk, n_tiles, fill;
};

__device__ __forceinline__ ScoreItem score_item(const FmhaParams& p, int item) {
  ScoreItem it;
  const int n_hg = p.Hq / p.pack_heads;
  const int wi = item / n_hg;
  it.h = (item - wi * n_hg) * p.pack_heads;   // first head; head group fastest: CTAs side by side share K pages
  it.g = it.h / p.hr;
  const int4 w = __ldg(p.work + 2 * wi), w2 = __ldg(p.work + 2 * wi + 1);
  it.tok0 = w.y;
  it.tokens = w.z & 1023;
  const int page_lo = w.z >> 10;
  it.qloc0 = w.w;
  it.kv_len = w2.x;
  it.qo_off = w2.y;
  it.kv_base = w2.z;
  it.fill = w2.w;   // 1: this entry also writes -inf for the pages above its own, up to max_k_tiles
  it.n_tiles = it.tokens * p.pack_heads > 128 ? 2 : 1;
  int vis = it.kv_len;   // keys visible to the last token of the entry
  if (p.causal) vis = min(vis, it.qloc0 + it.tokens + it.qo_off);
  it.n_pages = vis > 0 ? (vis + 127) >> 7 : 0;
  it.n_walk = max(0, it.n_pages - page_lo);
  return it;
}

// S[:, d .. d + N) = Q K^T for one pair (N = 256) or one page (N = 128)
template <class Cfg, int N>
__device__ __forceinline__ void issue_score_qk(uint32_t q_saddr, uint32_t k_saddr, uint32_t d, bool half_dim) {
  constexpr uint32_t desc_hi = smem_desc_hi(1024);
  const uint32_t qa = smem_desc_lo(q_saddr, 16), ka = smem_desc_lo(k_saddr, 16);
  if constexpr (Cfg::kKDirectFp8) {
    // Q_hi on the first 16 KiB of the Q tile, Q_lo on the second; 32 contraction bytes per step
    constexpr uint32_t idesc = make_idesc(128, N, 0, 0, 0, 0);
    if (half_dim) {
      // only the first 64 bytes of every K row were loaded: rows of 64 bytes under the 64-byte swizzle, eight of
      // them 512 bytes apart
      constexpr uint32_t k_hi = smem_desc_hi_sw64(512);
      umma_ss_f8_lohi2<0>(d, qa, desc_hi, ka, k_hi, idesc);
      umma_ss_f8_lohi2<1>(d, qa + 2, desc_hi, ka + 2, k_hi, idesc);
      umma_ss_f8_lohi2<1>(d, qa + 1024, desc_hi, ka, k_hi, idesc);
      umma_ss_f8_lohi2<1>(d, qa + 1026, desc_hi, ka + 2, k_hi, idesc);
    } else {
      umma_ss_lohi<0, 1>(d, qa, ka, desc_hi, idesc);
      umma_ss_lohi<1, 1>(d, qa + 2, ka + 2, desc_hi, idesc);
      umma_ss_lohi<1, 1>(d, qa + 4, ka + 4, desc_hi, idesc);
      umma_ss_lohi<1, 1>(d, qa + 6, ka + 6, desc_hi, idesc);
      umma_ss_lohi<1, 1>(d, qa + 1024, ka, desc_hi, idesc);
      umma_ss_lohi<1, 1>(d, qa + 1026, ka + 2, desc_hi, idesc);
      umma_ss_lohi<1, 1>(d, qa + 1028, ka + 4, desc_hi, idesc);
      umma_ss_lohi<1, 1>(d, qa + 1030, ka + 6, desc_hi, idesc);
    }
  } else {
    // 16-bit operands: the 64-element halves of Q are 16 KiB apart, those of a K pair 32 KiB (descriptor units
    // of 16 bytes: 1024 and 2048)
    constexpr uint32_t idesc = make_idesc(128, N, Cfg::kFmt16, Cfg::kFmt16, 0, 0);
    umma_ss_lohi<0, 0>(d, qa, ka, desc_hi, idesc);
    umma_ss_lohi<1, 0>(d, qa + 2, ka + 2, desc_hi, idesc);
    umma_ss_lohi<1, 0>(d, qa + 4, ka + 4, desc_hi, idesc);
    umma_ss_lohi<1, 0>(d, qa + 6, ka + 6, desc_hi, idesc);
    if (!half_dim) {
      umma_ss_lohi<1, 0>(d, qa + 1024, ka + 2048, desc_hi, idesc);
      umma_ss_lohi<1, 0>(d, qa + 1026, ka + 2050, desc_hi, idesc);
      umma_ss_lohi<1, 0>(d, qa + 1028, ka + 2052, desc_hi, idesc);
      umma_ss_lohi<1, 0>(d, qa + 1030, ka + 2054, desc_hi, idesc);
    }
  }
}

template <int KVMODE>
__global__ void __launch_bounds__(ScoreCfg<KVMODE>::kThreads, 1)
score_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                 const FmhaParams p) {
  using Cfg = ScoreCfg<KVMODE>;
  using Smem = ScoreSmem<KVMODE>;
  constexpr int QB = Cfg::kQBufs;
  constexpr int NRAW = Cfg::kRawStages > 0 ? Cfg::kRawStages : 1;
  extern __shared__ uint8_t smem_raw[];
  Smem& sm = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  volatile int* abort_flag = &sm.abort;
  MSA_TDECL

  if (tid == 0) {
    for (int b = 0; b < QB; ++b) {
      mbar_init(&sm.q_full[b], 1);
      mbar_init(&sm.q_ready[b], 8);     // one arrival per row-max warp
      mbar_init(&sm.q_empty[b], Cfg::kIssuers);
    }
    for (int t = 0; t < 2; ++t) {
      for (int e = 0; e < 2; ++e) {
        mbar_init(&sm.sc_full[t][e], 1);
        mbar_init(&sm.sc_free[t][e], 4);     // the four warps of the tile's row-max group
      }
    }
    for (int s = 0; s < Cfg::kMaxPairs; ++s) {
      mbar_init(&sm.k_full[s], Cfg::kKConvert ? Cfg::kCvtWarps : 1);
      mbar_init(&sm.k_empty[s], Cfg::kIssuers);
    }
    for (int s = 0; s < NRAW; ++s) {
      mbar_init(&sm.raw_full[s], 1);
      mbar_init(&sm.raw_empty[s], Cfg::kKConvert ? Cfg::kCvtWarps : 1);
    }
    sm.abort = 0;
    mbar_fence_init();
  }
  if (warp == Cfg::kMmaWarp) {
    tmem_alloc(&sm.tmem_base, 512);
    tmem_relinquish();
  }
  if (warp == Cfg::kProducerWarp && lane == 0) {
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;

  // The j-th item of this CTA that has pages to visit (the list is heaviest first; rounds alternate direction so
  // that the CTA with the heaviest item of one round takes the lightest of the next), or -1 past the end.
  auto item_of = [&](int j) {
    const int base = j * static_cast<int>(gridDim.x);
    const int idx = (j & 1) ? base + static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x)
                            : base + static_cast<int>(blockIdx.x);
    return (base < p.n_items && idx < p.n_items) ? idx : -1;
  };
  // every role walks the same sequence: items without a visible page are skipped by all of them
  auto next_item = [&](int& j, ScoreItem& it) -> bool {
    for (;; ++j) {
      const int item = item_of(j);
      if (item < 0) {
        if (j * static_cast<int>(gridDim.x) >= p.n_items) return false;
        continue;   // a hole in the last (partial) round
      }
      it = score_item(p, item);
      if (it.n_walk > 0) return true;
    }
  };
  // e4m3 K over the first 64 head-dim elements only: the TMA box is 64 bytes wide, a page takes 8 KiB
  const int pack_shift = 31 - __clz(p.pack_heads);   // pack_heads is a power of two
  const bool fp8_half = Cfg::kKDirectFp8 && p.half_dim != 0;
  const uint32_t page_stride = fp8_half ? kHalfBytes / 2 : kHalfBytes;   // second page: rows 128-255 of the operand
  const int NP = fp8_half ? Cfg::kPairsHalf : Cfg::kPairs;               // pairs in the K ring
  const uint32_t pair_bytes = fp8_half ? Cfg::kPairBytes / 2 : Cfg::kPairBytes;

  if (warp < 8) {
    // =========================================================================
    // row-max group of tile t
    // =========================================================================
    setmaxnreg_inc<Cfg::kRegsRowMax>();
    const int t = warp >> 2;
    const int r = tid & 127;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t s_cur = tmem + lane_base + t * 256;
    bool ok = true;
    uint32_t use_a = 0, use_b = 0;   // first / second pages of my tile so far (sc_full / sc_free phases)
    uint32_t n_q = 0;

    // My tile of Q item number nq (buffer nq % QB) into the operand format of the quantised modes; every warp
    // arrives, also when its tile does not exist.
    auto convert_q = [&](uint32_t nq, int n_tiles) {
      if constexpr (Cfg::kQuant) {
        const int qb = nq % QB;
        ok = ok && mbar_wait(&sm.q_full[qb], (nq / QB) & 1, abort_flag);
        if (ok && t < n_tiles) {
          if constexpr (Cfg::kKDirectFp8) {
            // my row -> two e4m3 rows (hi, lo) sharing one power-of-two scale; hi lands on the first
            // 64-column half of the bf16 tile, lo on the second, same row: in place, thread-private
            uint8_t* rowp = sm.q[qb][t] + r * 128;
            uint4 x[16];
#pragma unroll
            for (int c = 0; c < 16; ++c)
              x[c] = *reinterpret_cast<const uint4*>(rowp + (c >> 3) * kHalfBytes + (((c & 7) ^ (r & 7)) << 4));
            float amax = 0.f;
#pragma unroll
            for (int c = 0; c < 16; ++c) {
              const uint32_t v[4] = {x[c].x, x[c].y, x[c].z, x[c].w};
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                amax = fmaxf(amax, fabsf(__uint_as_float(v[i] << 16)));
                amax = fmaxf(amax, fabsf(__uint_as_float(v[i] & 0xffff0000u)));
              }
            }
            float sq = 1.0f;   // power of two that brings the row maximum into [224, 448]
            if (amax > 0.f && amax < 3.0e38f) {
              int e;
              frexpf(amax, &e);
              sq = ldexpf(1.0f, e - 9);
              if (amax / sq > 448.0f) sq *= 2.0f;
            }
            const float inv = 1.0f / sq;
            sm.q_row_scale[qb][t][r] = sq;
#pragma unroll
            for (int c8 = 0; c8 < 8; ++c8) {
              uint32_t hi4[4], lo4[4];
#pragma unroll
              for (int half = 0; half < 2; ++half) {
                const uint4 xv = x[c8 * 2 + half];
                const uint32_t v[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
                for (int i = 0; i < 4; i += 2) {
                  float y[4] = {__uint_as_float(v[i] << 16) * inv, __uint_as_float(v[i] & 0xffff0000u) * inv,
                                __uint_as_float(v[i + 1] << 16) * inv, __uint_as_float(v[i + 1] & 0xffff0000u) * inv};
                  const uint32_t h01 = f32x2_to_e4m3x2(y[0], y[1]), h23 = f32x2_to_e4m3x2(y[2], y[3]);
                  float f[4];
                  e4m3x2_to_f32x2(h01, f[0], f[1]);
                  e4m3x2_to_f32x2(h23, f[2], f[3]);
                  const uint32_t l01 = f32x2_to_e4m3x2(y[0] - f[0], y[1] - f[1]);
                  const uint32_t l23 = f32x2_to_e4m3x2(y[2] - f[2], y[3] - f[3]);
                  hi4[half * 2 + (i >> 1)] = h01 | (h23 << 16);
                  lo4[half * 2 + (i >> 1)] = l01 | (l23 << 16);
                }
              }
              const uint32_t off = ((c8 ^ (r & 7)) << 4);
              *reinterpret_cast<uint4*>(rowp + off) = make_uint4(hi4[0], hi4[1], hi4[2], hi4[3]);
              *reinterpret_cast<uint4*>(rowp + kHalfBytes + off) = make_uint4(lo4[0], lo4[1], lo4[2], lo4[3]);
            }
          } else {
            // bf16 -> f16 in place (the dequantised K tiles are f16 and the tensor core wants one format)
            uint4* qv = reinterpret_cast<uint4*>(sm.q[qb][t]);
            for (int i = r; i < kTileBytes / 16; i += 128) {
              uint4 xq = qv[i];
              xq.x = bf16x2_to_f16x2(xq.x);
              xq.y = bf16x2_to_f16x2(xq.y);
              xq.z = bf16x2_to_f16x2(xq.z);
              xq.w = bf16x2_to_f16x2(xq.w);
              qv[i] = xq;
            }
          }
          fence_proxy_async();
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm.q_ready[qb]);
      }
    };

    int j = 0, j_next = 0;
    ScoreItem it, it_next;
    bool have = next_item(j, it);
    if (have && QB == 2) convert_q(0, it.n_tiles);
    while (have && ok) {
      j_next = j + 1;
      const bool have_next = next_item(j_next, it_next);
      if (QB == 1) convert_q(n_q, it.n_tiles);   // a single Q buffer: rewritten when the item starts
      const int r_entry = t * 128 + r;                       // my row within the work entry
      const int tok_local = r_entry >> pack_shift;           // its token and head
      const int head = it.h + (r_entry & (p.pack_heads - 1));
      const bool row_valid = tok_local < it.tokens;
      int limit_base = -1;
      if (row_valid) {
        limit_base = it.kv_len - 1;
        if (p.causal) limit_base = min(limit_base, it.qloc0 + tok_local + it.qo_off);
      }
      float row_scale = 1.0f;
      float* dst = p.max_score + static_cast<long long>(head) * p.ms_head + it.tok0 + tok_local;
      const int n = it.n_pages, n_pairs = (it.n_walk + 1) >> 1;
      const bool mine = t < it.n_tiles;
      for (int pi = 0; pi < n_pairs && ok; ++pi) {
        if (mine) {
          const int page_a = n - 1 - 2 * pi, page_b = page_a - 1;   // pages are walked from the highest down
          const bool two = 2 * pi + 1 < it.n_walk;
          MSA_TBEGIN
          ok = mbar_wait(&sm.sc_full[t][0], use_a & 1, abort_flag);
          MSA_TEND(0)
          if (!ok) break;
          ++use_a;
          tc_fence_after();
          if (r == 0) { MSA_TRACE(t * 2, use_a, clock64()) }
          MSA_TBEGIN
          if constexpr (Cfg::kKDirectFp8) {
            if (pi == 0) row_scale = sm.q_row_scale[n_q % QB][t][r];
          }
          // 64-column chunks, two in flight: c0, c1 = first page, then second.  A chunk's registers take the next
          // load as soon as its maxima are folded in; each page's columns go back to the issuer as soon as they
          // are in registers, so the next pair's MMAs for the first page run while the second is being read.
          uint32_t c0[64], c1[64];
          tmem_ld32p(s_cur, c0);
          tmem_ld32p(s_cur + 32, c0 + 32);
          tmem_ld32p(s_cur + 64, c1);
          tmem_ld32p(s_cur + 96, c1 + 32);
          tmem_ld_wait();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&sm.sc_free[t][0]);
          const int limit_a = limit_base - (page_a << 7), limit_b = limit_a + 128;
          const bool vis_a = __all_sync(0xffffffffu, limit_a >= 127);
          auto fold = [&](uint32_t (&c)[64], int lim, bool all_visible, float& m0, float& m1, float& m2, float& m3) {
            if (!all_visible) {
#pragma unroll
              for (int e = 0; e < 64; ++e) c[e] = (e <= lim) ? c[e] : 0xff800000u;
            }
#pragma unroll
            for (int e = 0; e < 64; e += 8) {
              m0 = max3(m0, __uint_as_float(c[e]), __uint_as_float(c[e + 1]));
              m1 = max3(m1, __uint_as_float(c[e + 2]), __uint_as_float(c[e + 3]));
              m2 = max3(m2, __uint_as_float(c[e + 4]), __uint_as_float(c[e + 5]));
              m3 = max3(m3, __uint_as_float(c[e + 6]), __uint_as_float(c[e + 7]));
            }
          };
          float a0 = -INFINITY, a1 = -INFINITY, a2 = -INFINITY, a3 = -INFINITY;
          fold(c0, limit_a, vis_a, a0, a1, a2, a3);
          if (two) {
            ok = mbar_wait(&sm.sc_full[t][1], use_b & 1, abort_flag);
            if (!ok) break;
            ++use_b;
            tc_fence_after();
            tmem_ld32p(s_cur + 128, c0);
            tmem_ld32p(s_cur + 160, c0 + 32);
          }
          fold(c1, limit_a - 64, vis_a, a0, a1, a2, a3);
          // (a request longer than the score tensor's max_k_tiles pages is a caller error: its pages are not stored)
          if (row_valid && page_a < p.max_k_tiles)
            __stwt(dst + static_cast<long long>(page_a) * p.ms_tile, fmaxf(fmaxf(a0, a1), fmaxf(a2, a3)) * row_scale);
          if (two) {
            tmem_ld32p(s_cur + 192, c1);
            tmem_ld32p(s_cur + 224, c1 + 32);
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.sc_free[t][1]);
            const bool vis_b = __all_sync(0xffffffffu, limit_b >= 127);
            float b0 = -INFINITY, b1 = -INFINITY, b2 = -INFINITY, b3 = -INFINITY;
            fold(c0, limit_b, vis_b, b0, b1, b2, b3);
            fold(c1, limit_b - 64, vis_b, b0, b1, b2, b3);
            if (row_valid && page_b < p.max_k_tiles)
              __stwt(dst + static_cast<long long>(page_b) * p.ms_tile, fmaxf(fmaxf(b0, b1), fmaxf(b2, b3)) * row_scale);
          }
          MSA_TEND(1)
        }
        // Two Q buffers: Q of the next item is rewritten while the issuers still have this item's pairs in hand.
        // The producer issues that Q load right after K pair min(1, n_pairs - 1) of this item (see there), so
        // waiting for it at the same pair cannot dead-lock: the ring holds at least two pairs.
        if (QB == 2 && pi == min(1, n_pairs - 1) && have_next) convert_q(n_q + 1, it_next.n_tiles);
      }
      // the tiles nobody visits (beyond the causal frontier, beyond the request, padding up to max_k_tiles) read
      // -inf: written by the kernel when the caller asks for it, so that no separate pass has to pre-fill the
      // tensor -- here with packed e2m1 K, by the otherwise idle warp 11 in the other modes
      if (Cfg::kKConvert && p.fill_tail != 0 && it.fill != 0 && mine && row_valid && ok) {
        for (int pg = n; pg < p.max_k_tiles; ++pg) __stwt(dst + static_cast<long long>(pg) * p.ms_tile, -INFINITY);
      }
      ++n_q;
      have = have_next;
      it = it_next;
      j = j_next;
    }
    MSA_TFLUSH(r == 0 && t == 0, 0, 3)
  } else {
    setmaxnreg_dec<Cfg::kRegsHelper>();
    if (warp == Cfg::kProducerWarp) {
      // =======================================================================
      // producer: Q per item, K per pair (lane 0)
      // =======================================================================
      if (lane == 0) {
        bool ok = true;
        uint32_t n_q = 0, pair_seq = 0, raw_seq = 0;
        // the Q tiles of the item numbered n_q into buffer n_q % QB, once the item that last used the buffer is done
        auto load_q = [&](const ScoreItem& qi) {
          const int qb = n_q % QB;
          MSA_TBEGIN
          ok = mbar_wait(&sm.q_empty[qb], ((n_q / QB) & 1) ^ 1, abort_flag);
          MSA_TEND(12)
          if (!ok) return;
          ++n_q;
          mbar_expect_tx(&sm.q_full[qb], qi.n_tiles * kTileBytes);
          for (int t = 0; t < qi.n_tiles; ++t) {
            const int tok = qi.tok0 + t * (128 >> pack_shift);   // a box is 128 / hb tokens x hb heads
            tma_load_3d(sm.q[qb][t], &tmap_q, &sm.q_full[qb], 0, qi.h, tok);
            tma_load_3d(sm.q[qb][t] + kHalfBytes, &tmap_q, &sm.q_full[qb], 64, qi.h, tok);
          }
        };
        int j = 0, j_next = 0;
        ScoreItem it, it_next;
        bool have = next_item(j, it);
        if (have && QB == 2) load_q(it);
        while (have && ok) {
          j_next = j + 1;
          const bool have_next = next_item(j_next, it_next);
          if (QB == 1) load_q(it);
          if (!ok) break;
          const int n = it.n_pages, n_pairs = (it.n_walk + 1) >> 1;
          const int page_base = p.paged ? it.kv_base : 0;
          const int tok_base = p.paged ? 0 : it.kv_base;
          for (int pi = 0; pi < n_pairs && ok; ++pi, ++pair_seq) {
            const int np = min(2, it.n_walk - 2 * pi);
            const int kq = pair_seq % NP;
            if constexpr (Cfg::kKConvert) {
              for (int e = 0; e < np && ok; ++e, ++raw_seq) {
                const int page = n - 1 - (2 * pi + e);
                int phys = __ldg(p.kv_indices + page_base + page);
                if (static_cast<unsigned>(phys) >= static_cast<unsigned>(p.kv_pages)) {
                  atomicExch(p.status, MSA_ERR_BOUNDS);   // corrupt page table: reported, page 0 read instead
                  phys = 0;
                }
                const size_t tile = static_cast<size_t>(phys) * p.Hkv + it.g;
                const int s = raw_seq % NRAW;
                MSA_TBEGIN
                ok = mbar_wait(&sm.raw_empty[s], ((raw_seq / NRAW) & 1) ^ 1, abort_flag);
                MSA_TEND(13)
                if (!ok) break;
                mbar_expect_tx(&sm.raw_full[s], 8192 + p.k_scale_tile_bytes);
                bulk_load(sm.raw[s], p.k_raw + tile * 8192, 8192, &sm.raw_full[s]);
                bulk_load(sm.raw[s] + 8192, p.k_scale_bytes + tile * p.k_scale_tile_bytes, p.k_scale_tile_bytes,
                          &sm.raw_full[s]);
              }
            } else {
              MSA_TBEGIN
              ok = mbar_wait(&sm.k_empty[kq], ((pair_seq / NP) & 1) ^ 1, abort_flag);
              MSA_TEND(13)
              if (!ok) break;
              mbar_expect_tx(&sm.k_full[kq], np * (fp8_half ? Cfg::kPageBytes / 2 : Cfg::kPageBytes));
              for (int e = 0; e < np; ++e) {
                const int page = n - 1 - (2 * pi + e);
                int phys = p.paged ? __ldg(p.kv_indices + page_base + page) : 0;
                if (p.paged && static_cast<unsigned>(phys) >= static_cast<unsigned>(p.kv_pages)) {
                  atomicExch(p.status, MSA_ERR_BOUNDS);
                  phys = 0;
                }
                const int tok_k = tok_base + (page << 7);
                uint8_t* kdst = sm.k + kq * pair_bytes + e * page_stride;
                if constexpr (Cfg::kKDirectFp8) {
                  if (p.paged)
                    tma_load_4d(kdst, &tmap_k, &sm.k_full[kq], 0, 0, it.g, phys);
                  else
                    tma_load_3d(kdst, &tmap_k, &sm.k_full[kq], 0, it.g, tok_k);
                } else if (p.paged) {
                  tma_load_4d(kdst, &tmap_k, &sm.k_full[kq], 0, 0, it.g, phys);
                  tma_load_4d(kdst + kTileBytes, &tmap_k, &sm.k_full[kq], 64, 0, it.g, phys);
                } else {
                  tma_load_3d(kdst, &tmap_k, &sm.k_full[kq], 0, it.g, tok_k);
                  tma_load_3d(kdst + kTileBytes, &tmap_k, &sm.k_full[kq], 64, it.g, tok_k);
                }
              }
            }
            // two Q buffers: the next item's Q goes out early, so that it can be rewritten inside this item
            if (QB == 2 && ok && pi == min(1, n_pairs - 1) && have_next) load_q(it_next);
          }
          have = have_next;
          it = it_next;
          j = j_next;
        }
        MSA_TFLUSH(true, 12, 14)
      }
    } else if (warp == Cfg::kMmaWarp || warp == Cfg::kMmaWarp1) {
      // =======================================================================
      // MMA issuer: tile `me` with two issuers, both tiles with one.  tcgen05.commit covers the MMAs of the
      // committing thread only, hence K pairs and Q buffers are released by one arrival per issuer.
      // =======================================================================
      const int me = warp == Cfg::kMmaWarp ? 0 : 1;
      bool ok = true;
      uint32_t n_q = 0, pair_seq = 0;
      uint32_t use_seq[2][2] = {{0, 0}, {0, 0}};   // pages issued per tile and page of the pair (sc_free phase)
      int j = 0;
      ScoreItem it;
      while (ok && next_item(j, it)) {
        const int qb = n_q % QB;
        MSA_TBEGIN
        ok = mbar_wait(Cfg::kQuant ? &sm.q_ready[qb] : &sm.q_full[qb], (n_q / QB) & 1, abort_flag);
        MSA_TEND(14)
        if (!ok) break;
        ++n_q;
        const int n = it.n_pages, n_pairs = (it.n_walk + 1) >> 1;
        for (int pi = 0; pi < n_pairs && ok; ++pi, ++pair_seq) {
          const int np = min(2, it.n_walk - 2 * pi);
          const int kq = pair_seq % NP;
          MSA_TBEGIN
          ok = mbar_wait(&sm.k_full[kq], (pair_seq / NP) & 1, abort_flag);
          MSA_TEND(6)
          if (!ok) break;
          const uint32_t kaddr = smem_u32(sm.k + kq * pair_bytes);
#pragma unroll
          for (int t = me; t < 2; t += Cfg::kIssuers) {
            if (t < it.n_tiles) {
              const uint32_t qaddr = smem_u32(sm.q[qb][t]);
              // one page at a time (N = 128), each into its own 128 columns with its own barrier pair, so that the
              // row-max group reads the first page while the second is computed
              for (int e = 0; e < np && ok; ++e) {
                MSA_TBEGIN
                if (use_seq[t][e] >= 1) ok = mbar_wait(&sm.sc_free[t][e], (use_seq[t][e] + 1) & 1, abort_flag);
                MSA_TEND(4)
                if (!ok) break;
                ++use_seq[t][e];
                tc_fence_after();
                MSA_TBEGIN
                if (lane == 0) {
                  issue_score_qk<Cfg, 128>(qaddr, kaddr + e * page_stride, t * 256 + e * 128, p.half_dim != 0);
                  umma_commit(&sm.sc_full[t][e]);
                }
                __syncwarp();
                MSA_TEND(5)
              }
            }
          }
          if (!ok) break;
          if (lane == 0) {
            // my share of the K pair (and of Q after the item's last pair): freed when my MMAs above have read
            // it -- at once if I had no tile to issue for
            umma_commit(&sm.k_empty[kq]);
            if (pi + 1 == n_pairs) umma_commit(&sm.q_empty[qb]);
          }
          __syncwarp();
        }
        ++j;
      }
      MSA_TFLUSH(lane == 0 && me == 0, 4, 7)
      MSA_TFLUSH(lane == 0 && me == 0, 14, 15)
    } else if (!Cfg::kKConvert && warp == Cfg::kCvtWarp0) {
      // =======================================================================
      // -inf for the tiles above every flagged entry's pages (score_fill_tail): this warp has no other work in the
      // bf16 / e4m3 modes, so the stores overlap the MMAs instead of waiting at the end of every item
      // =======================================================================
      if (p.fill_tail != 0) {
        int j = 0;
        ScoreItem it;
        while (next_item(j, it)) {
          if (it.fill != 0) {
            float* dst[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              const int r_entry = e * 32 + lane;                  // rows of both tiles
              const int tok_local = r_entry >> pack_shift;
              const int head = it.h + (r_entry & (p.pack_heads - 1));
              dst[e] = tok_local < it.tokens
                           ? p.max_score + static_cast<long long>(head) * p.ms_head + it.tok0 + tok_local
                           : nullptr;
            }
            for (int pg = it.n_pages; pg < p.max_k_tiles; ++pg) {
              const long long off = static_cast<long long>(pg) * p.ms_tile;
#pragma unroll
              for (int e = 0; e < 8; ++e)
                if (dst[e] != nullptr) __stwt(dst[e] + off, -INFINITY);
            }
          }
          ++j;
        }
      }
    } else if constexpr (Cfg::kKConvert) {
      // =======================================================================
      // dequantise raw e2m1 pages into f16 operand tiles (warps 11-15).  Block scales: e4m3 per 16 values (two
      // 128x4 tiles per page) or, with k_mx, ue8m0 per 32 (one).
      // =======================================================================
      const int cw = warp - Cfg::kCvtWarp0;      // convert warp 0 .. kCvtWarps - 1
      const int r4 = lane >> 3, c8 = lane & 7;   // row within a group of 4, 16-value block of the row
      const bool mx = p.k_mx != 0;
      bool ok = cw < Cfg::kCvtWarps;
      uint32_t raw_seq = 0, pair_seq = 0;
      int j = 0;
      ScoreItem it;
      while (ok && next_item(j, it)) {
        const int n = it.n_pages, n_pairs = (it.n_walk + 1) >> 1;
        for (int pi = 0; pi < n_pairs && ok; ++pi, ++pair_seq) {
          const int np = min(2, it.n_walk - 2 * pi);
          const int kq = pair_seq % NP;
          ok = mbar_wait(&sm.k_empty[kq], ((pair_seq / NP) & 1) ^ 1, abort_flag);
          for (int e = 0; e < np && ok; ++e, ++raw_seq) {
            const int rs = raw_seq % NRAW;
            ok = mbar_wait(&sm.raw_full[rs], (raw_seq / NRAW) & 1, abort_flag);
            if (!ok) break;
            const uint8_t* rawp = sm.raw[rs];
            uint8_t* tile = sm.k + kq * pair_bytes + e * kHalfBytes + (c8 >> 2) * kTileBytes;
            // a warp takes every kCvtWarps-th group of four rows; block c8 of row `row`: 8 packed bytes in, two
            // 16-byte chunks of the 128-byte swizzled f16 row out.  Scale of (row, block): 128x4 tile offset
            // (row % 32) * 16 + (row / 32) * 4 + block % 4; with ue8m0 scales a block of 16 values shares the
            // scale of its group of 32 (block c8 -> group c8 / 2)
            const uint8_t* sc = mx ? rawp + 8192 + (c8 >> 1) : rawp + 8192 + (c8 >> 2) * 512 + (c8 & 3);
#pragma unroll 2
            for (int i = cw; i < 32; i += Cfg::kCvtWarps) {
              const int row = i * 4 + r4, r8 = row & 7;
              const uint2 x = *reinterpret_cast<const uint2*>(rawp + row * 64 + c8 * 8);
              const uint32_t sb = sc[(row & 31) * 16 + (row >> 5) * 4];
              uint32_t s2;
              if (mx) {
                // 2^(e - 127) as f16, exact for exponents -24 .. 15 (clamped outside)
                const int ex = min(max(static_cast<int>(sb) - 127, -24), 15);
                const uint32_t h = ex >= -14 ? static_cast<uint32_t>(ex + 15) << 10 : 1u << (ex + 24);
                s2 = h | (h << 16);
              } else {
                uint32_t s2hi;
                cvt_e4m3x4_f16x4(sb | (sb << 8), s2, s2hi);
              }
              uint32_t f0[4], f1[4];
              cvt_e2m1x8_f16x8(x.x, f0);
              cvt_e2m1x8_f16x8(x.y, f1);
              uint4 a, b;
              a.x = hmul2_u32(f0[0], s2);
              a.y = hmul2_u32(f0[1], s2);
              a.z = hmul2_u32(f0[2], s2);
              a.w = hmul2_u32(f0[3], s2);
              b.x = hmul2_u32(f1[0], s2);
              b.y = hmul2_u32(f1[1], s2);
              b.z = hmul2_u32(f1[2], s2);
              b.w = hmul2_u32(f1[3], s2);
              uint8_t* dst = tile + row * 128;
              *reinterpret_cast<uint4*>(dst + ((((c8 & 3) * 2) ^ r8) << 4)) = a;
              *reinterpret_cast<uint4*>(dst + ((((c8 & 3) * 2 + 1) ^ r8) << 4)) = b;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.raw_empty[rs]);
          }
          if (!ok) break;
          fence_proxy_async();
          __syncwarp();
          if (lane == 0) mbar_arrive(&sm.k_full[kq]);
        }
        ++j;
      }
    }
  }

  // ---- teardown ---------------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (warp == Cfg::kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
  if (tid == 0 && sm.abort) atomicExch(p.status, MSA_ERR_TIMEOUT);
}

}  // namespace msa
