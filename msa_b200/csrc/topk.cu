// Top-k page selector (stage 2): exact top-k of every (head, token) row of the
// max-score tensor [H, K, T] (T innermost), output [T, H, topk] ascending by
// page index with -1 at the tail.  Replaces SparseTopKSelect
// (csrc/include/sparse_topk_select.cuh:852-886 of the reference) without its
// transpose workspace: a CTA streams a [K-chunk x TOK tokens] slab of the score
// tensor into shared memory once (64-byte global segments for TOK = 16), then one
// warp per row finds the value of the k-th largest score and emits by threshold:
//   1. a lower bound on the k-th largest value from disjoint lane maxima,
//   2. candidates >= that bound (a few dozen of 1024) compacted by warp prefix,
//   3. warp bitonic sorts of 32-bit value keys merged into the running best k values,
//   4. every score above the k-th value, then the lowest-indexed ties, written in
//      index order from warp ballots -- no sort by index, no (value, index) pairs.
// Ties go to the lower page index; picks whose score is -inf are reported as -1.
// More than 1024 pages: the slabs are streamed a second time for step 4.
#include "common.cuh"
#include "msa_internal.h"

namespace msa {

constexpr int kTopkChunk = 1024;   // K values per slab (32 per lane)
constexpr uint32_t kNegInfKey = 0x007fffffu;   // ordered_key(-inf); 0 marks an empty slot

template <int NR, bool DESC, typename T>
__device__ __forceinline__ void warp_bitonic_sort(T (&x)[NR], int lane) {
  // element index e = reg * 32 + lane
#pragma unroll
  for (int k = 2; k <= 32 * NR; k <<= 1) {
#pragma unroll
    for (int j = k >> 1; j > 0; j >>= 1) {
      if (j >= 32) {
        const int jr = j >> 5;
#pragma unroll
        for (int r = 0; r < NR; ++r) {
          if ((r & jr) == 0) {
            const int e = r * 32 + lane;
            const bool up = ((e & k) == 0) != DESC;  // this block ends ascending
            const T a = x[r], b = x[r | jr];
            const bool sw = up ? (a > b) : (a < b);
            x[r] = sw ? b : a;
            x[r | jr] = sw ? a : b;
          }
        }
      } else {
#pragma unroll
        for (int r = 0; r < NR; ++r) {
          const T other = __shfl_xor_sync(0xffffffffu, x[r], j);
          const int e = r * 32 + lane;
          const bool up = ((e & k) == 0) != DESC;
          const bool lower = (lane & j) == 0;
          const T mn = x[r] < other ? x[r] : other;
          const T mx = x[r] < other ? other : x[r];
          x[r] = (lower == up) ? mn : mx;
        }
      }
    }
  }
}

// monotonic map float -> uint32 (no NaN, no -0.0 after sanitize) and back
__device__ __forceinline__ uint32_t ordered_key(float v) {
  const uint32_t u = __float_as_uint(v);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_value(uint32_t key) {
  return __uint_as_float((key & 0x80000000u) ? (key & 0x7fffffffu) : ~key);
}

// forced tiles rank as FLT_MAX, NaN never wins, +inf ranks with FLT_MAX, -0.0 becomes +0.0 (the two compare
// equal as floats, so they must tie)
__device__ __forceinline__ float sanitize(float v, bool forced) {
  if (forced) return 3.402823466e38f;
  if (!(v == v)) return -INFINITY;
  return fminf(v, 3.402823466e38f) + 0.0f;
}

// TOK tokens per slab: 16 (8 warps, two rows each) for throughput, 4 (4 warps, one row each) when the
// whole problem is only a few CTAs of the wide shape
template <int TOPK, int TOK>
__global__ void __launch_bounds__(TOK == 16 ? 256 : 128, TOK == 16 ? 3 : 8)
topk_select_kernel(const float* __restrict__ ms, int H, int K, int T, int nvp, int force_begin, int force_end,
                   int* __restrict__ out) {
  constexpr int WARPS = TOK == 16 ? 8 : 4;
  constexpr int ROWS = TOK / WARPS;                // rows per warp
  constexpr int NR = TOPK / 16;                    // registers per lane for 2 * TOPK value keys
  constexpr int PITCH = TOK + 1;
  extern __shared__ float slab[];                  // [kTopkChunk][PITCH]
  __shared__ uint32_t stage[WARPS][2 * TOPK];
  __shared__ uint32_t bitmap[WARPS][32];           // selected positions of one row and slab, bit kl

  const int h = blockIdx.y;
  const int t0 = blockIdx.x * TOK;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t lt_mask = (1u << lane) - 1u;
  const int keff = min(K, nvp);
  const int nchunks = (keff + kTopkChunk - 1) / kTopkChunk;
  const float* base = ms + static_cast<size_t>(h) * K * T;
  const bool vec_ok = (T % 4 == 0) && ((reinterpret_cast<uintptr_t>(ms) & 15) == 0) && (t0 + TOK <= T);

  // stream one slab in: the TOK consecutive tokens of one k are one global segment
  auto load_slab = [&](int k0, int klen) {
    if (vec_ok) {
      constexpr int Q = TOK / 4;                    // 128-bit loads per k
#pragma unroll 4
      for (int idx = tid; idx < klen * Q; idx += WARPS * 32) {
        const int kl = idx / Q, q4 = idx % Q;
        const int k = k0 + kl;
        float4 v = __ldcs(reinterpret_cast<const float4*>(base + static_cast<size_t>(k) * T + t0) + q4);
        const bool forced = k < force_begin || (k >= nvp - force_end && k < nvp);
        float* dst = slab + kl * PITCH + q4 * 4;
        dst[0] = sanitize(v.x, forced);
        dst[1] = sanitize(v.y, forced);
        dst[2] = sanitize(v.z, forced);
        dst[3] = sanitize(v.w, forced);
      }
    } else {
      for (int idx = tid; idx < klen * TOK; idx += WARPS * 32) {
        const int kl = idx / TOK, tt = idx % TOK;
        const int k = k0 + kl, t = t0 + tt;
        float v = -INFINITY;
        if (t < T) v = __ldcs(base + static_cast<size_t>(k) * T + t);
        slab[kl * PITCH + tt] = sanitize(v, k < force_begin || (k >= nvp - force_end && k < nvp));
      }
    }
  };

  uint32_t best[ROWS][NR];   // value keys, descending; slots [0, TOPK) hold the running best
  uint32_t cand[ROWS];       // candidate positions (bit j = slab row lane + 32 j) of the last slab
#pragma unroll
  for (int rr = 0; rr < ROWS; ++rr) {
    cand[rr] = 0u;
#pragma unroll
    for (int i = 0; i < NR; ++i) best[rr][i] = 0u;
  }

  // ---- pass A: the k-th largest value of every row ------------------------------------------
  for (int c = 0; c < nchunks; ++c) {
    const int k0 = c * kTopkChunk;
    const int klen = min(kTopkChunk, keff - k0);
    const int jmax = (klen + 31) >> 5;
    __syncthreads();
    load_slab(k0, klen);
    __syncthreads();
#pragma unroll
    for (int rr = 0; rr < ROWS; ++rr) {
      const int tt = warp * ROWS + rr;
      if (t0 + tt >= T) continue;  // warp-uniform
      float v[32];
      float gmax[NR];                  // maxima of 2 * TOPK disjoint groups (lane, j mod NR)
#pragma unroll
      for (int i = 0; i < NR; ++i) gmax[i] = -INFINITY;
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        v[j] = -INFINITY;
        if (j < jmax) {
          const int kl = lane + 32 * j;
          if (kl < klen) v[j] = slab[kl * PITCH + tt];
          gmax[j % NR] = fmaxf(gmax[j % NR], v[j]);
        }
      }
      // the TOPK-th largest group maximum: TOPK distinct elements are >= it, so it bounds the chunk's
      // TOPK-th largest from below, and only about 1.4 * TOPK elements reach it
      float thr;
      {
        uint32_t gk[NR];
#pragma unroll
        for (int i = 0; i < NR; ++i) gk[i] = ordered_key(gmax[i]);
        warp_bitonic_sort<NR, true>(gk, lane);
        const uint32_t tk = __shfl_sync(0xffffffffu, gk[(TOPK - 1) >> 5], (TOPK - 1) & 31);
        thr = tk > kNegInfKey ? key_value(tk) : -INFINITY;
      }
      // the running k-th best also bounds from below (strictly: earlier chunks win ties); -inf while unfilled
      const uint32_t kth = __shfl_sync(0xffffffffu, best[rr][(TOPK - 1) >> 5], (TOPK - 1) & 31);
      const float floor_v = kth > kNegInfKey ? key_value(kth) : -INFINITY;

      // one comparison per element: v >= thr && v > floor  <=>  v >= max(thr, the float after floor)
      float above_floor;   // smallest float greater than floor_v (floor_v is -inf, or finite and not -0.0)
      {
        const uint32_t fb = __float_as_uint(floor_v);
        above_floor = floor_v == -INFINITY ? -3.402823466e38f
                      : floor_v >= 0.0f    ? __uint_as_float(fb + 1u)
                                           : __uint_as_float(fb - 1u);
      }
      const float lower = fmaxf(thr, above_floor);
      uint32_t mask = 0;
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        if (j < jmax) mask |= (v[j] >= lower) ? (1u << j) : 0u;
      }
      cand[rr] = mask;
      const int cnt = __popc(mask);
      int pre = cnt;
#pragma unroll
      for (int s = 1; s < 32; s <<= 1) {
        const int o = __shfl_up_sync(0xffffffffu, pre, s);
        if (lane >= s) pre += o;
      }
      const int total = __shfl_sync(0xffffffffu, pre, 31);
      int rank = pre - cnt;  // rank of my next unstaged candidate (mine are consecutive)
      uint32_t m = mask;
      bool empty = (c == 0);           // nothing merged yet: the first batch may fill all 2 * TOPK slots
      for (int b0 = 0; b0 < total;) {
        const int cap = empty ? 2 * TOPK : TOPK;
        for (int i = lane; i < cap; i += 32) stage[warp][i] = 0u;
        __syncwarp();
        while (m != 0u && rank < b0 + cap) {
          const int j = __ffs(m) - 1;
          m &= m - 1;
          stage[warp][rank - b0] = ordered_key(slab[(lane + 32 * j) * PITCH + tt]);
          ++rank;
        }
        __syncwarp();
        // incoming keys occupy the element slots behind the running best
#pragma unroll
        for (int i = 0; i < NR; ++i) {
          const int e = i * 32 + lane;
          if (e >= 2 * TOPK - cap) best[rr][i] = stage[warp][e - (2 * TOPK - cap)];
        }
        warp_bitonic_sort<NR, true>(best[rr], lane);
        __syncwarp();
        b0 += cap;
        empty = false;
      }
    }
  }

  // ---- the cut of every row: value of the k-th largest and how many of its ties are taken ----------
  float cut[ROWS];
  int ties[ROWS], written[ROWS];
#pragma unroll
  for (int rr = 0; rr < ROWS; ++rr) {
    const uint32_t kth = __shfl_sync(0xffffffffu, best[rr][(TOPK - 1) >> 5], (TOPK - 1) & 31);
    written[rr] = 0;
    if (kth <= kNegInfKey) {          // fewer than TOPK scores above -inf: take them all
      cut[rr] = -INFINITY;
      ties[rr] = 0;
    } else {
      int gt = 0;
#pragma unroll
      for (int i = 0; i < NR; ++i) gt += (i * 32 + lane < TOPK && best[rr][i] > kth) ? 1 : 0;
      gt = __reduce_add_sync(0xffffffffu, gt);
      cut[rr] = key_value(kth);
      ties[rr] = TOPK - gt;
    }
  }

  // ---- pass B: emit in index order ------------------------------------------------------------
  for (int c = 0; c < nchunks; ++c) {
    const int k0 = c * kTopkChunk;
    const int klen = min(kTopkChunk, keff - k0);
    const int jmax = (klen + 31) >> 5;
    if (nchunks > 1) {
      __syncthreads();
      load_slab(k0, klen);
      __syncthreads();
    }
#pragma unroll
    for (int rr = 0; rr < ROWS; ++rr) {
      const int tt = warp * ROWS + rr;
      const int t = t0 + tt;
      if (t >= T) continue;  // warp-uniform
      int* o = out + (static_cast<size_t>(t) * H + h) * TOPK;
      // positions to test: the candidates of the only slab, or every position when the slabs were re-streamed
      uint32_t m;
      if (nchunks == 1) {
        m = cand[rr];
      } else {
        m = 0u;
        for (int j = 0; j < jmax; ++j) m |= (lane + 32 * j < klen) ? (1u << j) : 0u;
      }
      uint32_t m_gt = 0u, m_eq = 0u;
      while (m != 0u) {
        const int j = __ffs(m) - 1;
        m &= m - 1;
        const float x = slab[(lane + 32 * j) * PITCH + tt];
        if (x > cut[rr]) m_gt |= 1u << j;
        else if (x == cut[rr]) m_eq |= 1u << j;
      }
      uint32_t sel = m_gt;
      if (ties[rr] > 0) {
        const int n_eq = __reduce_add_sync(0xffffffffu, __popc(m_eq));
        if (n_eq <= ties[rr]) {
          sel |= m_eq;
          ties[rr] -= n_eq;
        } else {
          uint32_t any = __reduce_or_sync(0xffffffffu, m_eq);
          int taken = 0;
          while (any != 0u && taken < ties[rr]) {
            const int j = __ffs(any) - 1;
            any &= any - 1;
            const bool mine = (m_eq >> j) & 1u;
            const uint32_t b = __ballot_sync(0xffffffffu, mine);
            if (mine && taken + __popc(b & lt_mask) < ties[rr]) sel |= 1u << j;
            taken += __popc(b);
          }
          ties[rr] = 0;
        }
      }
      // index order without a sort: bit kl of a 1024-bit map, then lane L owns positions 32 L .. 32 L + 31
      bitmap[warp][lane] = 0u;
      __syncwarp();
      while (sel != 0u) {
        const int j = __ffs(sel) - 1;
        sel &= sel - 1;
        atomicOr(&bitmap[warp][j], 1u << lane);      // kl = lane + 32 j
      }
      __syncwarp();
      uint32_t w = bitmap[warp][lane];
      const int mine = __popc(w);
      int pos = mine;
#pragma unroll
      for (int s2 = 1; s2 < 32; s2 <<= 1) {
        const int o2 = __shfl_up_sync(0xffffffffu, pos, s2);
        if (lane >= s2) pos += o2;
      }
      int at = written[rr];
      const int total_sel = __shfl_sync(0xffffffffu, pos, 31);
      pos = at + pos - mine;
      while (w != 0u) {
        const int b = __ffs(w) - 1;
        w &= w - 1;
        if (pos < TOPK) o[pos] = k0 + 32 * lane + b;
        ++pos;
      }
      at += total_sel;
      __syncwarp();
      written[rr] = at;
    }
  }
#pragma unroll
  for (int rr = 0; rr < ROWS; ++rr) {
    const int t = t0 + warp * ROWS + rr;
    if (t >= T) continue;
    int* o = out + (static_cast<size_t>(t) * H + h) * TOPK;
    for (int e = written[rr] + lane; e < TOPK; e += 32) o[e] = -1;
  }
}

// ---------------------------------------------------------------------------------------------------
// Fast path: at most 1024 candidate pages per row, token count a multiple of 4 (the prefill and decode shapes).
// A CTA owns 16 consecutive tokens of one head: the [K x 16] slab goes to shared memory once (cp.async, 64-byte
// global segments), and the selection never sorts more than a few dozen values per row:
//   A. every row is cut into G = 2 * TOPK interleaved groups (group = page mod G, so that a run of visible pages
//      spreads over all groups); 16 threads per row take their groups' maxima.  The TOPK-th largest group maximum
//      is a lower bound `thr` of the TOPK-th largest score, and only ~1.5 * TOPK scores reach it.
//   B. the same threads collect the scores >= thr (and > -inf) as (score, page) candidates, at most 4 * TOPK;
//   C. a warp ranks a row's candidates against each other (score descending, page ascending: the lower page wins
//      a tie), keeps rank < TOPK, and writes the kept pages in ascending order.
// A row with more candidates than the buffer holds (masses of equal scores) is redone by its warp with a
// bit-by-bit search of the TOPK-th largest key over the slab: slower, exact, and rare.
// Semantics are those of topk_select_kernel: forced tiles rank as FLT_MAX, NaN never wins, +inf ranks with
// FLT_MAX, -0.0 ties with +0.0, a pick scoring -inf is not reported (-1 at the tail).
// ---------------------------------------------------------------------------------------------------
constexpr int kFastTok = 16;

template <int TOPK>
struct __align__(128) TopkFastSmem {
  static constexpr int G = 2 * TOPK;      // groups per row
  static constexpr int C = 4 * TOPK;      // candidate capacity per row
  float slab[kTopkChunk][kFastTok];       // four TMA boxes of 256 pages x 16 tokens
  uint64_t full[2];                       // pages [0, 512) / [512, 1024) have landed
  int abort;
  float gmax[G][kFastTok];
  float cand_v[kFastTok][C];
  short cand_k[kFastTok][C];
  short sel[kFastTok][TOPK];
  float thr[kFastTok];
  int cnt[kFastTok];
};

template <int TOPK>
__global__ void __launch_bounds__(256, TOPK == 16 ? 3 : 2)
topk_select_fast_kernel(const __grid_constant__ CUtensorMap tmap_ms, int H, int K, int T, int nvp, int force_begin,
                        int force_end, int* __restrict__ out, int* status) {
  using Smem = TopkFastSmem<TOPK>;
  constexpr int G = Smem::G, C = Smem::C;
  constexpr int GPT = G / 16;              // groups per thread (16 threads per row)
  extern __shared__ __align__(128) uint8_t topk_raw[];
  Smem& sm = *reinterpret_cast<Smem*>(topk_raw);

  const int h = blockIdx.y;
  const int t0 = blockIdx.x * kFastTok;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int keff = min(K, nvp);            // <= 1024 (host)
  volatile int* abort_flag = &sm.abort;

  // ---- slab in: four TMA boxes (256 pages x 16 tokens, 16 KiB each), issued by one thread; the group maxima of
  // the first two are taken while the last two are still arriving.  Pages past K and tokens past T read zero
  // (TMA fill) and are never looked at: every loop below stops at keff, and rows past T are not emitted. --------
  if (tid == 0) {
    mbar_init(&sm.full[0], 1);
    mbar_init(&sm.full[1], 1);
    sm.abort = 0;
    mbar_fence_init();
  }
  if (tid < kFastTok) sm.cnt[tid] = 0;
  __syncthreads();
  if (tid == 0) {
    tma_prefetch_desc(&tmap_ms);
    for (int half = 0; half < 2; ++half) {
      const int boxes = max(0, min(2, (keff - half * 512 + 255) / 256));
      if (boxes > 0) {
        mbar_expect_tx(&sm.full[half], boxes * 256 * kFastTok * 4);
        for (int b = 0; b < boxes; ++b)
          tma_load_3d(&sm.slab[half * 512 + b * 256][0], &tmap_ms, &sm.full[half], t0, half * 512 + b * 256, h);
      } else {
        mbar_arrive(&sm.full[half]);
      }
    }
  }
  const bool forced_any = force_begin + force_end > 0;
  bool ok = mbar_wait(&sm.full[0], 0, abort_flag);
  // forced tiles are patched after the whole slab is in: wait for everything first in that (uncommon) case
  if (forced_any && ok) ok = mbar_wait(&sm.full[1], 0, abort_flag);
  if (forced_any) __syncthreads();
  // forced tiles rank above everything (at most TOPK rows of the slab)
  for (int idx = tid; idx < (force_begin + force_end) * kFastTok; idx += 256) {
    const int f = idx / kFastTok, tt = idx % kFastTok;
    const int k = f < force_begin ? f : nvp - force_end + (f - force_begin);
    if (k >= 0 && k < keff) sm.slab[k][tt] = 3.402823466e38f;
  }
  if (forced_any) __syncthreads();

  // ---- A: group maxima.  Thread (u, t): pages u, u + 16, u + 32, ...; page u + 16 i belongs to group
  // (u + 16 i) mod G, i.e. local group i mod GPT ------------------------------------------------------------
  const int t = lane & 15, u = warp * 2 + (lane >> 4);
  float gm[GPT];
#pragma unroll
  for (int j = 0; j < GPT; ++j) gm[j] = -INFINITY;
  const int n_i = max(0, min(64, (keff - u + 15) >> 4));   // my pages: u + 16 i, i < n_i
  const float* col = &sm.slab[u][t];                       // page u + 16 i sits 16 * kFastTok floats further on
  // eight loads in flight per step: the loop is bound by shared-memory latency, not by instruction count.
  // A full row (1024 pages: every thread owns 64) takes the loop without the per-element bound checks.
  const bool full_row = keff == kTopkChunk;   // CTA-uniform
  if (full_row) {
#pragma unroll
    for (int i0 = 0; i0 < 64; i0 += 8) {
      if (i0 == 32 && !forced_any && ok) ok = mbar_wait(&sm.full[1], 0, abort_flag);   // pages from 512 on
      float v[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] = col[(i0 + e) * 16 * kFastTok];
      if constexpr (GPT <= 4) {
        // v[e] and v[e + GPT] belong to the same group: one three-input max for the two (NaN never wins)
#pragma unroll
        for (int e = 0; e < 8; ++e)
          if ((e / GPT) % 2 == 0) gm[e % GPT] = max3(gm[e % GPT], v[e], v[e + GPT]);
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) gm[(i0 + e) % GPT] = fmaxf(gm[(i0 + e) % GPT], v[e]);
      }
    }
  } else {
    for (int i0 = 0; i0 < 64; i0 += 8) {
      if (i0 == 32 && !forced_any && ok) ok = mbar_wait(&sm.full[1], 0, abort_flag);   // pages from 512 on
      float v[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] = (i0 + e < n_i) ? col[(i0 + e) * 16 * kFastTok] : -INFINITY;
#pragma unroll
      for (int e = 0; e < 8; ++e) gm[(i0 + e) % GPT] = fmaxf(gm[(i0 + e) % GPT], v[e]);   // NaN never wins
    }
  }
  bool saw_inf = false;
#pragma unroll
  for (int j = 0; j < GPT; ++j) saw_inf |= (gm[j] == INFINITY);
#pragma unroll
  for (int j = 0; j < GPT; ++j) sm.gmax[u + 16 * j][t] = fminf(gm[j], 3.402823466e38f);
  // +inf ranks with FLT_MAX: rewrite such scores in place (rare, CTA-uniform branch)
  if (__syncthreads_or(saw_inf ? 1 : 0)) {
    for (int i = 0; i < 64; ++i) {
      const int k = u + 16 * i;
      if (k < keff && sm.slab[k][t] == INFINITY) sm.slab[k][t] = 3.402823466e38f;
    }
    __syncthreads();
  }

  // ---- threshold of each row: the TOPK-th largest of its G group maxima (warp w: rows 2w, 2w + 1) ------------
  for (int rr = 0; rr < 2; ++rr) {
    const int row = warp * 2 + rr;
    uint32_t gk[G / 32];
#pragma unroll
    for (int a = 0; a < G / 32; ++a) gk[a] = ordered_key(sm.gmax[lane + 32 * a][row] + 0.0f);
    warp_bitonic_sort<G / 32, true>(gk, lane);       // descending
    const uint32_t tk = __shfl_sync(0xffffffffu, gk[(TOPK - 1) >> 5], (TOPK - 1) & 31);
    if (lane == 0) sm.thr[row] = key_value(tk);
  }
  __syncthreads();

  // ---- B: candidates ------------------------------------------------------------------------------------------
  {
    const float thr = sm.thr[t];
    // which of my 64 scores are candidates; slots are then reserved with one shared-memory atomic per pair of
    // threads (lanes l and l ^ 16 serve the same row) instead of one per candidate
    uint32_t m0 = 0u, m1 = 0u;
    // v >= thr && v > -inf  <=>  v >= max(thr, -FLT_MAX); NaN fails the comparison
    const float lower = fmaxf(thr, -3.402823466e38f);
    if (full_row) {
#pragma unroll
      for (int i0 = 0; i0 < 64; i0 += 8) {
        float v[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = col[(i0 + e) * 16 * kFastTok];
        uint32_t bits = 0u;
#pragma unroll
        for (int e = 0; e < 8; ++e) bits |= (v[e] >= lower) ? (1u << e) : 0u;
        if (i0 < 32) m0 |= bits << (i0 & 31);
        else m1 |= bits << (i0 & 31);
      }
    } else {
#pragma unroll
      for (int i0 = 0; i0 < 64; i0 += 8) {
        if (i0 < n_i) {
          float v[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) v[e] = (i0 + e < n_i) ? col[(i0 + e) * 16 * kFastTok] : -INFINITY;
          uint32_t bits = 0u;
#pragma unroll
          for (int e = 0; e < 8; ++e) bits |= (v[e] >= lower) ? (1u << e) : 0u;
          if (i0 < 32) m0 |= bits << (i0 & 31);
          else m1 |= bits << (i0 & 31);
        }
      }
    }
    const int mine = __popc(m0) + __popc(m1);
    const int pair = __shfl_xor_sync(0xffffffffu, mine, 16);
    int slot = 0;
    if (lane < 16 && mine + pair > 0) slot = atomicAdd(&sm.cnt[t], mine + pair);
    slot = __shfl_sync(0xffffffffu, slot, lane & 15) + (lane >= 16 ? pair : 0);
    while (m0 != 0u) {
      const int i = __ffs(m0) - 1;
      m0 &= m0 - 1;
      if (slot < C) {
        sm.cand_v[t][slot] = col[i * 16 * kFastTok] + 0.0f;   // -0.0 -> +0.0
        sm.cand_k[t][slot] = static_cast<short>(u + 16 * i);
      }
      ++slot;
    }
    while (m1 != 0u) {
      const int i = 32 + __ffs(m1) - 1;
      m1 &= m1 - 1;
      if (slot < C) {
        sm.cand_v[t][slot] = col[i * 16 * kFastTok] + 0.0f;
        sm.cand_k[t][slot] = static_cast<short>(u + 16 * i);
      }
      ++slot;
    }
  }
  __syncthreads();

  // ---- C: rank, keep, order, emit (warp w: rows 2w, 2w + 1) --------------------------------------------------
  // Both rows at once when each has at most one candidate per lane (the usual case): the steps below are chains of
  // shuffles and shared-memory round trips, and two independent chains hide each other's latency.  The method is
  // the one described at the single-row code that follows (which takes every other case).
  bool both_done = false;
  if (t0 + warp * 2 + 1 < T && sm.cnt[warp * 2] <= 32 && sm.cnt[warp * 2 + 1] <= 32) {
    const int row0 = warp * 2;
    int nn[2], ka[2], rank[2] = {0, 0};
    uint32_t key[2];
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      nn[q] = sm.cnt[row0 + q];
      const float va = lane < nn[q] ? sm.cand_v[row0 + q][lane] : 0.f;
      ka[q] = lane < nn[q] ? sm.cand_k[row0 + q][lane] : 0;
      key[q] = lane < nn[q] ? ordered_key(va) : 0u;
    }
    const int nmax = max(nn[0], nn[1]);
#pragma unroll 8
    for (int b = 0; b < nmax; ++b) {         // past a row's last candidate the key read is 0 and counts for nothing
#pragma unroll
      for (int q = 0; q < 2; ++q) rank[q] += (__shfl_sync(0xffffffffu, key[q], b) > key[q]) ? 1 : 0;
    }
    bool dup = false;
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      const uint32_t same = __match_any_sync(0xffffffffu, key[q]);
      dup |= lane < nn[q] && (same & (same - 1u)) != 0u;
    }
    if (__any_sync(0xffffffffu, dup)) {
      for (int b = 0; b < nmax; ++b) {
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          const uint32_t kb = __shfl_sync(0xffffffffu, key[q], b);
          const int pb = __shfl_sync(0xffffffffu, ka[q], b);
          rank[q] += (kb != 0u && kb == key[q] && pb < ka[q]) ? 1 : 0;
        }
      }
    }
    uint32_t* map0 = reinterpret_cast<uint32_t*>(sm.cand_v[row0]);
    uint32_t* map1 = reinterpret_cast<uint32_t*>(sm.cand_v[row0 + 1]);
    __syncwarp();
    map0[lane] = 0u;
    map1[lane] = 0u;
    __syncwarp();
    if (lane < nn[0] && rank[0] < TOPK) atomicOr(&map0[ka[0] >> 5], 1u << (ka[0] & 31));
    if (lane < nn[1] && rank[1] < TOPK) atomicOr(&map1[ka[1] >> 5], 1u << (ka[1] & 31));
    __syncwarp();
    uint32_t w[2] = {map0[lane], map1[lane]};
    int mine[2], pre[2];
#pragma unroll
    for (int q = 0; q < 2; ++q) pre[q] = mine[q] = __popc(w[q]);
#pragma unroll
    for (int s2 = 1; s2 < 32; s2 <<= 1) {
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        const int up = __shfl_up_sync(0xffffffffu, pre[q], s2);
        if (lane >= s2) pre[q] += up;
      }
    }
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      int* o = out + (static_cast<size_t>(t0 + row0 + q) * H + h) * TOPK;
      const int n_sel = __shfl_sync(0xffffffffu, pre[q], 31);
      int pos = pre[q] - mine[q];
      uint32_t ww = w[q];
      while (ww != 0u) {
        const int bit = __ffs(ww) - 1;
        ww &= ww - 1;
        o[pos++] = lane * 32 + bit;
      }
      for (int a = lane; a < TOPK; a += 32)
        if (a >= n_sel) o[a] = -1;
    }
    both_done = true;
  }
  for (int rr = 0; rr < 2 && !both_done; ++rr) {
    const int row = warp * 2 + rr;
    const int tok = t0 + row;
    if (tok >= T) continue;                // warp-uniform
    int* o = out + (static_cast<size_t>(tok) * H + h) * TOPK;
    const int n = sm.cnt[row];
    int n_sel = 0;
    if (n <= 32) {
      // The usual case, one candidate per lane, everything from registers: rank = candidates with a greater
      // score (one shuffle and one compare each); equal scores, rare, are ordered by page in a second loop that
      // runs only if some lanes hold the same score.  The kept pages leave in ascending order through a
      // 1024-bit map (the row's candidate buffer, free once the candidates are in registers): lane L owns pages
      // 32 L .. 32 L + 31, a prefix sum of the population counts gives its first output slot.
      const float va = lane < n ? sm.cand_v[row][lane] : 0.f;
      const int ka = lane < n ? sm.cand_k[row][lane] : 0;
      const uint32_t key = lane < n ? ordered_key(va) : 0u;    // > 0 for every candidate (finite scores)
      int rank = 0;
#pragma unroll 8
      for (int b = 0; b < n; ++b)            // n is warp-uniform
        rank += (__shfl_sync(0xffffffffu, key, b) > key) ? 1 : 0;
      const uint32_t same = __match_any_sync(0xffffffffu, key);
      if (__any_sync(0xffffffffu, lane < n && (same & (same - 1u)) != 0u)) {
        for (int b = 0; b < n; ++b) {
          const uint32_t kb = __shfl_sync(0xffffffffu, key, b);
          const int pb = __shfl_sync(0xffffffffu, ka, b);
          rank += (kb == key && pb < ka) ? 1 : 0;
        }
      }
      const bool keep = lane < n && rank < TOPK;
      uint32_t* map = reinterpret_cast<uint32_t*>(sm.cand_v[row]);
      __syncwarp();
      map[lane] = 0u;
      __syncwarp();
      if (keep) atomicOr(&map[ka >> 5], 1u << (ka & 31));
      __syncwarp();
      uint32_t w = map[lane];
      const int mine = __popc(w);
      int pre = mine;
#pragma unroll
      for (int s2 = 1; s2 < 32; s2 <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, pre, s2);
        if (lane >= s2) pre += up;
      }
      n_sel = __shfl_sync(0xffffffffu, pre, 31);
      int pos = pre - mine;
      while (w != 0u) {
        const int bit = __ffs(w) - 1;
        w &= w - 1;
        o[pos++] = lane * 32 + bit;
      }
      for (int a = lane; a < TOPK; a += 32)
        if (a >= n_sel) o[a] = -1;
      continue;
    }
    if (n <= 64) {
      // two candidates per lane (slots lane and lane + 32), same method
      const float va0 = sm.cand_v[row][lane], va1 = lane + 32 < n ? sm.cand_v[row][lane + 32] : 0.f;
      const int ka0 = sm.cand_k[row][lane], ka1 = lane + 32 < n ? sm.cand_k[row][lane + 32] : 0;
      const uint32_t key0 = ordered_key(va0), key1 = lane + 32 < n ? ordered_key(va1) : 0u;
      int rank0 = 0, rank1 = 0;
#pragma unroll 8
      for (int b = 0; b < 32; ++b) {
        const uint32_t kb = __shfl_sync(0xffffffffu, key0, b);
        rank0 += (kb > key0) ? 1 : 0;
        rank1 += (kb > key1) ? 1 : 0;
      }
      for (int b = 32; b < n; ++b) {
        const uint32_t kb = __shfl_sync(0xffffffffu, key1, b - 32);
        rank0 += (kb > key0) ? 1 : 0;
        rank1 += (kb > key1) ? 1 : 0;
      }
      // equal scores: ordered by page (the slower exact comparison, only when some score repeats)
      const uint32_t same0 = __match_any_sync(0xffffffffu, key0), same1 = __match_any_sync(0xffffffffu, key1);
      bool dup = (same0 & (same0 - 1u)) != 0u || (lane + 32 < n && (same1 & (same1 - 1u)) != 0u);
      // a score may also repeat across the two slots: compare against every key of the other slot
      for (int b = 0; b < n - 32; ++b) dup |= __shfl_sync(0xffffffffu, key1, b) == key0;
      if (__any_sync(0xffffffffu, dup)) {
        for (int b = 0; b < n; ++b) {
          const uint32_t kb = b < 32 ? __shfl_sync(0xffffffffu, key0, b) : __shfl_sync(0xffffffffu, key1, b - 32);
          const int pb = b < 32 ? __shfl_sync(0xffffffffu, ka0, b) : __shfl_sync(0xffffffffu, ka1, b - 32);
          rank0 += (kb == key0 && pb < ka0) ? 1 : 0;
          rank1 += (kb == key1 && pb < ka1) ? 1 : 0;
        }
      }
      const bool keep0 = rank0 < TOPK, keep1 = lane + 32 < n && rank1 < TOPK;
      uint32_t* map = reinterpret_cast<uint32_t*>(sm.cand_v[row]);
      __syncwarp();
      map[lane] = 0u;
      __syncwarp();
      if (keep0) atomicOr(&map[ka0 >> 5], 1u << (ka0 & 31));
      if (keep1) atomicOr(&map[ka1 >> 5], 1u << (ka1 & 31));
      __syncwarp();
      uint32_t w = map[lane];
      const int mine = __popc(w);
      int pre = mine;
#pragma unroll
      for (int s2 = 1; s2 < 32; s2 <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, pre, s2);
        if (lane >= s2) pre += up;
      }
      n_sel = __shfl_sync(0xffffffffu, pre, 31);
      int pos = pre - mine;
      while (w != 0u) {
        const int bit = __ffs(w) - 1;
        w &= w - 1;
        o[pos++] = lane * 32 + bit;
      }
      for (int a = lane; a < TOPK; a += 32)
        if (a >= n_sel) o[a] = -1;
      continue;
    }
    if (n <= C) {
      // every lane owns candidates lane, lane + 32, ...; rank = number of candidates that beat it
      for (int a0 = 0; a0 < n; a0 += 32) {
        const int a = a0 + lane;
        const float va = a < n ? sm.cand_v[row][a] : 0.f;
        const int ka = a < n ? sm.cand_k[row][a] : 0;
        int rank = 0;
        int b = 0;
        for (; b + 4 <= n; b += 4) {       // four broadcast reads in flight
          float vb[4];
          int kb[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            vb[e] = sm.cand_v[row][b + e];
            kb[e] = sm.cand_k[row][b + e];
          }
#pragma unroll
          for (int e = 0; e < 4; ++e) rank += (vb[e] > va || (vb[e] == va && kb[e] < ka)) ? 1 : 0;
        }
        for (; b < n; ++b) {
          const float vb = sm.cand_v[row][b];
          const int kb = sm.cand_k[row][b];
          rank += (vb > va || (vb == va && kb < ka)) ? 1 : 0;
        }
        const bool keep = a < n && rank < TOPK;
        const uint32_t m = __ballot_sync(0xffffffffu, keep);
        if (keep) sm.sel[row][n_sel + __popc(m & ((1u << lane) - 1u))] = static_cast<short>(ka);
        n_sel += __popc(m);
      }
    } else {
      // too many candidates (masses of equal scores): search the TOPK-th largest key of the row bit by bit
      const uint32_t* none = nullptr;
      (void)none;
      uint32_t prefix = 0u;
      int need = TOPK;                     // how many of the keys >= prefix-so-far are still wanted
      // keys of finite, non-NaN scores; -inf and NaN rank lowest and are never reported
      auto key_at = [&](int k) -> uint32_t {
        const float v = sm.slab[k][row];
        if (!(v == v) || v == -INFINITY) return 0u;
        return ordered_key(v + 0.0f);
      };
      for (int bit = 31; bit >= 0; --bit) {
        const uint32_t trial = prefix | (1u << bit);
        int c = 0;
        for (int k = lane; k < keff; k += 32) {
          const uint32_t key = key_at(k);
          c += ((key >> bit) == (trial >> bit)) ? 1 : 0;   // keys that match the prefix and have this bit set
        }
        c = __reduce_add_sync(0xffffffffu, c);
        if (c >= need) prefix = trial;       // the TOPK-th largest has this bit set
        else need -= c;                      // all of those are above it
      }
      // prefix = key of the TOPK-th largest (0 if fewer than TOPK reportable scores); `need` of its ties are taken
      int taken_eq = 0;
      for (int k0 = 0; k0 < keff; k0 += 32) {
        const int k = k0 + lane;
        const uint32_t key = k < keff ? key_at(k) : 0u;
        const bool gt = key > prefix && key != 0u;
        const bool eq = key == prefix && key != 0u;
        const uint32_t me = __ballot_sync(0xffffffffu, eq);
        const bool eq_take = eq && (taken_eq + __popc(me & ((1u << lane) - 1u)) < need);
        const bool keep = gt || eq_take;
        const uint32_t mk = __ballot_sync(0xffffffffu, keep);
        const int pos = n_sel + __popc(mk & ((1u << lane) - 1u));
        if (keep && pos < TOPK) sm.sel[row][pos] = static_cast<short>(k);
        n_sel = min(TOPK, n_sel + __popc(mk));
        taken_eq += __popc(me);
      }
    }
    __syncwarp();
    // ascending page order: position = number of kept pages below mine
    for (int a0 = 0; a0 < TOPK; a0 += 32) {
      const int a = a0 + lane;
      if (a < TOPK) {
        if (a < n_sel) {
          const int ka = sm.sel[row][a];
          int pos = 0;
          for (int b = 0; b < n_sel; ++b) pos += (sm.sel[row][b] < ka) ? 1 : 0;
          o[pos] = ka;
        } else {
          o[a] = -1;                       // slots n_sel .. TOPK-1
        }
      }
    }
    __syncwarp();
  }
  if (!ok && tid == 0 && status != nullptr) atomicExch(status, MSA_ERR_TIMEOUT);
}

// [H, K, T] -> [H, K, n_blocks]: max over the tokens of each query block.  A warp owns four consecutive
// blocks of one (head, page) row and has all their loads in flight before it reduces (one 128-token block is
// a single 16-byte load per lane, far too little to cover the memory latency on its own).
constexpr int kBlockMaxPerWarp = 8;
__global__ void block_max_kernel(const float* __restrict__ ms, int K, int T, const int* __restrict__ block_starts,
                                 int n_blocks, float* __restrict__ out) {
  const int warp = (blockIdx.y * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int hk = blockIdx.x;  // h * K + k
  const int b0 = warp * kBlockMaxPerWarp;
  if (b0 >= n_blocks) return;
  const float* row = ms + static_cast<size_t>(hk) * T;
  const bool row_vec = (T % 4 == 0) && ((reinterpret_cast<uintptr_t>(ms) & 15) == 0);
  float m[kBlockMaxPerWarp];
  int s[kBlockMaxPerWarp], e[kBlockMaxPerWarp];
#pragma unroll
  for (int i = 0; i < kBlockMaxPerWarp; ++i) {
    const int b = min(b0 + i, n_blocks - 1);
    s[i] = __ldg(block_starts + b);
    e[i] = __ldg(block_starts + b + 1);
    m[i] = -INFINITY;
  }
  // fast path: every block is at most 128 tokens, 16-byte aligned, a multiple of 4 long
  bool fast = row_vec;
#pragma unroll
  for (int i = 0; i < kBlockMaxPerWarp; ++i) fast = fast && ((s[i] & 3) == 0) && (((e[i] - s[i]) & 3) == 0) && (e[i] - s[i] <= 128);
  if (fast) {
    float4 v[kBlockMaxPerWarp];
#pragma unroll
    for (int i = 0; i < kBlockMaxPerWarp; ++i) {
      const int t = s[i] + lane * 4;
      v[i] = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
      if (t < e[i]) v[i] = __ldcs(reinterpret_cast<const float4*>(row + t));
    }
#pragma unroll
    for (int i = 0; i < kBlockMaxPerWarp; ++i) m[i] = fmaxf(fmaxf(v[i].x, v[i].y), fmaxf(v[i].z, v[i].w));
  } else {
#pragma unroll
    for (int i = 0; i < kBlockMaxPerWarp; ++i)
      for (int t = s[i] + lane; t < e[i]; t += 32) m[i] = fmaxf(m[i], __ldcs(row + t));
  }
#pragma unroll
  for (int i = 0; i < kBlockMaxPerWarp; ++i) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m[i] = fmaxf(m[i], __shfl_xor_sync(0xffffffffu, m[i], o));
    if (lane == 0 && b0 + i < n_blocks) out[static_cast<size_t>(hk) * n_blocks + b0 + i] = m[i];
  }
}

template <int TOPK, int TOK>
static int launch_topk_shape(const float* ms, int H, int K, int T, int nvp, int fb, int fe, int* out,
                             cudaStream_t st) {
  static DeviceSetup setup;
  constexpr int smem = kTopkChunk * (TOK + 1) * static_cast<int>(sizeof(float));
  const int rc = setup.ensure(nullptr, [] {
    return static_cast<int>(
        cudaFuncSetAttribute(topk_select_kernel<TOPK, TOK>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  });
  if (rc != MSA_OK) return rc;
  dim3 grid((T + TOK - 1) / TOK, H);
  topk_select_kernel<TOPK, TOK><<<grid, TOK == 16 ? 256 : 128, smem, st>>>(ms, H, K, T, nvp, fb, fe, out);
  return static_cast<int>(cudaGetLastError());
}

template <int TOPK>
static int launch_topk_fast(const float* ms, int H, int K, int T, int nvp, int fb, int fe, int* out, cudaStream_t st) {
  static DeviceSetup setup;
  constexpr int smem = static_cast<int>(sizeof(TopkFastSmem<TOPK>));
  const int rc = setup.ensure(nullptr, [] {
    return static_cast<int>(
        cudaFuncSetAttribute(topk_select_fast_kernel<TOPK>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  });
  if (rc != MSA_OK) return rc;
  CUtensorMap map;
  const int mrc = make_score_map(&map, ms, H, K, T, kFastTok, 256);
  if (mrc != MSA_OK) return mrc;
  dim3 grid((T + kFastTok - 1) / kFastTok, H);
  topk_select_fast_kernel<TOPK><<<grid, 256, smem, st>>>(map, H, K, T, nvp, fb, fe, out, nullptr);
  return static_cast<int>(cudaGetLastError());
}

template <int TOPK>
static int launch_topk(const float* ms, int H, int K, int T, int nvp, int fb, int fe, int* out, cudaStream_t st) {
  static DeviceSetup setup0;
  int sms0 = 0;
  const int rc0 = setup0.ensure(&sms0, [] { return static_cast<int>(MSA_OK); });
  if (rc0 != MSA_OK) return rc0;
  // up to 1024 candidate pages, 16-byte aligned token rows and enough rows to fill the GPU with 16-token CTAs:
  // the slab-in-shared-memory selection (decode-sized inputs keep the warp-per-row kernel below)
  if ((K < nvp ? K : nvp) <= kTopkChunk && T % 4 == 0 && (reinterpret_cast<uintptr_t>(ms) & 15) == 0 &&
      static_cast<long long>((T + kFastTok - 1) / kFastTok) * H >= 2LL * sms0)
    return launch_topk_fast<TOPK>(ms, H, K, T, nvp, fb, fe, out, st);
  // fewer wide CTAs than two per SM (decode-sized inputs): the narrow shape gives every row its own warp
  // and four times as many CTAs
  static DeviceSetup setup;
  int num_sms = 0;
  const int rc = setup.ensure(&num_sms, [] { return static_cast<int>(MSA_OK); });
  if (rc != MSA_OK) return rc;
  const long long wide_ctas = static_cast<long long>((T + 15) / 16) * H;
  if (wide_ctas < 2LL * num_sms) return launch_topk_shape<TOPK, 4>(ms, H, K, T, nvp, fb, fe, out, st);
  return launch_topk_shape<TOPK, 16>(ms, H, K, T, nvp, fb, fe, out, st);
}

int topk_select(const float* ms, int H, int K, int T, int topk, int nvp, int fb, int fe, int* out, cudaStream_t st) {
  if (ms == nullptr || out == nullptr || H <= 0 || K <= 0 || T < 0) return MSA_ERR_INVALID;
  if (nvp <= 0 || nvp > K || fb < 0 || fe < 0 || fb + fe > topk) return MSA_ERR_INVALID;
  if (H > 65535) return MSA_ERR_TOO_LARGE;
  if (T == 0) return MSA_OK;
  switch (topk) {
    case 16: return launch_topk<16>(ms, H, K, T, nvp, fb, fe, out, st);
    case 32: return launch_topk<32>(ms, H, K, T, nvp, fb, fe, out, st);
    case 64: return launch_topk<64>(ms, H, K, T, nvp, fb, fe, out, st);
    default: return MSA_ERR_UNSUPPORTED;
  }
}

int block_max(const float* ms, int H, int K, int T, const int* block_starts, int n_blocks, float* out,
              cudaStream_t st) {
  if (ms == nullptr || out == nullptr || block_starts == nullptr || H <= 0 || K <= 0) return MSA_ERR_INVALID;
  constexpr int per_cta = 8 * kBlockMaxPerWarp;   // 8 warps
  if ((n_blocks + per_cta - 1) / per_cta > 65535) return MSA_ERR_TOO_LARGE;
  if (n_blocks <= 0) return MSA_OK;
  dim3 grid(H * K, (n_blocks + per_cta - 1) / per_cta);
  block_max_kernel<<<grid, 256, 0, st>>>(ms, K, T, block_starts, n_blocks, out);
  return static_cast<int>(cudaGetLastError());
}

// [n_blocks, row] -> [T, row]: every token of block b receives the block's row (row = heads x topk page ids,
// a multiple of four ints).  One CTA per block; 16-byte stores.
__global__ void __launch_bounds__(256) expand_block_lists_kernel(const int4* __restrict__ lists,
                                                                const int* __restrict__ block_starts, int row4,
                                                                int4* __restrict__ out) {
  const int b = blockIdx.x;
  const int t0 = block_starts[b], t1 = block_starts[b + 1];
  const int n = (t1 - t0) * row4;
  const int4* src = lists + static_cast<size_t>(b) * row4;
  int4* dst = out + static_cast<size_t>(t0) * row4;
  for (int i = threadIdx.x; i < n; i += 256) dst[i] = __ldg(src + i % row4);
}

int expand_block_lists(const int* lists, const int* block_starts, int n_blocks, int H, int topk, int* out,
                       cudaStream_t st) {
  if (lists == nullptr || block_starts == nullptr || out == nullptr || H <= 0 || topk <= 0) return MSA_ERR_INVALID;
  if ((static_cast<long long>(H) * topk) % 4 != 0) return MSA_ERR_UNSUPPORTED;
  if (((reinterpret_cast<uintptr_t>(lists) | reinterpret_cast<uintptr_t>(out)) & 15) != 0) return MSA_ERR_INVALID;
  if (n_blocks <= 0) return MSA_OK;
  expand_block_lists_kernel<<<n_blocks, 256, 0, st>>>(reinterpret_cast<const int4*>(lists), block_starts,
                                                     H * topk / 4, reinterpret_cast<int4*>(out));
  return static_cast<int>(cudaGetLastError());
}

}  // namespace msa
