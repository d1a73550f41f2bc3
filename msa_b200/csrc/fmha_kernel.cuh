// Paged attention forward for sm_100a: one persistent kernel covers the dense pass
// (with or without per-page max score) and the block-sparse pass over the pages each
// query token selected.  (The score-only proxy pass is score_kernel.cuh.)
//
// One CTA per SM loops over work items; an item is one 128-token query tile x NT
// query heads of one KV group.  Roles (warps):
//   [0, 4*NT)     softmax warpgroups, one per query head ("tile"); thread = query row = TMEM lane
//   4*NT          producer: builds the page bitmap of the NEXT item while the current one computes,
//                 prefetches its Q tile, and issues the TMA loads of the K/V pages named by the walk
//   4*NT + 1      MMA issuer (one lane): S_t = Q_t K^T, O_t += P_t V with tcgen05, accumulators in TMEM
//   4*NT + 2, +3  (NVFP4 K/V; FP8 V in the f16-P build) dequantise raw pages into f16 UMMA tiles
// The last four warps form one warpgroup that gives registers back (setmaxnreg) to the softmax
// warpgroups, which keep a whole 128-column S row in registers.
// TMEM columns: S_t at t*128 (P_t aliases the first 64 columns of S_t, the first 32 when P is e4m3),
// O_t at 256 + t*128.
// Pages are walked from the highest logical page down, so the causally masked tile comes first.
//
// K/V formats:
//   bf16   K and V tiles come from TMA in the SW128 UMMA layout; bf16 x bf16 MMAs.
//   e4m3   K pages go to the tensor core as stored (kind::f8f6f4) against Q split into two e4m3
//          terms per row (q = s * (hi + lo), s a power of two).  V pages also feed the tensor core as
//          stored, as the MN-major B operand of kind::f8f6f4 MMAs whose A operand is P rounded to e4m3 in
//          TMEM; the row sum is taken from the unrounded f32 P.
//   e4m3 with f16 P (KV_FP8_F16P, chosen per call): K as above; V is dequantised to f16 by the convert warps
//          and P stays f16 -- slower, P exact to 11 bits.
//   nvfp4  K and V are dequantised (e2m1 x e4m3 block scale, exact in f16); Q is converted to f16.
#pragma once
#include "common.cuh"

namespace msa {

constexpr int kTileBytes = 128 * 128 * 2;  // one 128x128 16-bit operand tile
constexpr int kHalfBytes = kTileBytes / 2;  // one 64-column SW128 sub-tile; also one 128x128 8-bit tile
constexpr int kBitmapWords = 512;           // up to 16384 logical pages per request
constexpr float kRescaleThreshold = 8.0f;   // lazy O rescale: tolerate row-max growth of 2^8
constexpr float kRescaleThresholdE4 = 4.0f; // same when P is e4m3 (max 448): P is carried x2^4, so 2^4 more fits
// P leaves the softmax as a truncated 16-bit float built with integer ops (the f32 -> 16-bit conversion
// instruction shares a pipe with ex2, the unit this kernel saturates):
//   bf16: keep the upper 16 bits of exp2(x + log2(1 + 2^-9)); the added factor centres the truncation error.
//   f16 : exp2(x - 105 + log2(1 + 2^-11)) has the f16 exponent field already in place (f32 bias 127 =
//         f16 bias 15 + 112, and P is carried x2^7 so that values down to 2^-21 stay normal); bits >> 13
//         are the f16.  The row sum carries the same factors and the epilogue divides them out.
constexpr float kBiasBf16 = 0.0028150156f;             // log2(1 + 2^-9)
constexpr float kGainBf16 = 1.001953125f;              // 1 + 2^-9
constexpr float kBiasF16 = 0.00070426374f - 105.0f;    // log2(1 + 2^-11) - 105
constexpr float kGainF16 = 1.00048828125f / 5.1922968585348276e33f;  // (1 + 2^-11) / 2^112
//   e4m3: exp2(x - 116) has the e4m3 exponent field in place (f32 bias 127 = e4m3 bias 7 + 120, P carried
//         x2^4: weights down to 2^-10 of the row maximum stay normal, smaller ones are dropped); bits >> 20,
//         rounded to nearest, are the e4m3.  The gain
//         2^-120 is applied in two halves so that no intermediate of the normalisation leaves the normal
//         f32 range.
constexpr float kBiasE4 = -116.0f;
constexpr float kGainE4Num = 1.0f / 1.152921504606846976e18f;      // 2^-60
constexpr float kGainE4Den = 1.152921504606846976e18f;             // 2^60

enum KvMode : int { KV_BF16 = 0, KV_FP8 = 1, KV_NVFP4 = 2, KV_FP8_F16P = 3 };

// Optional per-role cycle accounting (build with -DMSA_ROLE_TIMING): lane 0 of one warp per role adds the
// cycles it spent in each wait / work phase to a [n_cta][16] int64 buffer set through
// msa_debug_set_timing_buffer().  Compiled out by default.
#ifdef MSA_ROLE_TIMING
#define MSA_TDECL long long tacc[16] = {0}; long long tmark = 0; (void)tmark;
#define MSA_TBEGIN tmark = clock64();
#define MSA_TEND(slot) tacc[slot] += clock64() - tmark;
#define MSA_TFLUSH(cond, lo, hi)                                                              \
  if ((cond) && p.timing != nullptr) {                                                        \
    for (int ti = lo; ti < hi; ++ti) p.timing[static_cast<size_t>(blockIdx.x) * 16 + ti] = tacc[ti]; \
  }
#define MSA_TRACE(slot, iter, val) if (blockIdx.x == 0 && p.timing != nullptr && (iter) >= 56 && (iter) < 88) p.timing[4096 + ((iter) - 56) * 16 + (slot)] = (val);
#else
#define MSA_TRACE(slot, iter, val)
#define MSA_TDECL
#define MSA_TBEGIN
#define MSA_TEND(slot)
#define MSA_TFLUSH(cond, lo, hi)
#endif

struct FmhaParams {
  __nv_bfloat16* out;            // [total_q, Hq, 128] or null
  float* lse;                    // [total_q, Hq] natural-log LSE or null
  float* max_score;              // [Hq, max_k_tiles, total_q] or null; element (h, tile, tok) at h * ms_head + tile * ms_tile + tok
  long long ms_tile, ms_head;
  const int4* work;              // per query tile, two int4: {request, first token (global), valid rows, first token
                                 // (request-local)}, {kv_len, causal offset, first page-table slot | first K/V token, 0}
  const int* kv_indices;         // flat page table (paged)
  const int* kv_block_indexes;   // [total_q, list_heads, topk] request-local page ids, ascending, -1 tail; or null
  const uint8_t* tile_uniform;   // [n_work, list_heads]: 1 = every row of the query tile has the same list; or null
  const uint8_t* k_scale_bytes;  // NVFP4: e4m3 block scales in 128x4 tiles, one 1 KiB block per (page, head)
  const uint8_t* v_scale_bytes;
  int k_scale_tile_bytes;        // score-only pass over packed e2m1 K: scale bytes per (page, head): 1024 (e4m3 per 16
                                 // values) or 512 (ue8m0 per 32 values, k_mx)
  int k_mx;
  int kv_pages;                  // paged K/V: physical pages in the pool (page-table entries are checked against it)
  int fill_tail;                 // score kernel: entries flagged in work[7] write -inf above their page range
  int pack_heads;                // score-only pass: query heads per 128-row tile (a power of two dividing hr), else 1
  const uint8_t* k_raw;          // NVFP4 raw page storage
  const uint8_t* v_raw;
  int Hq, Hkv, hr, topk, list_heads, total_q, max_k_tiles, n_work, n_head_groups, n_items;
  int causal, paged, sparse, do_pv, do_maxscore;
  int half_dim;                  // score kernel: only the first 64 of the 128 head-dim elements count
  float scale_log2;              // softmax scale * log2(e) * (q_scale * k_scale [* k_global])
  float out_scale;               // v_scale * o_scale [* v_global]
  int* status;
  long long* timing;             // role cycle accounting (MSA_ROLE_TIMING builds), else null
};

template <int NT, int KVMODE>
struct FmhaCfg {
  static constexpr bool kQuant = KVMODE != KV_BF16;
  static constexpr bool kKDirectFp8 = KVMODE == KV_FP8 || KVMODE == KV_FP8_F16P;   // K pages feed kind::f8f6f4 MMAs as stored
  static constexpr bool kKConvert = KVMODE == KV_NVFP4;     // K is dequantised by the convert warps
  static constexpr bool kPvFp8 = KVMODE == KV_FP8;          // P.V in e4m3 on the V pages as stored
  static constexpr bool kVConvert = kQuant && !kPvFp8;      // V is dequantised by the convert warps
  static constexpr bool kHasCvt = kKConvert || kVConvert;   // the convert warps have work
  static constexpr bool kQConvert = kQuant;                 // softmax threads rewrite Q (f16, or e4m3 hi/lo)
  static constexpr int kKBytes = kKDirectFp8 ? kHalfBytes : kTileBytes;
  // ring depth: two stages each (four, in the shared memory e4m3 P.V leaves free, measured 20 % slower)
  static constexpr int kKStages = 2;
  static constexpr int kVStages = 2;
  static constexpr int kVBytes = kPvFp8 ? kHalfBytes : kTileBytes;
  static constexpr int kRawStages = kHasCvt ? 2 : 0;
  static constexpr int kRawBytes = KVMODE == KV_NVFP4 ? 10240 : 16384;
  static constexpr int kSoftmaxWarps = 4 * NT;
  // output through shared-memory staging + TMA stores; the two-head NVFP4 variant has no shared memory left
  // for the staging buffers and keeps per-row stores
  static constexpr bool kStageOut = !(KVMODE == KV_NVFP4 && NT == 2);
  static constexpr int kProducerWarp = kSoftmaxWarps;
  static constexpr int kMmaWarp = kSoftmaxWarps + 1;
  static constexpr int kCvtWarp0 = kSoftmaxWarps + 2;
  static constexpr int kCvtThreads = 64;
  static constexpr int kWarps = kSoftmaxWarps + 4;
  static constexpr int kThreads = kWarps * 32;
  // Register split (NT == 2 only): the CTA is launched with 168 registers per thread (384 threads); the
  // helper warpgroup shrinks to 72 and the two softmax warpgroups grow to 216.  setmaxnreg.inc waits,
  // unbounded, for registers released inside the CTA's own launch allocation, so the totals must
  // balance exactly: 256 * 216 + 128 * 72 == 384 * 168.
  static constexpr bool kRebalance = NT == 2;
  static constexpr int kRegsLaunch = 168;
  static constexpr int kRegsSoftmax = 216;
  static constexpr int kRegsHelper = 72;
  static_assert(!kRebalance || (256 * kRegsSoftmax + 128 * kRegsHelper == 384 * kRegsLaunch),
                "setmaxnreg budget must balance or the CTA deadlocks");
  // UMMA operand format of the 16-bit MMAs (A and B must match): bf16 from TMA, f16 once K/V are dequantised
  static constexpr int kFmt16 = kQuant ? 0 : 1;
  // arrivals that release a bitmap buffer: one per softmax warp, the MMA warp, each convert warp
  static constexpr int kBmEmptyCount = kSoftmaxWarps + 1 + (kHasCvt ? 2 : 0);
};

template <int NT, int KVMODE>
struct __align__(1024) FmhaSmem {
  using Cfg = FmhaCfg<NT, KVMODE>;
  uint8_t q[NT][kTileBytes];
  uint8_t k[Cfg::kKStages][Cfg::kKBytes];
  uint8_t v[Cfg::kVStages][Cfg::kVBytes];
  uint8_t raw[Cfg::kRawStages > 0 ? Cfg::kRawStages : 1][Cfg::kRawStages > 0 ? Cfg::kRawBytes : 16];
  // output staging, one 32-row x 32-column bf16 piece (64-byte rows, 64-byte swizzle) per softmax warp: the
  // epilogue writes its rows here and a TMA store moves them out, instead of 16-byte stores scattered over
  // rows that lie num_qo_heads * 256 bytes apart
  alignas(1024) uint8_t o_stage[Cfg::kStageOut ? Cfg::kSoftmaxWarps : 1][Cfg::kStageOut ? 2048 : 16];
  uint64_t q_full, q_ready, q_empty;
  uint64_t k_full[Cfg::kKStages], k_empty[Cfg::kKStages];
  uint64_t v_full[Cfg::kVStages], v_empty[Cfg::kVStages];
  uint64_t raw_full[Cfg::kRawStages > 0 ? Cfg::kRawStages : 1], raw_empty[Cfg::kRawStages > 0 ? Cfg::kRawStages : 1];
  uint64_t s_full[NT], p_full[NT], o_final[NT];
  uint64_t bm_full[2], bm_empty[2];
  uint32_t tmem_base;
  int abort;
  int item_pages[2];   // pages in the walk of the item that owns bitmap buffer b (sparse)
  uint32_t bitmap[2][kBitmapWords];
  // Sparse pass, published by the producer together with the bitmap of buffer b so that no role waits on global
  // memory at an item boundary: the item's work record and, for a tile whose rows all carry one list, that
  // list's cursor (index and page of its last entry inside the request, page of the entry before it).
  int4 item_work[2][2];
  int item_uniform[2];
  int uni_cur[2][4];
};

template <int NT, int KVMODE>
constexpr int fmha_smem_bytes() {
  return static_cast<int>(sizeof(FmhaSmem<NT, KVMODE>)) + 1024;
}

// Walks the pages of one work item from the highest down: a plain countdown for
// the dense pass, the set bits of the union bitmap for the sparse pass.
struct PageWalk {
  const uint32_t* bm;
  uint32_t bits;
  int w;
  int sparse;
  int lo;   // dense walk: first page of the range (a KV split of a short-query call starts above page 0)
  __device__ __forceinline__ void init(int is_sparse, const uint32_t* bitmap, int n_pages, int first_page = 0) {
    sparse = is_sparse;
    bm = bitmap;
    bits = 0;
    lo = first_page;
    w = is_sparse ? (n_pages + 31) >> 5 : n_pages;
  }
  __device__ __forceinline__ int next() {
    if (!sparse) return --w >= 0 ? w + lo : -1;  // lo + n-1 ... lo, then -1
    while (bits == 0) {
      if (--w < 0) return -1;
      bits = bm[w];
    }
    const int b = 31 - __clz(bits);
    bits &= ~(1u << b);
    return (w << 5) + b;
  }
  __device__ __forceinline__ bool more() const {  // would next() return another page?
    if (!sparse) return w > 0;
    if (bits) return true;
    for (int i = w - 1; i >= 0; --i)
      if (bm[i]) return true;
    return false;
  }
};

// What every role needs to know about one work item.
struct ItemInfo {
  int req, tok0, rows, qloc0, h0, g, kv_len, qo_off, kv_base, n_pages_req, walk_n;
  int page_lo;   // dense walk starts at this page (KV splits of short-query calls), else 0
  int out_off;   // added to the token index of output / LSE rows (split s writes rows s * total_q + token)
  bool oversize;
};

// w, w2: the two int4 halves of the item's work record
// SPLITS: the work list may carry KV splits (dense calls with output only); elsewhere the two fields are constants,
// so that the kernels of the other modes carry no trace of them.
template <bool SPLITS>
__device__ __forceinline__ ItemInfo decode_item(const FmhaParams& p, int item, int nt, const int4 w, const int4 w2) {
  ItemInfo it;
  const int hg = item % p.n_head_groups;  // head group fastest: CTAs running side by side share K/V pages
  it.req = w.x;
  it.tok0 = w.y;
  it.rows = SPLITS ? (w.z & 1023) : w.z;     // rows | first page << 10
  it.page_lo = SPLITS ? (w.z >> 10) : 0;
  it.out_off = SPLITS ? w2.w : 0;
  it.qloc0 = w.w;
  it.h0 = hg * nt;
  it.g = it.h0 / p.hr;
  it.kv_len = w2.x;
  it.qo_off = w2.y;
  it.kv_base = w2.z;
  // the sparse pass keeps one bit per logical page of the request in shared memory: a longer request is not
  // walked at all (every role sees an empty item, the producer reports MSA_ERR_UNSUPPORTED in the status word)
  it.oversize = p.sparse && it.kv_len > kBitmapWords * 32 * 128;
  if (it.oversize) it.kv_len = 0;
  it.n_pages_req = (it.kv_len + 127) >> 7;
  int kv_vis = it.kv_len;  // keys visible to the last row of the tile bound the dense walk
  if (p.causal) kv_vis = min(it.kv_len, it.qloc0 + it.rows + it.qo_off);
  const int n_dense = kv_vis > 0 ? (kv_vis + 127) >> 7 : 0;
  it.walk_n = p.sparse ? it.n_pages_req : (SPLITS ? max(0, n_dense - it.page_lo) : n_dense);
  return it;
}
template <bool SPLITS>
__device__ __forceinline__ ItemInfo load_item(const FmhaParams& p, int item, int nt) {
  const int wi = item / p.n_head_groups;
  return decode_item<SPLITS>(p, item, nt, __ldg(p.work + 2 * wi), __ldg(p.work + 2 * wi + 1));
}

// Calls f(entry index, page) for the leading valid entries of one page list (ascending ids, -1 tail):
// 128-bit loads when the list length allows, all issued before the first use.
template <typename F>
__device__ __forceinline__ void for_each_list_entry(const int* list, int topk, F&& f) {
  if ((topk & 15) == 0) {
    // 16 entries at a time: four 128-bit loads issued before the first use
    for (int base = 0; base < topk; base += 16) {
      const int4* src = reinterpret_cast<const int4*>(list + base);
      const int4 v0 = __ldg(src), v1 = __ldg(src + 1), v2 = __ldg(src + 2), v3 = __ldg(src + 3);
      const int e[16] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w, v2.x, v2.y, v2.z, v2.w, v3.x, v3.y, v3.z, v3.w};
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        if (e[i] < 0) return;
        f(base + i, e[i]);
      }
    }
  } else {
    for (int e = 0; e < topk; ++e) {
      const int pg = __ldg(list + e);
      if (pg < 0) return;
      f(e, pg);
    }
  }
}

// e4m3 x4 (one 32-bit word) -> f16 x4, exact
__device__ __forceinline__ void cvt_e4m3x4_f16x4(uint32_t w, uint32_t& lo, uint32_t& hi) {
  asm("{\n"
      ".reg .b16 a, b;\n"
      "mov.b32 {a, b}, %2;\n"
      "cvt.rn.f16x2.e4m3x2 %0, a;\n"
      "cvt.rn.f16x2.e4m3x2 %1, b;\n"
      "}\n"
      : "=r"(lo), "=r"(hi)
      : "r"(w));
}
// e2m1 x8 (one 32-bit word, low nibble = even element) -> f16 x8, exact
__device__ __forceinline__ void cvt_e2m1x8_f16x8(uint32_t w, uint32_t (&o)[4]) {
  asm("{\n"
      ".reg .b8 b0, b1, b2, b3;\n"
      "mov.b32 {b0, b1, b2, b3}, %4;\n"
      "cvt.rn.f16x2.e2m1x2 %0, b0;\n"
      "cvt.rn.f16x2.e2m1x2 %1, b1;\n"
      "cvt.rn.f16x2.e2m1x2 %2, b2;\n"
      "cvt.rn.f16x2.e2m1x2 %3, b3;\n"
      "}\n"
      : "=r"(o[0]), "=r"(o[1]), "=r"(o[2]), "=r"(o[3])
      : "r"(w));
}
__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
// bf16x2 -> f16x2 (round to nearest)
__device__ __forceinline__ uint32_t bf16x2_to_f16x2(uint32_t x) {
  const float lo = __uint_as_float(x << 16);
  const float hi = __uint_as_float(x & 0xffff0000u);
  return pack_f16x2(lo, hi);
}
// two floats -> two e4m3 bytes (low byte = a), and back to floats
__device__ __forceinline__ uint32_t f32x2_to_e4m3x2(float a, float b) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(b), "f"(a));
  return r;
}
__device__ __forceinline__ void e4m3x2_to_f32x2(uint32_t v, float& a, float& b) {
  uint32_t h2;
  asm("{\n.reg .b16 t;\ncvt.u16.u32 t, %1;\ncvt.rn.f16x2.e4m3x2 %0, t;\n}\n" : "=r"(h2) : "r"(v));
  const __half2 h = *reinterpret_cast<__half2*>(&h2);
  a = __low2float(h);
  b = __high2float(h);
}

// MMA issue with everything but the dynamic shared-memory base known at compile time (tile, ring stage,
// k-step): operands then live on the uniform datapath instead of being moved there per instruction.
// TMEM addresses are absolute: the kernel owns all 512 columns, so the allocation starts at column 0.
// S_T (+ d_off columns) = Q_T K^T with the K tile at shared-memory address k_saddr
template <class Cfg, class Smem, int T>
__device__ __forceinline__ void issue_qk_at(Smem& sm, uint32_t k_saddr) {
  constexpr uint32_t desc_hi = smem_desc_hi(1024);
  const uint32_t qa = smem_desc_lo(smem_u32(sm.q[T]), 16), ka = smem_desc_lo(k_saddr, 16);
  constexpr uint32_t d = T * 128;
  if constexpr (Cfg::kKDirectFp8) {
    // S = Q_hi K^T + Q_lo K^T: 2 x 4 steps of 32 contraction bytes inside the 128-byte swizzle row
    constexpr uint32_t idesc = make_idesc(128, 128, 0, 0, 0, 0);
    umma_ss_lohi<0, 1>(d, qa, ka, desc_hi, idesc);
    umma_ss_lohi<1, 1>(d, qa + 2, ka + 2, desc_hi, idesc);
    umma_ss_lohi<1, 1>(d, qa + 4, ka + 4, desc_hi, idesc);
    umma_ss_lohi<1, 1>(d, qa + 6, ka + 6, desc_hi, idesc);
    umma_ss_lohi<1, 1>(d, qa + 1024, ka, desc_hi, idesc);
    umma_ss_lohi<1, 1>(d, qa + 1026, ka + 2, desc_hi, idesc);
    umma_ss_lohi<1, 1>(d, qa + 1028, ka + 4, desc_hi, idesc);
    umma_ss_lohi<1, 1>(d, qa + 1030, ka + 6, desc_hi, idesc);
  } else {
    // the first 64 elements are the first 128-byte swizzle sub-tile
    constexpr uint32_t idesc = make_idesc(128, 128, Cfg::kFmt16, Cfg::kFmt16, 0, 0);
    umma_ss_lohi<0, 0>(d, qa, ka, desc_hi, idesc);
    umma_ss_lohi<1, 0>(d, qa + 2, ka + 2, desc_hi, idesc);
    umma_ss_lohi<1, 0>(d, qa + 4, ka + 4, desc_hi, idesc);
    umma_ss_lohi<1, 0>(d, qa + 6, ka + 6, desc_hi, idesc);
    umma_ss_lohi<1, 0>(d, qa + 1024, ka + 1024, desc_hi, idesc);
    umma_ss_lohi<1, 0>(d, qa + 1026, ka + 1026, desc_hi, idesc);
    umma_ss_lohi<1, 0>(d, qa + 1028, ka + 1028, desc_hi, idesc);
    umma_ss_lohi<1, 0>(d, qa + 1030, ka + 1030, desc_hi, idesc);
  }
}
template <class Cfg, class Smem, int T, int S>
__device__ __forceinline__ void issue_pv_static(Smem& sm, uint32_t accumulate) {
  // B = V tile, MN-major: 16 keys per step = 2 KiB; d halves 16 KiB apart (LBO), 8-key groups 1 KiB apart (SBO)
  constexpr uint32_t desc_hi = smem_desc_hi(1024);
  const uint32_t va = smem_desc_lo(smem_u32(sm.v[S]), kHalfBytes);
  constexpr uint32_t d = 256 + T * 128, a = T * 128;
  if constexpr (Cfg::kPvFp8) {
    // e4m3 P (four per TMEM column) x e4m3 V as stored: a 128-byte row holds all 128 d of one key, 32 keys
    // per step = 4 KiB, 8-key groups 1 KiB apart (SBO); a single 128-byte block along d, so LBO is unused
    constexpr uint32_t idesc8 = make_idesc(128, 128, 0, 0, 0, 1);
    umma_ts_f8_lohi(d, a, va, desc_hi, idesc8, accumulate);
#pragma unroll
    for (int ks = 1; ks < 4; ++ks) umma_ts_f8_lohi(d, a + ks * 8, va + ks * 256, desc_hi, idesc8, 1u);
  } else {
    constexpr uint32_t idesc = make_idesc(128, 128, Cfg::kFmt16, Cfg::kFmt16, 0, 1);
    umma_ts_lohi(d, a, va, desc_hi, idesc, accumulate);
#pragma unroll
    for (int ks = 1; ks < 8; ++ks) umma_ts_lohi(d, a + ks * 8, va + ks * 128, desc_hi, idesc, 1u);
  }
}
// same with the ring stage known at the call site, so that the addresses are constants plus the buffer base
template <class Cfg, class Smem, int T, int S>
__device__ __forceinline__ void issue_qk_static(Smem& sm) {
  issue_qk_at<Cfg, Smem, T>(sm, smem_u32(sm.k[S]));
}
template <class Cfg, class Smem, int T>
__device__ __forceinline__ void issue_qk_stage(Smem& sm, int stage) {
  static_assert(Cfg::kKStages == 2, "one branch per ring stage");
  if (stage == 0) issue_qk_static<Cfg, Smem, T, 0>(sm);
  else issue_qk_static<Cfg, Smem, T, 1>(sm);
}
template <class Cfg, class Smem, int T>
__device__ __forceinline__ void issue_pv_stage(Smem& sm, int stage, uint32_t accumulate) {
  static_assert(Cfg::kVStages == 2, "one branch per ring stage");
  if (stage == 0) issue_pv_static<Cfg, Smem, T, 0>(sm, accumulate);
  else issue_pv_static<Cfg, Smem, T, 1>(sm, accumulate);
}

// (The score-only pass, per-page max of Q K^T with no softmax and no V, is a kernel of its own: score_kernel.cuh.)
// LISTS: 0 = no page lists (dense walk only), 1 = decided at run time by p.sparse (the variant page-list calls
// use).  The dense specialisation is measurably faster than the generic code on dense calls, while the
// generic code is the faster one on page-list calls, so each kind of call gets its own instantiation.
template <int NT, int KVMODE, int LISTS>
__global__ void __launch_bounds__(FmhaCfg<NT, KVMODE>::kThreads, 1)
fmha_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_o,
                const FmhaParams p) {
  using Cfg = FmhaCfg<NT, KVMODE>;
  using Smem = FmhaSmem<NT, KVMODE>;
  constexpr int NK = Cfg::kKStages, NV = Cfg::kVStages;
  constexpr bool kSplits = LISTS == 0;   // only dense calls are ever planned with KV splits
  const bool sparse = LISTS != 0 && p.sparse != 0;
  constexpr int NRAW = Cfg::kRawStages > 0 ? Cfg::kRawStages : 1;
  extern __shared__ uint8_t smem_raw[];
  Smem& sm = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  volatile int* abort_flag = &sm.abort;
  MSA_TDECL

  // ---- one-time setup ---------------------------------------------------------
  if (tid == 0) {
    mbar_init(&sm.q_full, 1);
    mbar_init(&sm.q_ready, 4 * NT);              // one arrival per softmax warp
    mbar_init(&sm.q_empty, 1);
    for (int s = 0; s < NK; ++s) {
      mbar_init(&sm.k_full[s], Cfg::kKConvert ? Cfg::kCvtThreads / 32 : 1);
      mbar_init(&sm.k_empty[s], 1);
    }
    for (int s = 0; s < NV; ++s) {
      mbar_init(&sm.v_full[s], Cfg::kVConvert ? Cfg::kCvtThreads / 32 : 1);
      mbar_init(&sm.v_empty[s], 1);
    }
    for (int s = 0; s < NRAW; ++s) {
      mbar_init(&sm.raw_full[s], 1);
      mbar_init(&sm.raw_empty[s], Cfg::kCvtThreads / 32);
    }
    for (int t = 0; t < NT; ++t) {
      mbar_init(&sm.s_full[t], 1);
      mbar_init(&sm.p_full[t], 128);              // every softmax thread arrives (measured faster than one per warp)
      mbar_init(&sm.o_final[t], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&sm.bm_full[b], 1);
      mbar_init(&sm.bm_empty[b], Cfg::kBmEmptyCount);
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
    tma_prefetch_desc(&tmap_v);
    tma_prefetch_desc(&tmap_o);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;
  // the MMA warp addresses TMEM absolutely (all 512 columns are ours, so the base can only be column 0)
  if (tmem != 0 && tid == 0) sm.abort = 1;
  __syncthreads();
  // The j-th item of this CTA, or -1 past the end.  The list is ordered heaviest first and the CTAs walk it in
  // rounds of gridDim.x items, forwards in even rounds and backwards in odd ones (a snake), so that the CTA
  // that drew the heaviest item of one round draws the lightest of the next.
  const int n_items_eff = (sm.abort == 0) ? p.n_items : 0;
  auto item_of = [&](int j) {
    const int base = j * static_cast<int>(gridDim.x);
    const int idx = (j & 1) ? base + static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x)
                            : base + static_cast<int>(blockIdx.x);
    return (base < n_items_eff && idx < n_items_eff) ? idx : -1;
  };

  if (warp < Cfg::kSoftmaxWarps) {
    // =========================================================================
    // softmax warpgroup of tile t
    // =========================================================================
    if constexpr (Cfg::kRebalance) setmaxnreg_inc<Cfg::kRegsSoftmax>();
    const int t = warp >> 2;
    const int r = tid & 127;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t s_addr = tmem + lane_base + t * 128;
    const uint32_t o_addr = tmem + lane_base + 256 + t * 128;
    constexpr float kBias = Cfg::kPvFp8 ? kBiasE4 : Cfg::kQuant ? kBiasF16 : kBiasBf16;
    constexpr float kGain = Cfg::kPvFp8 ? kGainE4Num : Cfg::kQuant ? kGainF16 : kGainBf16;
    constexpr float kGainDen = Cfg::kPvFp8 ? kGainE4Den : 1.0f;
    constexpr float kThreshold = Cfg::kPvFp8 ? kRescaleThresholdE4 : kRescaleThreshold;
    bool ok = true;
    uint32_t it_total = 0;   // S/P hand-overs so far (barrier phase)
    uint32_t n_q = 0;        // items with at least one page so far (q_full / q_ready phase)
    uint32_t n_fin = 0;      // o_final phase
    // Ring stages are handed back by one softmax thread of the last tile: S of that tile arriving means every
    // MMA issued before it has completed (in-order pipe), i.e. K of this page and V of the previous one are free.
    const bool releaser = (warp == (NT - 1) * 4) && lane == 0;
    uint32_t k_rel = 0, v_rel = 0;

    // state of the item being prepared (filled by setup) and of the item whose output is pending
    struct RowState {
      ItemInfo info;
      PageWalk walk;
      const int* list;
      int cur, cur_page, prev_page, limit_base, first_page, bm;
      float sl2;
      bool row_valid;
    } nx;
    struct Pending {
      float m_used, l_sum, sl2;
      int tok, h, n_iter;
      bool row_valid, valid;
    } pend;
    pend.valid = false;
    pend.m_used = -INFINITY;
    pend.l_sum = 0.f;
    pend.sl2 = 0.f;
    pend.tok = pend.h = pend.n_iter = 0;
    pend.row_valid = false;

    // prepares item `item` (index j in this CTA's sequence): row visibility, list cursor, Q rewrite
    auto setup = [&](int item, int j) {
      nx.bm = j & 1;
      if (sparse) {
        // the producer published the item's work record (and a uniform tile's list cursor) with the bitmap
        ok = ok && mbar_wait(&sm.bm_full[nx.bm], (j >> 1) & 1, abort_flag);
        nx.info = decode_item<kSplits>(p, item, NT, sm.item_work[nx.bm][0], sm.item_work[nx.bm][1]);
      } else {
        nx.info = load_item<kSplits>(p, item, NT);
      }
      const int r_tile = r;   // my row within the work entry
      nx.row_valid = r_tile < nx.info.rows;
      nx.limit_base = -1;
      nx.list = nullptr;
      nx.cur = -1;
      nx.cur_page = -1;
      nx.prev_page = -1;
      nx.sl2 = p.scale_log2;
      if (nx.row_valid) {
        nx.limit_base = nx.info.kv_len - 1;
        if (p.causal) nx.limit_base = min(nx.limit_base, nx.info.qloc0 + r_tile + nx.info.qo_off);
      }
      if (sparse && nx.row_valid) {
        const int lh = (p.list_heads == p.Hkv) ? nx.info.g : (nx.info.h0 + t);
        nx.list = p.kv_block_indexes + (static_cast<size_t>(nx.info.tok0 + r) * p.list_heads + lh) * p.topk;
        if (sm.item_uniform[nx.bm]) {
          nx.cur = sm.uni_cur[nx.bm][0];
          nx.cur_page = sm.uni_cur[nx.bm][1];
          nx.prev_page = sm.uni_cur[nx.bm][2];
        } else {
          int cur = -1, cur_page = -1, prev_page = -1;
          const int npr = nx.info.n_pages_req;
          for_each_list_entry(nx.list, p.topk, [&](int e, int pg) {
            if (pg < npr) {
              prev_page = cur_page;
              cur = e;
              cur_page = pg;
            }
          });
          nx.cur = cur;
          nx.cur_page = cur_page;
          nx.prev_page = prev_page;
        }
      }
      nx.walk.init(sparse, sm.bitmap[nx.bm], nx.info.walk_n, kSplits ? nx.info.page_lo : 0);
      nx.first_page = ok ? nx.walk.next() : -1;
      if (nx.first_page >= 0) {
        if constexpr (Cfg::kQConvert) {
          ok = ok && mbar_wait(&sm.q_full, n_q & 1, abort_flag);
          if (ok) {
            if constexpr (Cfg::kKDirectFp8) {
              // my row -> two e4m3 rows (hi, lo) sharing one power-of-two scale; hi lands on the first
              // 64-column half of the bf16 tile, lo on the second, same row: in place, thread-private
              uint8_t* rowp = sm.q[t] + r * 128;
              uint4 x[16];
#pragma unroll
              for (int c = 0; c < 16; ++c)
                x[c] = *reinterpret_cast<const uint4*>(rowp + (c >> 3) * kHalfBytes + (((c & 7) ^ (r & 7)) << 4));
              float amax = 0.f;
#pragma unroll
              for (int c = 0; c < 16; ++c) {
                const uint32_t w[4] = {x[c].x, x[c].y, x[c].z, x[c].w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  amax = fmaxf(amax, fabsf(__uint_as_float(w[i] << 16)));
                  amax = fmaxf(amax, fabsf(__uint_as_float(w[i] & 0xffff0000u)));
                }
              }
              // power-of-two scale that brings the row maximum into [224, 448]
              float sq = 1.0f;
              if (amax > 0.f && amax < 3.0e38f) {
                int e;
                frexpf(amax, &e);                  // amax = m * 2^e, m in [0.5, 1)
                sq = ldexpf(1.0f, e - 9);          // amax / sq in [256, 512) -> saturates only above 448
                if (amax / sq > 448.0f) sq *= 2.0f;
              }
              const float inv = 1.0f / sq;
              nx.sl2 = p.scale_log2 * sq;
#pragma unroll
              for (int c8 = 0; c8 < 8; ++c8) {     // 16 values -> 16 hi bytes + 16 lo bytes
                uint32_t hi4[4], lo4[4];
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                  const uint4 xv = x[c8 * 2 + half];
                  const uint32_t w[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
                  for (int i = 0; i < 4; i += 2) {
                    float y[4] = {__uint_as_float(w[i] << 16) * inv, __uint_as_float(w[i] & 0xffff0000u) * inv,
                                  __uint_as_float(w[i + 1] << 16) * inv, __uint_as_float(w[i + 1] & 0xffff0000u) * inv};
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
              // bf16 -> f16 in place (the dequantised K/V tiles are f16 and the tensor core wants one format)
              uint4* qv = reinterpret_cast<uint4*>(sm.q[t]);
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
          if (lane == 0) mbar_arrive(&sm.q_ready);
        }
        ++n_q;
      }
    };

    // writes the output of the finished item: O / l, LSE; called after the next item's setup so the
    // tensor core already works on it
    auto epilogue = [&]() {
      if (!pend.valid) return;
      pend.valid = false;
      if (pend.n_iter > 0) {
        ok = ok && mbar_wait(&sm.o_final[t], n_fin & 1, abort_flag);
        ++n_fin;
        tc_fence_after();
        if (releaser && ok) {   // the item's last V tile has been consumed
          mbar_arrive(&sm.v_empty[v_rel % NV]);
          ++v_rel;
        }
      }
      if (!ok) return;
      const float inv = (pend.l_sum > 0.f) ? p.out_scale * kGain / (pend.l_sum * kGainDen) : 0.f;
      __nv_bfloat16* orow = p.out + (static_cast<size_t>(pend.tok) * p.Hq + pend.h) * 128;
      // a warp whose 32 rows all exist stages its piece in shared memory and lets TMA write it (rows of other
      // requests follow a partial tile in the output, so such a tile keeps the per-row stores)
      const bool via_tma = Cfg::kStageOut && __all_sync(0xffffffffu, pend.row_valid);
      uint8_t* stage = sm.o_stage[Cfg::kStageOut ? warp : 0];
      const int row32 = r & 31;
      // the whole O row at once (the registers of the S row are free here): one TMEM round trip, not four
      uint32_t rg[128];
      if (pend.n_iter > 0) {
        tmem_ld32p(o_addr, rg);
        tmem_ld32p(o_addr + 32, rg + 32);
        tmem_ld32p(o_addr + 64, rg + 64);
        tmem_ld32p(o_addr + 96, rg + 96);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int e = 0; e < 128; ++e) rg[e] = 0u;
      }
      // O has been read: the next item's first PV may overwrite it (it waits for my next P anyway)
      tc_fence_before();
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint4 o[4];
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          const int e = c * 32 + v * 8;
          o[v].x = pack_bf16x2(__uint_as_float(rg[e + 0]) * inv, __uint_as_float(rg[e + 1]) * inv);
          o[v].y = pack_bf16x2(__uint_as_float(rg[e + 2]) * inv, __uint_as_float(rg[e + 3]) * inv);
          o[v].z = pack_bf16x2(__uint_as_float(rg[e + 4]) * inv, __uint_as_float(rg[e + 5]) * inv);
          o[v].w = pack_bf16x2(__uint_as_float(rg[e + 6]) * inv, __uint_as_float(rg[e + 7]) * inv);
        }
        if (via_tma) {
          if (lane == 0) tma_store_wait_read();   // the previous piece has left the staging buffer
          __syncwarp();
          // 64-byte swizzle: 16-byte chunk v of row i sits at chunk v ^ ((i >> 1) & 3)
#pragma unroll
          for (int v = 0; v < 4; ++v)
            *reinterpret_cast<uint4*>(stage + row32 * 64 + ((v ^ ((row32 >> 1) & 3)) << 4)) = o[v];
          fence_proxy_async();
          __syncwarp();
          if (lane == 0) {
            tma_store_3d(&tmap_o, stage, c * 32, pend.h, pend.tok - row32);
            tma_store_commit();
          }
        } else if (pend.row_valid) {
          uint4* dst = reinterpret_cast<uint4*>(orow + c * 32);
#pragma unroll
          for (int v = 0; v < 4; ++v) dst[v] = o[v];
        }
      }
      if (p.lse != nullptr && pend.row_valid) {
        const float v = (pend.l_sum > 0.f)
                            ? (pend.m_used * pend.sl2 + log2f(pend.l_sum) - kBias) * 0.6931471805599453f
                            : -INFINITY;
        p.lse[static_cast<size_t>(pend.tok) * p.Hq + pend.h] = v;
      }
    };

    // The loop starts one (virtual) item early: its first pass has nothing to compute and only prepares the
    // CTA's first item, so that setup -- a long unrolled piece of code -- has a single call site.
    for (int j = -1; ok; ++j) {
      if (j >= 0 && item_of(j) < 0) break;
      if (j >= 0) {
      // ---- main loop of the item prepared in nx -------------------------------
      const ItemInfo info = nx.info;
      const int h = info.h0 + t;
      const int tok = info.tok0 + r;
      const bool row_valid = nx.row_valid;
      const int limit_base = nx.limit_base;
      const int* list = nx.list;
      int cur = nx.cur, cur_page = nx.cur_page, prev_page = nx.prev_page;
      const float sl2 = nx.sl2;
      const float ms_scale = sl2 / p.scale_log2;   // un-does the per-row Q scale for the raw max score
      PageWalk walk = nx.walk;
      const int my_bm = nx.bm;
      float m_used = -INFINITY, l_sum = 0.f;
      int n_iter = 0;

      for (int page = nx.first_page; page >= 0 && ok; page = walk.next(), ++n_iter, ++it_total) {
        // visibility of this page for my row
        int limit = limit_base - (page << 7);
        if (sparse) {
          // the walk descends, so does the cursor; the entry below the current one is fetched one step
          // ahead so that its load latency never sits in front of a softmax step
          while (cur >= 0 && cur_page > page) {
            --cur;
            cur_page = prev_page;
            prev_page = cur > 0 ? __ldg(list + cur - 1) : -1;
          }
          if (!(cur >= 0 && cur_page == page)) limit = -1;
        }
        const bool full_vis = __all_sync(0xffffffffu, limit >= 127);

        MSA_TBEGIN
        ok = mbar_wait(&sm.s_full[t], it_total & 1, abort_flag);
        MSA_TEND(0)
        if (!ok) break;
        tc_fence_after();
        if (releaser) {
          mbar_arrive(&sm.k_empty[k_rel % NK]);
          ++k_rel;
          if (n_iter > 0) {
            mbar_arrive(&sm.v_empty[v_rel % NV]);
            ++v_rel;
          }
        }
        if (r == 0) { MSA_TRACE(t * 2, it_total, clock64()) }
        MSA_TBEGIN

        // the whole 128-column S row of this thread, one wait for the four loads
        uint32_t sr[128];
        tmem_ld32p(s_addr, sr);
        tmem_ld32p(s_addr + 32, sr + 32);
        tmem_ld32p(s_addr + 64, sr + 64);
        tmem_ld32p(s_addr + 96, sr + 96);
        tmem_ld_wait();
        if (!full_vis) {
#pragma unroll
          for (int c = 0; c < 128; ++c) sr[c] = (c <= limit) ? sr[c] : 0xff800000u;
        }
        float t0 = -INFINITY, t1 = -INFINITY, t2 = -INFINITY, t3 = -INFINITY;   // four chains, not one
#pragma unroll
        for (int c = 0; c < 128; c += 8) {
          t0 = max3(t0, __uint_as_float(sr[c]), __uint_as_float(sr[c + 1]));
          t1 = max3(t1, __uint_as_float(sr[c + 2]), __uint_as_float(sr[c + 3]));
          t2 = max3(t2, __uint_as_float(sr[c + 4]), __uint_as_float(sr[c + 5]));
          t3 = max3(t3, __uint_as_float(sr[c + 6]), __uint_as_float(sr[c + 7]));
        }
        const float tmax = fmaxf(fmaxf(t0, t1), fmaxf(t2, t3));
        if (p.do_maxscore && row_valid)
          __stwt(p.max_score + h * p.ms_head + page * p.ms_tile + tok, tmax * ms_scale);

        const float m_new = fmaxf(m_used, tmax);
        const bool first = (m_used == -INFINITY);
        const bool need = !first && ((m_new - m_used) * sl2 > kThreshold);
        if (__any_sync(0xffffffffu, need)) {
          // every MMA issued before the one that produced this S tile has completed, so O is quiescent;
          // eight columns at a time keeps the S row resident in registers
          const float alpha = need ? fast_exp2((m_used - m_new) * sl2) : 1.0f;
#pragma unroll 1
          for (int c = 0; c < 16; ++c) {
            uint32_t rg[8];
            tmem_ld8(o_addr + c * 8, rg);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 8; ++e) rg[e] = __float_as_uint(__uint_as_float(rg[e]) * alpha);
            tmem_st8(o_addr + c * 8, rg);
          }
          l_sum *= alpha;
        }
        if (need || first) m_used = m_new;
        const float mb = (m_used == -INFINITY) ? 0.f : m_used * sl2;

        // P = exp2(S * scale - m * scale) -> 16-bit pairs into the first 64 columns of S (packed fp32 math);
        // each S register dies as its exponential is taken
        const uint64_t sl2_2 = pack2(sl2, sl2), nmb_2 = pack2(kBias - mb, kBias - mb);
        uint64_t acc = 0ull;
        if constexpr (Cfg::kPvFp8) {
          // e4m3: four P per column, the first 32 columns of S
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t pk[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              const int col = c * 32 + 4 * e;
              float x0, x1, x2, x3;
              unpack2(fma2(pack2u(sr[col], sr[col + 1]), sl2_2, nmb_2), x0, x1);
              unpack2(fma2(pack2u(sr[col + 2], sr[col + 3]), sl2_2, nmb_2), x2, x3);
              const float p0 = fast_exp2(x0), p1 = fast_exp2(x1), p2 = fast_exp2(x2), p3 = fast_exp2(x3);
              const uint64_t p01 = pack2(p0, p1), p23 = pack2(p2, p3);
              acc = add2(acc, p01);
              acc = add2(acc, p23);
              // f32 bits [26:20] are the e4m3.  The upper halves of two values are packed into one word first
              // (bits [10:4] of each half); one shift-add then rounds both to nearest and leaves them in bytes 1
              // and 3 (the exponent field never passes 15, so nothing crosses from the lower half into the upper)
              const uint32_t lo = (__byte_perm(__float_as_uint(p0), __float_as_uint(p1), 0x7632) << 4) + 0x00800080u;
              const uint32_t hi = (__byte_perm(__float_as_uint(p2), __float_as_uint(p3), 0x7632) << 4) + 0x00800080u;
              pk[e] = __byte_perm(lo, hi, 0x7531);
            }
            tmem_st8(s_addr + c * 8, pk);
          }
        } else {
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          uint32_t pk[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const int col = c * 16 + 2 * e;
            float x0, x1;
            unpack2(fma2(pack2u(sr[col], sr[col + 1]), sl2_2, nmb_2), x0, x1);
            const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
            acc = add2(acc, pack2(p0, p1));
            pk[e] = Cfg::kQuant ? __byte_perm(__float_as_uint(p0) >> 13, __float_as_uint(p1) >> 13, 0x5410)
                                : __byte_perm(__float_as_uint(p0), __float_as_uint(p1), 0x7632);
          }
          tmem_st8(s_addr + c * 8, pk);
        }
        }
        {
          float a0, a1;
          unpack2(acc, a0, a1);
          l_sum += a0 + a1;
        }
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(&sm.p_full[t]);
        if (r == 0) { MSA_TRACE(t * 2 + 1, it_total, clock64()) }
        MSA_TEND(1)
      }
      // this item's bitmap is no longer needed by my warp
      if (sparse) {
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm.bm_empty[my_bm]);
      }
      pend.valid = true;
      pend.m_used = m_used;
      pend.l_sum = l_sum;
      pend.sl2 = sl2;
      pend.tok = kSplits ? tok + info.out_off : tok;
      pend.h = h;
      pend.n_iter = n_iter;
      pend.row_valid = row_valid;
      }
      // ---- drain this item's O, then prepare the next item.  The next Q was requested only when this item's
      // last QK completed and is still on its way from HBM: the drain fills that wait, and the Q rewrite that
      // follows finds its tile in shared memory.
      const int next_item = item_of(j + 1);
      MSA_TBEGIN
      epilogue();
      if (r == 0 && t == 0) { MSA_TRACE(10, it_total, clock64()) }
      MSA_TEND(10)
      MSA_TBEGIN
      if (r == 0 && t == 0) { MSA_TRACE(8, it_total, clock64()) }
      if (next_item >= 0 && ok) setup(next_item, j + 1);
      if (r == 0 && t == 0) { MSA_TRACE(9, it_total, clock64()) }
      MSA_TEND(2)
    }
    if (lane == 0) tma_store_wait_all();   // this warp's output pieces have left shared memory and are written
    MSA_TFLUSH(tid == 0, 0, 3)
    MSA_TFLUSH(tid == 0, 10, 11)
  } else {
    if constexpr (Cfg::kRebalance) setmaxnreg_dec<Cfg::kRegsHelper>();
    if (warp == Cfg::kProducerWarp) {
      // =======================================================================
      // producer: per item the page bitmap (sparse), Q, then K (and V) of every walked page
      // =======================================================================
      bool ok = true;
      uint32_t n_q = 0, k_seq = 0, v_seq = 0, raw_seq = 0;
      uint32_t pg_total = 0;   // pages issued so far (trace index of an item's first iteration)
      (void)pg_total;
      // Sparse pass: bitmap, page count and metadata of item `item` (the jj-th of this CTA) into buffer jj & 1.
      // All lanes take part.  It runs one item ahead, in the middle of the previous item's page loads (when the
      // rings are full and the warp would only wait), so its global-memory latency is off every critical path.
      auto build_bitmap = [&](int item, int jj) {
        const int b = jj & 1;
        const int wi = item / p.n_head_groups;
        const int4 w = __ldg(p.work + 2 * wi), w2 = __ldg(p.work + 2 * wi + 1);
        const ItemInfo info = decode_item<kSplits>(p, item, NT, w, w2);
        const int lh = (p.list_heads == p.Hkv) ? info.g : info.h0;
        const bool uniform = p.tile_uniform != nullptr &&
                             __ldg(p.tile_uniform + static_cast<size_t>(wi) * p.list_heads + lh) != 0;
        if (info.oversize && lane == 0) atomicExch(p.status, MSA_ERR_UNSUPPORTED);
        // the buffer was used by item jj - 2: wait until every walker released it
        ok = mbar_wait(&sm.bm_empty[b], ((jj >> 1) & 1) ^ 1, abort_flag);
        if (!ok) return;
        const int words = (info.n_pages_req + 31) >> 5;
        for (int x = lane; x < words; x += 32) sm.bitmap[b][x] = 0;
        __syncwarp();
        // the union of the pages any row of the tile selected and can see
        const int npr = info.n_pages_req;
        uint32_t* bmw = sm.bitmap[b];
        int cur = -1, cur_page = -1, prev_page = -1;
        if (uniform) {
          // one list for the whole tile (the usual case: pages are selected per query block): its entries,
          // one per lane, cut at what the tile's last row can see
          int lim = info.kv_len - 1;
          if (p.causal) lim = min(lim, info.qloc0 + info.rows - 1 + info.qo_off);
          const int* list = p.kv_block_indexes + (static_cast<size_t>(info.tok0) * p.list_heads + lh) * p.topk;
          for (int e0 = 0; e0 < p.topk; e0 += 32) {
            const int e = e0 + lane;
            const int pg = e < p.topk ? __ldg(list + e) : -1;
            const bool inside = pg >= 0 && pg < npr;
            if (inside && (pg << 7) <= lim) atomicOr(&bmw[pg >> 5], 1u << (pg & 31));
            // cursor: the last entry inside the request and the page before it (entries ascend, -1 only at the tail)
            const uint32_t m = __ballot_sync(0xffffffffu, inside);
            if (m != 0u) {
              const int last = 31 - __clz(m);
              const int pg_last = __shfl_sync(0xffffffffu, pg, last);
              const int pg_before = __shfl_sync(0xffffffffu, pg, last > 0 ? last - 1 : 0);
              prev_page = last > 0 ? pg_before : cur_page;
              cur = e0 + last;
              cur_page = pg_last;
            }
          }
        } else {
          for (int rr = lane; rr < info.rows; rr += 32) {
            int lim = info.kv_len - 1;
            if (p.causal) lim = min(lim, info.qloc0 + rr + info.qo_off);
            const int* list = p.kv_block_indexes + (static_cast<size_t>(info.tok0 + rr) * p.list_heads + lh) * p.topk;
            for_each_list_entry(list, p.topk, [&](int, int pg) {
              if (pg < npr && (pg << 7) <= lim) atomicOr(&bmw[pg >> 5], 1u << (pg & 31));
            });
          }
        }
        __syncwarp();
        int cnt = 0;
        for (int x = lane; x < words; x += 32) cnt += __popc(sm.bitmap[b][x]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
        if (lane == 0) {
          sm.item_pages[b] = cnt;
          sm.item_work[b][0] = w;
          sm.item_work[b][1] = w2;
          sm.item_uniform[b] = uniform ? 1 : 0;
          sm.uni_cur[b][0] = cur;
          sm.uni_cur[b][1] = cur_page;
          sm.uni_cur[b][2] = prev_page;
        }
        __threadfence_block();
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm.bm_full[b]);
      };
      MSA_TBEGIN
      if (sparse && item_of(0) >= 0) build_bitmap(item_of(0), 0);
      MSA_TEND(11)
      for (int j = 0; ok; ++j) {
        const int item = item_of(j);
        if (item < 0) break;
        if (lane == 0) { MSA_TRACE(11, pg_total, clock64()) }
        const int b = j & 1;
        const ItemInfo info = sparse ? decode_item<kSplits>(p, item, NT, sm.item_work[b][0], sm.item_work[b][1])
                                       : load_item<kSplits>(p, item, NT);
        const int next_item = item_of(j + 1);
        bool next_pending = sparse && next_item >= 0;
        if (lane == 0) { MSA_TRACE(12, pg_total, clock64()) }
        PageWalk walk;
        walk.init(sparse, sm.bitmap[b], info.walk_n, kSplits ? info.page_lo : 0);
        int page = walk.next();
        if (page >= 0) {
          // Q of this item: the tile buffer is free once the previous item's last QK has completed
          if (lane == 0) {
            MSA_TBEGIN
            ok = mbar_wait(&sm.q_empty, (n_q & 1) ^ 1, abort_flag);
            MSA_TEND(12)
            if (ok) {
              MSA_TRACE(13, pg_total, clock64())
              mbar_expect_tx(&sm.q_full, NT * kTileBytes);
              for (int t = 0; t < NT; ++t) {
                const int qh = info.h0 + t, qt = info.tok0;
                tma_load_3d(sm.q[t], &tmap_q, &sm.q_full, 0, qh, qt);
                tma_load_3d(sm.q[t] + kHalfBytes, &tmap_q, &sm.q_full, 64, qh, qt);
              }
            }
          }
          ++n_q;
          ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        }
        const int page_base = p.paged ? info.kv_base : 0;
        const int tok_base = p.paged ? 0 : info.kv_base;
        // K (and V) of one page into the next ring slots (lane 0)
        auto load_page = [&](int page) {
          int phys = p.paged ? __ldg(p.kv_indices + page_base + page) : 0;
          if (static_cast<unsigned>(phys) >= static_cast<unsigned>(p.kv_pages) && p.paged) {
            // a corrupt page table: report it and read page 0 instead of memory outside the pool
            atomicExch(p.status, MSA_ERR_BOUNDS);
            phys = 0;
          }
          const int tok_k = tok_base + (page << 7);
          const size_t tile = static_cast<size_t>(phys) * p.Hkv + info.g;
          // ---- K ----
          if constexpr (Cfg::kKConvert) {
            const int s = raw_seq % NRAW;
            ok = mbar_wait(&sm.raw_empty[s], ((raw_seq / NRAW) & 1) ^ 1, abort_flag);
            if (!ok) return;
            ++raw_seq;
            mbar_expect_tx(&sm.raw_full[s], 8192 + 1024);
            bulk_load(sm.raw[s], p.k_raw + tile * 8192, 8192, &sm.raw_full[s]);
            bulk_load(sm.raw[s] + 8192, p.k_scale_bytes + tile * 1024, 1024, &sm.raw_full[s]);
          } else {
            const int s = k_seq % NK;
            uint8_t* kdst = sm.k[s];
            MSA_TBEGIN
            ok = mbar_wait(&sm.k_empty[s], ((k_seq / NK) & 1) ^ 1, abort_flag);
            MSA_TEND(13)
            if (!ok) return;
            ++k_seq;
            mbar_expect_tx(&sm.k_full[s], Cfg::kKBytes);
            if constexpr (Cfg::kKDirectFp8) {
              if (p.paged)
                tma_load_4d(kdst, &tmap_k, &sm.k_full[s], 0, 0, info.g, phys);
              else
                tma_load_3d(kdst, &tmap_k, &sm.k_full[s], 0, info.g, tok_k);
            } else if (p.paged) {
              tma_load_4d(kdst, &tmap_k, &sm.k_full[s], 0, 0, info.g, phys);
              tma_load_4d(kdst + kHalfBytes, &tmap_k, &sm.k_full[s], 64, 0, info.g, phys);
            } else {
              tma_load_3d(kdst, &tmap_k, &sm.k_full[s], 0, info.g, tok_k);
              tma_load_3d(kdst + kHalfBytes, &tmap_k, &sm.k_full[s], 64, info.g, tok_k);
            }
          }
          // ---- V ----
          if constexpr (Cfg::kVConvert) {
            const int s = raw_seq % NRAW;
            ok = mbar_wait(&sm.raw_empty[s], ((raw_seq / NRAW) & 1) ^ 1, abort_flag);
            if (!ok) return;
            ++raw_seq;
            if constexpr (Cfg::kKDirectFp8) {
              mbar_expect_tx(&sm.raw_full[s], 16384);
              if (p.paged)
                tma_load_4d(sm.raw[s], &tmap_v, &sm.raw_full[s], 0, 0, info.g, phys);
              else
                tma_load_3d(sm.raw[s], &tmap_v, &sm.raw_full[s], 0, info.g, tok_k);
            } else {
              mbar_expect_tx(&sm.raw_full[s], 8192 + 1024);
              bulk_load(sm.raw[s], p.v_raw + tile * 8192, 8192, &sm.raw_full[s]);
              bulk_load(sm.raw[s] + 8192, p.v_scale_bytes + tile * 1024, 1024, &sm.raw_full[s]);
            }
          } else {
            const int s = v_seq % NV;
            ok = mbar_wait(&sm.v_empty[s], ((v_seq / NV) & 1) ^ 1, abort_flag);
            if (!ok) return;
            ++v_seq;
            mbar_expect_tx(&sm.v_full[s], Cfg::kPvFp8 ? kHalfBytes : kTileBytes);
            if constexpr (Cfg::kPvFp8) {
              if (p.paged)
                tma_load_4d(sm.v[s], &tmap_v, &sm.v_full[s], 0, 0, info.g, phys);
              else
                tma_load_3d(sm.v[s], &tmap_v, &sm.v_full[s], 0, info.g, tok_k);
            } else if (p.paged) {
              tma_load_4d(sm.v[s], &tmap_v, &sm.v_full[s], 0, 0, info.g, phys);
              tma_load_4d(sm.v[s] + kHalfBytes, &tmap_v, &sm.v_full[s], 64, 0, info.g, phys);
            } else {
              tma_load_3d(sm.v[s], &tmap_v, &sm.v_full[s], 0, info.g, tok_k);
              tma_load_3d(sm.v[s] + kHalfBytes, &tmap_v, &sm.v_full[s], 64, info.g, tok_k);
            }
          }
        };
        int issued = 0;
        for (; page >= 0 && ok; page = walk.next()) {
          ++pg_total;
          if (lane == 0) load_page(page);
          ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
          // three pages of this item are on their way: time to prepare the next item
          if (++issued == 3 && next_pending && ok) {
            MSA_TBEGIN
            build_bitmap(next_item, j + 1);
            MSA_TEND(11)
            next_pending = false;
          }
        }
        if (next_pending && ok) {
          MSA_TBEGIN
          build_bitmap(next_item, j + 1);
          MSA_TEND(11)
        }
      }
      MSA_TFLUSH(lane == 0, 11, 14)
      if (!ok && lane == 0) {
        // give copies in flight a bounded time to land before the CTA tears down
        const long long t0 = clock64();
        while (clock64() - t0 < (1LL << 22)) {
        }
      }
    } else if (warp == Cfg::kMmaWarp) {
      // =======================================================================
      // MMA issuer.  Its single issuing lane is the serial heart of the pipeline, so it does nothing but
      // wait for P / operand stages and issue: ring stages are released by a softmax thread (which sees
      // the same completion through S), and the walk length comes precomputed from the producer.
      // =======================================================================
      bool ok = true;
      uint32_t n_q = 0, k_seq = 0, v_seq = 0, it_total = 0;
      for (int j = 0; ok; ++j) {
        const int item = item_of(j);
        if (item < 0) break;
        const int b = j & 1;
        int count;
        if (sparse) {
          ok = mbar_wait(&sm.bm_full[b], (j >> 1) & 1, abort_flag);
          if (!ok) break;
          count = sm.item_pages[b];
        } else {
          count = load_item<kSplits>(p, item, NT).walk_n;
        }
        if (count > 0) {
          MSA_TBEGIN
          ok = mbar_wait(Cfg::kQConvert ? &sm.q_ready : &sm.q_full, n_q & 1, abort_flag);
          MSA_TEND(14)
          if (lane == 0) { MSA_TRACE(14, it_total, clock64()) }
          ++n_q;
          // Pass i = -1 has no P to wait for and only issues S_t(0) = Q_t K(0)^T, so that every MMA group has a
          // single issue site; pass i issues O_t += P_t(i) V(i) and S_t(i + 1) = Q_t K(i + 1)^T.
          for (int i = -1; i < count && ok; ++i) {
            const bool real = i >= 0;
            const bool has_next = i + 1 < count;
            int v_stage = 0, k_stage = 0;
            uint32_t k_this = 0;
            if (real) {
              v_stage = v_seq % NV;
              MSA_TBEGIN
              ok = mbar_wait(&sm.v_full[v_stage], (v_seq / NV) & 1, abort_flag);
              MSA_TEND(3)
              ++v_seq;
            }
            if (has_next) {
              k_this = k_seq;
              k_stage = k_seq % NK;
              ++k_seq;
            }
#pragma unroll
            for (int t = 0; t < NT; ++t) {
              if (!ok) break;
              if (real) {
                MSA_TBEGIN
                ok = mbar_wait(&sm.p_full[t], it_total & 1, abort_flag);
                MSA_TEND(4 + t)
                if (!ok) break;
              }
              if (t == 0 && has_next) {
                MSA_TBEGIN
                ok = mbar_wait(&sm.k_full[k_stage], (k_this / NK) & 1, abort_flag);
                MSA_TEND(6)
                if (!ok) break;
              }
              tc_fence_after();
              if (lane == 0) {
                MSA_TRACE(4 + t * 2, it_total, clock64())
                if (real) {
                  if (t == 0) issue_pv_stage<Cfg, Smem, 0>(sm, v_stage, i > 0 ? 1u : 0u);
                  else issue_pv_stage<Cfg, Smem, NT - 1>(sm, v_stage, i > 0 ? 1u : 0u);
                }
                if (has_next) {
                  if (t == 0) issue_qk_stage<Cfg, Smem, 0>(sm, k_stage);
                  else issue_qk_stage<Cfg, Smem, NT - 1>(sm, k_stage);
                  umma_commit(&sm.s_full[t]);
                  // the QK just issued for the last tile is the item's last: Q may be overwritten after it
                  if (t == NT - 1 && i + 2 == count) umma_commit(&sm.q_empty);
                } else if (real) {
                  umma_commit(&sm.o_final[t]);
                }
                MSA_TRACE(5 + t * 2, it_total, clock64())
              }
              __syncwarp();
            }
            if (real) ++it_total;
          }
        }
        if (sparse && lane == 0) mbar_arrive(&sm.bm_empty[b]);
        __syncwarp();
      }
      MSA_TFLUSH(lane == 0, 3, 7)
      MSA_TFLUSH(lane == 0, 14, 15)
    } else if (Cfg::kHasCvt && warp >= Cfg::kCvtWarp0) {
      if constexpr (Cfg::kHasCvt) {
        // =====================================================================
        // dequantise raw pages into the f16 UMMA tiles (the SW128 image a 16-bit TMA load would leave).
        // 64 threads; a thread owns one 16-value column group of every 8th row, so every shared-memory
        // offset below is a per-thread constant plus a compile-time step.
        // =====================================================================
        const int ct = tid - Cfg::kCvtWarp0 * 32;  // 0..63
        const int r8 = ct >> 3, c8 = ct & 7;       // row within a group of 8, 16-value column group
        const uint32_t dst_off = (c8 >> 2) * kHalfBytes + r8 * 128;
        const uint32_t sw0 = (((c8 & 3) * 2) ^ r8) << 4, sw1 = (((c8 & 3) * 2 + 1) ^ r8) << 4;
        bool ok = true;
        uint32_t raw_seq = 0, k_seq = 0, v_seq = 0;
        auto convert = [&](const uint8_t* rawp, uint8_t* dst) {
          if constexpr (Cfg::kKDirectFp8) {
            const uint8_t* src = rawp + ct * 16;   // row (it*8 + r8), bytes [c8*16, +16)
#pragma unroll 4
            for (int it = 0; it < 16; ++it) {
              const uint4 x = *reinterpret_cast<const uint4*>(src + it * 1024);
              uint4 a, b;
              cvt_e4m3x4_f16x4(x.x, a.x, a.y);
              cvt_e4m3x4_f16x4(x.y, a.z, a.w);
              cvt_e4m3x4_f16x4(x.z, b.x, b.y);
              cvt_e4m3x4_f16x4(x.w, b.z, b.w);
              *reinterpret_cast<uint4*>(dst + it * 1024 + sw0) = a;
              *reinterpret_cast<uint4*>(dst + it * 1024 + sw1) = b;
            }
          } else {
            // NVFP4: a row is 64 bytes (128 e2m1) with 8 block scales; my block is c8 of row it*8 + r8
            const uint8_t* src = rawp + ct * 8;
            const uint8_t* sc = rawp + 8192 + (c8 >> 2) * 512 + r8 * 16 + (c8 & 3);
#pragma unroll 4
            for (int it = 0; it < 16; ++it) {
              const uint2 x = *reinterpret_cast<const uint2*>(src + it * 512);
              // scale of (row, block): 128x4 tile offset (row % 32) * 16 + (row / 32) * 4 + block % 4
              const uint32_t sb = sc[(it & 3) * 128 + (it >> 2) * 4];
              uint32_t s2, s2hi;
              cvt_e4m3x4_f16x4(sb | (sb << 8), s2, s2hi);
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
              *reinterpret_cast<uint4*>(dst + it * 1024 + sw0) = a;
              *reinterpret_cast<uint4*>(dst + it * 1024 + sw1) = b;
            }
          }
        };
        for (int j = 0; ok; ++j) {
          const int item = item_of(j);
          if (item < 0) break;
          const ItemInfo info = load_item<kSplits>(p, item, NT);
          const int b = j & 1;
          if (sparse) {
            ok = mbar_wait(&sm.bm_full[b], (j >> 1) & 1, abort_flag);
            if (!ok) break;
          }
          const int count = sparse ? sm.item_pages[b] : info.walk_n;
          for (int pg = 0; pg < count && ok; ++pg) {
            if constexpr (Cfg::kKConvert) {
              const int rs = raw_seq % NRAW, st = k_seq % NK;
              ok = mbar_wait(&sm.raw_full[rs], (raw_seq / NRAW) & 1, abort_flag);
              if (ok) ok = mbar_wait(&sm.k_empty[st], ((k_seq / NK) & 1) ^ 1, abort_flag);
              if (!ok) break;
              ++raw_seq;
              ++k_seq;
              convert(sm.raw[rs], sm.k[st] + dst_off);
              fence_proxy_async();
              __syncwarp();
              if (lane == 0) {
                mbar_arrive(&sm.k_full[st]);
                mbar_arrive(&sm.raw_empty[rs]);
              }
            }
            const int rs = raw_seq % NRAW, st = v_seq % NV;
            MSA_TBEGIN
            ok = mbar_wait(&sm.raw_full[rs], (raw_seq / NRAW) & 1, abort_flag);
            MSA_TEND(7)
            MSA_TBEGIN
            if (ok) ok = mbar_wait(&sm.v_empty[st], ((v_seq / NV) & 1) ^ 1, abort_flag);
            MSA_TEND(8)
            if (!ok) break;
            ++raw_seq;
            ++v_seq;
            MSA_TBEGIN
            convert(sm.raw[rs], sm.v[st] + dst_off);
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
              mbar_arrive(&sm.v_full[st]);
              mbar_arrive(&sm.raw_empty[rs]);
            }
            MSA_TEND(9)
          }
          if (sparse) {
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.bm_empty[b]);
          }
        }
        MSA_TFLUSH(ct == 0, 7, 10)
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
