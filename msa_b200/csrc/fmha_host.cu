// Host side of the attention kernel: TMA tensor maps, variant dispatch, and the
// one-tile tensor-core self-test.
#include <mutex>

#include "fmha_kernel.cuh"
#include "score_kernel.cuh"
#include "msa_internal.h"

namespace msa {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// rank-3 or rank-4 tiled map; dims/strides innermost first, strides in bytes for dims 1..rank-1
static int make_map(CUtensorMap* m, CUtensorMapDataType dt, int rank, const void* base, const uint64_t* dims,
                    const uint64_t* strides, const uint32_t* box, CUtensorMapSwizzle sw) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return MSA_ERR_DRIVER;
  cuuint64_t gd[4], gs[3];
  cuuint32_t bx[4], es[4];
  for (int i = 0; i < rank; ++i) {
    gd[i] = dims[i];
    bx[i] = box[i];
    es[i] = 1;
  }
  for (int i = 0; i < rank - 1; ++i) gs[i] = strides[i];
  CUresult r = fn(m, dt, static_cast<cuuint32_t>(rank), const_cast<void*>(base), gd, gs, bx, es,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? MSA_OK : MSA_ERR_DRIVER;
}

// Output [total_q, Hq, 128] bf16 as 32-row x 32-column boxes (64-byte rows, 64-byte swizzle): one per softmax warp
// and column quarter
static int make_o_map(CUtensorMap* m, const void* o, int64_t total_q, int hq) {
  const uint64_t dims[3] = {128, static_cast<uint64_t>(hq), static_cast<uint64_t>(total_q)};
  const uint64_t strides[2] = {256, static_cast<uint64_t>(hq) * 256};
  const uint32_t box[3] = {32, 1, 32};
  return make_map(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, o, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_64B);
}

// pack_heads = hb > 1 (score-only pass over short requests): a tile is 128 / hb tokens x hb adjacent heads
static int make_q_map(CUtensorMap* m, const void* q, int64_t total_q, int hq, int pack_heads = 1) {
  const uint64_t dims[3] = {128, static_cast<uint64_t>(hq), static_cast<uint64_t>(total_q)};
  const uint64_t strides[2] = {256, static_cast<uint64_t>(hq) * 256};
  const uint32_t box[3] = {64, static_cast<uint32_t>(pack_heads), static_cast<uint32_t>(128 / pack_heads)};
  return make_map(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, q, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
}

// K or V pages.  bf16: two 64-column SW128 boxes per tile.  e4m3: one 128-byte-row box, swizzled when the
// tile feeds the tensor core as stored (K), plain when the convert warps read it (V).
// fp8_half: boxes over the first 64 bytes of every row only (score-only pass over a 64-wide slice), 64-byte swizzle.
static int make_kv_map(CUtensorMap* m, const void* kv, int64_t rows, int hkv, int paged, int fp8, int fp8_swizzle,
                       int fp8_half = 0) {
  const uint64_t es = fp8 ? 1 : 2;
  const CUtensorMapDataType dt = fp8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const CUtensorMapSwizzle sw = (fp8 && fp8_half)       ? CU_TENSOR_MAP_SWIZZLE_64B
                                : (fp8 && !fp8_swizzle) ? CU_TENSOR_MAP_SWIZZLE_NONE
                                                        : CU_TENSOR_MAP_SWIZZLE_128B;
  const uint32_t inner = fp8 ? (fp8_half ? 64 : 128) : 64;
  if (paged) {
    const uint64_t dims[4] = {128, 128, static_cast<uint64_t>(hkv), static_cast<uint64_t>(rows)};
    const uint64_t strides[3] = {128 * es, 128 * 128 * es, static_cast<uint64_t>(hkv) * 128 * 128 * es};
    const uint32_t box[4] = {inner, 128, 1, 1};
    return make_map(m, dt, 4, kv, dims, strides, box, sw);
  }
  const uint64_t dims[3] = {128, static_cast<uint64_t>(hkv), static_cast<uint64_t>(rows)};
  const uint64_t strides[2] = {128 * es, static_cast<uint64_t>(hkv) * 128 * es};
  const uint32_t box[3] = {inner, 1, 128};
  return make_map(m, dt, 3, kv, dims, strides, box, sw);
}

int make_score_map(void* tensor_map, const float* ms, int H, int K, int T, int box_t, int box_k) {
  const uint64_t dims[3] = {static_cast<uint64_t>(T), static_cast<uint64_t>(K), static_cast<uint64_t>(H)};
  const uint64_t strides[2] = {static_cast<uint64_t>(T) * 4, static_cast<uint64_t>(K) * T * 4};
  const uint32_t box[3] = {static_cast<uint32_t>(box_t), static_cast<uint32_t>(box_k), 1};
  return make_map(static_cast<CUtensorMap*>(tensor_map), CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, ms, dims, strides, box,
                  CU_TENSOR_MAP_SWIZZLE_NONE);
}

int make_paged_e4m3_map(void* tensor_map, const void* kv, int64_t pages, int hkv) {
  return make_kv_map(static_cast<CUtensorMap*>(tensor_map), kv, pages, hkv, 1, 1, 1);
}

static long long* g_timing_buffer = nullptr;
void set_timing_buffer(void* ptr) { g_timing_buffer = static_cast<long long*>(ptr); }

template <int NT, int KVMODE, int LISTS>
static int launch_fmha_mode(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& mo,
                       const FmhaParams& p, int max_ctas, cudaStream_t st) {
  using Cfg = FmhaCfg<NT, KVMODE>;
  static DeviceSetup setup;
  int num_sms = 0;
  constexpr int smem = fmha_smem_bytes<NT, KVMODE>();
  const int rc = setup.ensure(&num_sms, [] {
    cudaError_t e = cudaFuncSetAttribute(fmha_fwd_kernel<NT, KVMODE, LISTS>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (Cfg::kRebalance) {
      // the in-kernel register hand-over only balances if the CTA starts with exactly kRegsLaunch per thread
      cudaFuncAttributes fa;
      e = cudaFuncGetAttributes(&fa, fmha_fwd_kernel<NT, KVMODE, LISTS>);
      if (e != cudaSuccess) return static_cast<int>(e);
      if (fa.numRegs != Cfg::kRegsLaunch) return static_cast<int>(MSA_ERR_UNSUPPORTED);
    }
    return static_cast<int>(MSA_OK);
  });
  if (rc != MSA_OK) return rc;
  // persistent: one CTA per SM walks the item list with stride gridDim.x; max_ctas > 0 caps the grid
  int ctas = p.n_items < num_sms ? p.n_items : num_sms;
  if (max_ctas > 0 && max_ctas < ctas) ctas = max_ctas;
  fmha_fwd_kernel<NT, KVMODE, LISTS><<<static_cast<unsigned>(ctas), Cfg::kThreads, smem, st>>>(mq, mk, mv, mo, p);
  return static_cast<int>(cudaGetLastError());
}

// score-only pass: its own kernel, one (query tile, head) per work item
template <int KVMODE>
static int launch_score(const CUtensorMap& mq, const CUtensorMap& mk, const FmhaParams& p, int max_ctas,
                        cudaStream_t st) {
  using Cfg = ScoreCfg<KVMODE>;
  static DeviceSetup setup;
  int num_sms = 0;
  constexpr int smem = score_smem_bytes<KVMODE>();
  static_assert(smem <= 232448, "shared memory of the score kernel exceeds the 227 KiB a CTA can have");
  const int rc = setup.ensure(&num_sms, [] {
    cudaError_t e = cudaFuncSetAttribute(score_fwd_kernel<KVMODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    // the in-kernel register hand-over only balances if the CTA starts with exactly kRegsLaunch per thread
    cudaFuncAttributes fa;
    e = cudaFuncGetAttributes(&fa, score_fwd_kernel<KVMODE>);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (fa.numRegs != Cfg::kRegsLaunch) return static_cast<int>(MSA_ERR_UNSUPPORTED);
    return static_cast<int>(MSA_OK);
  });
  if (rc != MSA_OK) return rc;
  int ctas = p.n_items < num_sms ? p.n_items : num_sms;
  if (max_ctas > 0 && max_ctas < ctas) ctas = max_ctas;
  score_fwd_kernel<KVMODE><<<static_cast<unsigned>(ctas), Cfg::kThreads, smem, st>>>(mq, mk, p);
  return static_cast<int>(cudaGetLastError());
}

template <int NT, int KVMODE>
static int launch_fmha(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& mo,
                       const FmhaParams& p, int max_ctas, cudaStream_t st) {
  return p.sparse ? launch_fmha_mode<NT, KVMODE, 1>(mq, mk, mv, mo, p, max_ctas, st)
                  : launch_fmha_mode<NT, KVMODE, 0>(mq, mk, mv, mo, p, max_ctas, st);
}

int fmha_fwd(const msa_fmha_args* a, cudaStream_t st) {
  if (a == nullptr || a->q == nullptr || a->k == nullptr || a->work == nullptr || a->status == nullptr)
    return MSA_ERR_INVALID;
  if (a->out == nullptr && a->max_score == nullptr) return MSA_ERR_INVALID;
  if (a->out != nullptr && a->v == nullptr) return MSA_ERR_INVALID;
  if (a->num_kv_heads <= 0 || a->num_qo_heads <= 0 || a->num_qo_heads % a->num_kv_heads != 0) return MSA_ERR_INVALID;
  if (a->paged && a->kv_indices == nullptr) return MSA_ERR_INVALID;
  if (a->kv_dtype < MSA_KV_BF16 || a->kv_dtype > MSA_KV_NVFP4) return MSA_ERR_UNSUPPORTED;
  if (a->kv_dtype == MSA_KV_NVFP4 && (!a->paged || a->k_scale_128x4 == nullptr ||
                                      (a->out != nullptr && a->v_scale_128x4 == nullptr)))
    return MSA_ERR_INVALID;
  const bool sparse = a->kv_block_indexes != nullptr;
  if (sparse && (a->topk <= 0 ||
                 (a->list_heads != a->num_kv_heads && a->list_heads != a->num_qo_heads)))
    return MSA_ERR_INVALID;
  if (a->max_score != nullptr && a->max_k_tiles <= 0) return MSA_ERR_INVALID;
  if (a->max_score_tile_stride < 0 || a->max_score_head_stride < 0) return MSA_ERR_INVALID;
  if (a->max_score_tile_stride > 0 && a->max_score_tile_stride < a->total_q) return MSA_ERR_INVALID;
  if (a->qk_dim != 0 && a->qk_dim != 64 && a->qk_dim != 128) return MSA_ERR_INVALID;
  if (a->qk_dim == 64 && (a->out != nullptr || a->kv_dtype == MSA_KV_NVFP4)) return MSA_ERR_UNSUPPORTED;
  if (a->out_rows != 0 && (a->out_rows < a->total_q || a->out == nullptr || a->lse == nullptr)) return MSA_ERR_INVALID;
  const bool score_only = a->out == nullptr;
  if (score_only && sparse) return MSA_ERR_UNSUPPORTED;        // the pass over page lists has no max-score output
  if (a->k_scale_format != 0 && (a->k_scale_format != 1 || !score_only || a->kv_dtype != MSA_KV_NVFP4))
    return MSA_ERR_INVALID;
  // heads per query tile of the score-only pass: a power of two that divides the heads per KV head; a work entry
  // then covers up to 256 / hb tokens
  const int hb = a->score_pack_heads > 1 ? a->score_pack_heads : 1;
  if (hb > 1 && (!score_only || (hb & (hb - 1)) != 0 || hb > 128 ||
                 (a->num_qo_heads / a->num_kv_heads) % hb != 0 || a->tile_rows != 256 / hb))
    return MSA_ERR_INVALID;
  if (hb == 1 && a->tile_rows != 0 && a->tile_rows != 128 && a->tile_rows != 256) return MSA_ERR_INVALID;
  if (hb == 1 && a->tile_rows == 256 && !score_only) return MSA_ERR_UNSUPPORTED;
  if (a->n_work <= 0 || a->total_q <= 0) return MSA_OK;
  const int64_t out_rows = a->out_rows > 0 ? a->out_rows : a->total_q;

  FmhaParams p{};
  p.out = static_cast<__nv_bfloat16*>(a->out);
  p.lse = a->lse;
  p.max_score = a->max_score;
  p.ms_tile = a->max_score_tile_stride > 0 ? a->max_score_tile_stride : a->total_q;
  p.ms_head = a->max_score_head_stride > 0 ? a->max_score_head_stride : p.ms_tile * a->max_k_tiles;
  p.work = reinterpret_cast<const int4*>(a->work);
  p.kv_indices = a->kv_indices;
  p.kv_block_indexes = a->kv_block_indexes;
  p.tile_uniform = sparse ? a->tile_uniform : nullptr;
  p.k_scale_bytes = a->k_scale_128x4;
  p.v_scale_bytes = a->v_scale_128x4;
  p.k_scale_tile_bytes = a->k_scale_format == 1 ? 512 : 1024;
  p.k_mx = a->k_scale_format == 1;
  p.k_raw = static_cast<const uint8_t*>(a->k);
  p.v_raw = static_cast<const uint8_t*>(a->v);
  p.Hq = a->num_qo_heads;
  p.Hkv = a->num_kv_heads;
  p.hr = a->num_qo_heads / a->num_kv_heads;
  p.topk = a->topk;
  p.list_heads = a->list_heads;
  p.total_q = static_cast<int>(a->total_q);
  p.max_k_tiles = a->max_k_tiles;
  p.n_work = a->n_work;
  p.causal = a->causal;
  p.paged = a->paged;
  p.sparse = sparse ? 1 : 0;
  p.do_pv = a->out != nullptr;
  p.do_maxscore = a->max_score != nullptr;
  p.half_dim = a->qk_dim == 64;
  p.scale_log2 = a->sm_scale * a->qk_scale * 1.4426950408889634f;
  p.out_scale = a->v_scale;
  p.status = a->status;
  p.timing = g_timing_buffer;

  // two query heads share one K/V stream when they share a KV head and a page list
  int nt = (p.hr % 2 == 0 && (!sparse || a->list_heads == a->num_kv_heads)) ? 2 : 1;
  if (score_only) nt = hb;  // the score kernel takes hb heads per work item
  p.pack_heads = hb;
  p.fill_tail = score_only && a->score_fill_tail != 0;
  p.kv_pages = a->paged ? static_cast<int>(a->kv_rows < 0x7fffffffLL ? a->kv_rows : 0x7fffffffLL) : 0;
  p.n_head_groups = p.Hq / nt;
  const long long n_items = static_cast<long long>(p.n_work) * p.n_head_groups;
  if (n_items > 0x7fffffffLL) return MSA_ERR_TOO_LARGE;
  p.n_items = static_cast<int>(n_items);

  CUtensorMap mq, mk, mv, mo;
  int rc = make_q_map(&mq, a->q, a->total_q, p.Hq, score_only ? hb : 1);
  if (rc != MSA_OK) return rc;
  // score-only calls have no output: the map is never used then, but must be a valid one
  rc = make_o_map(&mo, a->out != nullptr ? a->out : a->q, a->out != nullptr ? out_rows : a->total_q, p.Hq);
  if (rc != MSA_OK) return rc;
  if (a->kv_dtype == MSA_KV_NVFP4) {
    mk = mq;  // pages are fetched with untiled bulk copies
    mv = mq;
  } else {
    const int fp8 = a->kv_dtype == MSA_KV_FP8_E4M3;
    rc = make_kv_map(&mk, a->k, a->kv_rows, p.Hkv, a->paged, fp8, 1, fp8 && score_only && p.half_dim);
    if (rc != MSA_OK) return rc;
    rc = make_kv_map(&mv, a->v != nullptr ? a->v : a->k, a->kv_rows, p.Hkv, a->paged, fp8, a->fp8_p_f16 == 0);
    if (rc != MSA_OK) return rc;
  }
  if (score_only) {
    switch (a->kv_dtype) {
      case MSA_KV_BF16: return launch_score<KV_BF16>(mq, mk, p, a->max_ctas, st);
      case MSA_KV_FP8_E4M3: return launch_score<KV_FP8>(mq, mk, p, a->max_ctas, st);
      case MSA_KV_NVFP4: return launch_score<KV_NVFP4>(mq, mk, p, a->max_ctas, st);
    }
    return MSA_ERR_UNSUPPORTED;
  }
  if (a->kv_dtype == MSA_KV_FP8_E4M3 && a->fp8_p_f16 != 0) {
    if (nt == 1) return launch_fmha<1, KV_FP8_F16P>(mq, mk, mv, mo, p, a->max_ctas, st);
    return launch_fmha<2, KV_FP8_F16P>(mq, mk, mv, mo, p, a->max_ctas, st);
  }
  switch (a->kv_dtype * 2 + (nt - 1)) {
    case 0: return launch_fmha<1, KV_BF16>(mq, mk, mv, mo, p, a->max_ctas, st);
    case 1: return launch_fmha<2, KV_BF16>(mq, mk, mv, mo, p, a->max_ctas, st);
    case 2: return launch_fmha<1, KV_FP8>(mq, mk, mv, mo, p, a->max_ctas, st);
    case 3: return launch_fmha<2, KV_FP8>(mq, mk, mv, mo, p, a->max_ctas, st);
    case 4: return launch_fmha<1, KV_NVFP4>(mq, mk, mv, mo, p, a->max_ctas, st);
    case 5: return launch_fmha<2, KV_NVFP4>(mq, mk, mv, mo, p, a->max_ctas, st);
  }
  return MSA_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------------------
// Merge of KV splits: a dense call with few query tiles is planned as n_splits work entries per tile, each over a
// range of the pages; every split leaves a normalised bf16 partial and its natural-log LSE.  One warp per
// (token, head) row: lane l owns columns 4l .. 4l + 3.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) fmha_combine_kernel(const uint2* __restrict__ part_o, const float* __restrict__ part_lse,
                                                          int n_splits, long long n_rows, uint2* __restrict__ out,
                                                          float* __restrict__ lse) {
  const long long row = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= n_rows) return;
  float m = -INFINITY;
  for (int s = lane; s < n_splits; s += 32) m = fmaxf(m, __ldg(part_lse + s * n_rows + row));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  float wsum = 0.f;
  if (m > -INFINITY) {
    for (int s = 0; s < n_splits; ++s) {
      const float l = __ldg(part_lse + s * n_rows + row);
      if (l == -INFINITY) continue;
      const float w = __expf(l - m);
      const uint2 v = __ldg(part_o + (s * n_rows + row) * 32 + lane);
      const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
      const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
      acc[0] += w * a.x;
      acc[1] += w * a.y;
      acc[2] += w * b.x;
      acc[3] += w * b.y;
      wsum += w;
    }
  }
  const float inv = wsum > 0.f ? 1.f / wsum : 0.f;
  uint2 r;
  const __nv_bfloat162 lo = __floats2bfloat162_rn(acc[0] * inv, acc[1] * inv);
  const __nv_bfloat162 hi = __floats2bfloat162_rn(acc[2] * inv, acc[3] * inv);
  r.x = *reinterpret_cast<const uint32_t*>(&lo);
  r.y = *reinterpret_cast<const uint32_t*>(&hi);
  out[row * 32 + lane] = r;
  if (lse != nullptr && lane == 0) lse[row] = wsum > 0.f ? m + logf(wsum) : -INFINITY;
}

int fmha_combine(const void* partial_out, const float* partial_lse, int n_splits, int64_t total_q, int num_qo_heads,
                 void* out, float* lse, cudaStream_t st) {
  if (partial_out == nullptr || partial_lse == nullptr || out == nullptr || n_splits <= 0 || num_qo_heads <= 0 ||
      total_q < 0)
    return MSA_ERR_INVALID;
  const long long n_rows = static_cast<long long>(total_q) * num_qo_heads;
  if (n_rows == 0) return MSA_OK;
  const long long blocks = (n_rows * 32 + 255) / 256;
  if (blocks > 0x7fffffffLL) return MSA_ERR_TOO_LARGE;
  fmha_combine_kernel<<<static_cast<unsigned>(blocks), 256, 0, st>>>(static_cast<const uint2*>(partial_out), partial_lse,
                                                                    n_splits, n_rows, static_cast<uint2*>(out), lse);
  return static_cast<int>(cudaGetLastError());
}

// ---------------------------------------------------------------------------
// Which query tiles have one page list for all their rows?  MSA selects pages per query block, so the per-token
// lists the API takes are usually 128 copies of one row; the attention kernel then builds a tile's page bitmap
// from a single row instead of 128.  One CTA per (tile, list head): row r is compared with row 0.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(128) list_uniform_kernel(const int4* __restrict__ work,
                                                          const int* __restrict__ lists, int list_heads, int topk,
                                                          uint8_t* __restrict__ flags) {
  const int wi = blockIdx.x, lh = blockIdx.y, r = threadIdx.x;
  const int4 w = __ldg(work + 2 * wi);   // {request, first token, rows, first local token}
  const int* row0 = lists + (static_cast<size_t>(w.y) * list_heads + lh) * topk;
  const int* mine = lists + (static_cast<size_t>(w.y + r) * list_heads + lh) * topk;
  int same = 1;
  if (r > 0 && r < (w.z & 1023)) {
    if ((topk & 3) == 0) {
      for (int e = 0; e < topk; e += 4) {
        const int4 a = __ldg(reinterpret_cast<const int4*>(row0 + e)), b = __ldg(reinterpret_cast<const int4*>(mine + e));
        same &= (a.x == b.x) & (a.y == b.y) & (a.z == b.z) & (a.w == b.w);
      }
    } else {
      for (int e = 0; e < topk; ++e) same &= __ldg(row0 + e) == __ldg(mine + e);
    }
  }
  same = __syncthreads_and(same);
  if (r == 0) flags[static_cast<size_t>(wi) * list_heads + lh] = static_cast<uint8_t>(same);
}

int list_uniformity(const int32_t* work, int n_work, const int32_t* lists, int list_heads, int topk, uint8_t* flags,
                    cudaStream_t st) {
  if (work == nullptr || lists == nullptr || flags == nullptr || list_heads <= 0 || list_heads > 65535 || topk <= 0)
    return MSA_ERR_INVALID;
  if (n_work <= 0) return MSA_OK;
  list_uniform_kernel<<<dim3(n_work, list_heads), 128, 0, st>>>(reinterpret_cast<const int4*>(work), lists, list_heads,
                                                                topk, flags);
  return static_cast<int>(cudaGetLastError());
}

// ---------------------------------------------------------------------------
// one-tile self-test: S = Q K^T (SS MMA, both operands K-major SW128) and
// O = P V (TS MMA, P in TMEM, V MN-major SW128)
// ---------------------------------------------------------------------------
struct __align__(1024) SelfTestSmem {
  uint8_t q[kTileBytes], k[kTileBytes], v[kTileBytes];
  uint64_t full, done_s, done_o;
  uint32_t tmem_base;
  int abort;
};

__global__ void __launch_bounds__(128, 1)
umma_selftest_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                     const __grid_constant__ CUtensorMap tmap_v, const __nv_bfloat16* __restrict__ pmat,
                     float* __restrict__ s_out, float* __restrict__ o_out, int* status, int skip_loads,
                     long long wait_limit) {
  extern __shared__ uint8_t smem_raw[];
  SelfTestSmem& sm = *reinterpret_cast<SelfTestSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid >> 5;
  volatile int* abort_flag = &sm.abort;
  if (tid == 0) {
    mbar_init(&sm.full, 1);
    mbar_init(&sm.done_s, 1);
    mbar_init(&sm.done_o, 1);
    sm.abort = 0;
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(&sm.tmem_base, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;
  // skip_loads: the loads are never issued, so the wait below can only run out -- the way a test drives the
  // timeout path (abort flag, every later step skipped, TMEM freed, status word written) without a fault
  if (tid == 0 && !skip_loads) {
    mbar_expect_tx(&sm.full, 3 * kTileBytes);
    tma_load_3d(sm.q, &tmap_q, &sm.full, 0, 0, 0);
    tma_load_3d(sm.q + kHalfBytes, &tmap_q, &sm.full, 64, 0, 0);
    tma_load_3d(sm.k, &tmap_k, &sm.full, 0, 0, 0);
    tma_load_3d(sm.k + kHalfBytes, &tmap_k, &sm.full, 64, 0, 0);
    tma_load_3d(sm.v, &tmap_v, &sm.full, 0, 0, 0);
    tma_load_3d(sm.v + kHalfBytes, &tmap_v, &sm.full, 64, 0, 0);
  }
  bool ok = mbar_wait(&sm.full, 0, abort_flag, wait_limit);
  constexpr uint32_t idesc_qk = make_idesc(128, 128, 1, 1, 0, 0);
  constexpr uint32_t idesc_pv = make_idesc(128, 128, 1, 1, 0, 1);
  if (ok && tid == 0) {
    tc_fence_after();
    const uint32_t qa = smem_u32(sm.q), ka = smem_u32(sm.k);
    for (int ks = 0; ks < 8; ++ks) {
      const uint32_t off = (ks >> 2) * kHalfBytes + (ks & 3) * 32;
      umma_ss(tmem, make_smem_desc(qa + off, 16, 1024), make_smem_desc(ka + off, 16, 1024), idesc_qk, ks > 0);
    }
    umma_commit(&sm.done_s);
  }
  __syncwarp();
  if (ok) ok = mbar_wait(&sm.done_s, 0, abort_flag, wait_limit);
  const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
  const int row = tid;
  if (ok) {
    tc_fence_after();
    uint32_t rg[32];
    for (int c = 0; c < 4; ++c) {
      tmem_ld32(tmem + lane_base + c * 32, rg);
      tmem_ld_wait();
      for (int e = 0; e < 32; ++e) s_out[row * 128 + c * 32 + e] = __uint_as_float(rg[e]);
    }
    // P (given, bf16 row-major) -> TMEM columns [0, 64) as packed pairs
    const uint32_t* prow = reinterpret_cast<const uint32_t*>(pmat + row * 128);
    for (int c = 0; c < 4; ++c) {
      uint32_t pk[16];
      for (int e = 0; e < 16; ++e) pk[e] = prow[c * 16 + e];
      tmem_st16(tmem + lane_base + c * 16, pk);
    }
    tmem_st_wait();
  }
  tc_fence_before();
  __syncthreads();
  if (ok && tid == 0) {
    tc_fence_after();
    const uint32_t va = smem_u32(sm.v);
    for (int ks = 0; ks < 8; ++ks)
      umma_ts(tmem + 128, tmem + ks * 8, make_smem_desc(va + ks * 2048, kHalfBytes, 1024), idesc_pv, ks > 0);
    umma_commit(&sm.done_o);
  }
  __syncwarp();
  if (ok) ok = mbar_wait(&sm.done_o, 0, abort_flag, wait_limit);
  if (ok) {
    tc_fence_after();
    uint32_t rg[32];
    for (int c = 0; c < 4; ++c) {
      tmem_ld32(tmem + lane_base + 128 + c * 32, rg);
      tmem_ld_wait();
      for (int e = 0; e < 32; ++e) o_out[row * 128 + c * 32 + e] = __uint_as_float(rg[e]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, 256);
  }
  if (tid == 0 && sm.abort) atomicExch(status, MSA_ERR_TIMEOUT);
}

int umma_selftest(const void* q, const void* k, const void* v, const void* pm, float* s_out, float* o_out,
                  int* status, int skip_loads, long long wait_cycles, cudaStream_t st) {
  if (!q || !k || !v || !pm || !s_out || !o_out || !status) return MSA_ERR_INVALID;
  CUtensorMap mq, mk, mv;
  int rc = make_q_map(&mq, q, 128, 1);
  if (rc == MSA_OK) rc = make_q_map(&mk, k, 128, 1);
  if (rc == MSA_OK) rc = make_q_map(&mv, v, 128, 1);
  if (rc != MSA_OK) return rc;
  constexpr int smem = static_cast<int>(sizeof(SelfTestSmem)) + 1024;
  static DeviceSetup setup;
  rc = setup.ensure(nullptr, [] {
    return static_cast<int>(
        cudaFuncSetAttribute(umma_selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  });
  if (rc != MSA_OK) return rc;
  if (wait_cycles <= 0 || wait_cycles > kWaitCycles) wait_cycles = kWaitCycles;
  umma_selftest_kernel<<<1, 128, smem, st>>>(mq, mk, mv, static_cast<const __nv_bfloat16*>(pm), s_out, o_out,
                                              status, skip_loads, wait_cycles);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace msa
