// Host-side planner and input validator behind msa_plan / msa_validate_inputs: plain C++ over host arrays,
// no device work.  What csrc/fmha_sm100_plan.cu:18-35 (the TVM-FFI `plan` function) and the asserts of
// python/fmha_sm100/api.py:128-263 are to the reference.  The persistent kernels take query tiles
// round-robin from an ordered list, so the plan is that order (heaviest tile first), the page-table offsets,
// and -- for the decode kernels -- the per-token (request, last visible key) pair and the split count.
#include <algorithm>
#include <cstring>
#include <vector>

#include "msa_internal.h"

namespace msa {

namespace {

constexpr int kPage = 128;

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

inline int tile_rows_of(const msa_plan_desc* d) { return d->tile_rows > 0 ? d->tile_rows : kPage; }

inline int kv_splits_of(const msa_plan_desc* d) { return d->dense_kv_splits > 1 ? d->dense_kv_splits : 1; }

int plan_check(const msa_plan_desc* d) {
  if (d == nullptr || d->batch < 0) return MSA_ERR_INVALID;
  if (d->tile_rows < 0 || d->tile_rows > 256) return MSA_ERR_INVALID;
  if (d->dense_kv_splits < 0 || d->dense_kv_splits > 1024) return MSA_ERR_INVALID;
  if (d->batch > 0 && (d->qo_lens == nullptr || d->kv_lens == nullptr)) return MSA_ERR_INVALID;
  if (d->num_qo_heads <= 0 || d->num_kv_heads <= 0 || d->num_qo_heads % d->num_kv_heads != 0) return MSA_ERR_INVALID;
  for (int b = 0; b < d->batch; ++b)
    if (d->qo_lens[b] < 0 || d->kv_lens[b] < 0) return MSA_ERR_INVALID;
  return MSA_OK;
}

inline int offset_of(const msa_plan_desc* d, int b, int max_kv) {
  if (!d->causal) return max_kv;                       // every key visible
  if (d->qo_offset != nullptr) return d->qo_offset[b];
  return d->kv_lens[b] - d->qo_lens[b];
}

}  // namespace

int plan_sizes(const msa_plan_desc* d, int32_t* n_work, int64_t* total_q, int64_t* total_pages) {
  const int rc = plan_check(d);
  if (rc != MSA_OK) return rc;
  int64_t nw = 0, tq = 0, tp = 0;
  for (int b = 0; b < d->batch; ++b) {
    nw += ceil_div(d->qo_lens[b], tile_rows_of(d)) * kv_splits_of(d);
    tq += d->qo_lens[b];
    tp += ceil_div(d->kv_lens[b], kPage);
  }
  if (nw > 0x7fffffffLL || tq * kv_splits_of(d) > 0x7fffffffLL || tp > 0x7fffffffLL) return MSA_ERR_TOO_LARGE;
  if (n_work != nullptr) *n_work = static_cast<int32_t>(nw);
  if (total_q != nullptr) *total_q = tq;
  if (total_pages != nullptr) *total_pages = tp;
  return MSA_OK;
}

int plan(const msa_plan_desc* d, int32_t* work, int32_t* kv_page_indptr, int32_t* token_request,
         int32_t* token_pos, int32_t* num_splits) {
  int32_t n_work = 0;
  int64_t total_q = 0;
  int rc = plan_sizes(d, &n_work, &total_q, nullptr);
  if (rc != MSA_OK) return rc;
  int max_kv = 0;
  for (int b = 0; b < d->batch; ++b) max_kv = std::max(max_kv, d->kv_lens[b]);

  if (kv_page_indptr != nullptr) {
    kv_page_indptr[0] = 0;
    for (int b = 0; b < d->batch; ++b)
      kv_page_indptr[b + 1] = kv_page_indptr[b] + static_cast<int32_t>(ceil_div(d->kv_lens[b], kPage));
  }

  if (work != nullptr && n_work > 0) {
    struct Tile {
      int cost;
      int32_t rec[8];
    };
    std::vector<Tile> tiles;
    tiles.reserve(n_work);
    int start = 0, kv_base = 0;
    for (int b = 0; b < d->batch; ++b) {
      const int ql = d->qo_lens[b], kl = d->kv_lens[b], off = offset_of(d, b, max_kv);
      const int tile = tile_rows_of(d);
      for (int t0 = 0; t0 < ql; t0 += tile) {
        const int rows = std::min(tile, ql - t0);
        const int64_t vis = d->causal ? std::min<int64_t>(kl, static_cast<int64_t>(t0) + rows + off) : kl;
        const int n_vis = static_cast<int>(std::max<int64_t>(0, ceil_div(vis, kPage)));
        const int n_splits = kv_splits_of(d);
        const int per = static_cast<int>(ceil_div(n_vis, n_splits));
        for (int s = 0; s < n_splits; ++s) {
          // split s walks pages [lo, hi) and writes output rows s * total_q + token; a split beyond the visible
          // pages still gets an entry (lo past the last page: nothing to walk), so that every partial row is written
          const int lo = std::min(n_vis, s * per), hi = std::min(n_vis, lo + per);
          if (lo > 0x1fffff) return MSA_ERR_TOO_LARGE;
          Tile t;
          t.cost = hi - lo;
          const int kl_s = (n_splits > 1 && hi > lo) ? std::min<int64_t>(kl, static_cast<int64_t>(hi) * kPage) : kl;
          const int32_t rec[8] = {b, start + t0, rows | (n_splits > 1 ? lo << 10 : 0), t0, kl_s, off, kv_base,
                                  static_cast<int32_t>(s * total_q)};
          std::memcpy(t.rec, rec, sizeof(rec));
          tiles.push_back(t);
        }
      }
      start += ql;
      kv_base += d->paged ? static_cast<int>(ceil_div(kl, kPage)) : kl;
    }
    // heaviest first; equal cost keeps batch order (a stable order makes plans reproducible)
    std::stable_sort(tiles.begin(), tiles.end(), [](const Tile& a, const Tile& b) { return a.cost > b.cost; });
    for (int i = 0; i < n_work; ++i) std::memcpy(work + static_cast<size_t>(i) * 8, tiles[i].rec, sizeof(tiles[i].rec));
  }

  if (token_request != nullptr || token_pos != nullptr) {
    int64_t t = 0;
    for (int b = 0; b < d->batch; ++b) {
      const int kl = d->kv_lens[b], off = offset_of(d, b, max_kv);
      for (int i = 0; i < d->qo_lens[b]; ++i, ++t) {
        if (token_request != nullptr) token_request[t] = b;
        if (token_pos != nullptr) {
          const int64_t pos = d->causal ? std::min<int64_t>(static_cast<int64_t>(i) + off, kl - 1) : kl - 1;
          token_pos[t] = static_cast<int32_t>(pos);
        }
      }
    }
  }

  if (num_splits != nullptr) {
    int splits = 1;
    const int kbn = d->kv_block_num;
    if (kbn > 0) {
      if (d->num_kv_splits > 0) {
        splits = std::min(d->num_kv_splits, kbn);
      } else {
        // Whole waves of resident CTAs: the GQA <= 8 kernel is persistent with one CTA per SM and every split
        // costs a prologue and a merge; the GQA > 8 kernel keeps two CTAs per SM resident.  At most 64 splits;
        // a split count that leaves the last splits empty is never better than the smaller count it equals.
        const int sms = d->num_sms > 0 ? d->num_sms : 148;
        const int hr = d->num_qo_heads / d->num_kv_heads;
        const int64_t resident = static_cast<int64_t>(sms) * (hr <= 8 ? 1 : 2);
        const int64_t rows = std::max<int64_t>(1, total_q * d->num_kv_heads);
        double best = -1e30;
        for (int s = 1; s <= std::min(kbn, 64); ++s) {
          if (s > 1 && ceil_div(kbn, s) == ceil_div(kbn, s - 1)) continue;
          const int64_t ctas = rows * s;
          const int64_t waves = ceil_div(ctas, resident);
          const double eff = static_cast<double>(ctas) / static_cast<double>(waves * resident);
          const int per = static_cast<int>(ceil_div(kbn, s));
          const double score = eff - 0.01 * s - (per < 2 ? 0.25 : 0.0);
          if (score > best) {
            best = score;
            splits = s;
          }
        }
      }
    }
    *num_splits = splits;
  }
  return MSA_OK;
}

// First violated rule of the index contract, checked in the order of python/fmha_sm100/api.py:128-263.
int validate_inputs(const msa_validate_args* a, int64_t* where) {
  if (where != nullptr) *where = -1;
  if (a == nullptr || a->batch < 0 || (a->batch > 0 && (a->qo_lens == nullptr || a->kv_lens == nullptr)))
    return MSA_ERR_INVALID;
  if (a->num_qo_heads <= 0 || a->num_kv_heads <= 0 || a->num_qo_heads % a->num_kv_heads != 0) return MSA_ERR_INVALID;
  int64_t sum_q = 0, sum_kv = 0, need_pages = 0;
  for (int b = 0; b < a->batch; ++b) {
    if (a->qo_lens[b] < 0 || a->kv_lens[b] < 0) return MSA_ERR_INVALID;
    sum_q += a->qo_lens[b];
    sum_kv += a->kv_lens[b];
    need_pages += ceil_div(a->kv_lens[b], kPage);
  }
  if (a->total_q != sum_q) return MSA_EVAL_Q_ROWS;
  if (a->paged) {
    if (a->kv_indices == nullptr || a->n_kv_indices != need_pages) return MSA_EVAL_PAGE_TABLE_LENGTH;
    for (int64_t i = 0; i < a->n_kv_indices; ++i)
      if (a->kv_indices[i] < 0 || a->kv_indices[i] >= a->kv_rows) {
        if (where != nullptr) *where = i;
        return MSA_EVAL_PAGE_TABLE_RANGE;
      }
  } else if (a->kv_rows != sum_kv) {
    return MSA_EVAL_KV_ROWS;
  }
  if (a->kv_block_indexes == nullptr) return MSA_OK;
  if (a->topk <= 0 || (a->list_heads != a->num_kv_heads && a->list_heads != a->num_qo_heads))
    return MSA_EVAL_LIST_SHAPE;
  // rule by rule over the whole tensor, so that the code names the first rule of the contract that is broken
  // anywhere (the reference asserts them in this order), and `where` the first element that breaks it
  const int64_t row_len = static_cast<int64_t>(a->list_heads) * a->topk;
  const int rules[4] = {MSA_EVAL_LIST_NEGATIVE, MSA_EVAL_LIST_PADDING, MSA_EVAL_LIST_RANGE, MSA_EVAL_LIST_ORDER};
  for (int rule : rules) {
    int64_t t = 0;
    for (int b = 0; b < a->batch; ++b) {
      const int n_pages = static_cast<int>(ceil_div(a->kv_lens[b], kPage));
      for (int i = 0; i < a->qo_lens[b]; ++i, ++t) {
        const int32_t* l = a->kv_block_indexes + t * row_len;
        for (int64_t x = 0; x < row_len; ++x) {
          const int e = static_cast<int>(x % a->topk);
          const int v = l[x];
          bool bad = false;
          switch (rule) {
            case MSA_EVAL_LIST_NEGATIVE: bad = v < -1; break;
            case MSA_EVAL_LIST_PADDING: bad = e > 0 && v != -1 && l[x - 1] == -1; break;
            case MSA_EVAL_LIST_RANGE: bad = v >= n_pages; break;
            default: bad = e > 0 && v != -1 && l[x - 1] != -1 && v <= l[x - 1]; break;
          }
          if (bad) {
            if (where != nullptr) *where = t * row_len + x;
            return rule;
          }
        }
      }
    }
  }
  return MSA_OK;
}

}  // namespace msa
