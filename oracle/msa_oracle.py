"""CPU oracle for the block-sparse attention hot path (TEST INFRASTRUCTURE ONLY).

This module is a plain PyTorch-on-CPU restatement of the reference algorithms
for the three stages (proxy max-score pass, top-k page selector, sparse paged
attention / decode) plus the quantised K/V formats.  It is the checker used by
``tests/``, by ``__graft_entry__.smoke()`` and by the ``cpu_baseline`` /
``--impl reference`` legs of ``bench.py``.  Nothing in ``msa_b200`` imports it
and it must never be on a product path.

Parity pinning: every function here is compared against outputs of the
reference's own PyTorch code (imported unmodified from the reference tree by
``tests/golden/make_golden.py``); the resulting fixtures live in
``tests/golden/*.npz`` and are checked by ``tests/test_oracle_golden.py``.
The one exception is NVFP4 *quantisation* (rounding and block-scale choice),
whose arithmetic lives in Transformer Engine, a third-party dependency that
is not vendored by the reference: for it only the storage layout and the
dequantisation formula are pinned ("parity unpinned" for the quantiser).

Reference citations use paths inside the reference project.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

PAGE = 128
NEG_INF = float("-inf")
FP8_MAX = 448.0
FP4_MAX = 6.0
NVFP4_BLOCK = 16

# e2m1 code -> value, python/fmha_sm100/cute/quantize.py:296-317
FP4_LUT = torch.tensor(
    [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0],
    dtype=torch.float32,
)


# ---------------------------------------------------------------------------
# helpers
# ---------------------------------------------------------------------------

def _as_list(x) -> List[int]:
    if isinstance(x, torch.Tensor):
        return [int(v) for v in x.tolist()]
    return [int(v) for v in x]


def page_indptr(kv_lens: Sequence[int], page_size: int = PAGE) -> List[int]:
    """Prefix sum of ceil(kv_len / page_size); python/fmha_sm100/api.py:405-409."""
    out = [0]
    for k in _as_list(kv_lens):
        out.append(out[-1] + (k + page_size - 1) // page_size)
    return out


def gather_request_kv(pages: torch.Tensor, kv_indices: torch.Tensor, indptr: Sequence[int], b: int,
                      kv_len: int) -> torch.Tensor:
    """Logical [kv_len, Hkv, D] view of request ``b`` from paged storage
    ``[total_pages, Hkv, page, D]`` through the flat page table."""
    ids = kv_indices[indptr[b]:indptr[b + 1]].long()
    x = pages[ids].float()  # [n, H, P, D]
    n, H, P, D = x.shape
    x = x.permute(0, 2, 1, 3).reshape(n * P, H, D)
    return x[:kv_len]


# ---------------------------------------------------------------------------
# stage 1: per-(token, head, 128-key tile) max of the raw q.k
# ---------------------------------------------------------------------------

def tile_max_score_paged(q: torch.Tensor, k_pages: torch.Tensor, kv_indices: torch.Tensor,
                         qo_lens, kv_lens, max_k_tiles: int, causal: bool = True,
                         qo_offset=None) -> torch.Tensor:
    """Per-tile max score, layout ``[Hq, max_k_tiles, total_q]`` float32.

    Restates ``ref_tile_max_score`` (tests/regression/test_correctness.py:123-163)
    for paged K: raw dot product (no softmax scale), tile = one 128-key page,
    causal rule ``i + qo_offset >= j``, ``-inf`` where a tile is invisible.
    """
    qo_lens, kv_lens = _as_list(qo_lens), _as_list(kv_lens)
    total_q, Hq, D = q.shape
    Hkv = k_pages.shape[1]
    hr = Hq // Hkv
    indptr = page_indptr(kv_lens)
    res = torch.full((Hq, max_k_tiles, total_q), NEG_INF, dtype=torch.float32)
    qoff = 0
    for b, (ql, kl) in enumerate(zip(qo_lens, kv_lens)):
        off = int(qo_offset[b]) if qo_offset is not None else kl - ql
        if ql == 0:
            continue
        qs = q[qoff:qoff + ql].float()                       # [ql, Hq, D]
        ks = gather_request_kv(k_pages, kv_indices, indptr, b, kl)  # [kl, Hkv, D]
        ks = ks.repeat_interleave(hr, dim=1)                 # [kl, Hq, D]
        n_tiles = (kl + PAGE - 1) // PAGE
        for t in range(n_tiles):
            k0, k1 = t * PAGE, min((t + 1) * PAGE, kl)
            s = torch.einsum("qhd,khd->qhk", qs, ks[k0:k1])
            if causal:
                qpos = torch.arange(ql).unsqueeze(1) + off
                kpos = torch.arange(k0, k1).unsqueeze(0)
                s = s.masked_fill(~(qpos >= kpos).unsqueeze(1), NEG_INF)
            res[:, t, qoff:qoff + ql] = s.max(dim=-1).values.permute(1, 0)
        qoff += ql
    return res


def block_max_score(max_score: torch.Tensor, block_starts: Sequence[int]) -> torch.Tensor:
    """Max over the tokens of each query block: ``[H, K, T] -> [H, K, n_blocks]``.
    ``block_starts`` has n_blocks + 1 entries (token offsets)."""
    bs = _as_list(block_starts)
    H, K, _ = max_score.shape
    out = torch.full((H, K, len(bs) - 1), NEG_INF, dtype=torch.float32)
    for i in range(len(bs) - 1):
        if bs[i + 1] > bs[i]:
            out[:, :, i] = max_score[:, :, bs[i]:bs[i + 1]].max(dim=-1).values
    return out


# ---------------------------------------------------------------------------
# stage 2: deterministic top-k page selector
# ---------------------------------------------------------------------------

def topk_select(max_score: torch.Tensor, topk: int, num_valid_pages: Optional[int] = None,
                force_begin: int = 0, force_end: int = 0) -> torch.Tensor:
    """Top-k tile indices per (token, head) row, ``[T, H, topk]`` int32.

    Contract of ``sparse_topk_select`` (python/fmha_sm100/api.py:1179-1290,
    csrc/include/sparse_topk_select.cuh:852-886): exact top-k by float32 value,
    output ascending by index, ``-1`` at the tail; the first ``force_begin`` and
    the last ``force_end`` of the ``num_valid_pages`` tiles are always selected
    (their score is replaced by FLT_MAX, sparse_topk_select.cuh:340-347).
    Two choices the reference leaves open are fixed here: ties are broken
    toward the lower index, and a pick whose score is ``-inf`` is reported as
    ``-1`` (the reference returns an arbitrary masked index there).
    """
    H, K, T = max_score.shape
    nvp = K if num_valid_pages is None else int(num_valid_pages)
    s = max_score.permute(2, 0, 1).contiguous().clone()  # [T, H, K]
    s[:, :, nvp:] = NEG_INF
    flt_max = torch.finfo(torch.float32).max
    if force_begin > 0:
        s[:, :, :min(force_begin, nvp)] = flt_max
    if force_end > 0:
        s[:, :, max(nvp - force_end, 0):nvp] = flt_max
    s = torch.nan_to_num(s, nan=NEG_INF, posinf=flt_max, neginf=NEG_INF)
    # stable descending sort => lower index first among equals
    order = torch.sort(s, dim=-1, descending=True, stable=True)
    kk = min(topk, K)
    idx = order.indices[..., :kk].to(torch.int64)
    val = order.values[..., :kk]
    big = torch.iinfo(torch.int32).max
    idx = torch.where(val == NEG_INF, torch.full_like(idx, big), idx)
    idx = torch.sort(idx, dim=-1).values
    idx = torch.where(idx == big, torch.full_like(idx, -1), idx)
    out = torch.full((T, H, topk), -1, dtype=torch.int32)
    out[..., :kk] = idx.to(torch.int32)
    return out


# ---------------------------------------------------------------------------
# stage 3: sparse paged attention with per-token page lists
# ---------------------------------------------------------------------------

def sparse_attention_paged(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                           kv_indices: torch.Tensor, qo_lens, kv_lens,
                           kv_block_indexes: torch.Tensor, sm_scale: Optional[float] = None,
                           qo_offset=None, causal: bool = True,
                           k_scale: float = 1.0, v_scale: float = 1.0,
                           token_chunk: int = 256) -> Tuple[torch.Tensor, torch.Tensor]:
    """Sparse attention over the pages each token selected.

    Restates ``sparse_ref`` (tests/regression/test_sparse_attn.py:46-75) and
    ``sparse_attention_ref`` (python/fmha_sm100/cute/test_sparse_atten.py:201-365):
    ``kv_block_indexes[token, kv_head, i]`` are request-local logical page ids
    (``-1`` = unused); masking uses the ORIGINAL key position
    ``page * 128 + o <= i + qo_offset`` and ``< kv_len``; rows with no visible
    key give 0 and ``lse = -inf``.  K/V may be any dtype convertible to float
    (bf16, e4m3): values are used as stored, times ``k_scale`` / ``v_scale``.
    Returns ``(out[total_q, Hq, D] float32, lse[total_q, Hq] float32)`` with the
    natural-log LSE of the scaled logits.
    """
    qo_lens, kv_lens = _as_list(qo_lens), _as_list(kv_lens)
    total_q, Hq, D = q.shape
    Hkv = k_pages.shape[1]
    hr = Hq // Hkv
    topk = kv_block_indexes.shape[-1]
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    indptr = page_indptr(kv_lens)
    out = torch.zeros(total_q, Hq, D, dtype=torch.float32)
    lse = torch.full((total_q, Hq), NEG_INF, dtype=torch.float32)
    qoff = 0
    for b, (ql, kl) in enumerate(zip(qo_lens, kv_lens)):
        off = int(qo_offset[b]) if qo_offset is not None else kl - ql
        table = kv_indices[indptr[b]:indptr[b + 1]].long()
        for c0 in range(0, ql, token_chunk):
            c1 = min(c0 + token_chunk, ql)
            n = c1 - c0
            idx = kv_block_indexes[qoff + c0:qoff + c1].long()       # [n, Hkv, topk]
            valid = idx >= 0
            safe = torch.where(valid, idx, torch.zeros_like(idx))
            phys = table[safe]                                        # [n, Hkv, topk]
            hsel = torch.arange(Hkv).view(1, Hkv, 1).expand_as(phys)
            kg = k_pages[phys, hsel].float() * k_scale                # [n, Hkv, topk, P, D]
            vg = v_pages[phys, hsel].float() * v_scale
            qs = q[qoff + c0:qoff + c1].float().view(n, Hkv, hr, D)
            s = torch.einsum("nghd,ngkpd->nghkp", qs, kg) * sm_scale  # [n,Hkv,hr,topk,P]
            kpos = safe.unsqueeze(-1) * PAGE + torch.arange(PAGE).view(1, 1, 1, PAGE)  # [n,Hkv,topk,P]
            vis = valid.unsqueeze(-1) & (kpos < kl)
            if causal:
                qpos = (torch.arange(c0, c1) + off).view(n, 1, 1, 1)
                vis = vis & (kpos <= qpos)
            s = s.masked_fill(~vis.unsqueeze(2), NEG_INF)
            s = s.reshape(n, Hkv, hr, topk * PAGE)
            l = torch.logsumexp(s, dim=-1)                            # [n,Hkv,hr]
            has = torch.isfinite(l)
            p = torch.exp(s - torch.where(has, l, torch.zeros_like(l)).unsqueeze(-1))
            p = torch.where(has.unsqueeze(-1), p, torch.zeros_like(p))
            o = torch.einsum("nghk,ngkd->nghd", p, vg.reshape(n, Hkv, topk * PAGE, D))
            out[qoff + c0:qoff + c1] = o.reshape(n, Hq, D)
            lse[qoff + c0:qoff + c1] = torch.where(has, l, torch.full_like(l, NEG_INF)).reshape(n, Hq)
        qoff += ql
    return out, lse


def dense_attention_paged(q, k_pages, v_pages, kv_indices, qo_lens, kv_lens, sm_scale=None,
                          qo_offset=None, causal=True, k_scale=1.0, v_scale=1.0,
                          token_chunk: int = 512) -> Tuple[torch.Tensor, torch.Tensor]:
    """Dense causal attention over paged K/V; the role ``sdpa_ref`` plays in
    tests/regression/test_correctness.py:33-94 (row i sees column j iff
    ``i + qo_offset >= j``)."""
    qo_lens, kv_lens = _as_list(qo_lens), _as_list(kv_lens)
    total_q, Hq, D = q.shape
    Hkv = k_pages.shape[1]
    hr = Hq // Hkv
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    indptr = page_indptr(kv_lens)
    out = torch.zeros(total_q, Hq, D, dtype=torch.float32)
    lse = torch.full((total_q, Hq), NEG_INF, dtype=torch.float32)
    qoff = 0
    for b, (ql, kl) in enumerate(zip(qo_lens, kv_lens)):
        off = int(qo_offset[b]) if qo_offset is not None else kl - ql
        ks = gather_request_kv(k_pages, kv_indices, indptr, b, kl) * k_scale   # [kl,Hkv,D]
        vs = gather_request_kv(v_pages, kv_indices, indptr, b, kl) * v_scale
        for c0 in range(0, ql, token_chunk):
            c1 = min(c0 + token_chunk, ql)
            n = c1 - c0
            qs = q[qoff + c0:qoff + c1].float().view(n, Hkv, hr, D)
            s = torch.einsum("nghd,kgd->nghk", qs, ks) * sm_scale
            if causal:
                vis = torch.arange(kl).view(1, kl) <= (torch.arange(c0, c1) + off).view(n, 1)
                s = s.masked_fill(~vis.view(n, 1, 1, kl), NEG_INF)
            l = torch.logsumexp(s, dim=-1)
            has = torch.isfinite(l)
            p = torch.exp(s - torch.where(has, l, torch.zeros_like(l)).unsqueeze(-1))
            p = torch.where(has.unsqueeze(-1), p, torch.zeros_like(p))
            o = torch.einsum("nghk,kgd->nghd", p, vs)
            out[qoff + c0:qoff + c1] = o.reshape(n, Hq, D)
            lse[qoff + c0:qoff + c1] = torch.where(has, l, torch.full_like(l, NEG_INF)).reshape(n, Hq)
        qoff += ql
    return out, lse


def dense_block_indexes(qo_lens, kv_lens, qo_offset=None) -> torch.Tensor:
    """Page lists that make ``sparse_attention_paged`` dense (all causally visible pages)."""
    qo_lens, kv_lens = _as_list(qo_lens), _as_list(kv_lens)
    maxp = max((k + PAGE - 1) // PAGE for k in kv_lens)
    rows = []
    for b, (ql, kl) in enumerate(zip(qo_lens, kv_lens)):
        off = int(qo_offset[b]) if qo_offset is not None else kl - ql
        for i in range(ql):
            nvis = max(0, min(kl, i + off + 1))
            npg = (nvis + PAGE - 1) // PAGE
            rows.append(list(range(npg)) + [-1] * (maxp - npg))
    return torch.tensor(rows, dtype=torch.int32)


# ---------------------------------------------------------------------------
# k2q CSR (reverse index), python/fmha_sm100/cute/sparse_index_utils.py:195-325
# ---------------------------------------------------------------------------

def build_k2q_csr(q2k: torch.Tensor, cu_seqlens_q, cu_seqlens_k, blk_kv: int = PAGE):
    """q2k ``[Hkv, total_q, topk]`` (request-local block ids, -1 unused) ->
    ``row_ptr[Hkv, total_rows + 1]``, ``q_indices[Hkv, total_q * topk]`` where a
    row is one (KV block, request) pair, block-major, and holds the ascending request-local query
    indices that selected it.  Unused tail of ``q_indices`` is -1."""
    Hkv, total_q, topk = q2k.shape
    cq, ck = _as_list(cu_seqlens_q), _as_list(cu_seqlens_k)
    B = len(cq) - 1
    nblk = [((ck[b + 1] - ck[b]) + blk_kv - 1) // blk_kv for b in range(B)]
    # rows are packed block-major: for kv block 0 all requests, then block 1, ...
    # (sparse_index_utils.py:176-192)
    row_map = [[-1] * max(nblk + [0]) for _ in range(B)]
    total_rows = 0
    for blk in range(max(nblk + [0])):
        for b in range(B):
            if blk < nblk[b]:
                row_map[b][blk] = total_rows
                total_rows += 1
    row_ptr = torch.zeros(Hkv, total_rows + 1, dtype=torch.int32)
    q_indices = torch.full((Hkv, total_q * topk), -1, dtype=torch.int32)
    for h in range(Hkv):
        buckets = [[] for _ in range(total_rows)]
        for b in range(B):
            for qi in range(cq[b], cq[b + 1]):
                for j in range(topk):
                    blk = int(q2k[h, qi, j])
                    if blk >= 0:
                        buckets[row_map[b][blk]].append(qi - cq[b])
        pos = 0
        for r, bk in enumerate(buckets):
            row_ptr[h, r] = pos
            bk.sort()
            for x in bk:
                q_indices[h, pos] = x
                pos += 1
        row_ptr[h, total_rows] = pos
    return row_ptr, q_indices


# ---------------------------------------------------------------------------
# FP8 e4m3 per-tensor quantisation (scale = amax / 448)
# ---------------------------------------------------------------------------

def quantize_fp8_per_tensor(x: torch.Tensor) -> Tuple[torch.Tensor, float]:
    """``x ~= q.float() * scale`` with ``q`` float8_e4m3fn, ``scale = amax / 448``."""
    amax = float(x.float().abs().max())
    scale = amax / FP8_MAX if amax > 0 else 1.0
    q = (x.float() / scale).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return q, scale


# ---------------------------------------------------------------------------
# NVFP4: packed e2m1 + e4m3 scale per 16 elements (128x4 tiled) + fp32 global scale
# ---------------------------------------------------------------------------

def nvfp4_scale_offset(row: torch.Tensor, col: torch.Tensor, scale_cols: int) -> torch.Tensor:
    """Flat offset of logical scale (row, col) in the 128x4-tiled scale storage;
    python/fmha_sm100/cute/quantize.py:58-90."""
    tiles_n = (scale_cols + 3) // 4
    return ((row // 128) * tiles_n + col // 4) * 512 + (row % 32) * 16 + ((row % 128) // 32) * 4 + col % 4


def _e2m1_round(x: torch.Tensor) -> torch.Tensor:
    """Round-to-nearest-even onto the e2m1 grid {0,.5,1,1.5,2,3,4,6} with
    saturation; returns the 4-bit code (sign in bit 3)."""
    a = x.abs().clamp(max=FP4_MAX)
    grid = FP4_LUT[:8]
    # nearest with ties to the even mantissa code (codes 0,2,4,6 have mantissa bit 0)
    d = (a.unsqueeze(-1) - grid).abs()
    best = d.min(dim=-1)
    code = best.indices
    # resolve ties: if the next grid point is equally near pick the even code
    nxt = (code + 1).clamp(max=7)
    tie = (d.gather(-1, nxt.unsqueeze(-1)).squeeze(-1) == best.values) & (nxt != code)
    code = torch.where(tie & (code % 2 == 1), nxt, code)
    sign = (x < 0) | ((x == 0) & (torch.signbit(x)))
    return (code + sign.long() * 8).to(torch.uint8)


def quantize_nvfp4(x: torch.Tensor):
    """Quantise ``x[..., D]`` (D % 16 == 0) to NVFP4.

    Storage contract (python/fmha_sm100/cute/quantize.py:145-159, 326-331 and
    atten_fwd_nvfp4_kv.py:1329-1336): two e2m1 codes per byte (low nibble = even
    element), one e4m3 scale per 16 elements stored in 128x4 tiles with logical
    row = flattened leading index, fp32 global scale = amax / (448 * 6).
    The rounding rules are this build's own (the reference delegates them to
    Transformer Engine): block scale = RNE-to-e4m3 of ``amax16 / (6 * global)``,
    element = RNE to e2m1 with saturation.  Returns
    ``(data uint8[..., D/2], scale_128x4 uint8[flat], global_scale float)``.
    """
    D = x.shape[-1]
    xf = x.float().reshape(-1, D)
    rows = xf.shape[0]
    scols = D // NVFP4_BLOCK
    amax = float(xf.abs().max())
    gscale = amax / (FP8_MAX * FP4_MAX) if amax > 0 else 1.0
    blk = xf.view(rows, scols, NVFP4_BLOCK)
    bamax = blk.abs().amax(dim=-1)
    bscale = (bamax / (FP4_MAX * gscale)).clamp(max=FP8_MAX).to(torch.float8_e4m3fn)
    bs = bscale.float()
    denom = torch.where(bs > 0, bs * gscale, torch.ones_like(bs)).unsqueeze(-1)
    codes = _e2m1_round(blk / denom).view(rows, D)
    data = (codes[:, 0::2] | (codes[:, 1::2] << 4)).to(torch.uint8)
    rows_pad = (rows + 127) // 128 * 128
    cols_pad = (scols + 3) // 4 * 4
    sflat = torch.zeros(rows_pad * cols_pad, dtype=torch.uint8)
    r = torch.arange(rows).view(-1, 1).expand(rows, scols)
    c = torch.arange(scols).view(1, -1).expand(rows, scols)
    sflat[nvfp4_scale_offset(r, c, scols).reshape(-1)] = bscale.view(torch.uint8).reshape(-1)
    return data.view(*x.shape[:-1], D // 2), sflat, gscale


def dequantize_nvfp4(data: torch.Tensor, scale_128x4: torch.Tensor, global_scale: float,
                     include_global_scale: bool = True) -> torch.Tensor:
    """``e2m1 * e4m3_block_scale * fp32_global`` -> float32 ``[..., D]``;
    python/fmha_sm100/cute/quantize.py:265-343 (without the final bf16 cast)."""
    D = data.shape[-1] * 2
    packed = data.reshape(-1, D // 2)
    rows = packed.shape[0]
    scols = D // NVFP4_BLOCK
    vals = torch.empty(rows, D, dtype=torch.float32)
    vals[:, 0::2] = FP4_LUT[(packed & 0x0F).long()]
    vals[:, 1::2] = FP4_LUT[(packed >> 4).long()]
    r = torch.arange(rows).view(-1, 1).expand(rows, scols)
    c = torch.arange(scols).view(1, -1).expand(rows, scols)
    s = scale_128x4.reshape(-1)[nvfp4_scale_offset(r, c, scols).reshape(-1)].view(rows, scols)
    s = s.view(torch.float8_e4m3fn).float().repeat_interleave(NVFP4_BLOCK, dim=1)
    out = vals * s
    if include_global_scale:
        out = out * float(global_scale)
    return out.view(*data.shape[:-1], D)


# ---------------------------------------------------------------------------
# KV-cache append (quantise new rows into the paged cache) in explicit float32 arithmetic
# ---------------------------------------------------------------------------

def _scatter_rows(cache: torch.Tensor, rows: torch.Tensor, slots: torch.Tensor) -> None:
    """``cache[pages, Hkv, 128, W]`` <- ``rows[tokens, Hkv, W]`` at ``slots`` (page * 128 + position); negative or
    out-of-range slots are skipped."""
    ok = (slots >= 0) & (slots < cache.shape[0] * PAGE)
    sl = slots[ok].long()
    cache[sl // PAGE, :, sl % PAGE] = rows[ok]


def kv_append_fp8(k_new, v_new, k_cache, v_cache, slots, k_scale: float, v_scale: float) -> None:
    """Per-tensor FP8 append: ``e4m3_rne(clamp(x * (1 / scale), +-448))`` -- the scale is first rounded to
    float32, its reciprocal is one float32 division, every element one float32 multiplication -- written into
    uint8 caches ``[pages, Hkv, 128, 128]`` in place.  ``scale`` is the dequant scale (``amax / 448`` by the
    convention this build restates for the reference's per-tensor FP8 K/V)."""
    one = torch.tensor(1.0, dtype=torch.float32)
    for new, cache, s in ((k_new, k_cache, k_scale), (v_new, v_cache, v_scale)):
        q = (new.float() * (one / torch.tensor(s, dtype=torch.float32))).clamp(-FP8_MAX, FP8_MAX)
        _scatter_rows(cache, q.to(torch.float8_e4m3fn).view(torch.uint8), slots)


def kv_append_nvfp4(k_new, v_new, k_cache, v_cache, k_block_scales, v_block_scales, slots,
                    k_global: float, v_global: float) -> None:
    """NVFP4 append with given global scales g (rounded to float32 first): block scale
    ``s = e4m3_rne(min(amax16 / (6 * g), 448))``, element ``e2m1_rne(x * (1 / (s * g)))`` saturating (``x * 1``
    when s == 0), every product and quotient a float32 operation (one division per block for the scale, one for
    the reciprocal, one multiplication per element).  Data go to uint8 caches ``[pages, Hkv, 128, 64]``
    (low nibble = even element, python/fmha_sm100/cute/quantize.py:326-331), scales to the flat 128x4-tiled
    storage at row ``(page * Hkv + head) * 128 + position`` (quantize.py:58-90,
    src/sm100/fwd/atten_fwd_nvfp4_kv.py:1329-1336)."""
    for new, cache, bsc, g in ((k_new, k_cache, k_block_scales, k_global), (v_new, v_cache, v_block_scales, v_global)):
        n, hkv, D = new.shape
        g32 = torch.tensor(g, dtype=torch.float32)
        blk = new.float().view(n, hkv, D // NVFP4_BLOCK, NVFP4_BLOCK)
        bamax = blk.abs().amax(dim=-1)
        bscale = (bamax / (torch.tensor(6.0, dtype=torch.float32) * g32)).clamp(max=FP8_MAX).to(torch.float8_e4m3fn)
        bs = bscale.float()
        den = torch.where(bs > 0, bs * g32, torch.ones_like(bs)).unsqueeze(-1)
        codes = _e2m1_round(blk * (torch.tensor(1.0, dtype=torch.float32) / den)).view(n, hkv, D)
        _scatter_rows(cache, (codes[..., 0::2] | (codes[..., 1::2] << 4)).to(torch.uint8), slots)
        ok = (slots >= 0) & (slots < cache.shape[0] * PAGE)
        sl = slots[ok].long()
        heads = torch.arange(hkv).view(1, hkv, 1)
        row = ((sl // PAGE).view(-1, 1, 1) * hkv + heads) * PAGE + (sl % PAGE).view(-1, 1, 1)
        col = torch.arange(D // NVFP4_BLOCK).view(1, 1, -1)
        off = nvfp4_scale_offset(row.expand(-1, hkv, D // NVFP4_BLOCK), col.expand(sl.numel(), hkv, -1),
                                 D // NVFP4_BLOCK)
        bsc.view(-1)[off.reshape(-1)] = bscale.view(torch.uint8)[ok].reshape(-1)   # flat or [rows, 8] storage


# ---------------------------------------------------------------------------
# end-to-end pipeline of the first BASELINE configuration (CPU-runnable)
# ---------------------------------------------------------------------------

def pipeline_block_sparse(q, k_pages, v_pages, kv_indices, qo_lens, kv_lens, topk, proxy_heads=1,
                          proxy_dim=64, sm_scale=None, q_block: int = PAGE):
    """Proxy pass on ``q[:, :proxy_heads, :proxy_dim]`` vs kv-head 0 of K ->
    max over each ``q_block`` query block -> top-k -> same list for every token
    of the block and every KV head -> sparse attention.  Returns
    ``(out, lse, kv_block_indexes[total_q, Hkv, topk], max_score)``."""
    qo_lens, kv_lens = _as_list(qo_lens), _as_list(kv_lens)
    Hkv = k_pages.shape[1]
    qp = q[:, :proxy_heads, :proxy_dim]
    kp = k_pages[:, :1, :, :proxy_dim]
    maxk = max((k + PAGE - 1) // PAGE for k in kv_lens)
    ms = tile_max_score_paged(qp, kp, kv_indices, qo_lens, kv_lens, maxk)
    starts, owner = [0], []
    off = 0
    for b, ql in enumerate(qo_lens):
        for s0 in range(0, ql, q_block):
            starts.append(off + min(s0 + q_block, ql))
            owner.append(b)
        off += ql
    bm = block_max_score(ms, starts)                       # [Hp, K, nblk]
    sel = topk_select(bm, topk, num_valid_pages=maxk)     # [nblk, Hp, topk]
    total_q = q.shape[0]
    idx = torch.empty(total_q, Hkv, topk, dtype=torch.int32)
    for i in range(len(starts) - 1):
        src = sel[i]
        if src.shape[0] != Hkv:
            src = src[:1].expand(Hkv, topk)
        idx[starts[i]:starts[i + 1]] = src.unsqueeze(0)
    out, lse = sparse_attention_paged(q, k_pages, v_pages, kv_indices, qo_lens, kv_lens, idx, sm_scale)
    return out, lse, idx, ms


# ---------------------------------------------------------------------------
# sub-sampled checks at full benchmark size
# ---------------------------------------------------------------------------

def sampled_sparse_error(out_rows, q_rows, k_pages, v_pages, table, kv_len, first_pos, idx_rows,
                         k_scale: float = 1.0, v_scale: float = 1.0, token_chunk: int = 16) -> float:
    """Max-abs difference between ``out_rows`` (``[n, Hq, D]``, any float dtype) and the oracle for ``n``
    consecutive query tokens of ONE request: token ``i`` sits at request position ``first_pos + i`` of a
    request with ``kv_len`` keys, ``table`` is that request's page table, ``idx_rows`` ``[n, Hkv, topk]`` its
    page lists.  ``k_pages`` / ``v_pages`` are the page pool (or any tensor ``table`` indexes into).  Lets a
    test compare a few (request, query block) slices of a benchmark-sized launch without running the oracle
    on all of it."""
    n = q_rows.shape[0]
    ref, _ = sparse_attention_paged(q_rows, k_pages, v_pages, table, [n], [kv_len], idx_rows,
                                    qo_offset=[first_pos], k_scale=k_scale, v_scale=v_scale,
                                    token_chunk=token_chunk)
    return float((out_rows.float() - ref).abs().max())


# ---------------------------------------------------------------------------
# FP4 indexer: per-page maxima of Q K^T with Q and K as packed e2m1 + block scales
# ---------------------------------------------------------------------------
_E2M1 = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0])
FP4_GROUPS = {"nvfp4": 8, "mxfp4": 4}


def fp4_scale_to_float(scale: torch.Tensor, fmt: str) -> torch.Tensor:
    """Block scales as float32: e4m3 (nvfp4) or ue8m0 = 2^(byte - 127) (mxfp4); raw uint8 bytes are accepted."""
    raw = scale.view(torch.uint8).cpu().to(torch.int64)
    if fmt == "mxfp4":
        return torch.ldexp(torch.ones(raw.shape), (raw - 127).to(torch.int32)).float()
    e, m = (raw >> 3) & 15, raw & 7
    mag = torch.where(e == 0, m.double() * 2.0 ** -9, torch.ldexp(1.0 + m.double() / 8.0, (e - 7).to(torch.int32)))
    return torch.where((raw & 0x80) != 0, -mag, mag).float()


def fp4_dequantize(packed: torch.Tensor, scale: torch.Tensor, fmt: str) -> torch.Tensor:
    """[..., 64] packed bytes (low nibble = even element) and logical scales [..., G] -> float32 [..., 128]; what
    ``_decode_fp4x2_to_f32`` / ``_dequantize_public_fp4`` do in
    python/fmha_sm100/cute/test_fp4_indexer.py:153-167."""
    raw = packed.view(torch.uint8).cpu().to(torch.int64)
    vals = torch.stack((_E2M1[raw & 15], _E2M1[(raw >> 4) & 15]), dim=-1).reshape(*packed.shape[:-1], 128)
    s = fp4_scale_to_float(scale, fmt)
    return vals * torch.repeat_interleave(s, 128 // FP4_GROUPS[fmt], dim=-1)


def fp4_mma_scale_offset(m, g, l, mn: int, groups: int):
    """Byte offset of scale (row m, group g, batch l) in the 128x4-tiled storage
    (fp4_indexer_mma_scale_storage_stride, python/fmha_sm100/cute/fp4_indexer_interface.py:243-249)."""
    rest_m, rest_g = (mn + 127) // 128, (groups + 3) // 4
    return (l * 512 * rest_m * rest_g + (m // 128) * 512 * rest_g + (g // 4) * 512 + (m % 32) * 16
            + ((m % 128) // 32) * 4 + g % 4)


def fp4_reorder_scales(q_scale: torch.Tensor, k_scale: torch.Tensor, fmt: str):
    """Logical Q [T, Hq, G] / K [P, Hk, 128, G] scale bytes -> flat uint8 storage in the 128x4-tiled layout
    (python/fmha_sm100/cute/src/sm100/fp4_indexer.py:83-199).  Padding bytes are zero."""
    G = FP4_GROUPS[fmt]
    qs, ks = q_scale.view(torch.uint8).cpu(), k_scale.view(torch.uint8).cpu()
    T, Hq, _ = qs.shape
    P, Hk, _, _ = ks.shape
    rest_g = (G + 3) // 4
    q_out = torch.zeros(Hq * ((T + 127) // 128) * rest_g * 512, dtype=torch.uint8)
    m, l, g = torch.meshgrid(torch.arange(T), torch.arange(Hq), torch.arange(G), indexing="ij")
    q_out[fp4_mma_scale_offset(m, g, l, T, G).reshape(-1)] = qs.reshape(-1)
    k_out = torch.zeros(P * Hk * rest_g * 512, dtype=torch.uint8)
    l, m, g = torch.meshgrid(torch.arange(P * Hk), torch.arange(128), torch.arange(G), indexing="ij")
    k_out[fp4_mma_scale_offset(m, g, l, 128, G).reshape(-1)] = ks.reshape(-1)
    return q_out, k_out


def fp4_indexer_block_scores(q_fp4, k_fp4, q_scale, k_scale, cu_seqlens_q, cu_seqlens_k, cu_page_offsets, kv_indices,
                             fmt: str, causal: bool = False, qo_offset=None) -> torch.Tensor:
    """``[Hq, max ceil(k_len / 128), total_q]`` float32, -inf where a page is beyond the request or wholly masked
    (row i of a request sees key j iff ``i + offset >= j``, offset = k_len - q_len unless given): the contract of
    ``fp4_indexer_block_scores`` as ``_reference_block_scores`` states it
    (python/fmha_sm100/cute/test_fp4_indexer.py:273-327), one matmul per (request, head) instead of Python loops."""
    q = fp4_dequantize(q_fp4, q_scale, fmt)
    k = fp4_dequantize(k_fp4, k_scale, fmt)
    cu_q, cu_k, cu_p = _as_list(cu_seqlens_q), _as_list(cu_seqlens_k), _as_list(cu_page_offsets)
    table = kv_indices.cpu().long()
    B = len(cu_q) - 1
    T, Hq, _ = q.shape
    Hk = k.shape[1]
    hr = Hq // Hk
    k_lens = [cu_k[b + 1] - cu_k[b] for b in range(B)]
    max_tiles = max((kl + PAGE - 1) // PAGE for kl in k_lens) if B else 0
    out = torch.full((Hq, max_tiles, T), NEG_INF, dtype=torch.float32)
    for b in range(B):
        q0, ql, kl = cu_q[b], cu_q[b + 1] - cu_q[b], k_lens[b]
        n = (kl + PAGE - 1) // PAGE
        if ql == 0 or n == 0:
            continue
        off = int(qo_offset[b]) if qo_offset is not None else kl - ql
        pages = table[cu_p[b]:cu_p[b] + n]
        for h in range(Hq):
            kk = k[pages, h // hr].reshape(n * PAGE, 128)                 # [n * 128, 128]
            s = q[q0:q0 + ql, h] @ kk.T                                   # [ql, n * 128]
            col = torch.arange(n * PAGE).view(1, -1)
            vis = col < kl
            if causal:
                vis = vis & (torch.arange(ql).view(-1, 1) + off >= col)
            s = torch.where(vis, s, torch.full_like(s, NEG_INF))
            out[h, :n, q0:q0 + ql] = s.view(ql, n, PAGE).amax(dim=2).T
    return out
