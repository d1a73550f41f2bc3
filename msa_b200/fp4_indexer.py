"""FP4 indexer: per-page maxima of Q K^T with Q and K stored as packed e2m1 and block scales -- the public
interface of python/fmha_sm100/cute/fp4_indexer_interface.py (``fp4_indexer_block_scores``, :745-1056; scale
storage helpers :220-249; ``fp4_indexer_reorder_scales_for_mma_cute``, :333-433), same names, arguments and
result layout.

The reference multiplies the packed operands with a block-scaled tensor-core instruction.  Here Q is dequantised
once to bf16 (``msa_fp4_dequant_rows``) and K page by page inside the score-only kernel, both exactly (e2m1 times
an e4m3 or power-of-two scale has at most six significant bits), and the products accumulate in float32 on the
tensor core -- the same numbers up to summation order.  MXFP4 scales outside 2^-24 .. 2^15 saturate in the K path.
"""
from __future__ import annotations

import ctypes
import math
from typing import Optional, Tuple

import torch

from . import _lib
from ._lib import FmhaArgs, MsaError, check, get_lib
from .api import TensorKeyedCache, _flag_fill_entries, _host_plan, _ptr, _stream

PAGE = 128
_GROUPS = {"mxfp4": 4, "nvfp4": 8}
_FORMAT_CODE = {"nvfp4": 0, "mxfp4": 1}
_PUBLIC, _MMA = "public", "preordered_mma"
_PLAN_CACHE = TensorKeyedCache(64)


def _fmt(fp4_format: str) -> str:
    f = str(fp4_format).lower()
    if f not in _GROUPS:
        raise ValueError(f"format must be one of {sorted(_GROUPS)}, got {fp4_format!r}")
    return f


def _scale_dtype(fmt: str):
    return torch.float8_e8m0fnu if fmt == "mxfp4" else torch.float8_e4m3fn


def _ceil_div(a: int, b: int) -> int:
    return (int(a) + int(b) - 1) // int(b)


def fp4_indexer_mma_scale_shape(mn: int, l: int, *, fp4_format: str) -> Tuple[int, ...]:
    """Semantic view ``(32, 4, restM, 4, restG, L)`` of the tiled scale storage."""
    return (32, 4, _ceil_div(mn, 128), 4, _ceil_div(_GROUPS[_fmt(fp4_format)], 4), int(l))


def fp4_indexer_mma_scale_stride(mn: int, l: int, *, fp4_format: str) -> Tuple[int, ...]:
    rest_m, rest_g = _ceil_div(mn, 128), _ceil_div(_GROUPS[_fmt(fp4_format)], 4)
    return (16, 4, 512 * rest_g, 1, 512, 512 * rest_m * rest_g)


def fp4_indexer_mma_scale_storage_shape(mn: int, l: int, *, fp4_format: str) -> Tuple[int, ...]:
    """Contiguous storage ``(L, restM, restG, 32, 4, 4)`` of preordered scales."""
    return (int(l), _ceil_div(mn, 128), _ceil_div(_GROUPS[_fmt(fp4_format)], 4), 32, 4, 4)


def fp4_indexer_mma_scale_storage_stride(mn: int, l: int, *, fp4_format: str) -> Tuple[int, ...]:
    rest_m, rest_g = _ceil_div(mn, 128), _ceil_div(_GROUPS[_fmt(fp4_format)], 4)
    return (512 * rest_m * rest_g, 512 * rest_g, 512, 16, 4, 1)


def _as_bytes(t: torch.Tensor, name: str, last: int, ndim: int) -> torch.Tensor:
    if not t.is_cuda or not t.is_contiguous():
        raise ValueError(f"{name} must be a contiguous CUDA tensor")
    if t.ndim != ndim or int(t.shape[-1]) != last:
        raise ValueError(f"{name} must have {ndim} dimensions with {last} packed bytes innermost, got {tuple(t.shape)}")
    if t.element_size() != 1:
        raise TypeError(f"{name} must use a one-byte packed FP4 storage dtype, got {t.dtype}")
    return t.view(torch.uint8)


def fp4_indexer_reorder_scales_for_mma_cute(q_scale: torch.Tensor, k_scale: torch.Tensor, *, fp4_format: str):
    """Logical scales ``q_scale [total_q, Hq, G]`` / ``k_scale [pages, Hk, 128, G]`` -> the two tensors in tiled
    storage (views shaped ``fp4_indexer_mma_scale_shape``, as the reference returns them)."""
    fmt = _fmt(fp4_format)
    G = _GROUPS[fmt]
    if q_scale.ndim != 3 or q_scale.shape[2] != G or k_scale.ndim != 4 or k_scale.shape[2] != PAGE or k_scale.shape[3] != G:
        raise ValueError(f"expected q_scale [T, Hq, {G}] and k_scale [P, Hk, 128, {G}]")
    if q_scale.dtype != _scale_dtype(fmt) or k_scale.dtype != _scale_dtype(fmt):
        raise TypeError(f"scales must have dtype {_scale_dtype(fmt)}")
    lib = get_lib()
    T, Hq = int(q_scale.shape[0]), int(q_scale.shape[1])
    P, Hk = int(k_scale.shape[0]), int(k_scale.shape[1])
    outs = []
    for src, mn, l, k_layout in ((q_scale, T, Hq, 0), (k_scale, PAGE, P * Hk, 1)):
        shape = fp4_indexer_mma_scale_storage_shape(mn, l, fp4_format=fmt)
        # rows of the last 128-row block that do not exist keep a zero byte
        store = torch.zeros(shape, dtype=torch.uint8, device=src.device)
        check(lib.msa_fp4_reorder_scales(_ptr(src.contiguous()), _FORMAT_CODE[fmt], mn, l, k_layout, _ptr(store),
                                         _stream()), "msa_fp4_reorder_scales")
        outs.append(store.view(_scale_dtype(fmt)).permute(3, 4, 1, 5, 2, 0))
    return outs[0], outs[1]


fp4_indexer_reorder_scales_for_mma = fp4_indexer_reorder_scales_for_mma_cute


def _check_mma_storage(scale: torch.Tensor, name: str, fmt: str, mn: int, l: int) -> None:
    """Accepts the permuted view the reorder function returns or its contiguous storage."""
    shape = fp4_indexer_mma_scale_storage_shape(mn, l, fp4_format=fmt)
    view = fp4_indexer_mma_scale_shape(mn, l, fp4_format=fmt)
    ok = (tuple(scale.shape) == shape and scale.is_contiguous()) or (
        tuple(scale.shape) == view and tuple(scale.stride()) == fp4_indexer_mma_scale_stride(mn, l, fp4_format=fmt))
    if not ok:
        raise ValueError(f"{name} must have MMA storage shape {shape} (or its view {view}), got {tuple(scale.shape)} "
                         f"with strides {tuple(scale.stride())}")
    if scale.element_size() != 1:
        raise TypeError(f"{name} must be a one-byte scale dtype, got {scale.dtype}")


def _plan(cu_q: torch.Tensor, cu_k: torch.Tensor, cu_p: torch.Tensor, qo_offset, causal: bool, Hq: int, Hk: int,
          max_q: int):
    """Work list of the score kernel for these prefix arrays (host copy once per distinct set of tensors)."""
    key_tensors, key_extra = (cu_q, cu_k, cu_p, qo_offset), (bool(causal), Hq, Hk, int(max_q))
    hit = _PLAN_CACHE.get(key_tensors, key_extra)
    if hit is not None:
        return hit
    cq, ck, cp = (t.detach().cpu().tolist() for t in (cu_q, cu_k, cu_p))
    ql = [cq[i + 1] - cq[i] for i in range(len(cq) - 1)]
    kl = [ck[i + 1] - ck[i] for i in range(len(ck) - 1)]
    if any(x < 0 for x in ql) or any(x < 0 for x in kl):
        raise ValueError("cu_seqlens must be non-decreasing")
    if causal:
        off = qo_offset.detach().cpu().tolist() if qo_offset is not None else [k - q for q, k in zip(ql, kl)]
    else:
        off = None
    # Requests with only a few tokens (decode): the heads of a GQA group share the 128 rows of a query tile, as the
    # reference's packed-Q decode path does (fp4_indexer_interface.py:913-948).  hb heads x 128 / hb tokens.
    hr = Hq // Hk
    pow2 = hr & -hr                                       # largest power of two dividing the heads per KV head
    need = 1 << max(0, int(max(ql + [1])) - 1).bit_length()  # tokens of the longest request, rounded up
    hb = max(1, min(pow2, 128 // min(128, need)))
    rows = 256 // hb
    sms = torch.cuda.get_device_properties(cu_q.device).multi_processor_count
    work = _host_plan(ql, kl, off, causal, True, Hq, Hk, tile_rows=rows)[0]
    items = int(work.shape[0]) * (Hq // hb)
    max_pages = max([(k + PAGE - 1) // PAGE for k in kl] + [0])
    # fewer work items than SMs: cut every entry's page range (per-page maxima need no merging afterwards)
    # into whole waves of one CTA per SM where possible, at least 16 pages per piece
    splits, best = 1, -1.0
    for n_s in range(1, max(1, min(max_pages // 16, 64)) + 1):
        if items == 0 or items * n_s > 64 * sms and n_s > 1:
            break
        eff = items * n_s / (math.ceil(items * n_s / sms) * sms) - 0.01 * n_s
        if eff > best:
            splits, best = n_s, eff
    if splits > 1:
        work = _host_plan(ql, kl, off, causal, True, Hq, Hk, tile_rows=rows, dense_kv_splits=splits)[0]
    if work.shape[0]:
        # page-table offsets as the caller gives them (they need not be the running sum of ceil(k_len / 128))
        work[:, 6] = [cp[r] for r in work[:, 0].tolist()]
    # the entry that covers a tile's highest pages also writes -inf above them (no pre-fill of the score tensor),
    # unless some tile sees no page at all
    fill = _flag_fill_entries(work, causal)
    plan = dict(fill=fill, work=torch.from_numpy(work).to(cu_q.device).contiguous(), n_work=int(work.shape[0]), pack_heads=hb,
                tile_rows=rows, status=torch.zeros(1, dtype=torch.int32, device=cu_q.device),
                max_kv=max(kl) if kl else 0)
    return _PLAN_CACHE.put(key_tensors, key_extra, plan)


def fp4_indexer_block_scores(
    q_fp4: torch.Tensor,
    k_fp4: torch.Tensor,
    q_scale: torch.Tensor,
    k_scale: torch.Tensor,
    cu_seqlens_q: torch.Tensor,
    cu_seqlens_k: torch.Tensor,
    cu_page_offsets: torch.Tensor,
    *,
    max_seqlen_q: int,
    max_seqlen_k: int,
    kv_indices: torch.Tensor,
    fp4_format: str,
    causal: bool = False,
    qo_offset: Optional[torch.Tensor] = None,
    scale_layout: str = _MMA,
) -> torch.Tensor:
    """FP4 QK max scores per 128-token KV page: ``[Hq, ceil(max_seqlen_k / 128), total_q]`` float32, -inf beyond a
    request's pages and where the causal rule hides a whole page.  Arguments as in the reference
    (python/fmha_sm100/cute/fp4_indexer_interface.py:745-818): ``q_fp4 [total_q, Hq, 64]``, ``k_fp4 [pages, Hk, 128,
    64]``, scales logical (``scale_layout="public"``: ``[total_q, Hq, G]`` / ``[pages, Hk, 128, G]``) or preordered
    (``"preordered_mma"``, the default)."""
    fmt = _fmt(fp4_format)
    if scale_layout not in (_PUBLIC, _MMA):
        raise ValueError(f"scale_layout must be 'public' or 'preordered_mma', got {scale_layout!r}")
    q_bytes = _as_bytes(q_fp4, "q_fp4", 64, 3)
    k_bytes = _as_bytes(k_fp4, "k_fp4", 64, 4)
    total_q, Hq, _ = (int(v) for v in q_bytes.shape)
    n_pages, Hk, page, _ = (int(v) for v in k_bytes.shape)
    if page != PAGE:
        raise ValueError(f"k_fp4 page_size must be 128, got {page}")
    if Hq % Hk != 0:
        raise ValueError("num_qo_heads must be divisible by num_kv_heads")
    for name, t in (("cu_seqlens_q", cu_seqlens_q), ("cu_seqlens_k", cu_seqlens_k), ("cu_page_offsets", cu_page_offsets)):
        if t.device != q_fp4.device or t.dtype != torch.int32 or t.ndim != 1 or not t.is_contiguous():
            raise ValueError(f"{name} must be a contiguous int32 vector on the device of q_fp4")
    if cu_seqlens_q.shape != cu_seqlens_k.shape or cu_seqlens_q.shape != cu_page_offsets.shape:
        raise ValueError("cu_seqlens_q, cu_seqlens_k, and cu_page_offsets must have shape [B + 1]")
    if kv_indices is None or kv_indices.device != q_fp4.device or kv_indices.dtype != torch.int32 or kv_indices.ndim != 1:
        raise ValueError("kv_indices must have shape [sum_pages], dtype torch.int32, and match q_fp4.device")
    if qo_offset is not None and not causal:
        raise ValueError("qo_offset is only valid when causal=True")
    G = _GROUPS[fmt]
    if scale_layout == _PUBLIC:
        if tuple(q_scale.shape) != (total_q, Hq, G) or tuple(k_scale.shape) != (n_pages, Hk, PAGE, G):
            raise ValueError(f"public scales must be [total_q, Hq, {G}] and [pages, Hk, 128, {G}]")
        if q_scale.dtype != _scale_dtype(fmt) or k_scale.dtype != _scale_dtype(fmt):
            raise TypeError(f"scales must have dtype {_scale_dtype(fmt)}")
    else:
        _check_mma_storage(q_scale, "q_scale", fmt, total_q, Hq)
        _check_mma_storage(k_scale, "k_scale", fmt, PAGE, n_pages * Hk)
    max_k_tiles = _ceil_div(int(max_seqlen_k), PAGE)
    if max_k_tiles == 0 or total_q == 0:
        return torch.full((Hq, max_k_tiles, total_q), -float("inf"), dtype=torch.float32, device=q_fp4.device)
    lib = get_lib()
    plan = _plan(cu_seqlens_q, cu_seqlens_k, cu_page_offsets, qo_offset, bool(causal), Hq, Hk, int(max_seqlen_q))
    if plan["fill"]:
        scores = torch.empty((Hq, max_k_tiles, total_q), dtype=torch.float32, device=q_fp4.device)
    else:
        scores = torch.full((Hq, max_k_tiles, total_q), -float("inf"), dtype=torch.float32, device=q_fp4.device)
    if plan["max_kv"] > max_k_tiles * PAGE:
        raise ValueError("max_seqlen_k is smaller than the longest KV segment")
    # K scales: the kernel reads the tiled storage; logical ones are tiled first (what the reference does too)
    if scale_layout == _PUBLIC:
        store = torch.zeros(fp4_indexer_mma_scale_storage_shape(PAGE, n_pages * Hk, fp4_format=fmt), dtype=torch.uint8,
                            device=q_fp4.device)
        check(lib.msa_fp4_reorder_scales(_ptr(k_scale.contiguous()), _FORMAT_CODE[fmt], PAGE, n_pages * Hk, 1,
                                         _ptr(store), _stream()), "msa_fp4_reorder_scales")
        k_sf = store
    else:
        k_sf = k_scale            # either form of the storage starts at the same address and is dense
    q16 = torch.empty(total_q, Hq, 128, dtype=torch.bfloat16, device=q_fp4.device)
    check(lib.msa_fp4_dequant_rows(_ptr(q_bytes), _ptr(q_scale), _FORMAT_CODE[fmt], 0 if scale_layout == _PUBLIC else 1,
                                   total_q, Hq, _ptr(q16), _stream()), "msa_fp4_dequant_rows")
    a = FmhaArgs()
    a.q, a.k, a.v = _ptr(q16), _ptr(k_bytes), None
    a.out, a.lse, a.max_score = None, None, _ptr(scores)
    a.work, a.n_work, a.tile_rows = _ptr(plan["work"]), plan["n_work"], plan["tile_rows"]
    a.score_pack_heads = plan["pack_heads"]
    a.score_fill_tail = 1 if plan["fill"] else 0
    a.kv_indices = _ptr(kv_indices.contiguous())
    a.k_scale_128x4 = _ptr(k_sf)
    a.k_scale_format = _FORMAT_CODE[fmt]
    a.total_q, a.kv_rows = total_q, n_pages
    a.num_qo_heads, a.num_kv_heads = Hq, Hk
    a.max_k_tiles = max_k_tiles
    a.kv_dtype, a.paged, a.causal = _lib.MSA_KV_NVFP4, 1, 1 if causal else 0
    a.sm_scale, a.qk_scale, a.v_scale = 1.0, 1.0, 1.0
    a.status = _ptr(plan["status"])
    check(lib.msa_fmha_fwd(ctypes.byref(a), _stream()), "msa_fmha_fwd")
    return scores


__all__ = [
    "fp4_indexer_block_scores",
    "fp4_indexer_reorder_scales_for_mma_cute",
    "fp4_indexer_reorder_scales_for_mma",
    "fp4_indexer_mma_scale_shape",
    "fp4_indexer_mma_scale_stride",
    "fp4_indexer_mma_scale_storage_shape",
    "fp4_indexer_mma_scale_storage_stride",
]
