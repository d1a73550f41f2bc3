"""Python surface of the hot path, same names and calling conventions as the
reference package: ``fmha_sm100_plan`` / ``fmha_sm100`` / ``sparse_topk_select``
(python/fmha_sm100/api.py:944, 1028, 1179 of MiniMax-AI/MSA).

Everything here is host plumbing (shape checks, metadata tensors, output
allocation) around the C-ABI calls of libmsa_b200.so; the arithmetic runs in
the sm_100a kernels only.  There is no CPU fallback.
"""
from __future__ import annotations

import contextlib
import ctypes
import math
import os
import weakref
from typing import Optional, Tuple, Union

import numpy as np
import torch

from . import _lib
from ._lib import DecodeArgs, FmhaArgs, MsaError, check, get_lib

PAGE = 128
HEAD_DIM = 128
_SPARSE_DECODE_QLEN = 32    # sparse calls with max q_len <= this take the split-KV decode kernel
_DENSE_DECODE_QLEN = 128    # python/fmha_sm100/api.py:125-126


def _prefill_qlen_threshold(sparse: bool) -> int:
    return _SPARSE_DECODE_QLEN if sparse else _DENSE_DECODE_QLEN


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


# Precision of P in attention over FP8 e4m3 K/V (msa_fmha_args.fp8_p_f16): "e4m3" multiplies a P rounded to e4m3
# by the V pages as stored; "f16" dequantises V to f16 and keeps P in f16 (about 13 % slower, P exact to 11 bits).
_FP8_PV_MODES = ("e4m3", "f16")
_fp8_pv = os.environ.get("MSA_B200_FP8_PV", "e4m3")
if _fp8_pv not in _FP8_PV_MODES:
    raise ValueError(f"MSA_B200_FP8_PV must be one of {_FP8_PV_MODES}, got {_fp8_pv!r}")


def set_fp8_pv_precision(mode: str) -> str:
    """Chooses how attention over FP8 K/V computes P.V from now on ("e4m3" or "f16"); returns the former setting."""
    global _fp8_pv
    if mode not in _FP8_PV_MODES:
        raise ValueError(f"mode must be one of {_FP8_PV_MODES}, got {mode!r}")
    old, _fp8_pv = _fp8_pv, mode
    return old


def get_fp8_pv_precision() -> str:
    return _fp8_pv


@contextlib.contextmanager
def fp8_pv_precision(mode: str):
    """``with fp8_pv_precision("f16"): ...`` -- the setting of set_fp8_pv_precision for the calls inside."""
    old = set_fp8_pv_precision(mode)
    try:
        yield
    finally:
        set_fp8_pv_precision(old)


def _require_cuda(t: torch.Tensor, name: str):
    if not t.is_cuda:
        raise MsaError(f"{name} must be a CUDA tensor: libmsa_b200 has no CPU path")


def _i32(x, device) -> torch.Tensor:
    if isinstance(x, torch.Tensor):
        return x.to(device=device, dtype=torch.int32).contiguous()
    return torch.tensor(np.asarray(x, dtype=np.int32), device=device)


class PlanInfo(dict):
    """Execution plan for one batch shape (python/fmha_sm100/api.py:431-438):
    per-request metadata on the device, the query-tile work list, and the
    split-KV workspace of the decode path.  Reusable across layers."""


def _np_i32(x) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(x, dtype=np.int32).reshape(-1))


def _np_ptr(a: Optional[np.ndarray]):
    return None if a is None else ctypes.c_void_p(a.ctypes.data)


def _host_plan(qo_lens, kv_lens, qo_offset, causal: bool, paged: bool, num_qo_heads: int = 1, num_kv_heads: int = 1,
               kv_block_num: int = -1, num_kv_splits: int = -1, num_sms: int = 0, decode: bool = False,
               tile_rows: int = 128, dense_kv_splits: int = 0):
    """Runs ``msa_plan`` (the host planner of libmsa_b200.so, standing in for
    csrc/fmha_sm100_plan.cu:18-35 and csrc/include/plan.cuh:899-1054 of the reference) and
    returns host arrays: ``(work[n_work, 8], kv_page_indptr[B + 1], token_request, token_pos, num_splits)``;
    the token arrays are ``None`` unless ``decode``."""
    lib = get_lib()
    ql, kl = _np_i32(qo_lens), _np_i32(kv_lens)
    off = None if qo_offset is None else _np_i32(qo_offset)
    d = _lib.PlanDesc()
    d.batch = int(ql.shape[0])
    d.qo_lens, d.kv_lens, d.qo_offset = _np_ptr(ql), _np_ptr(kl), _np_ptr(off)
    d.causal, d.paged = int(bool(causal)), int(bool(paged))
    d.num_qo_heads, d.num_kv_heads = int(num_qo_heads), int(num_kv_heads)
    d.kv_block_num, d.num_kv_splits, d.num_sms = int(kv_block_num), int(num_kv_splits or -1), int(num_sms)
    d.tile_rows = int(tile_rows)
    d.dense_kv_splits = int(dense_kv_splits)
    n_work, total_q, total_pages = ctypes.c_int32(0), ctypes.c_int64(0), ctypes.c_int64(0)
    check(lib.msa_plan_sizes(ctypes.byref(d), ctypes.byref(n_work), ctypes.byref(total_q), ctypes.byref(total_pages)),
          "msa_plan_sizes")
    work = np.zeros((n_work.value, 8), dtype=np.int32)
    indptr = np.zeros(d.batch + 1, dtype=np.int32)
    tok_req = np.zeros(total_q.value, dtype=np.int32) if decode else None
    tok_pos = np.zeros(total_q.value, dtype=np.int32) if decode else None
    splits = ctypes.c_int32(1)
    check(lib.msa_plan(ctypes.byref(d), _np_ptr(work), _np_ptr(indptr), _np_ptr(tok_req), _np_ptr(tok_pos),
                       ctypes.byref(splits)), "msa_plan")
    return work, indptr, tok_req, tok_pos, int(splits.value)


class TensorKeyedCache:
    """Host-side metadata derived from small device tensors (prefix sums, lengths), looked up by the identity and
    version of those tensors so that only the first call with them pays the device-to-host read.  An entry is valid
    only while the very same tensor objects are alive and unmodified: a new tensor that reuses the address of a
    freed one (version 0 again, same shape) must not hit, so every entry keeps weak references and compares them."""

    def __init__(self, max_entries: int = 32):
        self._max = max_entries
        self._entries: dict = {}

    @staticmethod
    def _key(tensors, extra):
        return tuple(None if t is None else (t.data_ptr(), t._version, tuple(t.shape), str(t.device))
                     for t in tensors) + tuple(extra)

    def get(self, tensors, extra=()):
        ent = self._entries.get(self._key(tensors, extra))
        if ent is None:
            return None
        refs, value = ent
        if all((r is None and t is None) or (r is not None and r() is t) for r, t in zip(refs, tensors)):
            return value
        return None

    def put(self, tensors, extra, value):
        if len(self._entries) >= self._max:
            self._entries.pop(next(iter(self._entries)))
        refs = tuple(None if t is None else weakref.ref(t) for t in tensors)
        self._entries[self._key(tensors, extra)] = (refs, value)
        return value


def _flag_fill_entries(work: np.ndarray, causal: bool) -> bool:
    """Score-only work list: sets field 7 to 1 on the entry of every (request, query tile) that covers the tile's
    highest pages -- the one that also writes -inf above them (``msa_fmha_args.score_fill_tail``) -- and 0 on the
    others.  Returns False when some query tile sees no page at all: it has no entry that runs, so the caller has
    to pre-fill the score tensor after all."""
    if work.shape[0] == 0:
        return True
    rows, lo = work[:, 2] & 1023, work[:, 2] >> 10
    vis = work[:, 4].astype(np.int64)
    if causal:
        vis = np.minimum(vis, work[:, 3].astype(np.int64) + rows + work[:, 5])
    n_pages = np.where(vis > 0, (vis + PAGE - 1) // PAGE, 0)
    walk = np.maximum(0, n_pages - lo)
    work[:, 7] = 0
    best = {}
    for i in np.nonzero(walk > 0)[0].tolist():
        key = (int(work[i, 0]), int(work[i, 1]))
        if key not in best or lo[i] > lo[best[key]]:
            best[key] = i
    work[list(best.values()), 7] = 1
    tiles = {(int(r[0]), int(r[1])) for r in work}
    return len(best) == len(tiles)


def build_work_list(qo_lens, kv_lens, qo_offset, causal: bool, paged: bool = True) -> np.ndarray:
    """One entry of 8 int32 per 128-row query tile: (request, first token (global),
    valid rows, first token (request-local), kv_len, causal offset, first page-table
    slot | first K/V token of the request, 0), heaviest tiles first -- the list the
    persistent CTAs take tiles from round-robin.  Built by ``msa_plan``."""
    return _host_plan(qo_lens, kv_lens, qo_offset, causal, paged)[0]


def _fmha_sm100_plan(
    qo_segment_lens: torch.Tensor,
    kv_segment_lens: torch.Tensor,
    num_qo_heads: int,
    num_kv_heads: int = -1,
    qo_offset: Optional[Union[int, torch.Tensor]] = None,
    num_kv_splits: int = -1,
    page_size: int = -1,
    output_maxscore: bool = False,
    kv_block_num: int = -1,
    usable_SM_count: int = -1,
    causal: bool = True,
    sparse_kernel_mode: str = "auto",
    use_fp8_kvcache: bool = False,
    device=None,
    stream=None,
) -> PlanInfo:
    """Same arguments as the reference planner (python/fmha_sm100/api.py:510-526)."""
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    device = torch.device(device) if not isinstance(device, torch.device) else device
    if device.type != "cuda":
        raise MsaError("plans are built for a CUDA device")
    if num_kv_heads == -1:
        num_kv_heads = num_qo_heads
    if num_qo_heads % num_kv_heads != 0:
        raise AssertionError(f"num_qo_heads ({num_qo_heads}) must be divisible by num_kv_heads ({num_kv_heads})")
    if page_size not in (-1, PAGE):
        raise MsaError(f"page_size must be {PAGE} (or -1 for ragged K/V), got {page_size}")
    qo_lens = [int(x) for x in qo_segment_lens.tolist()]
    kv_lens = [int(x) for x in kv_segment_lens.tolist()]
    B = len(qo_lens)
    if qo_offset is None:
        off = [kv_lens[i] - qo_lens[i] for i in range(B)]
    elif isinstance(qo_offset, int):
        off = [qo_offset] * B
    else:
        off = [int(x) for x in qo_offset.tolist()]
    max_kv_len = max(kv_lens) if kv_lens else 0
    if not causal:
        off = [max_kv_len] * B
    if max_kv_len > 16384 * PAGE:
        raise MsaError("kv_len beyond 16384 pages per request is not supported")

    qo_offsets = np.concatenate([[0], np.cumsum(qo_lens)]).astype(np.int32)
    kv_offsets = np.concatenate([[0], np.cumsum(kv_lens)]).astype(np.int32)
    max_qo_len = max(qo_lens) if qo_lens else 0
    total_q = int(qo_offsets[-1])
    # python/fmha_sm100/api.py:615-619
    max_k_tiles = math.ceil(math.ceil(max_kv_len / 128) / 128) * 128 if output_maxscore else -1
    if output_maxscore and num_qo_heads * max_k_tiles * total_q > (1 << 31):
        max_k_tiles = -1

    sparse = kv_block_num > 0
    use_decode = sparse and (sparse_kernel_mode == "decode" or
                             (sparse_kernel_mode == "auto" and max_qo_len <= _prefill_qlen_threshold(True)))
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    if usable_SM_count > 0:
        sms = min(sms, usable_SM_count)
    work, indptr, tok_req, tok_pos, splits = _host_plan(
        qo_lens, kv_lens, off, causal, page_size > 0, num_qo_heads, num_kv_heads, kv_block_num,
        num_kv_splits if num_kv_splits is not None else -1, sms, decode=use_decode)
    plan = PlanInfo()
    plan["MM-SA-Nv"] = False
    plan["device"] = device
    plan["batch_size"] = B
    plan["num_qo_heads"] = num_qo_heads
    plan["num_kv_heads"] = num_kv_heads
    plan["page_size"] = page_size
    plan["causal"] = bool(causal)
    plan["kv_block_num"] = kv_block_num
    plan["max_qo_len"] = max_qo_len
    plan["max_kv_len"] = max_kv_len
    plan["max_k_tiles"] = max_k_tiles
    plan["total_qo_len"] = total_q
    plan["qo_lens_host"] = qo_lens
    plan["kv_lens_host"] = kv_lens
    plan["total_pages_host"] = int(indptr[-1])
    plan["qo_segment_lens"] = _i32(qo_lens, device)
    plan["kv_segment_lens"] = _i32(kv_lens, device)
    plan["qo_segment_offsets"] = torch.from_numpy(qo_offsets).to(device)
    plan["kv_segment_offsets"] = torch.from_numpy(kv_offsets).to(device)
    plan["kv_page_indptr"] = torch.from_numpy(indptr).to(device)
    plan["qo_offset"] = _i32(off, device)
    plan["work"] = torch.from_numpy(work).to(device).contiguous()
    plan["n_work"] = int(work.shape[0])
    plan["dense_kv_splits"] = 1
    if not sparse and total_q > 0 and work.shape[0] > 0:
        # A dense call with few query tiles (a short query over a long context) cannot fill the GPU with one
        # CTA per (tile, head pair): each tile is split over ranges of its pages and the partial results are
        # merged afterwards (the role num_kv_splits has in python/fmha_sm100/api.py:944-1026).
        hr = num_qo_heads // num_kv_heads
        items = int(work.shape[0]) * (num_qo_heads // (2 if hr % 2 == 0 else 1))
        max_pages = max((min(kl, max(0, ql + o)) if causal else kl) for ql, kl, o in zip(qo_lens, kv_lens, off))
        max_pages = (max(0, max_pages) + PAGE - 1) // PAGE
        if num_kv_splits is not None and num_kv_splits >= 1:
            n_split = min(int(num_kv_splits), max(1, max_pages))     # forced; 1 = never split
        else:
            n_split = min(sms // max(1, items), max_pages // 8, 64)
        if n_split > 1:
            work_s = _host_plan(qo_lens, kv_lens, off, causal, page_size > 0, num_qo_heads, num_kv_heads,
                                dense_kv_splits=n_split)[0]
            plan["work_split"] = torch.from_numpy(work_s).to(device).contiguous()
            plan["dense_kv_splits"] = n_split
    if output_maxscore and not sparse:
        # the score-only pass takes two query tiles per work item (every K page is fetched once for both)
        work2 = _host_plan(qo_lens, kv_lens, off, causal, page_size > 0, num_qo_heads, num_kv_heads, tile_rows=256)[0]
        # the kernel writes -inf above every tile's pages itself, unless some tile has no page to visit
        plan["score_fill"] = _flag_fill_entries(work2, causal)
        plan["work_score"] = torch.from_numpy(work2).to(device).contiguous()
    plan["status"] = torch.zeros(1, dtype=torch.int32, device=device)
    plan["use_decode_kernel"] = bool(use_decode)
    plan["pack_factor"] = 1
    plan["orig_num_qo_heads"] = num_qo_heads
    plan["use_fp8_kvcache"] = bool(use_fp8_kvcache)
    plan["usable_SM_count"] = usable_SM_count
    if use_decode:
        # every token is its own row of the decode grid (python/fmha_sm100/api.py:398-429)
        plan["token_request"] = torch.from_numpy(tok_req).to(device)
        plan["token_pos"] = torch.from_numpy(tok_pos).to(device)
        plan["num_kv_splits"] = int(splits)
        ws = get_lib().msa_decode_workspace_bytes(total_q, num_qo_heads, int(splits))
        plan["workspace"] = torch.empty(max(ws, 16), dtype=torch.uint8, device=device)
    else:
        plan["num_kv_splits"] = 1
        plan["workspace"] = None
    return plan


def fmha_sm100_plan(
    qo_segment_lens: torch.Tensor,
    kv_segment_lens: torch.Tensor,
    *args,
    qo_offset: Optional[Union[int, torch.Tensor]] = None,
    split_prefill_decode=True,
    **kwargs,
):
    """Build a reusable plan; returns ``(has_mixed_prefill, split, batch_size,
    decode_plan, prefill_plan)`` exactly like python/fmha_sm100/api.py:944-1026.
    A batch ordered as short (decode) requests followed by long (prefill) ones
    is split at the first long request so each part takes its own kernel."""
    if qo_offset is None:
        qo_offset = kv_segment_lens - qo_segment_lens
    elif isinstance(qo_offset, int):
        qo_offset = torch.full_like(qo_segment_lens, qo_offset)
    batch_size = qo_segment_lens.shape[0]
    has_mixed_prefill = False
    split = 0
    qmax = int(qo_segment_lens.max().item()) if batch_size else 0
    sparse = kwargs.get("kv_block_num", -1) > 0
    thr = _prefill_qlen_threshold(sparse)
    if split_prefill_decode and qmax > thr:
        split = int((qo_segment_lens > thr).nonzero(as_tuple=False)[0, 0].item())
        has_mixed_prefill = split > 0
    if has_mixed_prefill:
        decode = _fmha_sm100_plan(qo_segment_lens[:split], kv_segment_lens[:split], *args,
                                  qo_offset=qo_offset[:split], **kwargs)
        prefill = _fmha_sm100_plan(qo_segment_lens[split:], kv_segment_lens[split:], *args,
                                   qo_offset=qo_offset[split:], **kwargs)
        return (True, split, batch_size, decode, prefill)
    plan = _fmha_sm100_plan(qo_segment_lens, kv_segment_lens, *args, qo_offset=qo_offset, **kwargs)
    return (False, 0, batch_size, plan, None)


def _validate_fmha_inputs(q, k, v, plan, kv_indices, kv_block_indexes, is_paged):
    """Host re-check of the index contract before a launch, by ``msa_validate_inputs`` of the library
    (the rules of python/fmha_sm100/api.py:128-263); raises ``AssertionError`` naming the first broken
    rule and the offending element, as the reference's asserts do.  Copies the index tensors to the host."""
    Hq, Hkv = plan["num_qo_heads"], plan["num_kv_heads"]
    if q.dim() != 3 or q.shape[1] != Hq:
        raise AssertionError(f"q must be [total_qo_len, {Hq}, head_dim], got {tuple(q.shape)}")
    if is_paged:
        if k.dim() != 4 or k.shape[1] != Hkv or k.shape[2] != PAGE:
            raise AssertionError(f"paged K must be [total_pages, {Hkv}, {PAGE}, D], got {tuple(k.shape)}")
        if v is not None and tuple(v.shape[:3]) != tuple(k.shape[:3]):
            raise AssertionError(f"paged V {tuple(v.shape)} does not match K {tuple(k.shape)}")
        if kv_indices is None:
            raise AssertionError("paged K/V needs kv_indices")
    ql, kl = _np_i32(plan["qo_lens_host"]), _np_i32(plan["kv_lens_host"])
    kvi = None if kv_indices is None else _np_i32(kv_indices.detach().cpu().numpy())
    bi = None
    a = _lib.ValidateArgs()
    if kv_block_indexes is not None:
        if kv_block_indexes.dim() != 3 or kv_block_indexes.shape[0] != q.shape[0]:
            raise AssertionError(f"kv_block_indexes must be [total_q, heads, topk], got {tuple(kv_block_indexes.shape)}")
        bi = _np_i32(kv_block_indexes.detach().cpu().numpy())
        a.list_heads, a.topk = int(kv_block_indexes.shape[1]), int(kv_block_indexes.shape[2])
    a.batch = int(ql.shape[0])
    a.qo_lens, a.kv_lens = _np_ptr(ql), _np_ptr(kl)
    a.total_q, a.kv_rows, a.paged = int(q.shape[0]), int(k.shape[0]), int(bool(is_paged))
    a.kv_indices, a.n_kv_indices = _np_ptr(kvi), 0 if kvi is None else int(kvi.shape[0])
    a.kv_block_indexes = _np_ptr(bi)
    a.num_qo_heads, a.num_kv_heads = int(Hq), int(Hkv)
    where = ctypes.c_int64(-1)
    lib = get_lib()
    rc = lib.msa_validate_inputs(ctypes.byref(a), ctypes.byref(where))
    if rc != 0:
        at = f" (flat element {where.value})" if where.value >= 0 else ""
        raise AssertionError(f"{lib.msa_error_string(rc).decode()}{at}")


def _kv_dtype_code(k: torch.Tensor) -> int:
    if k.dtype == torch.bfloat16:
        return _lib.MSA_KV_BF16
    if k.dtype == torch.float8_e4m3fn:
        return _lib.MSA_KV_FP8_E4M3
    raise MsaError(f"unsupported K/V dtype {k.dtype} (bf16 and float8_e4m3fn; NVFP4 goes through "
                   f"sparse_atten_nvfp4_kv_func)")


def _run_prefill(q, k, v, plan, kv_indices, kv_block_indexes, qo_offset_t, out, max_score, lse,
                 sm_scale, qk_scale, v_scale, kv_dtype, is_paged, k_sf=None, v_sf=None, qk_dim=0, fill_tail=False):
    lib = get_lib()
    a = FmhaArgs()
    a.qk_dim = int(qk_dim)
    a.q, a.k, a.v = _ptr(q), _ptr(k), _ptr(v)
    a.out, a.lse, a.max_score = _ptr(out), _ptr(lse), _ptr(max_score)
    score_pairs = out is None and kv_block_indexes is None and "work_score" in plan
    work = plan["work_score"] if score_pairs else plan["work"]
    n_split = 1
    if (out is not None and kv_block_indexes is None and "work_split" in plan
            and qo_offset_t is plan["qo_offset"]):
        # KV splits of a short dense call: every split writes a normalised partial and its LSE into buffers the
        # plan keeps, msa_fmha_combine merges them into out / lse
        work, n_split = plan["work_split"], plan["dense_kv_splits"]
        final_out, final_lse = out, lse
        if "split_out" not in plan:
            plan["split_out"] = torch.empty(n_split * q.shape[0], q.shape[1], HEAD_DIM, dtype=torch.bfloat16,
                                            device=q.device)
            plan["split_lse"] = torch.empty(n_split * q.shape[0], q.shape[1], dtype=torch.float32, device=q.device)
        out, lse = plan["split_out"], plan["split_lse"]
        a.out, a.lse = _ptr(out), _ptr(lse)
        a.out_rows = int(out.shape[0])
    if qo_offset_t is not plan["qo_offset"]:
        # runtime causal-offset override: patch column 5 of a copy of the work list
        work = work.clone()
        work[:, 5] = qo_offset_t.to(torch.int32)[work[:, 0].long()]
    if bool(is_paged) != (plan["page_size"] > 0):
        raise MsaError("the plan and the call disagree on paged vs ragged K/V (pass page_size to fmha_sm100_plan)")
    a.work, a.n_work = _ptr(work), int(work.shape[0])
    a.tile_rows = 256 if score_pairs else 128
    a.score_fill_tail = 1 if (fill_tail and score_pairs) else 0
    a.fp8_p_f16 = 1 if _fp8_pv == "f16" else 0
    a.kv_indices = _ptr(kv_indices)
    a.kv_block_indexes = _ptr(kv_block_indexes)
    a.k_scale_128x4, a.v_scale_128x4 = _ptr(k_sf), _ptr(v_sf)
    a.total_q = q.shape[0]
    a.kv_rows = k.shape[0]
    a.num_qo_heads, a.num_kv_heads = plan["num_qo_heads"], plan["num_kv_heads"]
    a.topk = kv_block_indexes.shape[2] if kv_block_indexes is not None else 0
    a.list_heads = kv_block_indexes.shape[1] if kv_block_indexes is not None else 0
    flags = None
    if kv_block_indexes is not None and a.n_work > 0:
        # which query tiles carry one list for all their rows (pages selected per query block): a short device
        # pass over the lists, then the attention kernel takes such a tile's page set from a single row
        flags = torch.empty(a.n_work * a.list_heads, dtype=torch.uint8, device=q.device)
        check(lib.msa_list_uniformity(_ptr(work), a.n_work, _ptr(kv_block_indexes), a.list_heads, a.topk,
                                      _ptr(flags), _stream()), "msa_list_uniformity")
    a.tile_uniform = _ptr(flags)
    a.max_k_tiles = max_score.shape[1] if max_score is not None else 0
    if max_score is not None:
        # a slice [.., .., t0:t1] of a larger score tensor is written in place through its strides
        if max_score.stride(2) != 1:
            raise MsaError("max_score must be contiguous along the token dimension")
        a.max_score_tile_stride, a.max_score_head_stride = int(max_score.stride(1)), int(max_score.stride(0))
    a.kv_dtype = kv_dtype
    a.paged = 1 if is_paged else 0
    a.causal = 1 if plan["causal"] else 0
    a.sm_scale, a.qk_scale, a.v_scale = float(sm_scale), float(qk_scale), float(v_scale)
    a.status = _ptr(plan["status"])
    a.max_ctas = max(0, int(plan.get("usable_SM_count", -1)))
    check(lib.msa_fmha_fwd(ctypes.byref(a), _stream()), "msa_fmha_fwd")
    if n_split > 1:
        check(lib.msa_fmha_combine(_ptr(out), _ptr(lse), n_split, int(q.shape[0]), int(q.shape[1]), _ptr(final_out),
                                   _ptr(final_lse), _stream()), "msa_fmha_combine")


def _run_decode(q, k, v, plan, kv_indices, kv_block_indexes, out, lse, sm_scale, qk_scale, v_scale,
                token_pos=None):
    lib = get_lib()
    a = DecodeArgs()
    a.q, a.k, a.v, a.out, a.lse = _ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(lse)
    a.kv_indices, a.kv_page_indptr = _ptr(kv_indices), _ptr(plan["kv_page_indptr"])
    a.kv_block_indexes = _ptr(kv_block_indexes)
    a.token_request = _ptr(plan["token_request"])
    a.token_pos = _ptr(plan["token_pos"] if token_pos is None else token_pos)
    a.num_tokens = q.shape[0]
    a.num_qo_heads, a.num_kv_heads = plan["num_qo_heads"], plan["num_kv_heads"]
    a.topk = kv_block_indexes.shape[2]
    a.num_splits = min(plan["num_kv_splits"], kv_block_indexes.shape[2])
    a.sm_scale, a.qk_scale, a.v_scale = float(sm_scale), float(qk_scale), float(v_scale)
    ws = plan["workspace"]
    need = lib.msa_decode_workspace_bytes(a.num_tokens, a.num_qo_heads, a.num_splits)
    if ws is None or ws.numel() < need:
        ws = torch.empty(max(need, 16), dtype=torch.uint8, device=q.device)
        plan["workspace"] = ws
    a.workspace, a.workspace_bytes = _ptr(ws), ws.numel()
    a.num_pages = k.shape[0]
    a.status = _ptr(plan["status"])
    check(lib.msa_decode_fwd(ctypes.byref(a), _stream()), "msa_decode_fwd")


def _fmha_sm100(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    plan_info: PlanInfo,
    kv_indices: Optional[torch.Tensor] = None,
    kv_block_indexes: Optional[torch.Tensor] = None,
    q_offset_override: Optional[Union[int, torch.Tensor]] = None,
    out: Optional[torch.Tensor] = None,
    max_score: Optional[torch.Tensor] = None,
    sm_scale: Optional[float] = None,
    q_scale: Optional[float] = None,
    k_scale: Optional[float] = None,
    v_scale: Optional[float] = None,
    o_scale: Optional[float] = None,
    output_maxscore: bool = True,
    output_o: bool = True,
    check_input_valid: bool = False,
    return_lse: bool = False,
    score_dim: Optional[int] = None,
):
    """One sub-plan (python/fmha_sm100/api.py:750-941).  Two additions: ``return_lse`` appends the
    natural-log LSE ``[total_q, Hq]`` to the result; ``score_dim=64`` tells a score-only call
    (``output_o=False``) that only the first 64 elements of q and k are non-zero -- a 64-wide proxy
    zero-padded to the 128-wide layout -- so that the kernel skips the other half of the contraction."""
    plan = plan_info
    _require_cuda(q, "q")
    _require_cuda(k, "k")
    nnz_qo, num_qo_heads, head_dim = q.shape
    if head_dim != HEAD_DIM or k.shape[-1] != HEAD_DIM:
        raise MsaError("head_dim must be 128")
    is_paged = kv_indices is not None
    if num_qo_heads != plan["num_qo_heads"]:
        raise MsaError(f"q has {num_qo_heads} heads, the plan was made for {plan['num_qo_heads']}")
    if nnz_qo != plan["total_qo_len"]:
        raise MsaError(f"q has {nnz_qo} tokens, the plan was made for {plan['total_qo_len']}")
    if check_input_valid:
        _validate_fmha_inputs(q, k, v, plan, kv_indices, kv_block_indexes, is_paged)
    sm_scale = 1.0 / math.sqrt(head_dim) if sm_scale is None else sm_scale
    q_scale = 1.0 if q_scale is None else q_scale
    k_scale = 1.0 if k_scale is None else k_scale
    v_scale = 1.0 if v_scale is None else v_scale
    o_scale = 1.0 if o_scale is None else o_scale
    assert output_o or output_maxscore
    max_k_tiles = plan["max_k_tiles"]
    if kv_block_indexes is not None:
        output_maxscore = False          # the sparse pass has no max-score output (sparse_fmha_adapter.py:67-202)
    fill_in_kernel = False
    if not output_maxscore or max_k_tiles == -1:
        max_score = None
        output_o = True
    elif max_score is None:
        # untouched entries (beyond the causal frontier, padding tiles) must read -inf: the score-only kernel writes
        # them itself (no separate pass over the tensor); the attention kernel's Full mode needs the pre-fill
        fill_in_kernel = (not output_o and kv_block_indexes is None and plan.get("score_fill", False)
                          and q_offset_override is None and not plan["use_decode_kernel"] and nnz_qo > 0)
        alloc = torch.empty if fill_in_kernel else (lambda *a, **k: torch.full(*a, -float("inf"), **k))
        max_score = alloc((num_qo_heads, max_k_tiles, nnz_qo), dtype=torch.float32, device=q.device)
    if not output_o:
        out = None
    elif out is None:
        out = torch.empty(nnz_qo, num_qo_heads, HEAD_DIM, device=q.device, dtype=torch.bfloat16)
    lse = torch.empty(nnz_qo, num_qo_heads, dtype=torch.float32, device=q.device) if (return_lse and output_o) else None

    if q.dtype == torch.float8_e4m3fn:
        q = q.to(torch.bfloat16)         # exact; q_scale carries the magnitude
    if q.dtype != torch.bfloat16:
        raise MsaError(f"q must be bfloat16 or float8_e4m3fn, got {q.dtype}")
    q = q.contiguous()
    k = k.contiguous()
    v = v.contiguous() if v is not None else None
    kv_dtype = _kv_dtype_code(k)
    if kv_indices is not None:
        kv_indices = kv_indices.to(torch.int32).contiguous()
    if kv_block_indexes is not None:
        kv_block_indexes = kv_block_indexes.to(torch.int32).contiguous()

    qo_offset_t = plan["qo_offset"]
    token_pos = None
    if q_offset_override is not None:
        if isinstance(q_offset_override, int):
            qo_offset_t = torch.full_like(plan["qo_offset"], q_offset_override)
        else:
            qo_offset_t = q_offset_override.to(device=q.device, dtype=torch.int32).contiguous()
        if plan["use_decode_kernel"]:
            req = plan["token_request"].long()
            local = torch.arange(nnz_qo, device=q.device) - plan["qo_segment_offsets"].long()[req]
            token_pos = torch.minimum(local + qo_offset_t.long()[req],
                                      plan["kv_segment_lens"].long()[req] - 1).to(torch.int32)

    if nnz_qo > 0:
        if (kv_block_indexes is not None and plan["use_decode_kernel"] and kv_dtype == _lib.MSA_KV_FP8_E4M3
                and kv_block_indexes.shape[1] == plan["num_kv_heads"]
                and num_qo_heads // plan["num_kv_heads"] <= 16):
            _run_decode(q, k, v, plan, kv_indices, kv_block_indexes, out, lse, sm_scale, q_scale * k_scale,
                        v_scale * o_scale, token_pos)
        else:
            if score_dim not in (None, 64, 128):
                raise MsaError("score_dim must be 64 or 128")
            if score_dim == 64 and (output_o or kv_dtype == _lib.MSA_KV_NVFP4):
                raise MsaError("score_dim=64 is for the score-only pass over bf16 or fp8 K")
            _run_prefill(q, k, v, plan, kv_indices, kv_block_indexes, qo_offset_t, out, max_score, lse,
                         sm_scale, q_scale * k_scale, v_scale * o_scale, kv_dtype, is_paged,
                         qk_dim=0 if score_dim is None else score_dim, fill_tail=fill_in_kernel)
    if return_lse:
        return out, max_score, lse
    return out, max_score


def fmha_sm100(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    plan_info,
    kv_indices: Optional[torch.Tensor] = None,
    kv_block_indexes: Optional[torch.Tensor] = None,
    q_offset_override: Optional[Union[int, torch.Tensor]] = None,
    out: Optional[torch.Tensor] = None,
    max_score: Optional[torch.Tensor] = None,
    **kwargs,
) -> Tuple[Optional[torch.Tensor], Optional[torch.Tensor]]:
    """Dense, paged, score-only or block-sparse attention with a precomputed plan;
    arguments, defaults and the ``(out, max_score)`` result follow
    python/fmha_sm100/api.py:1028-1171.

    q ``[total_q, Hq, 128]`` bf16 (or e4m3); k/v ragged ``[total_kv, Hkv, 128]`` or
    paged ``[pages, Hkv, 128, 128]`` in bf16 or e4m3 (e4m3 K/V with bf16 Q is
    dequantised in the load path; pass the per-tensor scales as ``k_scale`` /
    ``v_scale``); ``kv_indices`` flat int32 page table; ``kv_block_indexes``
    ``[total_q, Hkv | Hq, K]`` int32 request-local page ids, ascending, -1 tail.
    ``max_score[Hq, max_k_tiles, total_q]`` holds the raw (unscaled) q.k maximum of
    every visible 128-key tile and -inf elsewhere.
    """
    has_mixed, split, batch_size, decode, prefill = plan_info
    if not has_mixed:
        return _fmha_sm100(q, k, v, decode, out=out, max_score=max_score, kv_indices=kv_indices,
                           kv_block_indexes=kv_block_indexes, q_offset_override=q_offset_override, **kwargs)
    # Mixed batch: the leading short requests take the decode sub-plan, the rest the prefill sub-plan, and both
    # write straight into their token ranges of one output / one score tensor (no concatenation afterwards).
    n_dec, nnz, Hq = decode["total_qo_len"], q.shape[0], q.shape[1]
    paged = kv_indices is not None
    want_o = bool(kwargs.get("output_o", True)) or kv_block_indexes is not None
    want_ms = bool(kwargs.get("output_maxscore", True)) and kv_block_indexes is None
    tiles = [pl["max_k_tiles"] for pl in (decode, prefill)]
    if min(tiles) == -1:
        want_ms = False
    if not want_ms:
        want_o = True
    if want_o and out is None:
        out = torch.empty(nnz, Hq, HEAD_DIM, device=q.device, dtype=torch.bfloat16)
    if want_ms and max_score is None:
        max_score = torch.full((Hq, max(tiles), nnz), -float("inf"), dtype=torch.float32, device=q.device)
    lses = []
    for part, pl, tok in ((0, decode, slice(0, n_dec)), (1, prefill, slice(n_dec, nnz))):
        req = slice(0, split) if part == 0 else slice(split, batch_size)
        if paged:
            n_pg = decode["total_pages_host"]
            pages = slice(0, n_pg) if part == 0 else slice(n_pg, None)
            k_part, v_part, idx_part = k, v, kv_indices[pages]
        else:
            n_kv = sum(decode["kv_lens_host"])
            rows = slice(0, n_kv) if part == 0 else slice(n_kv, None)
            k_part, v_part, idx_part = k[rows], (v[rows] if v is not None else None), None
        if isinstance(q_offset_override, torch.Tensor):
            off_part = q_offset_override[req]
        else:
            off_part = q_offset_override
        res = _fmha_sm100(q[tok], k_part, v_part, pl, kv_indices=idx_part,
                          kv_block_indexes=None if kv_block_indexes is None else kv_block_indexes[tok],
                          q_offset_override=off_part, out=out[tok] if want_o else None,
                          max_score=max_score[:, :pl["max_k_tiles"], tok] if want_ms else None, **kwargs)
        if len(res) > 2:
            lses.append(res[2])
    result = (out if want_o else None, max_score if want_ms else None)
    if lses:
        result = result + (torch.cat(lses, dim=0),)
    return result


def plan_status(plan_info) -> int:
    """Read (synchronising) the device status word of a plan: 0, or a negative
    MSA_ERR_* code such as MSA_ERR_TIMEOUT when a bounded device wait gave up."""
    worst = 0
    for p in (plan_info[3], plan_info[4]):
        if p is not None:
            worst = min(worst, int(p["status"].item()))
    return worst


def sparse_topk_select(
    max_score: torch.Tensor,
    topk: int,
    num_valid_pages: Optional[int] = None,
    output: Optional[torch.Tensor] = None,
    force_begin_blocks: int = 0,
    force_end_blocks: int = 0,
    q_block_starts: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Top-k KV-tile indices per (token, head) row of ``max_score[H, K, T]``;
    returns int32 ``[T, H, topk]`` ascending with -1 at the tail
    (python/fmha_sm100/api.py:1179-1290).

    Differences from the reference, all supersets of its contract: ``topk`` may be
    16, 32 or 64; ties go to the lower tile index; a pick whose score is -inf is
    reported as -1 (the reference returns an arbitrary masked tile there).
    ``q_block_starts`` (int32 ``[n_blocks + 1]`` token offsets) is an addition:
    the scores are first reduced by max over each query block, one list is
    selected per block and written to every token of the block.
    """
    assert max_score.dtype == torch.float32, f"max_score must be float32, got {max_score.dtype}"
    assert max_score.dim() == 3, f"max_score must be 3D, got {max_score.shape}"
    assert max_score.is_contiguous(), "max_score must be contiguous"
    assert topk in (16, 32, 64), f"topk must be 16, 32 or 64, got {topk}"
    _require_cuda(max_score, "max_score")
    H, K, T = max_score.shape
    if num_valid_pages is not None:
        assert 0 < num_valid_pages <= K, f"num_valid_pages={num_valid_pages} must be in (0, max_k_tiles={K}]"
        nvp = int(num_valid_pages)
    else:
        nvp = int(K)
    assert force_begin_blocks >= 0 and force_end_blocks >= 0
    assert force_begin_blocks + force_end_blocks <= topk, (
        f"force_begin_blocks({force_begin_blocks}) + force_end_blocks({force_end_blocks}) exceeds topk={topk}")
    lib = get_lib()
    dev = max_score.device
    if q_block_starts is None:
        out = output if output is not None else torch.empty(T, H, topk, dtype=torch.int32, device=dev)
        assert out.is_contiguous() and out.dtype == torch.int32 and tuple(out.shape) == (T, H, topk)
        check(lib.msa_topk_select(_ptr(max_score), H, K, T, topk, nvp, int(force_begin_blocks),
                                  int(force_end_blocks), _ptr(out), _stream()), "msa_topk_select")
        return out
    starts = q_block_starts.to(device=dev, dtype=torch.int32).contiguous()
    nblk = starts.numel() - 1
    bm = torch.empty(H, K, nblk, dtype=torch.float32, device=dev)
    check(lib.msa_block_max(_ptr(max_score), H, K, T, _ptr(starts), nblk, _ptr(bm), _stream()), "msa_block_max")
    sel = torch.empty(nblk, H, topk, dtype=torch.int32, device=dev)
    check(lib.msa_topk_select(_ptr(bm), H, K, nblk, topk, nvp, int(force_begin_blocks), int(force_end_blocks),
                              _ptr(sel), _stream()), "msa_topk_select")
    out = output if output is not None else torch.empty(T, H, topk, dtype=torch.int32, device=dev)
    assert out.is_contiguous() and out.dtype == torch.int32 and tuple(out.shape) == (T, H, topk)
    check(lib.msa_expand_block_lists(_ptr(sel), _ptr(starts), nblk, H, topk, _ptr(out), _stream()),
          "msa_expand_block_lists")
    return out
