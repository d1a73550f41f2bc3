"""CSR-driven entry points of the reference's second stack, same names and
arguments: ``sparse_atten_func``, ``sparse_atten_nvfp4_kv_func``,
``build_k2q_csr`` (python/fmha_sm100/cute/interface.py:600-991,
python/fmha_sm100/cute/sparse_index_utils.py:331) and the paged FP8 decode
wrapper (interface.py:1125-1423).

The reference executes KV-outer (one CTA per KV block and the queries that
picked it) and therefore wants the reverse index (k2q CSR).  The kernels here
are query-stationary and walk each query tile's own page lists, so the CSR is
turned back into per-query lists on the device (tensor ops, no host loop) and
the same attention kernel as ``fmha_sm100`` runs.
"""
from __future__ import annotations

import math
from typing import Optional

import numpy as np
import torch

from . import _lib
from ._lib import MsaError
from .api import PAGE, TensorKeyedCache, _fmha_sm100_plan, _ptr, _run_decode, _run_prefill, _stream
from .quant import Nvfp4QuantizedTensor  # noqa: F401  (re-export for callers of the nvfp4 entry point)


def _row_map(kv_lens, blk_kv, device):
    """Block-major packing of CSR rows: row ids for kv block 0 of every request,
    then block 1, ... (python/fmha_sm100/cute/sparse_index_utils.py:176-192).
    Returns (row_request[total_rows], row_block[total_rows])."""
    nblk = [(k + blk_kv - 1) // blk_kv for k in kv_lens]
    reqs, blks = [], []
    for blk in range(max(nblk + [0])):
        for b, n in enumerate(nblk):
            if blk < n:
                reqs.append(b)
                blks.append(blk)
    return (torch.tensor(reqs, dtype=torch.int64, device=device), torch.tensor(blks, dtype=torch.int64, device=device))


def build_k2q_csr(q2k_indices: torch.Tensor, cu_seqlens_q: torch.Tensor, cu_seqlens_k: torch.Tensor,
                  blk_kv: int = PAGE, **_hints):
    """q2k ``[Hkv, total_q, topK]`` (request-local KV block ids, -1 unused) ->
    ``(k2q_row_ptr[Hkv, total_rows + 1], k2q_q_indices[Hkv, total_q * topK])``:
    for every (KV block, request) row the ascending request-local queries that
    selected it; unused tail is -1 (python/fmha_sm100/cute/sparse_index_utils.py:331).
    CUDA tensors go through ``msa_build_k2q_csr`` (four small kernels, deterministic);
    CPU tensors through the tensor-op version below.  The reference's size hints
    (``total_k``, ``max_seqlen_k``, ...) are accepted and not needed."""
    if q2k_indices.is_cuda:
        return _build_k2q_csr_device(q2k_indices, cu_seqlens_q, cu_seqlens_k, blk_kv)
    return _build_k2q_csr_host(q2k_indices, cu_seqlens_q, cu_seqlens_k, blk_kv)


_CSR_WORKSPACE_LIMIT = 1 << 30


def _build_k2q_csr_device(q2k, cu_seqlens_q, cu_seqlens_k, blk_kv):
    lib = _lib.get_lib()
    dev = q2k.device
    Hkv, total_q, topk = q2k.shape
    cq = np.asarray(cu_seqlens_q.tolist(), dtype=np.int64)
    ck = np.asarray(cu_seqlens_k.tolist(), dtype=np.int64)
    B = len(cq) - 1
    nblk = ((ck[1:] - ck[:-1]) + blk_kv - 1) // blk_kv
    rr, rb = _row_map_np((ck[1:] - ck[:-1]).tolist(), blk_kv)
    total_rows, maxb = int(rr.shape[0]), int(max(1, nblk.max() if B else 1))
    lut = np.full((max(B, 1), maxb), -1, dtype=np.int32)
    lut[rr, rb] = np.arange(total_rows, dtype=np.int32)
    chunk = 256
    c_req, c_q0, c_len, first = [], [], [], [0]
    for b in range(B):
        for s0 in range(int(cq[b]), int(cq[b + 1]), chunk):
            c_req.append(b)
            c_q0.append(s0)
            c_len.append(min(chunk, int(cq[b + 1]) - s0))
        first.append(len(c_req))
    n_chunks = len(c_req)
    ws_bytes = lib.msa_build_k2q_csr_workspace_bytes(Hkv, n_chunks, maxb, total_rows)
    if ws_bytes > _CSR_WORKSPACE_LIMIT or B == 0:
        rp, qi = _build_k2q_csr_host(q2k, cu_seqlens_q, cu_seqlens_k, blk_kv)
        return rp, qi
    i32 = lambda x: torch.tensor(np.asarray(x, dtype=np.int32), device=dev)  # noqa: E731
    meta = [i32(c_req), i32(c_q0), i32(c_len), i32(cq), i32(first), i32(nblk), torch.from_numpy(lut).to(dev)]
    q2k_c = q2k.to(torch.int32).contiguous()
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=dev)
    row_ptr = torch.empty(Hkv, total_rows + 1, dtype=torch.int32, device=dev)
    q_indices = torch.empty(Hkv, total_q * topk, dtype=torch.int32, device=dev)
    a = _lib.CsrBuildArgs()
    a.q2k = q2k_c.data_ptr()
    (a.chunk_request, a.chunk_first_query, a.chunk_len, a.cu_seqlens_q, a.request_first_chunk, a.request_blocks,
     a.row_of_block) = (m.data_ptr() for m in meta)
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    a.row_ptr, a.q_indices = row_ptr.data_ptr(), q_indices.data_ptr()
    a.total_q, a.q_indices_stride = total_q, total_q * topk
    a.num_kv_heads, a.topk, a.n_chunks, a.batch, a.max_blocks, a.total_rows = Hkv, topk, n_chunks, B, maxb, total_rows
    import ctypes
    _lib.check(lib.msa_build_k2q_csr(ctypes.byref(a), _stream()), "msa_build_k2q_csr")
    return row_ptr, q_indices


def _build_k2q_csr_host(q2k_indices: torch.Tensor, cu_seqlens_q: torch.Tensor, cu_seqlens_k: torch.Tensor,
                        blk_kv: int = PAGE):
    """The same index with tensor ops (any device; the CPU tests and the fallback for outsized workspaces)."""
    Hkv, total_q, topk = q2k_indices.shape
    dev = q2k_indices.device
    cq = [int(x) for x in cu_seqlens_q.tolist()]
    ck = [int(x) for x in cu_seqlens_k.tolist()]
    B = len(cq) - 1
    kv_lens = [ck[i + 1] - ck[i] for i in range(B)]
    row_req, row_blk = _row_map(kv_lens, blk_kv, dev)
    total_rows = row_req.numel()
    maxb = max([(k + blk_kv - 1) // blk_kv for k in kv_lens] + [1])
    lut = torch.full((B, maxb), -1, dtype=torch.int64, device=dev)
    lut[row_req, row_blk] = torch.arange(total_rows, device=dev)
    owner = torch.repeat_interleave(torch.arange(B, device=dev), torch.tensor([cq[i + 1] - cq[i] for i in range(B)],
                                                                              device=dev), output_size=total_q)
    qlocal = torch.arange(total_q, device=dev) - torch.tensor(cq, device=dev)[owner]
    row_ptr = torch.zeros(Hkv, total_rows + 1, dtype=torch.int32, device=dev)
    q_indices = torch.full((Hkv, total_q * topk), -1, dtype=torch.int32, device=dev)
    if total_rows == 0 or total_q == 0:
        return row_ptr, q_indices
    idx = q2k_indices.long()
    valid = idx >= 0
    rows = lut[owner.view(1, -1, 1).expand_as(idx), idx.clamp(min=0)]
    key = torch.where(valid, rows * total_q + qlocal.view(1, -1, 1), torch.full_like(rows, total_rows * total_q))
    key = key.reshape(Hkv, -1)
    skey, _ = torch.sort(key, dim=1)
    nvalid = valid.reshape(Hkv, -1).sum(dim=1)
    pos = torch.arange(total_q * topk, device=dev).view(1, -1)
    q_indices = torch.where(pos < nvalid.view(-1, 1), (skey % total_q), torch.full_like(skey, -1)).to(torch.int32)
    counts = torch.zeros(Hkv, total_rows + 1, dtype=torch.int64, device=dev)
    counts.scatter_add_(1, torch.where(valid, rows, torch.full_like(rows, total_rows)).reshape(Hkv, -1),
                        torch.ones_like(key))
    row_ptr[:, 1:] = counts[:, :total_rows].cumsum(dim=1).to(torch.int32)
    return row_ptr, q_indices.contiguous()


def k2q_csr_to_q2k(k2q_row_ptr: torch.Tensor, k2q_q_indices: torch.Tensor, topK: int, cu_seqlens_q, kv_lens,
                   blk_kv: int = PAGE) -> torch.Tensor:
    """Inverse of ``build_k2q_csr``: ``kv_block_indexes[total_q, Hkv, topK]``
    (ascending request-local block ids, -1 tail)."""
    dev = k2q_row_ptr.device
    Hkv = k2q_row_ptr.shape[0]
    cq = [int(x) for x in cu_seqlens_q.tolist()]
    total_q = cq[-1]
    row_req, row_blk = _row_map(kv_lens, blk_kv, dev)
    total_rows = row_req.numel()
    out = torch.full((total_q, Hkv, topK), -1, dtype=torch.int32, device=dev)
    if total_rows == 0 or total_q == 0:
        return out
    cq_t = torch.tensor(cq, device=dev)
    for h in range(Hkv):
        rp = k2q_row_ptr[h].long()
        nnz = int(rp[-1].item())
        if nnz == 0:
            continue
        e = torch.arange(nnz, device=dev)
        row = torch.searchsorted(rp, e, right=True) - 1
        qg = k2q_q_indices[h, :nnz].long() + cq_t[row_req[row]]
        blk = row_blk[row]
        order = torch.argsort(qg * (total_rows + 1) + blk)
        qs, bs = qg[order], blk[order]
        first = torch.searchsorted(qs, qs, right=False)
        rank = torch.arange(nnz, device=dev) - first
        keep = rank < topK
        out[qs[keep], h, rank[keep]] = bs[keep].to(torch.int32)
    return out


def _flat_page_table(page_table: torch.Tensor, kv_lens, blk_kv: int) -> torch.Tensor:
    parts = [page_table[b, :(kl + blk_kv - 1) // blk_kv] for b, kl in enumerate(kv_lens)]
    return torch.cat(parts).to(torch.int32).contiguous()


def _row_map_np(kv_caps, blk_kv):
    """``_row_map`` on the host with numpy: (row_request, row_block) int32 arrays."""
    nblk = np.asarray([(k + blk_kv - 1) // blk_kv for k in kv_caps], dtype=np.int64)
    maxb = int(nblk.max()) if nblk.size else 0
    blk, req = np.meshgrid(np.arange(maxb), np.arange(nblk.size), indexing="ij")
    keep = blk < nblk[req]
    return req[keep].astype(np.int32), blk[keep].astype(np.int32)


def k2q_csr_to_lists(k2q_row_ptr: torch.Tensor, k2q_q_indices: torch.Tensor, topK: int, cu_seqlens_q: torch.Tensor,
                     row_request: torch.Tensor, row_block: torch.Tensor, total_q: int) -> torch.Tensor:
    """Device inverse of ``build_k2q_csr`` through ``msa_k2q_csr_to_lists``: int32
    ``kv_block_indexes[total_q, Hkv, topK]`` (ascending request-local block ids, -1 tail).
    ``row_request`` / ``row_block`` give the (request, block) of every CSR row (block-major packing)."""
    lib = _lib.get_lib()
    dev = k2q_row_ptr.device
    Hkv = k2q_row_ptr.shape[0]
    rp = k2q_row_ptr.to(torch.int32)
    qi = k2q_q_indices.to(torch.int32)
    if rp.stride(1) != 1:
        rp = rp.contiguous()
    if qi.stride(1) != 1:
        qi = qi.contiguous()
    out = torch.empty(total_q, Hkv, topK, dtype=torch.int32, device=dev)
    counters = torch.empty(max(1, total_q * Hkv), dtype=torch.int32, device=dev)
    cq = cu_seqlens_q.to(device=dev, dtype=torch.int32).contiguous()
    _lib.check(lib.msa_k2q_csr_to_lists(_ptr(rp), _ptr(qi), _ptr(row_request), _ptr(row_block), _ptr(cq), Hkv,
                                        int(row_request.numel()), rp.stride(0), qi.stride(0), total_q, topK,
                                        _ptr(counters), _ptr(out), _stream()), "msa_k2q_csr_to_lists")
    return out


# Host metadata of recent CSR calls, keyed by the identity and version of the length tensors: a model calls
# the attention once per layer with the same cu_seqlens / seqused_k tensors, and only the first call of a
# step has to read them back to the host and plan.
_CSR_PLAN_CACHE = TensorKeyedCache(16)


def _csr_plan(q, k, topK, cu_seqlens_q, cu_seqlens_k, blk_kv, causal, page_table, seqused_k):
    Hq, Hkv = q.shape[1], k.shape[1]
    key_tensors = (cu_seqlens_q, cu_seqlens_k, seqused_k, page_table)
    key_extra = (Hq, Hkv, topK, bool(causal), str(q.device))
    hit = _CSR_PLAN_CACHE.get(key_tensors, key_extra)
    if hit is not None:
        return hit
    cq = [int(x) for x in cu_seqlens_q.tolist()]
    B = len(cq) - 1
    qo_lens = [cq[i + 1] - cq[i] for i in range(B)]
    paged = page_table is not None
    ck = [int(x) for x in cu_seqlens_k.tolist()]
    if seqused_k is not None:
        kv_lens = [int(x) for x in seqused_k.tolist()]
    elif paged:
        kv_lens = [int(page_table.shape[1]) * blk_kv] * B
    else:
        kv_lens = [ck[i + 1] - ck[i] for i in range(B)]
    # the CSR rows are laid out over the KV capacity the caller built it with
    cap_csr = [ck[i + 1] - ck[i] for i in range(B)] if paged else kv_lens
    rr, rb = _row_map_np(cap_csr, blk_kv)
    plan = _fmha_sm100_plan(torch.tensor(qo_lens), torch.tensor(kv_lens), Hq, Hkv,
                            qo_offset=None if causal else 0, page_size=PAGE if paged else -1,
                            kv_block_num=topK, causal=causal, sparse_kernel_mode="prefill", device=q.device)
    ent = {
        "plan": plan,
        "row_request": torch.from_numpy(rr).to(q.device),
        "row_block": torch.from_numpy(rb).to(q.device),
        "kv_indices": _flat_page_table(page_table, kv_lens, blk_kv) if paged else None,
        "total_q": cq[-1],
    }
    return _CSR_PLAN_CACHE.put(key_tensors, key_extra, ent)


def _csr_forward(q, k, v, k2q_row_ptr, k2q_q_indices, topK, cu_seqlens_q, cu_seqlens_k, blk_kv, causal,
                 softmax_scale, return_softmax_lse, page_table, seqused_k, kv_dtype, qk_scale, v_scale,
                 k_sf=None, v_sf=None, usable_SM_count=-1, lse_temperature_scale=1.0, return_temperature_lse=False):
    if blk_kv != PAGE:
        raise MsaError(f"blk_kv must be {PAGE}")
    if topK not in (4, 8, 16, 32, 64):
        raise ValueError(f"topK must be one of 4, 8, 16, 32, 64, got {topK}")
    if not q.is_cuda:
        raise MsaError("q must be a CUDA tensor: libmsa_b200 has no CPU path")
    ent = _csr_plan(q, k, topK, cu_seqlens_q, cu_seqlens_k, blk_kv, causal, page_table, seqused_k)
    plan = ent["plan"]
    plan["usable_SM_count"] = usable_SM_count
    paged = page_table is not None
    q2k = k2q_csr_to_lists(k2q_row_ptr, k2q_q_indices, topK, cu_seqlens_q, ent["row_request"], ent["row_block"],
                           ent["total_q"])
    Hq = q.shape[1]
    out = torch.empty(q.shape[0], Hq, 128, dtype=torch.bfloat16, device=q.device)
    lse = torch.empty(q.shape[0], Hq, dtype=torch.float32, device=q.device) if return_softmax_lse else None
    qq = q.to(torch.bfloat16).contiguous() if q.dtype != torch.bfloat16 else q.contiguous()
    kc, vc = k.contiguous(), v.contiguous()
    _run_prefill(qq, kc, vc, plan, ent["kv_indices"], q2k, plan["qo_offset"], out, None, lse,
                 softmax_scale, qk_scale, v_scale, kv_dtype, paged, k_sf, v_sf)
    if return_temperature_lse:
        # LSE of the logits scaled by softmax_scale / lse_temperature_scale (python/fmha_sm100/cute/interface.py:
        # 665-699): a second pass of the same kernel at that scale, whose LSE is kept and whose output is dropped --
        # the price of an output few callers ask for, instead of a second exponential per score in every call
        lse_t = torch.empty_like(lse)
        scratch = torch.empty_like(out)
        _run_prefill(qq, kc, vc, plan, ent["kv_indices"], q2k, plan["qo_offset"], scratch, None, lse_t,
                     softmax_scale / lse_temperature_scale, qk_scale, v_scale, kv_dtype, paged, k_sf, v_sf)
        return out, lse, lse_t
    return (out, lse) if return_softmax_lse else out


def sparse_atten_func(q, k, v, k2q_row_ptr, k2q_q_indices, topK, *, cu_seqlens_q, cu_seqlens_k, max_seqlen_q,
                      max_seqlen_k, blk_kv: int = 128, causal: bool = False, softmax_scale: Optional[float] = None,
                      lse_temperature_scale: float = 1.0, return_temperature_lse: bool = False,
                      partial_dtype: torch.dtype = torch.bfloat16, return_softmax_lse: bool = False,
                      page_table: Optional[torch.Tensor] = None, seqused_k: Optional[torch.Tensor] = None,
                      schedule=None, usable_SM_count: int = -1, qk_dtype=None, pv_dtype=None):
    """Block-sparse varlen attention from k2q CSR metadata; signature of
    python/fmha_sm100/cute/interface.py:600-625.  q ``[total_q, Hq, 128]`` bf16;
    k/v ragged ``[total_k, Hkv, 128]`` or paged ``[pages, Hkv, 128, 128]`` in bf16
    or e4m3 (cast, no scale, as the reference does).  Returns bf16
    ``[total_q, Hq, 128]`` (and the natural-log LSE if asked).  ``partial_dtype``,
    ``schedule`` and the ``*_dtype`` knobs of the KV-outer reference kernel have no
    effect here: nothing is split, accumulation is fp32 in TMEM."""
    if softmax_scale is None:
        softmax_scale = q.shape[-1] ** -0.5
    lse_temperature_scale = float(lse_temperature_scale)
    if not math.isfinite(lse_temperature_scale) or lse_temperature_scale <= 0.0:
        raise ValueError(f"lse_temperature_scale must be finite and > 0, got {lse_temperature_scale}")
    if return_temperature_lse and not return_softmax_lse:
        raise ValueError("return_temperature_lse=True requires return_softmax_lse=True")
    if cu_seqlens_q is None or cu_seqlens_k is None:
        raise ValueError("sparse_atten_func requires CSR varlen metadata: pass cu_seqlens_q and cu_seqlens_k")
    kv_dtype = _lib.MSA_KV_FP8_E4M3 if k.dtype == torch.float8_e4m3fn else _lib.MSA_KV_BF16
    return _csr_forward(q, k, v, k2q_row_ptr, k2q_q_indices, int(topK), cu_seqlens_q, cu_seqlens_k, int(blk_kv),
                        bool(causal), float(softmax_scale), bool(return_softmax_lse), page_table, seqused_k,
                        kv_dtype, 1.0, 1.0, usable_SM_count=int(usable_SM_count),
                        lse_temperature_scale=lse_temperature_scale, return_temperature_lse=bool(return_temperature_lse))


def sparse_atten_nvfp4_kv_func(q, k, v, k_scale_128x4, v_scale_128x4, k_global_scale, v_global_scale, k2q_row_ptr,
                               k2q_q_indices, topK, *, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k,
                               blk_kv: int = 128, causal: bool = False, softmax_scale: Optional[float] = None,
                               lse_temperature_scale: float = 1.0, return_temperature_lse: bool = False,
                               partial_dtype: torch.dtype = torch.bfloat16, return_softmax_lse: bool = False,
                               page_table: Optional[torch.Tensor] = None, seqused_k: Optional[torch.Tensor] = None,
                               schedule=None):
    """Same with packed NVFP4 K/V (python/fmha_sm100/cute/interface.py:768-991):
    k/v uint8 ``[pages, Hkv, 128, 64]``, e4m3 block scales in 128x4 tiles with row
    ``(page * Hkv + head) * 128 + token``, optional fp32 global scales.  Paged only."""
    if page_table is None:
        raise MsaError("NVFP4 K/V requires the paged layout")
    if softmax_scale is None:
        softmax_scale = q.shape[-1] ** -0.5
    kg = 1.0 if k_global_scale is None else float(k_global_scale.reshape(-1)[0])
    vg = 1.0 if v_global_scale is None else float(v_global_scale.reshape(-1)[0])
    return _csr_forward(q, k.view(torch.uint8), v.view(torch.uint8), k2q_row_ptr, k2q_q_indices, int(topK),
                        cu_seqlens_q, cu_seqlens_k, int(blk_kv), bool(causal), float(softmax_scale),
                        bool(return_softmax_lse), page_table, seqused_k, _lib.MSA_KV_NVFP4, kg, vg,
                        k_scale_128x4.view(torch.uint8).contiguous(), v_scale_128x4.view(torch.uint8).contiguous(),
                        lse_temperature_scale=float(lse_temperature_scale),
                        return_temperature_lse=bool(return_temperature_lse))


def sparse_prefill_nvfp4(q, k_q, v_q, plan_info, kv_indices, kv_block_indexes, sm_scale=None, return_lse=False):
    """NVFP4 sparse prefill driven by per-query page lists (the ``fmha_sm100``
    calling convention): ``k_q`` / ``v_q`` are ``Nvfp4QuantizedTensor`` of paged
    K/V ``[pages, Hkv, 128, 128]``; ``plan_info`` comes from ``fmha_sm100_plan``."""
    plan = plan_info[3]
    if plan_info[0]:
        raise MsaError("mixed decode/prefill plans are not supported for NVFP4")
    sm_scale = q.shape[-1] ** -0.5 if sm_scale is None else sm_scale
    out = torch.empty(q.shape[0], q.shape[1], 128, dtype=torch.bfloat16, device=q.device)
    lse = torch.empty(q.shape[0], q.shape[1], dtype=torch.float32, device=q.device) if return_lse else None
    _run_prefill(q.contiguous(), k_q.data.contiguous(), v_q.data.contiguous(), plan, kv_indices.to(torch.int32).contiguous(),
                 kv_block_indexes.to(torch.int32).contiguous(), plan["qo_offset"], out, None, lse, sm_scale,
                 float(k_q.global_scale.reshape(-1)[0]), float(v_q.global_scale.reshape(-1)[0]), _lib.MSA_KV_NVFP4,
                 True, k_q.scale_128x4, v_q.scale_128x4)
    return (out, lse) if return_lse else out


class SparseDecodePagedAttentionWrapper:
    """Paged FP8 decode with a plan/run split; keyword signatures of
    python/fmha_sm100/cute/interface.py:1125-1423.  ``plan`` takes the page table and
    lengths once per batch shape; ``run`` attends each request's ``seqlen_q`` new tokens to
    all of its pages (dense decode) or, when ``q2k_indices`` was planned, to the selected
    pages only.  Differences from the reference: q may be bf16 as well as e4m3, any GQA ratio
    up to 16 and any ``seqlen_q`` are accepted, and ``run`` also takes per-tensor
    ``k_scale`` / ``v_scale`` and per-call ``kv_block_indexes`` ``[total_q, Hkv, topK]``.
    ``enable_cuda_graph`` needs nothing here (``run`` launches a fixed sequence of kernels with
    no host read-back); ``max_grid_size`` caps the SM count the split choice assumes,
    ``fixed_split_size`` (pages per split) and ``disable_split_kv`` override it."""

    def __init__(self, *, blk_kv: int = 128, causal: bool = True):
        if int(blk_kv) != PAGE:
            raise MsaError(f"blk_kv must be {PAGE}")
        self.blk_kv = int(blk_kv)
        self.causal = bool(causal)
        self._plan = None
        self._lists = None
        self.batch = self.num_qo_heads = self.num_kv_heads = self.head_dim = None
        self.page_table = self.seqused_k = self.q2k_indices = None
        self.seqlen_q = self.max_seqlen_k = None
        self.is_sparse = False
        self.split_kv = False

    def plan(self, page_table: Optional[torch.Tensor] = None, seqused_k: Optional[torch.Tensor] = None, *,
             seqlen_q: int = 1, max_seqlen_k: Optional[int] = None, q2k_indices: Optional[torch.Tensor] = None,
             num_qo_heads: Optional[int] = None, num_kv_heads: Optional[int] = None, head_dim: Optional[int] = 128,
             enable_cuda_graph: bool = False, max_grid_size: Optional[int] = None,
             fixed_split_size: Optional[int] = None, disable_split_kv: bool = False, num_kv_splits: int = -1):
        if page_table is None or seqused_k is None:
            raise ValueError("decode plan requires page_table and seqused_k")
        if page_table.ndim != 2:
            raise ValueError("decode plan requires page_table with shape [B, max_num_pages_per_seq]")
        if seqused_k.shape != (int(page_table.shape[0]),):
            raise ValueError("decode plan requires seqused_k with shape [B]")
        if not page_table.is_cuda:
            raise ValueError("decode plan requires page_table and seqused_k to be CUDA tensors")
        if num_qo_heads is None or num_kv_heads is None or head_dim is None:
            raise ValueError("decode plan requires num_qo_heads, num_kv_heads, and head_dim")
        if int(head_dim) != 128:
            raise NotImplementedError("decode plan currently supports only head_dim=128")
        if int(num_qo_heads) % int(num_kv_heads) != 0:
            raise ValueError("decode plan requires num_qo_heads divisible by num_kv_heads")
        if int(seqlen_q) <= 0:
            raise ValueError("decode plan requires positive seqlen_q")
        kv_lens = [int(x) for x in seqused_k.tolist()]
        B = len(kv_lens)
        if max_seqlen_k is not None and int(max_seqlen_k) < max(kv_lens + [0]):
            raise ValueError(f"max_seqlen_k={max_seqlen_k} is below the longest request ({max(kv_lens)})")
        dev = page_table.device
        self.batch, self.num_qo_heads, self.num_kv_heads, self.head_dim = B, int(num_qo_heads), int(num_kv_heads), 128
        self.page_table, self.seqused_k = page_table, seqused_k
        self.seqlen_q, self.max_seqlen_k = int(seqlen_q), int(max_seqlen_k or max(kv_lens + [0]))
        self.is_sparse = q2k_indices is not None
        self._kv_indices = _flat_page_table(page_table, kv_lens, self.blk_kv)
        maxp = max([(k + PAGE - 1) // PAGE for k in kv_lens] + [1])
        total_q = B * self.seqlen_q
        if self.is_sparse:
            if q2k_indices.dtype != torch.int32:
                raise TypeError("decode plan requires q2k_indices to be torch.int32")
            if q2k_indices.ndim != 3 or q2k_indices.shape[0] != self.num_kv_heads or q2k_indices.shape[1] != total_q:
                raise ValueError("decode plan requires q2k_indices with shape [Hkv, total_q, topK]")
            self.q2k_indices = q2k_indices
            self._lists = q2k_indices.permute(1, 0, 2).contiguous()
            list_len = int(q2k_indices.shape[2])
        else:
            dense = torch.arange(maxp, dtype=torch.int32, device=dev).view(1, 1, maxp)
            npg = torch.tensor([(k + PAGE - 1) // PAGE for k in kv_lens], device=dev)
            npg = torch.repeat_interleave(npg, self.seqlen_q).view(-1, 1, 1)
            self._lists = torch.where(dense < npg, dense, torch.full_like(dense, -1)).expand(
                total_q, self.num_kv_heads, maxp).contiguous()
            list_len = maxp
        if disable_split_kv:
            num_kv_splits = 1
        elif fixed_split_size is not None and int(fixed_split_size) > 0:
            num_kv_splits = max(1, -(-list_len // int(fixed_split_size)))
        self._plan = _fmha_sm100_plan(torch.tensor([self.seqlen_q] * B), torch.tensor(kv_lens), self.num_qo_heads,
                                      self.num_kv_heads, page_size=PAGE, kv_block_num=list_len, causal=self.causal,
                                      sparse_kernel_mode="decode", num_kv_splits=num_kv_splits,
                                      usable_SM_count=-1 if max_grid_size is None else int(max_grid_size), device=dev)
        self.split_kv = self._plan["num_kv_splits"] > 1
        return self

    def run(self, q, k, v, *, softmax_scale: Optional[float] = None, return_softmax_lse: bool = False,
            out: Optional[torch.Tensor] = None, lse: Optional[torch.Tensor] = None, k_scale: float = 1.0,
            v_scale: float = 1.0, kv_block_indexes: Optional[torch.Tensor] = None):
        if self._plan is None:
            raise RuntimeError("decode wrapper must be planned before run")
        if k.dtype != torch.float8_e4m3fn or v.dtype != torch.float8_e4m3fn:
            raise MsaError("the decode kernel takes e4m3 K/V")
        if q.shape[0] != self.batch * self.seqlen_q or q.shape[1] != self.num_qo_heads:
            raise ValueError(f"q must be [{self.batch * self.seqlen_q}, {self.num_qo_heads}, 128], got {tuple(q.shape)}")
        sm = q.shape[-1] ** -0.5 if softmax_scale is None else softmax_scale
        qq = q.to(torch.bfloat16).contiguous()
        lists = self._lists if kv_block_indexes is None else kv_block_indexes.to(torch.int32).contiguous()
        if out is None:
            out = torch.empty(qq.shape[0], qq.shape[1], 128, dtype=torch.bfloat16, device=q.device)
        if return_softmax_lse and lse is None:
            lse = torch.empty(qq.shape[0], qq.shape[1], dtype=torch.float32, device=q.device)
        _run_decode(qq, k.contiguous(), v.contiguous(), self._plan, self._kv_indices, lists, out,
                    lse if return_softmax_lse else None, sm, k_scale, v_scale)
        return (out, lse) if return_softmax_lse else out


def sparse_decode_atten_func(q, k, v, q2k_indices: Optional[torch.Tensor] = None, *, page_table: torch.Tensor,
                             seqused_k: torch.Tensor, seqlen_q: int, max_seqlen_k: int, blk_kv: int = 128,
                             causal: bool = True, softmax_scale: Optional[float] = None,
                             return_softmax_lse: bool = False, schedule=None, O_partial=None, LSE_partial=None):
    """One-shot paged FP8 decode (python/fmha_sm100/cute/interface.py:994-1122): plans and runs.
    ``q2k_indices`` ``[Hkv, total_q, topK]`` selects pages, ``None`` attends to every page.
    ``schedule`` / ``O_partial`` / ``LSE_partial`` belong to the reference's scheduler and are not needed:
    the split-KV workspace is owned by the plan."""
    w = SparseDecodePagedAttentionWrapper(blk_kv=blk_kv, causal=causal)
    w.plan(page_table=page_table, seqused_k=seqused_k, seqlen_q=seqlen_q, max_seqlen_k=max_seqlen_k,
           q2k_indices=q2k_indices, num_qo_heads=int(q.shape[1]), num_kv_heads=int(k.shape[1]), head_dim=int(q.shape[2]))
    return w.run(q, k, v, softmax_scale=softmax_scale, return_softmax_lse=return_softmax_lse)
