"""KV-cache append: quantise new BF16 K/V rows on the device and scatter them into the paged cache.

The reference fills its compressed caches with PyTorch / Transformer Engine calls outside the attention path
(per-tensor FP8: python/fmha_sm100/cute/test_sparse_atten.py:1229-1235; NVFP4 with 128x4-tiled block scales:
python/fmha_sm100/cute/quantize.py:162-232).  Here one kernel launch (``msa_kv_append``) converts K and V of a
batch of new tokens straight into the cache layout the attention kernels read, so a serving loop never
materialises an intermediate quantised tensor or a separate scale swizzle.
"""
from __future__ import annotations

import ctypes
from typing import Tuple

import torch

from . import _lib
from ._lib import KvAppendArgs, MsaError, check, get_lib

PAGE = 128
HEAD_DIM = 128
FP8_MAX = 448.0
FP4_MAX = 6.0


def _stream(t: torch.Tensor) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def absmax_bf16(x: torch.Tensor, out: torch.Tensor = None) -> torch.Tensor:
    """max |x| of a BF16 CUDA tensor as float32 [1] on the device (no synchronisation).  With ``out`` the
    result is folded into it (running maximum over several calls)."""
    if not x.is_cuda or x.dtype != torch.bfloat16:
        raise MsaError("absmax_bf16 needs a CUDA bf16 tensor")
    x = x.contiguous()
    if out is None:
        out = torch.zeros(1, dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        check(get_lib().msa_absmax_bf16(ctypes.c_void_p(x.data_ptr()), x.numel(), ctypes.c_void_p(out.data_ptr()),
                                        _stream(x)), "msa_absmax_bf16")
    return out


def fp8_scale_from_amax(amax: float) -> float:
    """Per-tensor FP8 dequant scale, ``amax / 448`` (1 for an all-zero tensor)."""
    return float(amax) / FP8_MAX if amax > 0 else 1.0


def nvfp4_global_scale_from_amax(amax: float) -> float:
    """NVFP4 global dequant scale, ``amax / (448 * 6)`` (python/fmha_sm100/cute/quantize.py:145-159)."""
    return float(amax) / (FP8_MAX * FP4_MAX) if amax > 0 else 1.0


def alloc_fp8_cache(num_pages: int, num_kv_heads: int, device) -> Tuple[torch.Tensor, torch.Tensor]:
    shape = (num_pages, num_kv_heads, PAGE, HEAD_DIM)
    return (torch.zeros(shape, dtype=torch.float8_e4m3fn, device=device),
            torch.zeros(shape, dtype=torch.float8_e4m3fn, device=device))


def alloc_nvfp4_cache(num_pages: int, num_kv_heads: int, device):
    """``(k_data, v_data, k_block_scales, v_block_scales)``: uint8 [pages, Hkv, 128, 64] and the 128x4-tiled
    e4m3 scale storage, uint8 [pages * Hkv * 128, 8] (the rank-2 shape the reference's NVFP4 entry points take,
    python/fmha_sm100/cute/interface.py:355-416)."""
    shape = (num_pages, num_kv_heads, PAGE, HEAD_DIM // 2)
    sshape = (num_pages * num_kv_heads * PAGE, HEAD_DIM // 16)
    mk = lambda *s: torch.zeros(*s, dtype=torch.uint8, device=device)  # noqa: E731
    return mk(shape), mk(shape), mk(sshape), mk(sshape)


def _append(fmt, k_new, v_new, k_cache, v_cache, k_bs, v_bs, slots, k_scale, v_scale):
    if not (k_new.is_cuda and v_new.is_cuda and k_cache.is_cuda and v_cache.is_cuda and slots.is_cuda):
        raise MsaError("kv append needs CUDA tensors")
    if k_new.dtype != torch.bfloat16 or v_new.dtype != torch.bfloat16:
        raise MsaError("k_new / v_new must be bf16")
    if k_new.dim() != 3 or k_new.shape != v_new.shape or k_new.shape[2] != HEAD_DIM:
        raise MsaError("k_new / v_new must be [tokens, Hkv, 128] of equal shape")
    n, hkv = int(k_new.shape[0]), int(k_new.shape[1])
    last = HEAD_DIM if fmt == _lib.MSA_KV_FP8_E4M3 else HEAD_DIM // 2
    for name, c in (("k_cache", k_cache), ("v_cache", v_cache)):
        if c.dim() != 4 or c.shape[1] != hkv or c.shape[2] != PAGE or c.shape[3] != last or c.element_size() != 1:
            raise MsaError(f"{name} must be one byte per element, [pages, {hkv}, 128, {last}]")
        if not c.is_contiguous():
            raise MsaError(f"{name} must be contiguous")
    if k_cache.shape != v_cache.shape:
        raise MsaError("k_cache and v_cache differ in shape")
    if slots.dtype != torch.int32 or slots.numel() != n:
        raise MsaError("slots must be int32 [tokens]")
    pages = int(k_cache.shape[0])
    if fmt == _lib.MSA_KV_NVFP4:
        need = pages * hkv * PAGE * (HEAD_DIM // 16)
        for name, s in (("k_block_scales", k_bs), ("v_block_scales", v_bs)):
            if s is None or not s.is_cuda or s.element_size() != 1 or s.numel() < need or not s.is_contiguous():
                raise MsaError(f"{name} must be a contiguous CUDA byte tensor of at least {need} elements")
    k_new, v_new, slots = k_new.contiguous(), v_new.contiguous(), slots.contiguous()
    a = KvAppendArgs()
    a.struct_size = ctypes.sizeof(KvAppendArgs)
    a.format = fmt
    a.k_new, a.v_new = k_new.data_ptr(), v_new.data_ptr()
    a.k_cache, a.v_cache = k_cache.data_ptr(), v_cache.data_ptr()
    a.k_block_scales = k_bs.data_ptr() if k_bs is not None else None
    a.v_block_scales = v_bs.data_ptr() if v_bs is not None else None
    a.slots = slots.data_ptr()
    a.num_tokens, a.num_kv_heads, a.head_dim, a.num_pages = n, hkv, HEAD_DIM, pages
    a.k_scale, a.v_scale = float(k_scale), float(v_scale)
    with torch.cuda.device(k_new.device):
        check(get_lib().msa_kv_append(ctypes.byref(a), _stream(k_new)), "msa_kv_append")


def append_kv_fp8(k_new: torch.Tensor, v_new: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                  slots: torch.Tensor, k_scale: float, v_scale: float) -> None:
    """Write ``e4m3(clamp(x / scale))`` of the new rows into ``k_cache`` / ``v_cache``
    ([pages, Hkv, 128, 128], float8_e4m3fn or uint8) at ``slots`` (physical page * 128 + position; negative =
    skip).  ``k_scale`` / ``v_scale`` are the dequant scales the attention call is later given."""
    _append(_lib.MSA_KV_FP8_E4M3, k_new, v_new, k_cache, v_cache, None, None, slots, k_scale, v_scale)


def append_kv_nvfp4(k_new: torch.Tensor, v_new: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                    k_block_scales: torch.Tensor, v_block_scales: torch.Tensor, slots: torch.Tensor,
                    k_global_scale: float, v_global_scale: float) -> None:
    """NVFP4 variant: packed e2m1 codes into ``k_cache`` / ``v_cache`` (uint8 [pages, Hkv, 128, 64]) and the
    e4m3 block scales into the 128x4-tiled ``*_block_scales`` at row ``(page * Hkv + head) * 128 + position``."""
    _append(_lib.MSA_KV_NVFP4, k_new, v_new, k_cache, v_cache, k_block_scales, v_block_scales, slots,
            k_global_scale, v_global_scale)
