"""K/V cache quantisers for the two compressed formats of the hot path.

FP8: e4m3 with one float32 scale per tensor (``scale = amax / 448``).
NVFP4: two e2m1 codes per byte (low nibble = even element), one e4m3 scale per
16 values stored in 128x4 tiles, one float32 global scale
(``amax / (448 * 6)``) -- the storage contract of
python/fmha_sm100/cute/quantize.py:58-90, 145-159, 326-331 in the reference.
The reference delegates the NVFP4 rounding itself to Transformer Engine; here
the block scale is RNE-to-e4m3 of ``amax16 / (6 * global)`` and elements are
rounded to nearest-even on the e2m1 grid with saturation.
Pure torch tensor code; runs on whatever device the input lives on.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple

import torch

FP8_MAX = 448.0
FP4_MAX = 6.0
NVFP4_BLOCK = 16


def quantize_fp8_per_tensor(x: torch.Tensor) -> Tuple[torch.Tensor, float]:
    """Returns ``(x_e4m3, scale)`` with ``x ~= x_e4m3.float() * scale``."""
    amax = float(x.float().abs().max())
    scale = amax / FP8_MAX if amax > 0 else 1.0
    q = (x.float() / scale).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return q, scale


def nvfp4_scale_128x4_offset(row: torch.Tensor, col: torch.Tensor, scale_cols: int) -> torch.Tensor:
    """Flat offset of logical scale (row, col) in 128x4-tiled storage."""
    tiles_n = (scale_cols + 3) // 4
    return ((row // 128) * tiles_n + col // 4) * 512 + (row % 32) * 16 + ((row % 128) // 32) * 4 + col % 4


@dataclass
class Nvfp4QuantizedTensor:
    data: torch.Tensor          # uint8 [..., D/2]
    scale_128x4: torch.Tensor   # uint8 [round_up(rows, 128), round_up(D/16, 4)], e4m3 bits in 128x4-tiled storage
    global_scale: torch.Tensor  # float32 [1]
    logical_scale_shape: Tuple[int, int]
    original_shape: Tuple[int, ...]


def _e2m1_codes(a: torch.Tensor) -> torch.Tensor:
    """|x| (already divided by its scale) -> 3-bit e2m1 magnitude code, RNE, saturating."""
    a = a.clamp(max=FP4_MAX)
    # thresholds are the midpoints of {0,.5,1,1.5,2,3,4,6}; ties go to the even code
    code = torch.zeros_like(a, dtype=torch.int32)
    mids = [0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0]
    for i, m in enumerate(mids):
        up_is_even = ((i + 1) % 2 == 0)
        code = code + ((a >= m) if up_is_even else (a > m)).to(torch.int32)
    return code


def quantize_bf16_to_nvfp4_128x4(x: torch.Tensor) -> Nvfp4QuantizedTensor:
    """Quantise ``x[..., D]`` (D % 16 == 0); the flattened leading index is the scale row."""
    D = x.shape[-1]
    assert D % NVFP4_BLOCK == 0
    xf = x.float().reshape(-1, D)
    rows, scols = xf.shape[0], D // NVFP4_BLOCK
    amax = float(xf.abs().max())
    gscale = amax / (FP8_MAX * FP4_MAX) if amax > 0 else 1.0
    blk = xf.view(rows, scols, NVFP4_BLOCK)
    bscale = (blk.abs().amax(dim=-1) / (FP4_MAX * gscale)).clamp(max=FP8_MAX).to(torch.float8_e4m3fn)
    bs = bscale.float()
    denom = torch.where(bs > 0, bs * gscale, torch.ones_like(bs)).unsqueeze(-1)
    y = blk / denom
    code = _e2m1_codes(y.abs()) + (torch.signbit(y).to(torch.int32) << 3)
    code = code.view(rows, D).to(torch.uint8)
    data = code[:, 0::2] | (code[:, 1::2] << 4)
    rows_pad, cols_pad = (rows + 127) // 128 * 128, (scols + 3) // 4 * 4
    sflat = torch.zeros(rows_pad * cols_pad, dtype=torch.uint8, device=x.device)
    r = torch.arange(rows, device=x.device).view(-1, 1).expand(rows, scols)
    c = torch.arange(scols, device=x.device).view(1, -1).expand(rows, scols)
    sflat[nvfp4_scale_128x4_offset(r, c, scols).reshape(-1)] = bscale.view(torch.uint8).reshape(-1)
    return Nvfp4QuantizedTensor(data=data.view(*x.shape[:-1], D // 2), scale_128x4=sflat.view(rows_pad, cols_pad),
                                global_scale=torch.tensor([gscale], dtype=torch.float32, device=x.device),
                                logical_scale_shape=(rows, scols), original_shape=tuple(x.shape))


def quantize_kv_bf16_to_nvfp4_128x4(k: torch.Tensor, v: torch.Tensor):
    return quantize_bf16_to_nvfp4_128x4(k), quantize_bf16_to_nvfp4_128x4(v)


_FP4_LUT = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0]


def dequantize_nvfp4_128x4(qx: Nvfp4QuantizedTensor, include_global_scale: bool = True) -> torch.Tensor:
    """``e2m1 * e4m3 block scale * global`` as float32 in the original shape."""
    D = qx.original_shape[-1]
    packed = qx.data.reshape(-1, D // 2)
    rows, scols = packed.shape[0], D // NVFP4_BLOCK
    lut = torch.tensor(_FP4_LUT, dtype=torch.float32, device=packed.device)
    vals = torch.empty(rows, D, dtype=torch.float32, device=packed.device)
    vals[:, 0::2] = lut[(packed & 0x0F).long()]
    vals[:, 1::2] = lut[(packed >> 4).long()]
    r = torch.arange(rows, device=packed.device).view(-1, 1).expand(rows, scols)
    c = torch.arange(scols, device=packed.device).view(1, -1).expand(rows, scols)
    s = qx.scale_128x4.reshape(-1)[nvfp4_scale_128x4_offset(r, c, scols).reshape(-1)].view(rows, scols)
    s = s.view(torch.float8_e4m3fn).float().repeat_interleave(NVFP4_BLOCK, dim=1)
    out = vals * s
    if include_global_scale:
        out = out * qx.global_scale.reshape(-1)[0]
    return out.view(qx.original_shape)
