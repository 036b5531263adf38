"""Host codec of the NVFP4 key/value page format (the oracle of the append and read kernels).

Row layout (`csrc/include/kv_fp4.cuh`): ``D/2`` code bytes (value 2j in the low nibble of byte j, value 2j+1 in the high
nibble; bit 3 of a nibble is the sign, bits 0..2 index {0, .5, 1, 1.5, 2, 3, 4, 6}), ``D/16`` UE4M3 block scales (one per 16
values), zero padding to a multiple of 16 bytes; one fp32 scale per row (``max|row| / (6 * 448)``) is kept beside the pool.
``value = e2m1(code) * e4m3(block scale) * row scale``.  Every operation below mirrors the kernels' fp32 arithmetic
(correctly rounded multiplications and divisions), so codes and scales are expected to match the device bit for bit.

Reference counterpart: the 4-bit KV block codec ``include/phaseshift/quantization/psq/psq4_kv.h:1-79``
(``psq4_lsq1_encode_block``), whose 32-value blocks with codebook codes and a bf16 scale play the role of the 16-value
E2M1 blocks with E4M3 scales here.
"""
from __future__ import annotations

from typing import Tuple

import torch

from .formats import _e2m1_index, _e2m1_value, _from_e4m3_bytes, _to_e4m3_bytes


def nvfp4_row_bytes(head_dim: int) -> int:
    return ((head_dim // 2 + head_dim // 16) + 15) & ~15


def bits_per_value(kv_dtype: str, head_dim: int) -> float:
    """Storage cost of one cached value, row scale included."""
    if kv_dtype == "nvfp4":
        return (nvfp4_row_bytes(head_dim) + 4) * 8 / head_dim
    if kv_dtype == "fp8_e4m3":
        return (head_dim + 4) * 8 / head_dim
    return 16.0


def encode_nvfp4_rows(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``x [..., D]`` (any float dtype; D a multiple of 32) -> (rows ``[..., row_bytes]`` uint8, row scales ``[...]`` fp32)."""
    D = x.shape[-1]
    if D % 32:
        raise ValueError("head size must be a multiple of 32")
    xf = x.to(torch.float32)
    lead = xf.shape[:-1]
    amax = xf.abs().amax(dim=-1)
    ts = torch.where(amax > 0, amax * torch.tensor(1.0 / (6.0 * 448.0), dtype=torch.float32), torch.ones_like(amax))
    blocks = xf.reshape(*lead, D // 16, 16)
    bmax = blocks.abs().amax(dim=-1)
    sf = _to_e4m3_bytes(bmax / (6.0 * ts).unsqueeze(-1))
    sf_f = _from_e4m3_bytes(sf)
    denom = sf_f * ts.unsqueeze(-1)
    inv = torch.where(sf_f > 0, 1.0 / denom, torch.zeros_like(denom))
    scaled = blocks * inv.unsqueeze(-1)
    idx = _e2m1_index(scaled.abs()).to(torch.uint8)
    nib = idx | (((scaled < 0) & (idx != 0)).to(torch.uint8) << 3)      # no negative zero (the device may store one; it decodes to 0)
    nib = nib.reshape(*lead, D // 2, 2)
    codes = nib[..., 0] | (nib[..., 1] << 4)
    rows = torch.zeros(*lead, nvfp4_row_bytes(D), dtype=torch.uint8, device=x.device)
    rows[..., : D // 2] = codes
    rows[..., D // 2: D // 2 + D // 16] = sf
    return rows, ts


def decode_nvfp4_rows(rows: torch.Tensor, scale: torch.Tensor, head_dim: int) -> torch.Tensor:
    """Inverse of `encode_nvfp4_rows`: fp32 values ``[..., D]``."""
    D = head_dim
    codes = rows[..., : D // 2]
    sf = _from_e4m3_bytes(rows[..., D // 2: D // 2 + D // 16].contiguous())
    nib = torch.stack((codes & 0xF, codes >> 4), dim=-1).reshape(*rows.shape[:-1], D)
    mag = _e2m1_value(nib & 7)
    val = torch.where((nib & 8) != 0, -mag, mag)
    val = val.reshape(*rows.shape[:-1], D // 16, 16) * sf.unsqueeze(-1)
    return val.reshape(*rows.shape[:-1], D) * scale.to(torch.float32).unsqueeze(-1)
