"""Kernel-side weight layout ("tiled"): the engine's counterpart of the reference's mandatory native
preshuffle (docs/developer/psq_canonical_soa_payload.md:474-511,674-708).  Canonical row-major payloads
are never fed to kernels; after tensor-parallel slicing and quantisation each matrix is rearranged once
so that the bytes one warp consumes together are contiguous:

    block(quad q, k-step s) at byte offset (q * steps + s) * block_bytes
      = [4 rows x 512 B codes][4 rows x scale_row B block scales]

with N padded to a multiple of 4 rows and K to whole k-steps (zero codes, neutral scales).
k-step = 256 bf16 / 1024 nvfp4 / 512 mxfp8 weights per row (32 lanes x 16 bytes).
"""
from __future__ import annotations

import torch

from .formats import QuantizedTensor

STEP_K = {"bf16": 256, "nvfp4": 1024, "mxfp8": 512}
SCALE_ROW = {"bf16": 0, "nvfp4": 64, "mxfp8": 16}
BLOCK_BYTES = {f: 2048 + 4 * SCALE_ROW[f] for f in STEP_K}


def tiled_steps(fmt: str, k: int) -> int:
    return -(-k // STEP_K[fmt])


def tiled_nbytes(fmt: str, n: int, k: int) -> int:
    return -(-n // 4) * tiled_steps(fmt, k) * BLOCK_BYTES[fmt]


def tile_weight(q: QuantizedTensor) -> torch.Tensor:
    """QuantizedTensor (canonical) -> flat uint8 tensor in tiled layout, on the same device."""
    fmt = q.fmt
    n, _ = q.shape
    kp = q.k_padded
    steps = tiled_steps(fmt, kp)
    quads = -(-n // 4)
    dev = q.codes.device
    if fmt == "bf16":
        codes = q.codes.contiguous().view(torch.uint8).reshape(n, kp * 2)
    else:
        codes = q.codes.reshape(n, -1)
    row_bytes = steps * 512
    cb = torch.zeros(quads * 4, row_bytes, dtype=torch.uint8, device=dev)
    cb[:n, :codes.shape[1]] = codes
    cb = cb.reshape(quads, 4, steps, 512).permute(0, 2, 1, 3).reshape(quads, steps, 2048)
    sr = SCALE_ROW[fmt]
    if sr == 0:
        return cb.reshape(-1).contiguous()
    sc = torch.zeros(quads * 4, steps * sr, dtype=torch.uint8, device=dev)
    if fmt == "mxfp8":
        sc.fill_(127)          # 2^0 for padding blocks (their codes are zero anyway)
    sc[:n, :q.scales.shape[1]] = q.scales
    sc = sc.reshape(quads, 4, steps, sr).permute(0, 2, 1, 3).reshape(quads, steps, 4 * sr)
    return torch.cat([cb, sc], dim=2).reshape(-1).contiguous()


def untile_weight(t: torch.Tensor, fmt: str, n: int, k_padded: int) -> QuantizedTensor:
    """Inverse of tile_weight (tests; tensor_scale must be restored by the caller)."""
    steps = tiled_steps(fmt, k_padded)
    quads = -(-n // 4)
    sr = SCALE_ROW[fmt]
    blk = t.reshape(quads, steps, BLOCK_BYTES[fmt])
    cb = blk[:, :, :2048].reshape(quads, steps, 4, 512).permute(0, 2, 1, 3).reshape(quads * 4, steps * 512)[:n]
    if fmt == "bf16":
        codes = cb[:, :k_padded * 2].contiguous().view(torch.bfloat16)
        return QuantizedTensor(fmt, (n, k_padded), k_padded, codes, None, 1.0)
    width = k_padded // 2 if fmt == "nvfp4" else k_padded
    codes = cb[:, :width].contiguous()
    sc = blk[:, :, 2048:].reshape(quads, steps, 4, sr).permute(0, 2, 1, 3).reshape(quads * 4, steps * sr)[:n]
    sw = k_padded // 16 if fmt == "nvfp4" else k_padded // 32
    return QuantizedTensor(fmt, (n, k_padded), k_padded, codes, sc[:, :sw].contiguous(), 1.0)
