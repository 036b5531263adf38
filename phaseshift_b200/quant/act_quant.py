"""Activation quantisation for the block-scaled tensor-core projections, and the scale-factor layout
those kernels read.

The sm_100a block-scaled MMA needs both operands in the same block format, so activations are
quantised on the fly (the reference quantises activations to per-row-scaled E4M3 in front of its
quantised GEMMs, src/phaseshift/models/qwen35/kernels/optimized/activation_quantize.hip:65-317):

* NVFP4 weights -> NVFP4 activations: blocks of 16, UE4M3 block scale, and ONE fixed fp32 scale ``gs``
  per projection input site (``LinearW.act_scale``, calibrated, see ``calibrate_act_scale``):
  ``sf = e4m3(amax / (6 gs))``, ``q = e2m1(v / (sf gs))``, ``v ~= q sf gs``.
* MXFP8 weights -> MXFP8 activations: blocks of 32, UE8M0 exponent ``e`` = smallest with
  ``amax / 2^e <= 448``, ``q = e4m3(v / 2^e)``.

The functions here restate the CUDA quantisers (csrc/kernels/gemm_bs.cu) operation for operation in
fp32 PyTorch; they are the oracle of the kernel tests and what the CPU reference ops use to mimic the
tensor-core path.
"""
from __future__ import annotations

import torch

from .formats import _e2m1_index, _e2m1_value, _from_e4m3_bytes, _to_e4m3_bytes

PANEL_K = {"nvfp4": 256, "mxfp8": 128}        # K extent of one 128-byte operand panel
ATOMS_PER_PANEL = {"nvfp4": 4, "mxfp8": 1}    # 512-byte scale atoms per panel and 128 rows
SF_BLOCK = {"nvfp4": 16, "mxfp8": 32}
ACT_SCALE_TARGET_SF = 32.0                    # calibrated amax maps to a block scale of 32 (14x headroom to 448)


def calibrate_act_scale(amax: float) -> float:
    """Fixed NVFP4 activation scale for a site whose calibration run saw `amax`."""
    amax = max(float(amax), 1e-6)
    return amax / (6.0 * ACT_SCALE_TARGET_SF)


DEFAULT_ACT_SCALE = calibrate_act_scale(8.0)


def _blocks(x: torch.Tensor, b: int) -> torch.Tensor:
    m, k = x.shape
    kp = -(-k // b) * b
    if kp != k:
        x = torch.nn.functional.pad(x, (0, kp - k))
    return x.reshape(m, kp // b, b)


def fake_quant_nvfp4(x: torch.Tensor, gs: float) -> torch.Tensor:
    """fp32 [M, K] -> the values the NVFP4 activation quantiser represents (fp32 [M, K])."""
    m, k = x.shape
    f32 = torch.float32
    v = _blocks(x.to(f32), 16)
    gs_t = torch.tensor(gs, dtype=f32, device=x.device)
    c1 = torch.tensor(1.0, dtype=f32, device=x.device) / (torch.tensor(6.0, dtype=f32, device=x.device) * gs_t)
    amax = v.abs().amax(-1, keepdim=True)
    sf = _from_e4m3_bytes(_to_e4m3_bytes(amax * c1))
    inv = torch.where(sf > 0, 1.0 / (sf * gs_t), torch.zeros_like(sf))
    t = v * inv
    idx = _e2m1_index(t.abs())
    q = _e2m1_value(idx) * torch.sign(t)
    return (q * sf * gs_t).reshape(m, -1)[:, :k]


def fake_quant_mxfp8(x: torch.Tensor) -> torch.Tensor:
    """fp32 [M, K] -> the values the MXFP8 activation quantiser represents."""
    m, k = x.shape
    v = _blocks(x.to(torch.float32), 32)
    amax = v.abs().amax(-1, keepdim=True)
    mant, ex = torch.frexp(amax)                     # amax = mant * 2^ex, mant in [0.5, 1)
    e = (ex - 1) - 8 + (mant * 2.0 > 1.75).to(ex.dtype)
    e = e.clamp(-126, 126)
    live = amax >= 1e-30
    e = torch.where(live, e, torch.zeros_like(e))
    scale = torch.ldexp(torch.ones_like(amax), e)
    q = _from_e4m3_bytes(_to_e4m3_bytes(v / scale))
    q = torch.where(live, q, torch.zeros_like(q))
    return (q * scale).reshape(m, -1)[:, :k]


def fake_quant(x: torch.Tensor, fmt: str, gs: float) -> torch.Tensor:
    if fmt == "nvfp4":
        return fake_quant_nvfp4(x, gs)
    if fmt == "mxfp8":
        return fake_quant_mxfp8(x)
    return x


def pack_sf_atoms(scales: torch.Tensor, fmt: str, k: int) -> torch.Tensor:
    """Canonical block scales uint8 [N, blocks] -> scale atoms uint8 [ceil(N/128), panels * app, 512].

    Inside an atom (128 rows x 4 consecutive K-blocks) the factor of row r, block j sits at byte
    ``(r % 32) * 16 + (r // 32) * 4 + j``: one `tcgen05.cp.32x128b.warpx4` moves it into the four
    tensor-memory columns the block-scaled MMA reads.  Rows past N and blocks past K hold 0, which
    both UE4M3 (0.0) and UE8M0 (2^-127) decode to a finite value, so zero padding codes stay zero."""
    n, nb = scales.shape
    panels = -(-k // PANEL_K[fmt])
    atoms_k = panels * ATOMS_PER_PANEL[fmt]
    tiles = -(-n // 128)
    full = torch.zeros(tiles * 128, atoms_k * 4, dtype=torch.uint8, device=scales.device)
    full[:n, :min(nb, atoms_k * 4)] = scales[:, :atoms_k * 4]
    a = full.reshape(tiles, 4, 32, atoms_k, 4).permute(0, 3, 2, 1, 4)       # [tile, atom, r%32, r//32, j]
    return a.reshape(tiles, atoms_k, 512).contiguous()


def unpack_sf_atoms(atoms: torch.Tensor, n: int, nb: int) -> torch.Tensor:
    """Inverse of pack_sf_atoms (tests)."""
    tiles, atoms_k, _ = atoms.shape
    a = atoms.reshape(tiles, atoms_k, 32, 4, 4).permute(0, 3, 2, 1, 4).reshape(tiles * 128, atoms_k * 4)
    return a[:n, :nb].contiguous()
