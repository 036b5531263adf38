"""Block-scaled weight formats: NVFP4 (replaces PSQ4) and MXFP8 (replaces PSQ8), plus BF16.

Canonical payload (what the quantised safetensors directory stores; K contiguous, one row per output
feature, ``padded_k = align_up(k, 32)`` with zero padding, metadata never crossing a row -- the same
shape rules as the reference's canonical SoA payload, docs/developer/psq_canonical_soa_payload.md:77-89):

* ``nvfp4``: codes uint8 [N, Kp/2], sequential nibbles ``byte[j] = q[2j] | q[2j+1] << 4`` where
  q = sign<<3 | index into {0, .5, 1, 1.5, 2, 3, 4, 6}; metadata1 = UE4M3 scale per 16 weights
  [N, Kp/16]; metadata2 = one fp32 per-tensor scale.  w ~= E2M1[q] * e4m3(scale) * tensor_scale. 4.5 bpw.
* ``mxfp8``: codes = E4M3 bytes [N, Kp]; metadata1 = UE8M0 exponent per 32 weights [N, Kp/32].
  w ~= e4m3(code) * 2^(e-127).  8.25 bpw.

Two further formats are understood as *interchange* formats (checkpoints produced elsewhere), the
counterparts of the reference's FP8-block128 and MXFP4 kernels (src/phaseshift/models/qwen35/kernels/
optimized/linear/fp8_block128.hip, mxfp4.hip).  They have no kernels of their own: `to_kernel_format`
re-expresses them in a format the sm_100a kernels consume.

* ``mxfp4``: E2M1 nibbles as in ``nvfp4``; metadata1 = UE8M0 exponent per 32 weights.  4.25 bpw.  Runs as
  NVFP4 without any loss: every MXFP4 block scale 2^e is representable as e4m3(2^(e-t)) * 2^t.
* ``fp8_block128``: E4M3 bytes [N, Kp]; metadata1 = fp32 scale per 128 x 128 block [ceil(N/128), Kp/128].
  Runs as MXFP8 after one re-quantisation (its scales are not powers of two).

Block scales are chosen by a small search around the max-abs scale that minimises the block's
squared error, the counterpart of the reference's 65-candidate PSQ scale search
(src/phaseshift/quantization/psq/psq.cpp:39-74); an optional per-input-channel importance vector
(imatrix) weights the error like the reference's GPU quantiser does
(src/phaseshift/quantization/offline/gpu_quantizer.hip:8-32).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
_E2M1_BOUNDS = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)
FORMATS = ("bf16", "nvfp4", "mxfp8")
INTERCHANGE_FORMATS = ("mxfp4", "fp8_block128")
BLOCK = {"bf16": 16, "nvfp4": 16, "mxfp8": 32, "mxfp4": 32, "fp8_block128": 128}
K_ALIGN = 32
DEFAULT_SEARCH = 2      # scale-search half-width used by quantize() (0 = plain max-abs scales)


def align_up(x: int, a: int) -> int:
    return (x + a - 1) // a * a


def _e2m1_index(mag: torch.Tensor) -> torch.Tensor:
    """Nearest E2M1 magnitude index; exact midpoints go to the even index (round-half-even on codes)."""
    b = torch.tensor(_E2M1_BOUNDS, dtype=mag.dtype, device=mag.device)
    idx = torch.bucketize(mag, b, right=False)           # mag == bound -> lower index
    # midpoints: lower index is idx; choose even of (idx, idx+1)
    at_mid = torch.zeros_like(mag, dtype=torch.bool)
    for j, bd in enumerate(_E2M1_BOUNDS):
        at_mid |= (mag == bd)
    idx = torch.where(at_mid & (idx % 2 == 1), idx + 1, idx)
    return idx.clamp_(max=7)


def _e2m1_value(idx: torch.Tensor, dtype=torch.float32) -> torch.Tensor:
    lut = torch.tensor(E2M1_VALUES, dtype=dtype, device=idx.device)
    return lut[idx.long()]


def _to_e4m3_bytes(x: torch.Tensor) -> torch.Tensor:
    return x.clamp(-448.0, 448.0).to(torch.float8_e4m3fn).view(torch.uint8)


def _from_e4m3_bytes(b: torch.Tensor) -> torch.Tensor:
    return b.view(torch.float8_e4m3fn).to(torch.float32)


@dataclass
class QuantizedTensor:
    fmt: str
    shape: tuple                      # logical (N, K)
    k_padded: int
    codes: torch.Tensor               # bf16 [N, Kp] | uint8 [N, Kp/2] | uint8 [N, Kp]
    scales: Optional[torch.Tensor] = None      # uint8 block scales
    tensor_scale: float = 1.0

    def to(self, device) -> "QuantizedTensor":
        return QuantizedTensor(self.fmt, self.shape, self.k_padded, self.codes.to(device),
                               None if self.scales is None else self.scales.to(device), self.tensor_scale)

    @property
    def nbytes(self) -> int:
        n = self.codes.numel() * self.codes.element_size()
        if self.scales is not None:
            n += self.scales.numel()
        return n


def _pad_k(w: torch.Tensor) -> torch.Tensor:
    n, k = w.shape
    kp = align_up(k, K_ALIGN)
    if kp == k:
        return w
    out = w.new_zeros(n, kp)
    out[:, :k] = w
    return out


USE_CUDA_KERNELS = True     # CUDA tensors go through the dedicated quantiser kernels (bit-equal to the C++ ones)


def _kernel_quantize(wf: torch.Tensor, fmt: str, k: int, kp: int, importance, search: int, tensor_scale: float):
    """Row quantiser kernels (csrc/kernels/quant_kernels.cu).  `wf` is fp32 [N, kp] on a CUDA device."""
    import ctypes
    from ..ops import _lib
    n = wf.shape[0]
    dev = wf.device
    nv = fmt == "nvfp4"
    codes = torch.empty(n, kp // 2 if nv else kp, dtype=torch.uint8, device=dev)
    scales = torch.empty(n, kp // (16 if nv else 32), dtype=torch.uint8, device=dev)
    imp = None
    if importance is not None:
        imp = importance.float().reshape(-1).to(dev).contiguous()
    with torch.cuda.device(dev):
        _lib.call("ps_quantize_rows", ctypes.c_int(1 if nv else 0), ctypes.c_void_p(wf.data_ptr()), ctypes.c_longlong(wf.stride(0)),
                  ctypes.c_int(n), ctypes.c_int(k), ctypes.c_int(kp), ctypes.c_float(tensor_scale), ctypes.c_int(search),
                  ctypes.c_void_p(imp.data_ptr() if imp is not None else None), ctypes.c_void_p(codes.data_ptr()),
                  ctypes.c_void_p(scales.data_ptr()))
    return codes, scales


def _kernels_ok(w: torch.Tensor) -> bool:
    if not (USE_CUDA_KERNELS and w.is_cuda):
        return False
    try:
        from ..ops import _lib
        _lib.lib()
        return True
    except Exception:
        return False


def quantize_nvfp4(w: torch.Tensor, importance: Optional[torch.Tensor] = None, search: int = 2,
                   tensor_scale: Optional[float] = None) -> QuantizedTensor:
    """w [N, K] float -> NVFP4.  ``search`` = number of e4m3 scale steps tried on each side."""
    n, k = w.shape
    wf = _pad_k(w.float())
    kp = wf.shape[1]
    amax_t = float(wf.abs().max())
    if tensor_scale is None:
        tensor_scale = amax_t / (6.0 * 448.0) if amax_t > 0 else 1.0
    if _kernels_ok(wf):
        ts = float(torch.tensor(tensor_scale, dtype=torch.float32))
        codes, scales = _kernel_quantize(wf.contiguous(), "nvfp4", k, kp, importance, search, ts)
        return QuantizedTensor("nvfp4", (n, k), kp, codes, scales, float(tensor_scale))
    blk = wf.reshape(n, kp // 16, 16)
    imp = None
    if importance is not None:
        imp = _pad_k(importance.float().reshape(1, -1)).reshape(1, kp // 16, 16).to(wf.device)
    base = blk.abs().amax(-1) / 6.0 / tensor_scale                      # ideal block scale in e4m3 units
    base_b = _to_e4m3_bytes(base).to(torch.int16)
    best_err = None
    best_sb = None
    best_q = None
    for step in range(-search, search + 1):
        sb = (base_b + step).clamp(0, 0x7E)                              # stay finite and non-negative
        s = _from_e4m3_bytes(sb.to(torch.uint8)) * tensor_scale
        s_safe = torch.where(s > 0, s, torch.ones_like(s))
        r = blk / s_safe[..., None]
        idx = _e2m1_index(r.abs())
        deq = _e2m1_value(idx) * torch.sign(r) * s[..., None]
        e = (deq - blk) ** 2
        if imp is not None:
            e = e * imp
        err = e.sum(-1)
        q = idx.to(torch.uint8) | ((r < 0).to(torch.uint8) << 3)
        q = torch.where(idx == 0, torch.zeros_like(q), q)                # no negative zero
        if best_err is None:
            best_err, best_sb, best_q = err, sb, q
        else:
            take = err < best_err
            best_err = torch.where(take, err, best_err)
            best_sb = torch.where(take, sb, best_sb)
            best_q = torch.where(take[..., None], q, best_q)
    q = best_q.reshape(n, kp)
    codes = (q[:, 0::2] | (q[:, 1::2] << 4)).contiguous()
    return QuantizedTensor("nvfp4", (n, k), kp, codes, best_sb.to(torch.uint8).contiguous(), float(tensor_scale))


def dequantize_nvfp4(q: QuantizedTensor) -> torch.Tensor:
    n, k = q.shape
    c = q.codes
    lo, hi = c & 0xF, c >> 4
    nib = torch.stack([lo, hi], -1).reshape(n, q.k_padded)
    mag = _e2m1_value(nib & 7)
    sign = torch.where((nib & 8) != 0, -1.0, 1.0)
    s = _from_e4m3_bytes(q.scales) * q.tensor_scale
    w = (mag * sign).reshape(n, q.k_padded // 16, 16) * s[..., None]
    return w.reshape(n, q.k_padded)[:, :k].contiguous()


def quantize_mxfp8(w: torch.Tensor, importance: Optional[torch.Tensor] = None, search: int = 1) -> QuantizedTensor:
    n, k = w.shape
    wf = _pad_k(w.float())
    kp = wf.shape[1]
    if _kernels_ok(wf):
        codes, scales = _kernel_quantize(wf.contiguous(), "mxfp8", k, kp, importance, search, 1.0)
        return QuantizedTensor("mxfp8", (n, k), kp, codes, scales, 1.0)
    blk = wf.reshape(n, kp // 32, 32)
    imp = None
    if importance is not None:
        imp = _pad_k(importance.float().reshape(1, -1)).reshape(1, kp // 32, 32).to(wf.device)
    amax = blk.abs().amax(-1)
    # ceil(log2(amax / 448)) in exact integer arithmetic (same as the C++ and CUDA quantisers)
    fm, fe = torch.frexp(torch.where(amax > 0, amax, torch.ones_like(amax)) / 448.0)
    e0 = torch.where(fm == 0.5, fe - 1, fe).to(wf.dtype)
    best_err = best_e = best_c = None
    for step in range(-search, search + 1):
        e = (e0 + step).clamp(-126, 127)
        s = torch.exp2(e)
        cb = _to_e4m3_bytes(blk / s[..., None])
        deq = _from_e4m3_bytes(cb) * s[..., None]
        er = (deq - blk) ** 2
        if imp is not None:
            er = er * imp
        err = er.sum(-1)
        if best_err is None:
            best_err, best_e, best_c = err, e, cb
        else:
            take = err < best_err
            best_err = torch.where(take, err, best_err)
            best_e = torch.where(take, e, best_e)
            best_c = torch.where(take[..., None], cb, best_c)
    scales = (best_e + 127).to(torch.uint8).contiguous()
    return QuantizedTensor("mxfp8", (n, k), kp, best_c.reshape(n, kp).contiguous(), scales, 1.0)


def dequantize_mxfp8(q: QuantizedTensor) -> torch.Tensor:
    n, k = q.shape
    s = torch.exp2(q.scales.float() - 127.0)
    w = _from_e4m3_bytes(q.codes).reshape(n, q.k_padded // 32, 32) * s[..., None]
    return w.reshape(n, q.k_padded)[:, :k].contiguous()


def quantize(w: torch.Tensor, fmt: str, importance: Optional[torch.Tensor] = None) -> QuantizedTensor:
    if fmt == "nvfp4":
        return quantize_nvfp4(w, importance, search=DEFAULT_SEARCH)
    if fmt == "mxfp8":
        return quantize_mxfp8(w, importance, search=min(DEFAULT_SEARCH, 1))
    if fmt == "bf16":
        n, k = w.shape
        return QuantizedTensor("bf16", (n, k), k, w.to(torch.bfloat16).contiguous(), None, 1.0)
    if fmt == "mxfp4":
        return quantize_mxfp4(w)
    if fmt == "fp8_block128":
        return quantize_fp8_block128(w)
    raise ValueError(f"unknown weight format {fmt!r}")


def quantize_mxfp4(w: torch.Tensor) -> QuantizedTensor:
    """OCP MXFP4: E2M1 codes with one power-of-two scale per 32 weights (scale = 2^(floor(log2(amax)) - 2))."""
    n, k = w.shape
    wf = _pad_k(w.float())
    kp = wf.shape[1]
    blk = wf.reshape(n, kp // 32, 32)
    amax = blk.abs().amax(-1)
    _, fe = torch.frexp(torch.where(amax > 0, amax, torch.ones_like(amax)))     # amax = f * 2^fe, f in [0.5, 1)
    e = (fe - 1 - 2).clamp(-127, 127)                                           # emax of E2M1 is 2
    r = blk / torch.exp2(e.float())[..., None]
    idx = _e2m1_index(r.abs())
    q = idx.to(torch.uint8) | ((r < 0).to(torch.uint8) << 3)
    q = torch.where(idx == 0, torch.zeros_like(q), q).reshape(n, kp)
    codes = (q[:, 0::2] | (q[:, 1::2] << 4)).contiguous()
    return QuantizedTensor("mxfp4", (n, k), kp, codes, (e + 127).to(torch.uint8).contiguous(), 1.0)


def dequantize_mxfp4(q: QuantizedTensor) -> torch.Tensor:
    n, k = q.shape
    c = q.codes
    nib = torch.stack([c & 0xF, c >> 4], -1).reshape(n, q.k_padded)
    v = _e2m1_value(nib & 7) * torch.where((nib & 8) != 0, -1.0, 1.0)
    s = torch.exp2(q.scales.float() - 127.0)
    return (v.reshape(n, q.k_padded // 32, 32) * s[..., None]).reshape(n, q.k_padded)[:, :k].contiguous()


def quantize_fp8_block128(w: torch.Tensor) -> QuantizedTensor:
    """E4M3 codes with one fp32 scale (amax / 448) per 128 x 128 block; `scales` is a float32 tensor."""
    n, k = w.shape
    kp = align_up(k, 128)
    npad = align_up(n, 128)
    wf = w.new_zeros(npad, kp, dtype=torch.float32)
    wf[:n, :k] = w.float()
    blk = wf.reshape(npad // 128, 128, kp // 128, 128)
    amax = blk.abs().amax(dim=(1, 3))
    s = torch.where(amax > 0, amax / 448.0, torch.ones_like(amax))
    codes = _to_e4m3_bytes(blk / s[:, None, :, None]).reshape(npad, kp)[:n].contiguous()
    return QuantizedTensor("fp8_block128", (n, k), kp, codes, s.contiguous(), 1.0)


def dequantize_fp8_block128(q: QuantizedTensor) -> torch.Tensor:
    n, k = q.shape
    s = q.scales.float().repeat_interleave(128, 0)[:n].repeat_interleave(128, 1)[:, :q.k_padded]
    return (_from_e4m3_bytes(q.codes) * s)[:, :k].contiguous()


def to_kernel_format(q: QuantizedTensor) -> QuantizedTensor:
    """Re-express an interchange-format tensor in a format the kernels execute (identity otherwise)."""
    if q.fmt == "mxfp4":
        # lossless: codes unchanged, scale 2^e per 32 -> the same UE4M3 byte for both 16-blocks, with a
        # power-of-two tensor scale chosen so every block exponent fits UE4M3's normal range [2^-6, 2^8]
        e = q.scales.to(torch.int32) - 127
        live = q.codes.reshape(q.shape[0], -1, 16).ne(0).any(-1)                # all-zero blocks may take any scale
        t = int(e[live].max()) - 8 if bool(live.any()) else 0
        rel = (e - t).clamp(min=-6)
        if bool((rel[live] < -6).any()):
            return quantize_nvfp4(dequantize_mxfp4(q), search=DEFAULT_SEARCH)   # range too wide: re-quantise
        sb = ((rel + 7) << 3).to(torch.uint8)                                   # e4m3 byte of 2^rel (mantissa 0)
        return QuantizedTensor("nvfp4", q.shape, q.k_padded, q.codes, sb.repeat_interleave(2, 1).contiguous(), float(2.0 ** t))
    if q.fmt == "fp8_block128":
        return quantize_mxfp8(dequantize_fp8_block128(q), search=min(DEFAULT_SEARCH, 1))
    return q


def dequantize(q: QuantizedTensor) -> torch.Tensor:
    if q.fmt == "nvfp4":
        return dequantize_nvfp4(q)
    if q.fmt == "mxfp8":
        return dequantize_mxfp8(q)
    if q.fmt == "mxfp4":
        return dequantize_mxfp4(q)
    if q.fmt == "fp8_block128":
        return dequantize_fp8_block128(q)
    return q.codes.float()[:, :q.shape[1]]


def bits_per_weight(fmt: str) -> float:
    return {"bf16": 16.0, "nvfp4": 4.5, "mxfp8": 8.25, "mxfp4": 4.25, "fp8_block128": 8.002}[fmt]
