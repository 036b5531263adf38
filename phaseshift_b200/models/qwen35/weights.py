"""Qwen3.5 weights: HF tensor names, random initialisation, and the engine's fused layout.

HF names follow the reference's binder (src/phaseshift/models/qwen35/weights/model_weights.cpp:24-35,
177-225,322-340).  ``build_engine_weights`` turns HF tensors into what the kernels consume:

* GDN layer: ``in_proj`` = rows [q | k | v | z] of in_proj_qkv + in_proj_z (one projection, one
  launch), ``ba_proj`` = rows [b | a] kept in BF16 ("GDN-small" tensors stay BF16 in the reference's
  preset, src/phaseshift/quantization/fpx/profile.cpp:96-128), conv taps, A_log, dt_bias, head norm,
  ``out_proj``.
* Attention layer: ``qkv_proj`` = rows [q_proj (per head q|gate) | k_proj | v_proj], ``o_proj``.
* MLP: ``gate_up`` with rows interleaved (gate_0, up_0, gate_1, up_1, ...) so SwiGLU is a GEMV/GEMM
  epilogue; ``down``.

Tensor parallelism slices the HF tensors *before* fusing and quantising (partition, then layout), the
ordering the reference requires in docs/developer/tensor_partition.md:129-183.
"""
from __future__ import annotations

import zlib
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional

import torch

from ...quant.formats import QuantizedTensor, dequantize, quantize, to_kernel_format
from .config import Qwen35Config

P = "model.language_model."


def hf_tensor_shapes(cfg: Qwen35Config) -> Dict[str, tuple]:
    h, i = cfg.hidden_size, cfg.intermediate_size
    s = {P + "embed_tokens.weight": (cfg.vocab_size, h), P + "norm.weight": (h,)}
    if not cfg.tie_word_embeddings:
        s[P + "lm_head.weight"] = (cfg.vocab_size, h)
    for l, lt in enumerate(cfg.layer_types):
        lp = f"{P}layers.{l}."
        s[lp + "input_layernorm.weight"] = (h,)
        s[lp + "post_attention_layernorm.weight"] = (h,)
        s[lp + "mlp.gate_proj.weight"] = (i, h)
        s[lp + "mlp.up_proj.weight"] = (i, h)
        s[lp + "mlp.down_proj.weight"] = (h, i)
        if lt == 0:
            a = lp + "linear_attn."
            s[a + "in_proj_qkv.weight"] = (cfg.gdn_conv_dim, h)
            s[a + "in_proj_z.weight"] = (cfg.gdn_v_dim, h)
            s[a + "in_proj_b.weight"] = (cfg.linear_num_value_heads, h)
            s[a + "in_proj_a.weight"] = (cfg.linear_num_value_heads, h)
            s[a + "conv1d.weight"] = (cfg.gdn_conv_dim, 1, 4)
            s[a + "norm.weight"] = (cfg.linear_value_head_dim,)
            s[a + "dt_bias"] = (cfg.linear_num_value_heads,)
            s[a + "A_log"] = (cfg.linear_num_value_heads,)
            s[a + "out_proj.weight"] = (h, cfg.gdn_v_dim)
        else:
            a = lp + "self_attn."
            s[a + "q_proj.weight"] = (2 * cfg.attn_q_dim, h)
            s[a + "k_proj.weight"] = (cfg.attn_kv_dim, h)
            s[a + "v_proj.weight"] = (cfg.attn_kv_dim, h)
            s[a + "o_proj.weight"] = (h, cfg.attn_q_dim)
            s[a + "q_norm.weight"] = (cfg.head_dim,)
            s[a + "k_norm.weight"] = (cfg.head_dim,)
    return s


def random_tensor(name: str, shape: tuple, seed: int, device="cpu", std: float = 0.02) -> torch.Tensor:
    """Deterministic per-tensor init: matrices N(0, std); norm weights small; A_log/dt_bias in a sane
    range.  Values are rounded to bf16 so every backend starts from identical numbers."""
    g = torch.Generator(device=device)
    g.manual_seed((seed * 1000003 + zlib.crc32(name.encode())) & 0x7FFFFFFF)
    if name.endswith("A_log"):
        t = torch.empty(shape, device=device).uniform_(-2.0, 1.0, generator=g)
    elif name.endswith("dt_bias"):
        t = torch.empty(shape, device=device).uniform_(-1.0, 1.0, generator=g)
    elif name.endswith("conv1d.weight"):
        t = torch.randn(shape, device=device, generator=g) * 0.3
    elif name.endswith("norm.weight") or name.endswith("layernorm.weight"):
        t = torch.randn(shape, device=device, generator=g) * 0.05
        if name.endswith("linear_attn.norm.weight"):
            t = t + 1.0        # direct (not 1+w) scale
    else:
        t = torch.randn(shape, device=device, generator=g) * std
    return t.to(torch.bfloat16)


def random_hf_weights(cfg: Qwen35Config, seed: int = 0, device="cpu") -> Dict[str, torch.Tensor]:
    return {n: random_tensor(n, s, seed, device) for n, s in hf_tensor_shapes(cfg).items()}


def random_getter(cfg: Qwen35Config, seed: int = 0, device="cpu") -> Callable[[str], torch.Tensor]:
    shapes = hf_tensor_shapes(cfg)
    return lambda name: random_tensor(name, shapes[name], seed, device)


# ----------------------------------------------------------------------------------------------
# engine-side containers


@dataclass
class LinearW:
    """One projection.  ``q`` is the canonical row-major payload (what files store, what the CPU ops and
    dequantisation use); ``tiled`` is the kernel-side layout built from it on a CUDA device
    (quant/tiling.py).  ``drop_canonical()`` frees ``q``'s device tensors once ``tiled`` exists."""
    q: QuantizedTensor
    _deq: Optional[torch.Tensor] = None
    tiled: Optional[torch.Tensor] = None
    _shape: Optional[tuple] = None
    _kpad: int = 0
    _fmt: str = ""
    _tscale: float = 1.0
    sf_atoms: Optional[torch.Tensor] = None    # block scales in the tensor-core layout (quant/act_quant.pack_sf_atoms)
    codes: Optional[torch.Tensor] = None       # canonical code matrix kept for the tensor-core path (TMA reads it as is)
    act_scale: float = 0.0                     # fixed NVFP4 activation scale of this projection's input site

    def __post_init__(self):
        self._shape, self._kpad, self._fmt, self._tscale = self.q.shape, self.q.k_padded, self.q.fmt, self.q.tensor_scale
        if self.act_scale <= 0.0:
            from ...quant.act_quant import DEFAULT_ACT_SCALE
            self.act_scale = DEFAULT_ACT_SCALE

    def make_umma(self, keep_canonical: bool = True) -> "LinearW":
        """Prepare the block-scaled tensor-core operands: the code matrix stays canonical (row-major; the TMA
        tile load swizzles it on the fly), the block scales are re-laid into 512-byte atoms once."""
        if self._fmt not in ("nvfp4", "mxfp8"):
            raise ValueError("only block-quantised projections have tensor-core operands")
        if self.sf_atoms is None:
            from ...quant.act_quant import pack_sf_atoms
            self.codes = self.q.codes.contiguous()
            self.sf_atoms = pack_sf_atoms(self.q.scales, self._fmt, self._kpad)
        if not keep_canonical:
            self.q = None
        return self

    def make_tiled(self, keep_canonical: bool = True) -> "LinearW":
        from ...quant.tiling import tile_weight
        if self.tiled is None:
            self.tiled = tile_weight(self.q)
        if not keep_canonical:
            self.q = None
        return self

    @property
    def rowmajor_bf16(self) -> Optional[torch.Tensor]:
        """bf16 weights in plain row-major form [N, k_padded] (the canonical payload, when it is still resident):
        what the bf16 tensor-core GEMMs read through TMA.  None for block-quantised weights."""
        if self._fmt == "bf16" and self.q is not None and self.q.codes.is_cuda:
            return self.q.codes
        return None

    @property
    def N(self) -> int:
        return self._shape[0]

    @property
    def K(self) -> int:
        return self._shape[1]

    @property
    def k_padded(self) -> int:
        return self._kpad

    @property
    def fmt(self) -> str:
        return self._fmt

    @property
    def tensor_scale(self) -> float:
        return self._tscale

    @property
    def nbytes(self) -> int:
        if self.tiled is not None:
            return self.tiled.numel()          # also with both layouts resident: what a single-row step streams
        if self.sf_atoms is not None:
            # what a step streams: codes + one scale byte per block (atom padding is not read for real rows)
            return self.codes.numel() * self.codes.element_size() + self.N * (self._kpad // (16 if self._fmt == "nvfp4" else 32))
        return self.q.nbytes

    def dense(self) -> torch.Tensor:
        """fp32 [N, K] (dequantised); cached, used by the CPU/reference ops."""
        if self._deq is None:
            q = self.q
            if q is None and self.tiled is None and self.sf_atoms is not None:
                from ...quant.act_quant import unpack_sf_atoms
                nb = self._kpad // (16 if self._fmt == "nvfp4" else 32)
                q = QuantizedTensor(self._fmt, self._shape, self._kpad, self.codes,
                                    unpack_sf_atoms(self.sf_atoms, self._shape[0], nb), self._tscale)
            elif q is None:
                from ...quant.tiling import untile_weight
                q = untile_weight(self.tiled, self._fmt, self._shape[0], self._kpad)
                q.tensor_scale = self._tscale
                q.shape = self._shape
            self._deq = dequantize(q)
        return self._deq


@dataclass
class GdnW:
    in_proj: LinearW
    ba_proj: LinearW
    conv_w: torch.Tensor      # [local_conv_dim, 4] bf16
    A_log: torch.Tensor       # [Hv_local] f32
    dt_bias: torch.Tensor     # [Hv_local] f32
    norm_w: torch.Tensor      # [Dv] bf16
    out_proj: LinearW


@dataclass
class AttnW:
    qkv_proj: LinearW
    q_norm: torch.Tensor
    k_norm: torch.Tensor
    o_proj: LinearW


@dataclass
class LayerW:
    kind: int
    input_norm: torch.Tensor
    mixer: object
    post_norm: torch.Tensor
    gate_up: LinearW
    down: LinearW


@dataclass
class EngineWeights:
    cfg: Qwen35Config
    embed: LinearW                    # table [vocab, H]: bf16 or mxfp8
    layers: List[LayerW]
    final_norm: torch.Tensor
    lm_head: LinearW
    tp_rank: int = 0
    tp_size: int = 1
    preset: str = "bf16"
    layout: str = "canonical"

    def weight_bytes(self) -> int:
        n = self.embed.nbytes + self.lm_head.nbytes
        for l in self.layers:
            n += l.gate_up.nbytes + l.down.nbytes
            m = l.mixer
            if l.kind == 0:
                n += m.in_proj.nbytes + m.ba_proj.nbytes + m.out_proj.nbytes
            else:
                n += m.qkv_proj.nbytes + m.o_proj.nbytes
        return n

    def linears(self) -> List[LinearW]:
        """Every projection a step multiplies by (the embedding table is a gather, not a projection)."""
        out = [self.lm_head]
        for l in self.layers:
            m = l.mixer
            out += [l.gate_up, l.down] + ([m.in_proj, m.ba_proj, m.out_proj] if l.kind == 0 else [m.qkv_proj, m.o_proj])
        return out

    def decode_read_bytes(self) -> int:
        """Weight bytes one decode step must stream from HBM (everything except the embedding table)."""
        return self.weight_bytes() - self.embed.nbytes


# role -> format.  "nvfp4" mirrors the reference's `psq` preset with NVFP4 for PSQ4 and MXFP8 for PSQ8
# (src/phaseshift/quantization/fpx/profile.cpp:7-47,96-128).
def format_for(preset: str, role: str, layer: int) -> str:
    if preset == "bf16":
        return "bf16"
    if preset == "mxfp8":
        return "bf16" if role in ("gdn_small",) else "mxfp8"
    if preset == "nvfp4":
        if role in ("embed", "lm_head"):
            return "mxfp8"
        if role == "gdn_small":
            return "bf16"
        if role in ("ffn_down", "gdn_qkvz", "gdn_out"):
            return "mxfp8" if layer % 4 == 0 else "nvfp4"
        return "nvfp4"
    if preset in ("mxfp4", "fp8_block128"):
        # interchange presets: big projections in the named format (re-expressed for the kernels at load),
        # vocabulary matrices in MXFP8, the small GDN projections in BF16
        if role in ("embed", "lm_head"):
            return "mxfp8"
        return "bf16" if role == "gdn_small" else preset
    raise ValueError(f"unknown preset {preset!r}")


@dataclass
class TpGeometry:
    """Rank-local head geometry (reference: src/phaseshift/models/qwen35/model/tensor_parallel_context.cpp:16-65,
    generalised to tp in {1,2,4,8} with KV-head replication when tp > num_key_value_heads)."""
    tp_rank: int
    tp_size: int
    q_heads: range
    kv_heads: range
    gdn_k_heads: range
    gdn_v_heads: range
    inter: range

    @staticmethod
    def make(cfg: Qwen35Config, tp_rank: int, tp_size: int) -> "TpGeometry":
        def split(n, what):
            if n % tp_size:
                raise ValueError(f"{what}={n} is not divisible by tp_size={tp_size}")
            c = n // tp_size
            return range(tp_rank * c, (tp_rank + 1) * c)
        q = split(cfg.num_attention_heads, "num_attention_heads")
        if cfg.num_key_value_heads % tp_size == 0:
            kv = split(cfg.num_key_value_heads, "num_key_value_heads")
        else:
            if tp_size % cfg.num_key_value_heads:
                raise ValueError("tp_size must divide or be a multiple of num_key_value_heads")
            group = cfg.num_attention_heads // cfg.num_key_value_heads
            first = q.start // group
            if (q.stop - 1) // group != first:
                raise ValueError("a rank's query heads would span two KV heads")
            kv = range(first, first + 1)        # replicated KV head
        return TpGeometry(tp_rank, tp_size, q, kv, split(cfg.linear_num_key_heads, "linear_num_key_heads"),
                          split(cfg.linear_num_value_heads, "linear_num_value_heads"),
                          split(cfg.intermediate_size, "intermediate_size"))


def _rows(t: torch.Tensor, heads: range, dim: int) -> torch.Tensor:
    return t[heads.start * dim: heads.stop * dim]


class DenseSource:
    """Weights given as full-precision HF tensors; projections are quantised here according to the preset."""

    def __init__(self, get: Callable[[str], torch.Tensor], preset: str, device,
                 importance: Optional[Callable[[str], Optional[torch.Tensor]]] = None):
        self.get, self.preset, self.device, self.importance = get, preset, device, importance

    def tensor(self, name: str) -> torch.Tensor:
        return self.get(name)

    def linear(self, parts, role: str, layer: int, interleave: bool = False) -> QuantizedTensor:
        """parts: [(hf_name, row_range | None, k_range | None)] concatenated along rows."""
        ws = []
        for (name, rr, kr) in parts:
            w = self.get(name)
            if w.dim() > 2:
                w = w.reshape(w.shape[0], -1)
            if rr is not None:
                w = w[rr.start:rr.stop]
            if kr is not None:
                w = w[:, kr.start:kr.stop]
            ws.append(w)
        if interleave:
            w = torch.stack(ws, 1).reshape(len(ws) * ws[0].shape[0], ws[0].shape[1])
        else:
            w = torch.cat(ws, 0) if len(ws) > 1 else ws[0]
        fmt = format_for(self.preset, role, layer)
        imp = self.importance(parts[0][0]) if self.importance is not None else None
        if imp is not None and parts[0][2] is not None:
            imp = imp[parts[0][2].start:parts[0][2].stop]
        return to_kernel_format(quantize(w.to(self.device), fmt, imp))


class QuantizedSource:
    """Weights read from a quantised model directory: canonical payloads are sliced and concatenated as
    stored (never re-quantised).  K ranges must fall on block boundaries (reference rule:
    docs/developer/tensor_partition.md:60-127)."""

    def __init__(self, collection, manifest, device):
        self.col, self.man, self.device = collection, manifest, device
        self.entries = manifest.by_name()

    def tensor(self, name: str) -> torch.Tensor:
        name = self.man.aliases.get(name, name)
        e = self.entries[name]
        if e.encoding != "bf16":
            raise ValueError(f"{name} is stored as {e.encoding}, expected a plain bf16 tensor")
        return self.col.tensor(e.data)

    def _payload(self, name: str):
        name = self.man.aliases.get(name, name)
        e = self.entries[name]
        if e.encoding == "bf16":
            return e, self.col.tensor(e.data).reshape(e.logical_shape[0], -1), None
        return e, self.col.tensor(e.codes), self.col.tensor(e.metadata1)

    def linear(self, parts, role: str, layer: int, interleave: bool = False) -> QuantizedTensor:
        codes, scales, fmt, tscale, k_log = [], [], None, None, None
        for (name, rr, kr) in parts:
            e, c, sc = self._payload(name)
            if fmt is None:
                fmt, tscale = e.encoding, (e.metadata2 if e.metadata2 is not None else 1.0)
            elif e.encoding != fmt or abs((e.metadata2 or 1.0) - tscale) > 1e-12 * max(1.0, abs(tscale)):
                raise ValueError(f"tensors fused into one projection must share encoding and tensor scale ({name})")
            k = e.logical_shape[1]
            if rr is not None:
                c = c[rr.start:rr.stop]
                sc = None if sc is None else sc[rr.start:rr.stop]
            if kr is not None:
                blk = {"bf16": 1, "nvfp4": 32, "mxfp8": 32, "mxfp4": 32}[fmt]
                if kr.start % blk or kr.stop % blk:
                    raise ValueError(f"K range {kr} of {name} is not aligned to {blk}")
                if fmt == "nvfp4":
                    c, sc = c[:, kr.start // 2:kr.stop // 2], sc[:, kr.start // 16:kr.stop // 16]
                elif fmt == "mxfp8":
                    c, sc = c[:, kr.start:kr.stop], sc[:, kr.start // 32:kr.stop // 32]
                elif fmt == "mxfp4":
                    c, sc = c[:, kr.start // 2:kr.stop // 2], sc[:, kr.start // 32:kr.stop // 32]
                else:
                    c = c[:, kr.start:kr.stop]
                k = kr.stop - kr.start
            k_log = k
            codes.append(c)
            scales.append(sc)
        if interleave:
            cat = lambda xs: torch.stack(xs, 1).reshape(len(xs) * xs[0].shape[0], xs[0].shape[1])
        else:
            cat = lambda xs: torch.cat(xs, 0) if len(xs) > 1 else xs[0]
        c = cat(codes).contiguous().to(self.device)
        sc = None if scales[0] is None else cat(scales).contiguous().to(self.device)
        n = c.shape[0]
        if fmt not in ("bf16", "nvfp4", "mxfp8", "mxfp4"):
            raise ValueError(f"{parts[0][0]}: encoding {fmt!r} cannot be loaded from a model directory")
        kp = {"bf16": c.shape[1], "nvfp4": c.shape[1] * 2, "mxfp8": c.shape[1], "mxfp4": c.shape[1] * 2}[fmt]
        return to_kernel_format(QuantizedTensor(fmt, (n, k_log), kp, c, sc, float(tscale)))


def build_engine_weights(cfg: Qwen35Config, get, preset: str = "bf16", device="cpu", tp_rank: int = 0,
                         tp_size: int = 1, importance: Optional[Callable[[str], Optional[torch.Tensor]]] = None,
                         keep_canonical: bool = True, layout: Optional[str] = None) -> EngineWeights:
    """Build the engine's fused, (optionally) quantised and tiled weights for one tensor-parallel rank.

    ``get`` is either a callable ``name -> full HF tensor`` (weights are quantised here per ``preset``) or
    a source object (``DenseSource`` / ``QuantizedSource``).  Work proceeds one layer at a time so a 27B
    model never needs more than one layer of BF16 weights resident.

    ``layout`` picks the kernel-side form of block-quantised projections on a CUDA device: ``"tc"`` (default;
    canonical codes + scale atoms for the block-scaled tensor-core kernel, activations quantised to the weights'
    block format), ``"stream"`` (quad-tiled blocks for the CUDA-core streaming kernel, bf16 activations) or
    ``"both"`` (either kernel can run: single-row decode streams, everything else uses the tensor cores; costs a
    second copy of the block codes).
    The ``PS_LINEAR_LAYOUT`` environment variable overrides the default."""
    import os
    layout = layout or os.environ.get("PS_LINEAR_LAYOUT", "tc")
    if layout not in ("tc", "stream", "both"):
        raise ValueError(f"unknown linear layout {layout!r}")
    src = get if hasattr(get, "linear") else DenseSource(get, preset, device, importance)
    geo = TpGeometry.make(cfg, tp_rank, tp_size)
    Dk, Dv, D = cfg.linear_key_head_dim, cfg.linear_value_head_dim, cfg.head_dim
    qk = cfg.gdn_qk_dim
    on_cuda = torch.device(device).type == "cuda"

    def lin(parts, role: str, layer: int, interleave: bool = False) -> LinearW:
        lw = LinearW(src.linear(parts, role, layer, interleave))
        if on_cuda and role != "embed":
            if layout in ("tc", "both") and lw.fmt in ("nvfp4", "mxfp8"):
                if layout == "both":
                    lw.make_tiled(True)
                lw.make_umma(keep_canonical)
            else:
                # the GDN kernel reads b/a rows row-major; bf16 matrices keep their row-major form for the tensor-core GEMMs
                lw.make_tiled(keep_canonical or role == "gdn_small" or (lw.fmt == "bf16" and layout != "stream"))
        return lw

    def dev(t: torch.Tensor, dtype=torch.bfloat16) -> torch.Tensor:
        return t.to(device=device, dtype=dtype).contiguous()

    def hr(heads: range, dim: int, base: int = 0) -> range:
        return range(base + heads.start * dim, base + heads.stop * dim)

    layers = []
    for l, lt in enumerate(cfg.layer_types):
        lp = f"{P}layers.{l}."
        if lt == 0:
            a = lp + "linear_attn."
            kh, vh = geo.gdn_k_heads, geo.gdn_v_heads
            in_proj = lin([(a + "in_proj_qkv.weight", hr(kh, Dk), None), (a + "in_proj_qkv.weight", hr(kh, Dk, qk), None),
                           (a + "in_proj_qkv.weight", hr(vh, Dv, 2 * qk), None), (a + "in_proj_z.weight", hr(vh, Dv), None)],
                          "gdn_qkvz", l)
            ba = lin([(a + "in_proj_b.weight", hr(vh, 1), None), (a + "in_proj_a.weight", hr(vh, 1), None)], "gdn_small", l)
            cw = src.tensor(a + "conv1d.weight").reshape(cfg.gdn_conv_dim, 4)
            cw = torch.cat([_rows(cw[:qk], kh, Dk), _rows(cw[qk:2 * qk], kh, Dk), _rows(cw[2 * qk:], vh, Dv)], 0)
            out_proj = lin([(a + "out_proj.weight", None, hr(vh, Dv))], "gdn_out", l)
            mixer = GdnW(in_proj, ba, dev(cw), dev(_rows(src.tensor(a + "A_log"), vh, 1), torch.float32),
                         dev(_rows(src.tensor(a + "dt_bias"), vh, 1), torch.float32), dev(src.tensor(a + "norm.weight")),
                         out_proj)
        else:
            a = lp + "self_attn."
            qkv = lin([(a + "q_proj.weight", hr(geo.q_heads, 2 * D), None), (a + "k_proj.weight", hr(geo.kv_heads, D), None),
                       (a + "v_proj.weight", hr(geo.kv_heads, D), None)], "attn_qkv", l)
            o_proj = lin([(a + "o_proj.weight", None, hr(geo.q_heads, D))], "attn_o", l)
            mixer = AttnW(qkv, dev(src.tensor(a + "q_norm.weight")), dev(src.tensor(a + "k_norm.weight")), o_proj)
        gu = lin([(lp + "mlp.gate_proj.weight", geo.inter, None), (lp + "mlp.up_proj.weight", geo.inter, None)],
                 "ffn_gate_up", l, interleave=True)
        down = lin([(lp + "mlp.down_proj.weight", None, geo.inter)], "ffn_down", l)
        layers.append(LayerW(lt, dev(src.tensor(lp + "input_layernorm.weight")), mixer,
                             dev(src.tensor(lp + "post_attention_layernorm.weight")), gu, down))
    embed = lin([(P + "embed_tokens.weight", None, None)], "embed", 0)
    if cfg.tie_word_embeddings:
        lm_head = LinearW(embed.q)
        if on_cuda:
            if layout in ("tc", "both") and lm_head.fmt in ("nvfp4", "mxfp8"):
                if layout == "both":
                    lm_head.make_tiled(True)
                lm_head.make_umma(True)
            else:
                lm_head.make_tiled(True)
    else:
        lm_head = lin([(P + "lm_head.weight", None, None)], "lm_head", 0)
    ew = EngineWeights(cfg, embed, layers, dev(src.tensor(P + "norm.weight")), lm_head, tp_rank, tp_size, preset)
    ew.layout = layout if on_cuda else "canonical"
    return ew


# Tensors that are fused into one projection and must therefore share an NVFP4 per-tensor scale.
def scale_groups(cfg: Qwen35Config) -> List[List[str]]:
    groups = []
    for l, lt in enumerate(cfg.layer_types):
        lp = f"{P}layers.{l}."
        groups.append([lp + "mlp.gate_proj.weight", lp + "mlp.up_proj.weight"])
        if lt == 0:
            groups.append([lp + "linear_attn.in_proj_qkv.weight", lp + "linear_attn.in_proj_z.weight"])
        else:
            a = lp + "self_attn."
            groups.append([a + "q_proj.weight", a + "k_proj.weight", a + "v_proj.weight"])
    return groups


def load_engine_weights(model_dir, device="cpu", preset: Optional[str] = None, tp_rank: int = 0, tp_size: int = 1,
                        keep_canonical: bool = True, verify_weights: bool = False,
                        layout: Optional[str] = None) -> EngineWeights:
    """Load a model directory: quantised (manifest present, auto-detected) or plain BF16 (quantised on the
    fly when ``preset`` asks for it)."""
    from ...io.model_dir import ShardCollection, is_quantized_dir
    from ...quant.manifest import Manifest
    cfg = Qwen35Config.from_dir(model_dir)
    col = ShardCollection(model_dir)
    if is_quantized_dir(model_dir):
        man = Manifest.load(model_dir)
        if verify_weights:
            from ...quant.offline import verify_crc
            verify_crc(col, man)
        src = QuantizedSource(col, man, device)
        return build_engine_weights(cfg, src, man.preset, device, tp_rank, tp_size, keep_canonical=keep_canonical,
                                    layout=layout)
    return build_engine_weights(cfg, lambda n: col.tensor(n), preset or "bf16", device, tp_rank, tp_size,
                                keep_canonical=keep_canonical, layout=layout)
