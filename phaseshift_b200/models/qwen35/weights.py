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

from ...quant.formats import QuantizedTensor, dequantize, quantize
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

    def __post_init__(self):
        self._shape, self._kpad, self._fmt, self._tscale = self.q.shape, self.q.k_padded, self.q.fmt, self.q.tensor_scale

    def make_tiled(self, keep_canonical: bool = True) -> "LinearW":
        from ...quant.tiling import tile_weight
        if self.tiled is None:
            self.tiled = tile_weight(self.q)
        if not keep_canonical:
            self.q = None
        return self

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
            return self.tiled.numel()
        return self.q.nbytes

    def dense(self) -> torch.Tensor:
        """fp32 [N, K] (dequantised); cached, used by the CPU/reference ops."""
        if self._deq is None:
            q = self.q
            if q is None:
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


def build_engine_weights(cfg: Qwen35Config, get: Callable[[str], torch.Tensor], preset: str = "bf16",
                         device="cpu", tp_rank: int = 0, tp_size: int = 1,
                         importance: Optional[Callable[[str], Optional[torch.Tensor]]] = None,
                         keep_canonical: bool = True) -> EngineWeights:
    """``get(name)`` returns the full HF tensor; slicing, fusing and quantisation happen here, one layer
    at a time so a 27B model never needs more than one layer of BF16 weights resident."""
    geo = TpGeometry.make(cfg, tp_rank, tp_size)
    Dk, Dv, D = cfg.linear_key_head_dim, cfg.linear_value_head_dim, cfg.head_dim
    qk = cfg.gdn_qk_dim

    def lin(w: torch.Tensor, role: str, layer: int, name: str = "") -> LinearW:
        fmt = format_for(preset, role, layer)
        imp = importance(name) if (importance is not None and name) else None
        lw = LinearW(quantize(w.to(device), fmt, imp))
        if torch.device(device).type == "cuda" and role != "embed":
            lw.make_tiled(keep_canonical or role == "gdn_small")   # the GDN kernel reads b/a rows row-major
        return lw

    def dev(t: torch.Tensor, dtype=torch.bfloat16) -> torch.Tensor:
        return t.to(device=device, dtype=dtype).contiguous()

    layers = []
    for l, lt in enumerate(cfg.layer_types):
        lp = f"{P}layers.{l}."
        if lt == 0:
            a = lp + "linear_attn."
            qkv = get(a + "in_proj_qkv.weight")
            wq, wk, wv = qkv[:qk], qkv[qk:2 * qk], qkv[2 * qk:]
            seg = [_rows(wq, geo.gdn_k_heads, Dk), _rows(wk, geo.gdn_k_heads, Dk), _rows(wv, geo.gdn_v_heads, Dv),
                   _rows(get(a + "in_proj_z.weight"), geo.gdn_v_heads, Dv)]
            in_proj = lin(torch.cat(seg, 0), "gdn_qkvz", l, a + "in_proj_qkv.weight")
            ba = torch.cat([_rows(get(a + "in_proj_b.weight"), geo.gdn_v_heads, 1),
                            _rows(get(a + "in_proj_a.weight"), geo.gdn_v_heads, 1)], 0)
            cw = get(a + "conv1d.weight").reshape(cfg.gdn_conv_dim, 4)
            cw = torch.cat([_rows(cw[:qk], geo.gdn_k_heads, Dk), _rows(cw[qk:2 * qk], geo.gdn_k_heads, Dk),
                            _rows(cw[2 * qk:], geo.gdn_v_heads, Dv)], 0)
            out_w = get(a + "out_proj.weight")[:, geo.gdn_v_heads.start * Dv: geo.gdn_v_heads.stop * Dv]
            mixer = GdnW(in_proj, lin(ba, "gdn_small", l), dev(cw),
                         dev(_rows(get(a + "A_log"), geo.gdn_v_heads, 1), torch.float32),
                         dev(_rows(get(a + "dt_bias"), geo.gdn_v_heads, 1), torch.float32),
                         dev(get(a + "norm.weight")), lin(out_w, "gdn_out", l, a + "out_proj.weight"))
        else:
            a = lp + "self_attn."
            wq = _rows(get(a + "q_proj.weight"), geo.q_heads, 2 * D)
            wk = _rows(get(a + "k_proj.weight"), geo.kv_heads, D)
            wv = _rows(get(a + "v_proj.weight"), geo.kv_heads, D)
            o_w = get(a + "o_proj.weight")[:, geo.q_heads.start * D: geo.q_heads.stop * D]
            mixer = AttnW(lin(torch.cat([wq, wk, wv], 0), "attn_qkv", l, a + "q_proj.weight"),
                          dev(get(a + "q_norm.weight")), dev(get(a + "k_norm.weight")),
                          lin(o_w, "attn_o", l, a + "o_proj.weight"))
        g = get(lp + "mlp.gate_proj.weight")[geo.inter.start: geo.inter.stop]
        u = get(lp + "mlp.up_proj.weight")[geo.inter.start: geo.inter.stop]
        gu = torch.stack([g, u], 1).reshape(2 * g.shape[0], g.shape[1])
        down = get(lp + "mlp.down_proj.weight")[:, geo.inter.start: geo.inter.stop]
        layers.append(LayerW(lt, dev(get(lp + "input_layernorm.weight")), mixer,
                             dev(get(lp + "post_attention_layernorm.weight")),
                             lin(gu, "ffn_gate_up", l, lp + "mlp.gate_proj.weight"),
                             lin(down, "ffn_down", l, lp + "mlp.down_proj.weight")))
    embed_w = get(P + "embed_tokens.weight")
    embed = lin(embed_w, "embed", 0)
    if cfg.tie_word_embeddings:
        lm_head = LinearW(embed.q)
        if torch.device(device).type == "cuda":
            lm_head.make_tiled(True)
    else:
        lm_head = lin(get(P + "lm_head.weight"), "lm_head", 0, P + "lm_head.weight")
    return EngineWeights(cfg, embed, layers, dev(get(P + "norm.weight")), lm_head, tp_rank, tp_size, preset)
