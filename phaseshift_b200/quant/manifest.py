"""Quantised-model manifest ``phaseshift_quantization.json`` and the role -> encoding profile.

Same container idea as the reference (include/phaseshift/quantization/fpx/quantized_manifest.h:11-84,
docs/developer/psq_canonical_soa_payload.md:93-149): every logical tensor becomes independent
structure-of-arrays tensors ``<name>.__phaseshift_codes`` and ``<name>.__phaseshift_metadata1`` (block
scales); NVFP4 also records its fp32 per-tensor scale in the manifest entry (``metadata2``).  BF16
tensors keep a plain ``data`` reference.  Each entry carries role, encoding, layout, logical shape,
padded K and a CRC32 per stored tensor so ``verify`` can detect corruption.
"""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Dict, List, Optional

FORMAT = "phaseshift-b200-safetensors"
FORMAT_VERSION = 1
CODES = ".__phaseshift_codes"
META1 = ".__phaseshift_metadata1"

ROLES = ("embed", "lm_head", "norm", "gdn_small", "attn_qkv", "attn_o", "ffn_gate_up", "ffn_down", "gdn_qkvz",
         "gdn_out", "dflash_linear", "dflash_small", "other")


@dataclass
class TensorEntry:
    name: str
    role: str
    encoding: str                 # bf16 | nvfp4 | mxfp8
    layout: str                   # "row_major_k_contiguous"
    logical_shape: List[int]
    k_padded: int
    codes: Optional[str] = None   # stored tensor names
    metadata1: Optional[str] = None
    metadata2: Optional[float] = None     # NVFP4 per-tensor scale
    data: Optional[str] = None    # bf16 tensors
    crc32: Dict[str, int] = field(default_factory=dict)


@dataclass
class Manifest:
    format: str = FORMAT
    format_version: int = FORMAT_VERSION
    preset: str = "nvfp4"
    source_fingerprint: str = ""
    imatrix: Optional[dict] = None
    aliases: Dict[str, str] = field(default_factory=dict)     # e.g. tied lm_head -> embed_tokens
    tensors: List[TensorEntry] = field(default_factory=list)

    def save(self, model_dir) -> None:
        d = asdict(self)
        (Path(model_dir) / "phaseshift_quantization.json").write_text(json.dumps(d, indent=1))

    @staticmethod
    def load(model_dir) -> "Manifest":
        raw = json.loads((Path(model_dir) / "phaseshift_quantization.json").read_text())
        if raw.get("format") != FORMAT:
            raise ValueError(f"not a {FORMAT} manifest: {raw.get('format')!r}")
        if raw.get("format_version") != FORMAT_VERSION:
            raise ValueError(f"unsupported manifest version {raw.get('format_version')}")
        ts = [TensorEntry(**t) for t in raw.pop("tensors")]
        m = Manifest(**{k: v for k, v in raw.items() if k != "tensors"})
        m.tensors = ts
        return m

    def by_name(self) -> Dict[str, TensorEntry]:
        return {t.name: t for t in self.tensors}


def classify_qwen35(name: str) -> str:
    """HF tensor name -> role (reference: src/phaseshift/quantization/offline/qwen35_adapter.cpp)."""
    if name.endswith("embed_tokens.weight"):
        return "embed"
    if name.endswith("lm_head.weight"):
        return "lm_head"
    if "linear_attn" in name:
        if name.endswith("in_proj_qkv.weight") or name.endswith("in_proj_z.weight"):
            return "gdn_qkvz"
        if name.endswith("out_proj.weight"):
            return "gdn_out"
        return "gdn_small"        # in_proj_a/b, conv1d, norm, A_log, dt_bias
    if "self_attn" in name:
        if name.endswith(("q_proj.weight", "k_proj.weight", "v_proj.weight")):
            return "attn_qkv"
        if name.endswith("o_proj.weight"):
            return "attn_o"
        return "norm"
    if "mlp." in name:
        return "ffn_down" if name.endswith("down_proj.weight") else "ffn_gate_up"
    if name.endswith("norm.weight") or name.endswith("layernorm.weight"):
        return "norm"
    return "other"


def layer_of(name: str) -> int:
    parts = name.split(".")
    if "layers" in parts:
        return int(parts[parts.index("layers") + 1])
    return 0
