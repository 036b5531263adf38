"""Qwen3.5-style hybrid decoder configuration.

Keys and defaults follow the reference's text config reader
(include/phaseshift/models/qwen35/model/qwen35_config.h:11-38, src/.../model/qwen35_config.cpp):
a layer is Gated-DeltaNet (linear attention) unless ``(index + 1) % full_attention_interval == 0``
or ``layer_types`` says otherwise.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field, asdict
from pathlib import Path
from typing import List, Optional


@dataclass
class Qwen35Config:
    vocab_size: int = 151936
    hidden_size: int = 5120
    intermediate_size: int = 17408
    num_hidden_layers: int = 64
    full_attention_interval: int = 4
    linear_num_key_heads: int = 16
    linear_num_value_heads: int = 48
    linear_key_head_dim: int = 128
    linear_value_head_dim: int = 128
    linear_conv_kernel_dim: int = 4
    num_attention_heads: int = 24
    num_key_value_heads: int = 4
    head_dim: int = 256
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e7
    partial_rotary_factor: float = 0.25
    tie_word_embeddings: bool = False
    layer_types: Optional[List[int]] = None       # 0 = GDN, 1 = full attention
    eos_token_ids: List[int] = field(default_factory=list)
    name: str = "qwen35"

    def __post_init__(self):
        if self.layer_types is None:
            self.layer_types = [1 if (i + 1) % self.full_attention_interval == 0 else 0
                                for i in range(self.num_hidden_layers)]
        if len(self.layer_types) != self.num_hidden_layers:
            raise ValueError("layer_types length must equal num_hidden_layers")
        if self.linear_conv_kernel_dim != 4:
            raise ValueError("only a short-conv kernel of 4 is supported")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ValueError("num_attention_heads must be a multiple of num_key_value_heads")
        if self.linear_num_value_heads % self.linear_num_key_heads:
            raise ValueError("linear_num_value_heads must be a multiple of linear_num_key_heads")

    # ---- derived geometry
    @property
    def rotary_dim(self) -> int:
        return int(self.head_dim * self.partial_rotary_factor)

    @property
    def gdn_qk_dim(self) -> int:
        return self.linear_num_key_heads * self.linear_key_head_dim

    @property
    def gdn_v_dim(self) -> int:
        return self.linear_num_value_heads * self.linear_value_head_dim

    @property
    def gdn_conv_dim(self) -> int:
        return 2 * self.gdn_qk_dim + self.gdn_v_dim

    @property
    def attn_q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def attn_kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def gdn_layers(self) -> List[int]:
        return [i for i, t in enumerate(self.layer_types) if t == 0]

    @property
    def attn_layers(self) -> List[int]:
        return [i for i, t in enumerate(self.layer_types) if t == 1]

    def param_count(self) -> int:
        h = self.hidden_size
        n = 2 * self.vocab_size * h if not self.tie_word_embeddings else self.vocab_size * h
        for t in self.layer_types:
            n += 3 * h * self.intermediate_size
            if t == 0:
                n += h * (self.gdn_conv_dim + self.gdn_v_dim + 2 * self.linear_num_value_heads) + self.gdn_v_dim * h
            else:
                n += h * (2 * self.attn_q_dim + 2 * self.attn_kv_dim) + self.attn_q_dim * h
        return n

    def to_hf_dict(self) -> dict:
        d = asdict(self)
        d.pop("name")
        eos = d.pop("eos_token_ids")
        d["architectures"] = ["Qwen3_5ForCausalLM"]
        d["model_type"] = "qwen3_5_text"
        d["eos_token_id"] = eos
        return d

    def save(self, model_dir) -> None:
        Path(model_dir).mkdir(parents=True, exist_ok=True)
        (Path(model_dir) / "config.json").write_text(json.dumps(self.to_hf_dict(), indent=1))

    @staticmethod
    def from_dir(model_dir) -> "Qwen35Config":
        raw = json.loads((Path(model_dir) / "config.json").read_text())
        raw = raw.get("text_config", raw)
        kw = {}
        for f in Qwen35Config.__dataclass_fields__:
            if f in raw:
                kw[f] = raw[f]
        if "attention_head_dim" in raw:
            kw["head_dim"] = raw["attention_head_dim"]
        lt = raw.get("layer_types")
        if lt and isinstance(lt[0], str):
            kw["layer_types"] = [0 if "linear" in s else 1 for s in lt]
        eos = raw.get("eos_token_id", [])
        gen = Path(model_dir) / "generation_config.json"
        if gen.exists():
            eos = json.loads(gen.read_text()).get("eos_token_id", eos)
        if isinstance(eos, int):
            eos = [eos]
        kw["eos_token_ids"] = list(eos or [])
        kw.pop("name", None)
        return Qwen35Config(**kw)


def tiny_config(**over) -> Qwen35Config:
    """Hidden 256, 4 layers (3 GDN + 1 full attention), the CPU token-exactness fixture."""
    kw = dict(vocab_size=4096, hidden_size=256, intermediate_size=768, num_hidden_layers=4,
              linear_num_key_heads=4, linear_num_value_heads=8, linear_key_head_dim=64, linear_value_head_dim=64,
              num_attention_heads=4, num_key_value_heads=2, head_dim=64, name="qwen35-tiny")
    kw.update(over)
    return Qwen35Config(**kw)


def qwen35_4b_config(**over) -> Qwen35Config:
    kw = dict(vocab_size=151936, hidden_size=2560, intermediate_size=9216, num_hidden_layers=32,
              linear_num_key_heads=16, linear_num_value_heads=32, linear_key_head_dim=128,
              linear_value_head_dim=128, num_attention_heads=16, num_key_value_heads=4, head_dim=256,
              name="qwen35-4b")
    kw.update(over)
    return Qwen35Config(**kw)


def qwen35_27b_config(**over) -> Qwen35Config:
    kw = dict(name="qwen35-27b")
    kw.update(over)
    return Qwen35Config(**kw)


PRESETS = {"tiny": tiny_config, "4b": qwen35_4b_config, "27b": qwen35_27b_config}
