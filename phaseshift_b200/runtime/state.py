"""Device-resident sequence state: paged KV pools, GDN conv/recurrent pools, block tables.

Layouts (chosen for Blackwell: every (page, kv-head) tile is one contiguous 8 KB / 4 KB block that a
single bulk copy can fetch; the reference interleaves heads inside a token,
include/phaseshift/models/qwen35/state/paged_kv_pool.h:59-140):

* K/V pool per attention layer: ``[num_pages, Hkv, page_tokens, D]`` in bf16 or E4M3 bytes, FP8 pools
  carry ``[num_pages, Hkv, page_tokens]`` f32 scales (one per token x head, like the reference's
  FP8_E4M3 KV mode, state/kv_cache_types.h:11-46).
* GDN conv history per GDN layer: ``[slots, Hv, ring, 2*Dk+Dv]`` bf16, position p in slot p % ring.
* GDN recurrent state per GDN layer: ``[slots, Hv, Dk, Dv]`` f32 (reference: gdn_state_pool.h:16-105).
* Block table: ``[slots, max_blocks]`` int32, -1 = unmapped.

Sizing rules follow docs/developer/runtime.md:109-119:
``max_blocks = ceil((max_seq_len+1)/page)+1``, ``pages = ceil(capacity_tokens/page)+1``.
Page 0 is never handed out, so a zeroed block table entry cannot alias live data.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch

from ..models.qwen35.config import Qwen35Config
from ..models.qwen35.weights import TpGeometry

KV_DTYPES = ("bf16", "fp8_e4m3", "nvfp4")
# names accepted on the command line for the reference's block-coded caches (src/apps/compute/main.hip:47-81): its 4-bit
# format is served by the NVFP4 pools, its 8-bit format by the FP8 pools (same E4M3 codes, one scale per row instead of
# one per 32 values)
KV_DTYPE_ALIASES = {"psq4": "nvfp4", "psq8": "fp8_e4m3"}
KV_FMT = {"bf16": 0, "fp8_e4m3": 1, "nvfp4": 2}


def kv_row_bytes(kv_dtype: str, head_dim: int) -> int:
    """Bytes of one cached row (a token of one KV head) in the pools of `kv_dtype`, without the fp32 row scale."""
    if kv_dtype == "nvfp4":
        return ((head_dim // 2 + head_dim // 16) + 15) & ~15          # codes, block scales, padded to 16 bytes
    return head_dim * (1 if kv_dtype == "fp8_e4m3" else 2)


@dataclass
class StateConfig:
    max_slots: int = 1
    max_seq_len: int = 512
    page_tokens: int = 16
    kv_capacity_tokens: int = 0          # 0 = one full context per slot
    kv_dtype: str = "bf16"
    conv_ring: int = 4                   # >= 4; 3 + max speculative rows when rollback is needed
    spec_rows: int = 0                   # > 0 allocates the alternate recurrent state + update log

    def max_blocks(self) -> int:
        return -(-(self.max_seq_len + 1) // self.page_tokens) + 1

    def num_pages(self) -> int:
        cap = self.kv_capacity_tokens or self.max_slots * (self.max_seq_len + 1)
        return -(-cap // self.page_tokens) + 1 + self.max_slots


class KVLayer:
    __slots__ = ("k", "v", "k_scale", "v_scale")

    def __init__(self, k, v, k_scale, v_scale):
        self.k, self.v, self.k_scale, self.v_scale = k, v, k_scale, v_scale


class GdnLayerState:
    __slots__ = ("conv", "rec", "rec_alt")

    def __init__(self, conv, rec, rec_alt):
        self.conv, self.rec, self.rec_alt = conv, rec, rec_alt


class ModelState:
    """All per-sequence device state of one rank."""

    def __init__(self, cfg: Qwen35Config, sc: StateConfig, device, act_dtype=torch.bfloat16,
                 geo: Optional[TpGeometry] = None, arenas=None):
        """``arenas`` (a core.arena.ArenaSet, CUDA only): the KV pages and the recurrent / conv state are carved from
        the named arenas "kv" and "state" (stable virtual addresses, physical memory committed for exactly what the
        configuration needs, all under the set's byte budget) instead of the framework allocator."""
        if sc.kv_dtype not in KV_DTYPES:
            raise ValueError(f"kv dtype {sc.kv_dtype!r} not in {KV_DTYPES}")
        if sc.conv_ring < 4:
            raise ValueError("conv_ring must be >= 4")
        self.cfg, self.sc, self.device = cfg, sc, device
        geo = geo or TpGeometry.make(cfg, 0, 1)
        self.geo = geo
        self.hkv = len(geo.kv_heads)
        self.hv = len(geo.gdn_v_heads)
        self.num_pages = sc.num_pages()
        self.max_blocks = sc.max_blocks()
        D, pt = cfg.head_dim, sc.page_tokens
        fp8 = sc.kv_dtype == "fp8_e4m3"
        self.kv_fp8 = fp8
        self.kv_fmt = KV_FMT[sc.kv_dtype]            # 0 bf16, 1 FP8-E4M3 + row scale, 2 NVFP4 rows + row scale
        Drow = D                                     # last extent of the pools
        if act_dtype == torch.float32:
            kvt = torch.float32          # CPU reference keeps full precision
            fp8 = self.kv_fp8 = False
            self.kv_fmt = 0
        elif self.kv_fmt == 2:
            if D % 32 or D > 256:
                raise ValueError("NVFP4 key/value pages need a head size that is a multiple of 32, at most 256")
            kvt, Drow = torch.uint8, kv_row_bytes("nvfp4", D)
        else:
            kvt = torch.uint8 if fp8 else torch.bfloat16
        scaled = self.kv_fmt != 0                    # pools with an fp32 scale per (page, head, token)
        self.kv: List[Optional[KVLayer]] = []
        self.gdn: List[Optional[GdnLayerState]] = []
        Dk, Dv = cfg.linear_key_head_dim, cfg.linear_value_head_dim
        self.arenas = arenas
        esz = lambda dt: torch.empty(0, dtype=dt).element_size()
        n_attn = sum(1 for lt in cfg.layer_types if lt == 1)
        n_gdn = len(cfg.layer_types) - n_attn
        kv_need = n_attn * (2 * self.num_pages * self.hkv * pt * Drow * esz(kvt) + (2 * self.num_pages * self.hkv * pt * 4 if scaled else 0) + 1024)
        st_need = n_gdn * (sc.max_slots * self.hv * (sc.conv_ring * (2 * Dk + Dv) * esz(act_dtype)
                                                      + Dk * Dv * 4 * (2 if sc.spec_rows > 0 else 1)) + 1024)
        kv_arena = arenas.get("kv", kv_need + (2 << 20)) if arenas is not None and n_attn else None
        st_arena = arenas.get("state", st_need + (2 << 20)) if arenas is not None and n_gdn else None

        def pool(arena, shape, dtype, fill=0):
            if arena is None:
                return torch.full(shape, fill, dtype=dtype, device=device) if fill else torch.zeros(shape, dtype=dtype, device=device)
            t = arena.alloc(shape, dtype)
            return t.fill_(fill) if fill else t.zero_()
        for lt in cfg.layer_types:
            if lt == 1:
                k = pool(kv_arena, (self.num_pages, self.hkv, pt, Drow), kvt)
                v = pool(kv_arena, (self.num_pages, self.hkv, pt, Drow), kvt)
                ks = vs = None
                if scaled:
                    ks = pool(kv_arena, (self.num_pages, self.hkv, pt), torch.float32, 1)
                    vs = pool(kv_arena, (self.num_pages, self.hkv, pt), torch.float32, 1)
                self.kv.append(KVLayer(k, v, ks, vs))
                self.gdn.append(None)
            else:
                conv = pool(st_arena, (sc.max_slots, self.hv, sc.conv_ring, 2 * Dk + Dv), act_dtype)
                rec = pool(st_arena, (sc.max_slots, self.hv, Dk, Dv), torch.float32)
                alt = pool(st_arena, (sc.max_slots, self.hv, Dk, Dv), torch.float32) if sc.spec_rows > 0 else None
                self.gdn.append(GdnLayerState(conv, rec, alt))
                self.kv.append(None)
        self.block_table = torch.full((sc.max_slots, self.max_blocks), -1, dtype=torch.int32, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)

    def kv_bytes(self) -> int:
        n = 0
        for l in self.kv:
            if l is not None:
                n += 2 * l.k.numel() * l.k.element_size()
                if l.k_scale is not None:
                    n += 2 * l.k_scale.numel() * 4
        return n

    def reset_slot(self, slot: int) -> None:
        """Fresh sequence: zero recurrent state (conv history needs no clearing: taps before position 0
        are defined as zero by the kernels)."""
        for g in self.gdn:
            if g is not None:
                g.rec[slot].zero_()

    def copy_slot(self, dst: int, src: int) -> None:
        for g in self.gdn:
            if g is not None:
                g.rec[dst].copy_(g.rec[src])
                g.conv[dst].copy_(g.conv[src])
