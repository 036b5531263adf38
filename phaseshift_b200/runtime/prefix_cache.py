"""GPU-resident prefix cache: exact-token prefix index (C++ PrefixIndex) + device snapshots.

Policy follows the reference (docs/developer/prefix_cache.md:27-141, src/phaseshift/models/qwen35/runtime/
prefix_cache.cpp): separate cache storage, no refcount / copy-on-write, restore = device-to-device copy
into the request's own pages; lookup = longest stored sequence that is a strict prefix of the prompt;
LRU eviction; entries shorter than ``min_tokens`` or larger than the capacity are skipped silently.
A snapshot holds, for the first n tokens: every attention layer's K/V pages (and FP8 scales) and every
GDN layer's recurrent state + conv history ring.  All copies are issued on the engine's stream, so no
extra synchronisation is needed, and every tensor-parallel rank snapshots its own shard.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch

from ..core.native import runtime


@dataclass
class _Snapshot:
    tokens: int
    kv: list          # per attention layer: (k, v, k_scale, v_scale) with a leading [n_pages] dim
    gdn: list         # per GDN layer: (rec [Hv,Dk,Dv], conv [Hv,ring,CH])


@dataclass
class PrefixHitInfo:
    entry: int
    tokens: int


class PrefixCache:
    def __init__(self, engine, capacity_tokens: int, max_entries: int = 16, min_tokens: int = 64):
        self.engine = engine
        self.index = runtime().PrefixIndex(max_entries, capacity_tokens, min_tokens)
        self.snaps: Dict[int, _Snapshot] = {}
        self.stats = {"saved_tokens": 0, "restored_tokens": 0}

    def lookup(self, prompt: Sequence[int]) -> Optional[PrefixHitInfo]:
        h = self.index.lookup(list(prompt))
        if h.entry < 0 or h.entry not in self.snaps:
            return None
        return PrefixHitInfo(h.entry, h.tokens)

    def save(self, tokens: Sequence[int], slot: int, pages: Sequence[int]) -> bool:
        """Snapshot the first len(tokens) positions of the sequence in `slot` (its state must currently be
        exactly at that position)."""
        entry, evicted = self.index.insert(list(tokens))
        for e in evicted:
            self.snaps.pop(e, None)
        if entry < 0:
            return False
        st = self.engine.state
        n = len(tokens)
        n_pages = -(-n // st.sc.page_tokens)
        idx = torch.tensor(list(pages[:n_pages]), dtype=torch.long, device=st.device)
        kv, gdn = [], []
        for l in st.kv:
            if l is None:
                continue
            kv.append((l.k[idx].clone(), l.v[idx].clone(),
                       None if l.k_scale is None else l.k_scale[idx].clone(),
                       None if l.v_scale is None else l.v_scale[idx].clone()))
        for g in st.gdn:
            if g is None:
                continue
            gdn.append((g.rec[slot].clone(), g.conv[slot].clone()))
        self.snaps[entry] = _Snapshot(n, kv, gdn)
        self.stats["saved_tokens"] += n
        return True

    def restore(self, hit: PrefixHitInfo, slot: int, pages: Sequence[int]) -> None:
        snap = self.snaps[hit.entry]
        st = self.engine.state
        idx = torch.tensor(list(pages), dtype=torch.long, device=st.device)
        assert idx.numel() == snap.kv[0][0].shape[0] if snap.kv else True
        ki = 0
        for l in st.kv:
            if l is None:
                continue
            k, v, ks, vs = snap.kv[ki]
            ki += 1
            l.k[idx] = k
            l.v[idx] = v
            if ks is not None:
                l.k_scale[idx] = ks
                l.v_scale[idx] = vs
        gi = 0
        for g in st.gdn:
            if g is None:
                continue
            rec, conv = snap.gdn[gi]
            gi += 1
            g.rec[slot].copy_(rec)
            g.conv[slot].copy_(conv)
        self.stats["restored_tokens"] += snap.tokens

    def summary(self) -> dict:
        i = self.index
        return dict(entries=i.entries(), used_tokens=i.used_tokens(), hits=i.hits, misses=i.misses, inserts=i.inserts,
                    evictions=i.evictions, skipped=i.skipped, **self.stats)
