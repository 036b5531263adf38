"""GPU-resident prefix cache: exact-token prefix index (C++ PrefixIndex) + device snapshots.

Policy follows the reference (docs/developer/prefix_cache.md:27-141, src/phaseshift/models/qwen35/runtime/
prefix_cache.cpp): separate cache storage, no refcount / copy-on-write, restore = device-to-device copy
into the request's own pages; lookup = longest stored sequence that is a strict prefix of the prompt;
LRU eviction; entries shorter than ``min_tokens`` or larger than the capacity are skipped silently.
A snapshot holds, for the first n tokens: every attention layer's K/V pages (and FP8 scales) and every
GDN layer's recurrent state + conv history ring, stored in a pool that is allocated once and bounds the cache's
device memory.  All copies are issued on the engine's stream, so no
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
    pages: List[int]  # pool pages holding this prefix's K/V, in block order
    state_slot: int   # row of the pooled GDN state
    extra: object = None   # caller-owned companion state (e.g. a drafter's context ring), cloned by the caller


@dataclass
class PrefixHitInfo:
    entry: int
    tokens: int


class PrefixCache:
    """Storage is a POOL allocated once: ``capacity_tokens`` worth of K/V pages per attention layer (plus FP8 scales)
    and ``max_entries`` recurrent-state rows per GDN layer -- the cache can never hold more device memory than that,
    whatever is saved (the index evicts by LRU before the pool runs out; a save that still finds no room is skipped)."""

    def __init__(self, engine, capacity_tokens: int, max_entries: int = 16, min_tokens: int = 64):
        self.engine = engine
        self.index = runtime().PrefixIndex(max_entries, capacity_tokens, min_tokens)
        self.snaps: Dict[int, _Snapshot] = {}
        self.stats = {"saved_tokens": 0, "restored_tokens": 0, "skipped_no_room": 0}
        st = engine.state
        pt = st.sc.page_tokens
        self.pool_pages = -(-capacity_tokens // pt) + max_entries          # every entry may end in a partial page
        self.free_pages: List[int] = list(range(self.pool_pages))
        self.free_slots: List[int] = list(range(max_entries))
        dev = st.device
        self.kv_pool, self.gdn_pool = [], []
        for l in st.kv:
            if l is None:
                continue
            shp = (self.pool_pages,) + tuple(l.k.shape[1:])
            ks = vs = None
            if l.k_scale is not None:
                sshp = (self.pool_pages,) + tuple(l.k_scale.shape[1:])
                ks, vs = torch.ones(sshp, dtype=l.k_scale.dtype, device=dev), torch.ones(sshp, dtype=l.k_scale.dtype, device=dev)
            self.kv_pool.append((torch.zeros(shp, dtype=l.k.dtype, device=dev), torch.zeros(shp, dtype=l.k.dtype, device=dev), ks, vs))
        for g in st.gdn:
            if g is None:
                continue
            self.gdn_pool.append((torch.zeros((max_entries,) + tuple(g.rec.shape[1:]), dtype=g.rec.dtype, device=dev),
                                  torch.zeros((max_entries,) + tuple(g.conv.shape[1:]), dtype=g.conv.dtype, device=dev)))
        pin = dev.type == "cuda"
        self._h_idx = torch.zeros(2, max(1, st.max_blocks), dtype=torch.long, pin_memory=pin)
        self._d_idx = torch.zeros(2, max(1, st.max_blocks), dtype=torch.long, device=dev)

    def pool_bytes(self) -> int:
        n = 0
        for k, v, ks, vs in self.kv_pool:
            n += 2 * k.numel() * k.element_size() + (2 * ks.numel() * ks.element_size() if ks is not None else 0)
        for rec, conv in self.gdn_pool:
            n += rec.numel() * rec.element_size() + conv.numel() * conv.element_size()
        return n

    def _index_pair(self, a: Sequence[int], b: Sequence[int]):
        """Two equally long page lists as device index tensors through one pinned staging buffer (no pageable copy)."""
        n = len(a)
        self._h_idx[0, :n] = torch.as_tensor(list(a), dtype=torch.long)
        self._h_idx[1, :n] = torch.as_tensor(list(b), dtype=torch.long)
        self._d_idx[:, :n].copy_(self._h_idx[:, :n], non_blocking=True)
        return self._d_idx[0, :n], self._d_idx[1, :n]

    def _drop(self, entry: int) -> None:
        snap = self.snaps.pop(entry, None)
        if snap is not None:
            self.free_pages.extend(snap.pages)
            self.free_slots.append(snap.state_slot)

    def lookup(self, prompt: Sequence[int]) -> Optional[PrefixHitInfo]:
        h = self.index.lookup(list(prompt))
        if h.entry < 0 or h.entry not in self.snaps:
            return None
        return PrefixHitInfo(h.entry, h.tokens)

    def save(self, tokens: Sequence[int], slot: int, pages: Sequence[int], extra=None) -> bool:
        """Snapshot the first len(tokens) positions of the sequence in `slot` (its state must currently be
        exactly at that position).  ``extra`` rides along with the entry and is returned by ``restore``."""
        entry, evicted = self.index.insert(list(tokens))
        for e in evicted:
            self._drop(e)
        if entry < 0:
            return False
        self._drop(entry)                            # re-insert of a known prefix: refresh it
        st = self.engine.state
        n = len(tokens)
        n_pages = -(-n // st.sc.page_tokens)
        if n_pages > len(self.free_pages) or not self.free_slots or n_pages > self._h_idx.shape[1]:
            self.stats["skipped_no_room"] += 1
            self.index.erase(entry) if hasattr(self.index, "erase") else None
            return False
        mine = [self.free_pages.pop() for _ in range(n_pages)]
        ss = self.free_slots.pop()
        src, dst = self._index_pair(pages[:n_pages], mine)
        ki = 0
        for l in st.kv:
            if l is None:
                continue
            pk, pv, pks, pvs = self.kv_pool[ki]
            ki += 1
            pk.index_copy_(0, dst, l.k.index_select(0, src))
            pv.index_copy_(0, dst, l.v.index_select(0, src))
            if pks is not None:
                pks.index_copy_(0, dst, l.k_scale.index_select(0, src))
                pvs.index_copy_(0, dst, l.v_scale.index_select(0, src))
        gi = 0
        for g in st.gdn:
            if g is None:
                continue
            rec, conv = self.gdn_pool[gi]
            gi += 1
            rec[ss].copy_(g.rec[slot])
            conv[ss].copy_(g.conv[slot])
        self.snaps[entry] = _Snapshot(n, mine, ss, extra)
        self.stats["saved_tokens"] += n
        return True

    def restore(self, hit: PrefixHitInfo, slot: int, pages: Sequence[int]):
        """Copy the cached prefix into the request's own pages and slot; returns the entry's ``extra``."""
        snap = self.snaps[hit.entry]
        st = self.engine.state
        assert len(pages) == len(snap.pages), (len(pages), len(snap.pages))
        dst, src = self._index_pair(pages, snap.pages)
        ki = 0
        for l in st.kv:
            if l is None:
                continue
            pk, pv, pks, pvs = self.kv_pool[ki]
            ki += 1
            l.k.index_copy_(0, dst, pk.index_select(0, src))
            l.v.index_copy_(0, dst, pv.index_select(0, src))
            if pks is not None:
                l.k_scale.index_copy_(0, dst, pks.index_select(0, src))
                l.v_scale.index_copy_(0, dst, pvs.index_select(0, src))
        gi = 0
        for g in st.gdn:
            if g is None:
                continue
            rec, conv = self.gdn_pool[gi]
            gi += 1
            g.rec[slot].copy_(rec[snap.state_slot])
            g.conv[slot].copy_(conv[snap.state_slot])
        self.stats["restored_tokens"] += snap.tokens
        return snap.extra

    def summary(self) -> dict:
        i = self.index
        return dict(entries=i.entries(), used_tokens=i.used_tokens(), hits=i.hits, misses=i.misses, inserts=i.inserts,
                    evictions=i.evictions, skipped=i.skipped, pool_bytes=self.pool_bytes(),
                    pool_pages_free=len(self.free_pages), **self.stats)
