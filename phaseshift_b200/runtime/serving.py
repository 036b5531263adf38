"""Continuous-batching serving loop: C++ batcher (admission, KV banker, scheduling) + step engine +
prefix cache + token constraints.

One ``step()`` does what the reference's ``ContinuousBatcher::step`` does
(src/phaseshift/models/qwen35/runtime/continuous_batcher.cpp:281-560): admit queued requests (slot,
state reset, prefix-cache restore), plan a mixed decode/prefill batch under the token budget, fill
constraint masks, execute, read back the sampled ids, commit or fail the step, save prefix
checkpoints, emit events.  Under tensor parallelism every rank runs this loop on the same request
stream; all decisions are host-deterministic, so ranks stay in lockstep without exchanging plans, and
prefix restores happen symmetrically on every rank (the reference disables its prefix cache under TP,
docs/developer/tensor_parallel_execution.md:219-220).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch

from ..core.native import runtime
from .batch import SeqRows
from .engine import Engine
from .prefix_cache import PrefixCache


@dataclass
class ServeEvent:
    kind: str                   # token | done | error
    request_id: int
    token_id: int = -1
    info: dict = field(default_factory=dict)


class ServingEngine:
    def __init__(self, engine: Engine, max_step_tokens: int = 2048, max_step_requests: int = 0,
                 prefix_cache_tokens: int = 0, prefix_cache_entries: int = 16, prefix_min_tokens: int = 64,
                 full_claim: bool = False, constraint_compiler=None, terminal_checkpoints: bool = False):
        rt = runtime()
        self.rt, self.engine = rt, engine
        cfg = rt.BatcherConfig()
        cfg.max_slots = engine.sc.max_slots
        cfg.num_pages = engine.state.num_pages
        cfg.page_tokens = engine.sc.page_tokens
        cfg.max_seq_len = engine.sc.max_seq_len
        cfg.max_step_tokens = max_step_tokens
        cfg.max_step_requests = max_step_requests
        cfg.full_claim = full_claim
        self.batcher = rt.Batcher(cfg)
        self.prefix = PrefixCache(engine, prefix_cache_tokens, prefix_cache_entries, prefix_min_tokens) \
            if prefix_cache_tokens > 0 else None
        self.constraints = constraint_compiler
        self.matchers: Dict[int, object] = {}
        # terminal checkpoints (reference: src/phaseshift/models/qwen35/runtime/prefix_cache.cpp:229,391): when a request
        # finishes, everything it fed to the model (prompt + all generated tokens but the last) is cached, so the next
        # turn of the same conversation restores it instead of prefilling it again
        self.terminal_checkpoints = terminal_checkpoints and self.prefix is not None
        self.stops: Dict[int, frozenset] = {}
        self.stats = {"steps": 0, "tokens": 0, "prefill_tokens": 0, "failed_steps": 0, "terminal_checkpoints": 0}

    # ------------------------------------------------------------------ requests
    def submit(self, prompt: Sequence[int], max_new_tokens: int, temperature: float = 0.0, top_p: float = 1.0,
               top_k: int = 0, seed: int = 0, stop_tokens: Sequence[int] = (), checkpoint_position: int = 0,
               grammar: Optional[str] = None, structural_tag: Optional[str] = None) -> int:
        s = self.rt.Sampling(temperature, top_p, top_k, seed)
        rid = self.batcher.submit(list(prompt), max_new_tokens, s, list(stop_tokens), checkpoint_position)
        self.stops[rid] = frozenset(int(t) for t in stop_tokens)
        if grammar is not None or structural_tag is not None:
            if self.constraints is None:
                self.batcher.cancel(rid)
                raise ValueError("structured output requested but no constraint compiler is configured")
            self.matchers[rid] = self.constraints.matcher(grammar=grammar, structural_tag=structural_tag)
        return rid

    def cancel(self, rid: int) -> bool:
        ok = self.batcher.cancel(rid)
        self.engine.apply_block_updates(self.batcher.take_release_updates())
        self.matchers.pop(rid, None)
        return ok

    def request(self, rid: int) -> Optional[dict]:
        return self.batcher.request(rid)

    def idle(self) -> bool:
        return self.batcher.idle()

    # ------------------------------------------------------------------ one step
    def step(self) -> List[ServeEvent]:
        eng, b = self.engine, self.batcher
        events: List[ServeEvent] = []
        for rid in b.admit():
            r = b.request(rid)
            eng.state.reset_slot(r["slot"])
            if self.prefix is not None:
                hit = self.prefix.lookup(r["prompt"])
                if hit is not None:
                    ups = b.restore_prefix(rid, hit.tokens)
                    eng.apply_block_updates(ups)
                    self.prefix.restore(hit, r["slot"], [p for (_, _, p) in ups])
        plan = b.plan()
        if plan.empty():
            # requests rejected at admission (can never fit) surface as errors
            return events
        d = plan.to_dict()
        eng.apply_block_updates(d["block_updates"])
        toks = d["tokens"]
        rows, masked = [], []
        for (rid, slot, pos, off, n, sample, is_decode, sidx) in d["seqs"]:
            r = b.request(rid)
            rows.append(SeqRows(slot, pos, toks[off:off + n], (n - 1,) if sample else (),
                                temperature=r["temperature"], top_p=r["top_p"], top_k=r["top_k"], seed=r["seed"],
                                sample_index=sidx))
            if sample:
                masked.append(rid)
            if not is_decode:
                self.stats["prefill_tokens"] += n
        mask = mask_active = None
        if self.matchers and any(rid in self.matchers for rid in masked):
            mask, mask_active = self._fill_masks(masked)
        sampled, out, status = eng.run_rows(rows, mask=mask, mask_active=mask_active)
        self.stats["steps"] += 1
        if status != 0:
            self.stats["failed_steps"] += 1
            self.stats["last_status"] = int(status)
            for (kind, rid, tok) in b.fail(plan, f"device status {status}"):
                events.append(ServeEvent("error", rid, info={"message": f"device status {status}"}))
            eng.apply_block_updates(b.take_release_updates())
            return events
        # constraint bookkeeping before commit: advance matchers with the tokens they produced
        for rid, tok in zip(masked, sampled):
            m = self.matchers.get(rid)
            if m is not None and tok >= 0 and not m.accept(tok):
                sampled[masked.index(rid)] = -1
        if self.terminal_checkpoints:
            self._save_terminal(masked, sampled)
        for (kind, rid, tok) in b.commit(plan, list(sampled)):
            if kind == 0:
                self.stats["tokens"] += 1
                events.append(ServeEvent("token", rid, tok))
            else:
                r = b.request(rid)
                self._maybe_save_terminal(r)
                events.append(ServeEvent("done" if kind == 1 else "error", rid, info=self._done_info(r)))
                self.matchers.pop(rid, None)
        # prompt-boundary checkpoints reached by this step
        if self.prefix is not None:
            for (rid, slot, pos, off, n, sample, is_decode, sidx) in d["seqs"]:
                if is_decode:
                    continue
                r = b.request(rid)
                cp = r["checkpoint_position"]
                if cp and pos + n == cp and r["state"] == 1:
                    self.prefix.save(r["prompt"][:cp], slot, r["pages"])
        eng.apply_block_updates(b.take_release_updates())
        return events

    def run_until_idle(self, max_steps: int = 1_000_000) -> List[ServeEvent]:
        ev: List[ServeEvent] = []
        for _ in range(max_steps):
            if self.batcher.idle():
                break
            ev += self.step()
        return ev

    # ------------------------------------------------------------------ helpers
    def _done_info(self, r: dict) -> dict:
        return {"generated_ids": r["generated"], "finish_reason": r["finish_reason"], "prompt_tokens": r["prompt_tokens"],
                "restored_tokens": r["restored_tokens"], "prefill_tokens": r["prefill_tokens"],
                "cache_checkpoint_tokens": r["checkpoint_position"] if r["checkpoint_saved"] else 0,
                "message": r["error"]}

    def _maybe_save_terminal(self, r: dict) -> None:
        self.stops.pop(r["id"], None)

    def _save_terminal(self, rids: List[int], sampled) -> None:
        """Before the step is committed (the requests still own their pages): snapshot every request this step's
        token finishes.  The device state covers exactly the tokens fed so far = prompt + generated (the token
        sampled now has not been fed), which is what a follow-up prompt will start with."""
        b = self.batcher
        for rid, tok in zip(rids, sampled):
            r = b.request(rid)
            if r is None or tok < 0:
                continue
            fed = list(r["prompt"]) + list(r["generated"])
            if r["position"] + 0 < len(r["prompt"]):
                continue                                   # still prefilling (cannot finish)
            finishing = tok in self.stops.get(rid, ()) or len(r["generated"]) + 1 >= r["max_new_tokens"]
            if finishing and self.prefix.save(fed, r["slot"], r["pages"]):
                self.stats["terminal_checkpoints"] += 1

    def _fill_masks(self, rids: List[int]):
        vocab = self.engine.cfg.vocab_size
        words = (vocab + 31) // 32
        mask = torch.full((len(rids), words), -1, dtype=torch.int32)
        active = torch.zeros(len(rids), dtype=torch.uint8)
        for i, rid in enumerate(rids):
            m = self.matchers.get(rid)
            if m is not None:
                m.fill_next_mask(mask[i])
                active[i] = 1
        return mask.to(self.engine.device), active.to(self.engine.device)
