"""Serving loop for speculative decoding: the interface of ``ServingEngine`` (submit / cancel / step / events) on top
of ``DFlash2SpecDecoder`` rounds.

Speculative serving advances ONE request at a time, as the reference does (``serve_step_dflash``,
src/apps/compute/main.hip:1077-1124): requests queue up, the active one is prefilled chunk by chunk (each chunk's
tapped hidden states go to the drafter's ring), then every ``step()`` is one propose -> verify -> commit round that
emits 1..K+1 tokens.  Structured output works as in plain serving: the request's grammar matcher masks the first
token and every verify row (``DFlash2SpecDecoder.round(matcher=...)``).
"""
from __future__ import annotations

from collections import deque
from typing import Deque, Dict, List, Optional, Sequence

from .serving import ServeEvent


class _QueueFacade:
    """The two batcher calls the stdio loop makes (``cancel_all`` at shutdown, ``retire`` after a done event)."""

    def __init__(self, owner: "SpecServingEngine"):
        self.owner = owner

    def cancel_all(self) -> None:
        for rid in list(self.owner.requests):
            self.owner.cancel(rid)

    def retire(self, rid: int) -> None:
        self.owner.requests.pop(rid, None)


class SpecServingEngine:
    def __init__(self, decoder, prefill_chunk: int = 2048, constraint_compiler=None, prefix_cache_tokens: int = 0,
                 prefix_cache_entries: int = 8, prefix_min_tokens: int = 64, terminal_checkpoints: bool = True):
        """``prefix_cache_tokens`` > 0: prompt-boundary and terminal checkpoints as in plain serving; an entry also
        keeps the drafter's context ring, so a restored prefix is drafted from at once."""
        self.dec, self.engine = decoder, decoder.eng
        self.prefill_chunk = prefill_chunk
        self.constraints = constraint_compiler
        self.prefix = None
        if prefix_cache_tokens > 0 and hasattr(decoder.drafter, "snapshot"):
            from .prefix_cache import PrefixCache
            self.prefix = PrefixCache(self.engine, prefix_cache_tokens, prefix_cache_entries, prefix_min_tokens)
        self.terminal_checkpoints = terminal_checkpoints
        self.requests: Dict[int, dict] = {}
        self.queue: Deque[int] = deque()
        self.active: Optional[int] = None
        self.seq = None
        self.next_id = 1
        self.batcher = _QueueFacade(self)
        self.stats = {"steps": 0, "tokens": 0, "prefill_tokens": 0, "rounds": 0}

    # ------------------------------------------------------------------ requests
    def submit(self, prompt: Sequence[int], max_new_tokens: int, temperature: float = 0.0, top_p: float = 1.0, top_k: int = 0,
               seed: int = 0, stop_tokens: Sequence[int] = (), checkpoint_position: int = 0, grammar: Optional[str] = None,
               structural_tag: Optional[str] = None) -> int:
        prompt = list(prompt)
        if not prompt:
            raise ValueError("empty prompt")
        if len(prompt) + 1 > self.engine.sc.max_seq_len:
            raise ValueError("prompt does not fit max_seq_len")
        matcher = None
        if grammar is not None or structural_tag is not None:
            if self.constraints is None:
                raise ValueError("structured output requested but no constraint compiler is configured")
            matcher = self.constraints.matcher(grammar=grammar, structural_tag=structural_tag)
        rid = self.next_id
        self.next_id += 1
        self.requests[rid] = dict(id=rid, prompt=prompt, max_new_tokens=int(max_new_tokens), generated=[], state="queued",
                                  samp=dict(temperature=temperature, top_p=top_p, top_k=top_k, seed=seed),
                                  stop=set(int(t) for t in stop_tokens), matcher=matcher, prefilled=0, finish_reason="",
                                  prompt_tokens=len(prompt), restored_tokens=0, prefill_tokens=0, error="",
                                  checkpoint_position=int(checkpoint_position), checkpoint_saved=False)
        self.queue.append(rid)
        return rid

    def request(self, rid: int) -> Optional[dict]:
        return self.requests.get(rid)

    def cancel(self, rid: int) -> bool:
        r = self.requests.get(rid)
        if r is None or r["state"] in ("done", "cancelled"):
            return False
        if rid == self.active:
            self._release()
        elif rid in self.queue:
            self.queue.remove(rid)
        r["state"], r["finish_reason"] = "cancelled", "cancelled"
        return True

    def idle(self) -> bool:
        return self.active is None and not self.queue

    def _release(self) -> None:
        if self.seq is not None:
            self.engine.close_sequence(self.seq)
        self.seq, self.active = None, None

    # ------------------------------------------------------------------ one step
    def step(self) -> List[ServeEvent]:
        ev: List[ServeEvent] = []
        if self.active is None:
            if not self.queue:
                return ev
            self.active = self.queue.popleft()
            r = self.requests[self.active]
            r["state"] = "prefill"
            self.dec.drafter.reset()
            self.seq = self.engine.open_sequence()
            self._restore_prefix(r)
        rid = self.active
        r = self.requests[rid]
        self.stats["steps"] += 1
        try:
            if r["state"] == "prefill":
                c0 = r["prefilled"]
                end = c0 + self.prefill_chunk
                cp = r["checkpoint_position"]
                if self.prefix is not None and c0 < cp < min(end, len(r["prompt"])):
                    end = cp                                 # a chunk ends exactly at the checkpoint so it can be saved
                ids = r["prompt"][c0:end]
                last = c0 + len(ids) >= len(r["prompt"])
                tok = self.dec.prefill_chunk(self.seq, ids, last, r["samp"], r["matcher"])
                r["prefilled"] += len(ids)
                r["prefill_tokens"] += len(ids)
                self.stats["prefill_tokens"] += len(ids)
                if self.prefix is not None and cp and r["prefilled"] == cp and not last:
                    r["checkpoint_saved"] = self._save_prefix(r["prompt"][:cp])
                if not last:
                    return ev
                r["state"] = "decode"
                emitted = [tok]
            else:
                out = r["generated"]
                emitted = self.dec.round(self.seq, out[-1], out[:-1], r["max_new_tokens"] - len(out), r["samp"], r["matcher"])
                self.stats["rounds"] += 1
        except Exception as e:                      # poisoned sequence, device status, constraint failure
            r["state"], r["finish_reason"], r["error"] = "done", "error", str(e)
            self._release()
            ev.append(ServeEvent("error", rid, info={"message": str(e)}))
            return ev
        for t in emitted:
            if t < 0:
                r["finish_reason"] = "constraint"
                break
            r["generated"].append(t)
            self.stats["tokens"] += 1
            ev.append(ServeEvent("token", rid, t))
            if t in r["stop"]:
                r["finish_reason"] = "stop"
                break
            if len(r["generated"]) >= r["max_new_tokens"]:
                r["finish_reason"] = "length"
                break
        if not r["finish_reason"] and self.seq.position + 1 >= self.engine.sc.max_seq_len:
            r["finish_reason"] = "length"
        if r["finish_reason"]:
            r["state"] = "done"
            if self.prefix is not None and self.terminal_checkpoints and r["finish_reason"] in ("stop", "length"):
                fed = (r["prompt"] + r["generated"])[:self.seq.position]     # what the device state covers
                self._save_prefix(fed)
            self._release()
            ev.append(ServeEvent("done", rid, info={"generated_ids": list(r["generated"]), "finish_reason": r["finish_reason"],
                                                    "prompt_tokens": r["prompt_tokens"], "restored_tokens": r["restored_tokens"],
                                                    "prefill_tokens": r["prefill_tokens"],
                                                    "cache_checkpoint_tokens": r["checkpoint_position"] if r["checkpoint_saved"] else 0,
                                                    "message": ""}))
        return ev

    # ------------------------------------------------------------------ prefix cache
    def _save_prefix(self, tokens: Sequence[int]) -> bool:
        s = self.seq
        if s.position != len(tokens) or len(tokens) == 0:
            return False
        return self.prefix.save(list(tokens), s.slot, s.pages, extra=self.dec.drafter.snapshot())

    def _restore_prefix(self, r: dict) -> None:
        if self.prefix is None:
            return
        hit = self.prefix.lookup(r["prompt"])
        if hit is None or hit.tokens >= len(r["prompt"]):
            return
        s = self.seq
        self.engine._reserve(s, hit.tokens)
        n_pages = -(-hit.tokens // self.engine.sc.page_tokens)
        ring = self.prefix.restore(hit, s.slot, s.pages[:n_pages])
        if ring is None:
            return
        self.dec.drafter.restore(ring)
        s.position = hit.tokens
        r["prefilled"] = r["restored_tokens"] = hit.tokens

    def run_until_idle(self, max_steps: int = 1_000_000) -> List[ServeEvent]:
        ev: List[ServeEvent] = []
        for _ in range(max_steps):
            if self.idle():
                break
            ev += self.step()
        return ev
