"""DFlash2 speculative decoding round state machine.

One round (reference: src/phaseshift/models/qwen35/runtime/dflash2_spec_decoder.cpp:416-650,
docs/developer/dflash2.md:746-807,942-962):

1. ``K = min(num_drafts, remaining - 1, room - 1)``; K == 0 falls back to a plain decode step.
2. The drafter proposes K tokens from the pending (anchor) token and its context ring.
3. The target verifies rows ``[anchor, d1..dK]`` in ONE forward in Exact numeric mode (every row is
   computed with the arithmetic of a single-row decode), sampling one token per row; GDN layers keep
   their old recurrent state and log (k, delta, decay) per row instead.
4. ``spec_greedy_accept``: longest prefix where draft == target sample; the next token is the target's
   sample at the first mismatch (correction) or after the last draft (bonus).
5. Commit ``accepted + 1`` rows: replay the GDN log prefix onto the old state, advance the position
   (conv history and KV pages beyond it are simply overwritten later), trim surplus KV pages, append the
   committed rows' hidden taps to the drafter's ring.

With temperature 0 the emitted stream equals target-only greedy decoding token for token; with
temperature > 0 drafts are compared against the target's own samples (sample-and-compare), each row using
``sample_index = tokens generated so far + row``.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ...core.native import runtime
from ...runtime.batch import SeqRows
from .model import DFlash2Config, DFlash2Drafter


def embed_rows(table, ids: torch.Tensor) -> torch.Tensor:
    """Rows of the target's embedding table (bf16 or MXFP8 canonical payload) as fp32."""
    q = table.q
    if q.fmt == "bf16":
        return q.codes[ids].float()
    if q.fmt == "mxfp8":
        c = q.codes[ids].view(torch.float8_e4m3fn).float()
        s = torch.exp2(q.scales[ids].float() - 127.0)
        return (c.reshape(len(ids), -1, 32) * s[..., None]).reshape(len(ids), -1)[:, :q.shape[1]]
    raise ValueError("unsupported embedding format " + q.fmt)


class DFlash2SpecDecoder:
    def __init__(self, engine, drafter, num_drafts: int = 7, ngram_tail: int = 0, ngram_n: int = 0):
        """``drafter``: a ``DFlash2Drafter`` or any object with the same interface (``cfg.target_layer_ids``,
        ``reset``, ``append_context``, ``propose``), e.g. the built-in MTP head (models/qwen35/mtp.py)."""
        if engine.sc.spec_rows < num_drafts + 1 + ngram_tail:
            raise ValueError("engine state was not sized for this many speculative rows (StateConfig.spec_rows)")
        if engine.sc.conv_ring < 3 + num_drafts + 1 + ngram_tail:
            raise ValueError("conv_ring must be >= 3 + speculative rows so history survives a rollback")
        self.eng, self.drafter, self.k = engine, drafter, num_drafts
        self.ngram_tail, self.ngram_n = ngram_tail, ngram_n
        self.rt = runtime()
        self.verify_exact = True       # Exact numeric mode: every verified row uses single-row-decode arithmetic
        # verification rows and plain single-row steps must run the same projection arithmetic
        if hasattr(engine, "set_uniform_arithmetic"):
            engine.set_uniform_arithmetic(True)
        if hasattr(engine.ops, "topk"):
            drafter.topk_fn = engine.ops.topk              # exact radix top-k kernel for the candidate sets
        if hasattr(drafter, "bind"):
            drafter.bind(self._embed, self._lm_head)
        self.taps = list(drafter.cfg.target_layer_ids)
        cfg = engine.cfg
        rows = 16 if num_drafts + 1 + ngram_tail > 8 else 8
        st = engine.state
        dev = engine.device
        Dk, Dv = cfg.linear_key_head_dim, cfg.linear_value_head_dim
        self.logs: Dict[int, tuple] = {}
        for li, g in enumerate(st.gdn):
            if g is not None:
                self.logs[li] = (torch.zeros(rows, st.hv, Dk, device=dev), torch.zeros(rows, st.hv, Dv, device=dev),
                                 torch.zeros(rows, st.hv, device=dev))
        self.stats = {"rounds": 0, "accepted": 0, "proposed": 0, "emitted": 0, "plain_steps": 0}
        self.commit_graphs = True          # device-draft rounds: the commit (log replay + ring append) is one graph replay
        self._commit_graphs: Dict[tuple, object] = {}
        self._commit_ctl = self._commit_host = None

    @staticmethod
    def from_dir(engine, drafter_dir, num_drafts: int = 7, ngram_tail: int = 0, ngram_n: int = 0, native: Optional[bool] = None,
                 fmt: str = "nvfp4", target_model_dir=None):
        """``native`` (default: whenever the engine runs the CUDA op set and the drafter's shape fits the kernels):
        the drafter on the engine's own kernels (native.py) instead of torch tensor ops."""
        if native is None:
            native = engine.device.type == "cuda" and hasattr(engine.ops, "linear_bs")
            if native:
                c = DFlash2Config.from_dir(drafter_dir)
                native = c.head_dim == 128 and c.num_attention_heads // c.num_key_value_heads <= 4
        if native:
            from . import draft_vocab
            from .native import DFlash2NativeDrafter
            dr = DFlash2NativeDrafter.from_dir(drafter_dir, engine, fmt)
            # fixed draft vocabulary: only when the environment asks for it (off by default, like the reference)
            dv = draft_vocab.resolve(target_model_dir, engine.cfg.vocab_size, engine.cfg.hidden_size, dr.cfg.selector_top_k)
            if dv is not None:
                dr.set_draft_vocab(dv.ids.tolist())
            return DFlash2SpecDecoder(engine, dr, num_drafts, ngram_tail, ngram_n)
        dt = torch.float32 if engine.device.type == "cpu" else torch.bfloat16
        return DFlash2SpecDecoder(engine, DFlash2Drafter.from_dir(drafter_dir, engine.device, dt), num_drafts, ngram_tail,
                                  ngram_n)

    # ------------------------------------------------------------------ target bridges
    def _embed(self, ids: torch.Tensor) -> torch.Tensor:
        return embed_rows(self.eng.runner.w.embed, ids)

    def _lm_head(self, h: torch.Tensor) -> torch.Tensor:
        ops = self.eng.ops
        x = h.to(ops.act_dtype).contiguous()
        return ops.linear(x, self.eng.runner.w.lm_head, name="dflash_logits", out_f32=True).float()

    def _append_taps(self, out, n_rows: int, pos_start: int, tokens: Sequence[int]) -> None:
        taps = [out.taps[l][:n_rows] for l in self.taps]
        if getattr(self.drafter, "native", False):              # reads the taps side by side, as the step wrote them
            cat = out.taps_cat[:n_rows] if getattr(out, "taps_cat", None) is not None else None
            self.drafter.append_context(taps, pos_start, cat=cat)
        elif getattr(self.drafter, "wants_tokens", False):     # e.g. the MTP head pairs hidden j with token j + 1
            self.drafter.append_context(taps, pos_start, tokens=list(tokens[:n_rows]))
        else:
            self.drafter.append_context(taps, pos_start)

    def _commit_captured(self, out, n_rows: int, keep: int, slot: int, pos0: int) -> None:
        """Commit `keep` of the verified rows -- replay of the recurrent-state log of every GDN layer and the append of
        the kept rows' taps to the drafter's ring -- as ONE graph replay: the row count, slot and position travel in a
        device control word, so the same graph serves every outcome of the acceptance test."""
        eng, st = self.eng, self.eng.state
        if self._commit_ctl is None:
            self._commit_ctl = torch.zeros(1, 4, dtype=torch.int32, device=eng.device)
            self._commit_host = torch.zeros(1, 4, dtype=torch.int32, pin_memory=True)
        h = self._commit_host
        h[0, 0], h[0, 1], h[0, 2], h[0, 3] = 0, keep, slot, pos0
        self._commit_ctl.copy_(h, non_blocking=True)
        cat = out.taps_cat[:n_rows]
        key = (n_rows, cat.data_ptr())

        def run():
            for li, g in enumerate(st.gdn):
                if g is not None:
                    eng.ops.gdn_replay(g, st.hv, self._commit_ctl, 1, self.logs[li])
            self.drafter.append_context([], 0, cat=cat, ctl=self._commit_ctl)
        g = self._commit_graphs.get(key)
        if g is None:
            from ...utils.graphs import capture as capture_graph
            run()                                           # this round's commit, eagerly (also the warm-up)
            torch.cuda.current_stream().synchronize()
            self._commit_graphs[key] = capture_graph(eng.device, run)[0]
        else:
            g.replay()
        self.drafter.context_len = pos0 + keep

    # ------------------------------------------------------------------ phases
    def _masks(self, matcher, drafts: Sequence[int]):
        """Allowed-token bitmasks for verify rows [anchor, drafts...] under a grammar matcher: row i constrains the
        token that follows drafts[:i] (reference: dflash2_spec_decoder.cpp:99, token_constraint.cpp:114).  Drafts the
        grammar rejects, and everything after them, are dropped from the block.  Returns (kept drafts, mask, active)."""
        words = (self.eng.cfg.vocab_size + 31) // 32
        mask = torch.full((len(drafts) + 1, words), -1, dtype=torch.int32)
        ok = matcher.fill_draft_masks(list(drafts), mask)
        dev = self.eng.device
        return list(drafts[:ok]), mask[:ok + 1].to(dev), torch.ones(ok + 1, dtype=torch.uint8).to(dev)

    def prefill_chunk(self, s, ids: Sequence[int], last: bool, samp: dict, matcher=None) -> Optional[int]:
        """One prefill chunk: runs the target on it, appends its tapped hidden states to the drafter's ring (the
        reference appends per chunk too, dflash2_spec_decoder.cpp:416-520); the last chunk samples the first token."""
        pos0 = s.position
        kw = {}
        if last and matcher is not None:
            _, kw["mask"], kw["mask_active"] = self._masks(matcher, [])
        toks, out = self.eng.step([SeqRows(s.slot, pos0, list(ids), (len(ids) - 1,) if last else (), sample_index=0, **samp)],
                                  [s], tap_layers=self.taps, **kw)
        self._append_taps(out, len(ids), pos0, ids)
        if toks and matcher is not None:
            matcher.accept(toks[0])
        return toks[0] if toks else None

    def prefill(self, s, prompt: Sequence[int], chunk: int, samp: dict, matcher=None) -> int:
        tok = None
        for c0 in range(0, len(prompt), chunk):
            t = self.prefill_chunk(s, prompt[c0:c0 + chunk], c0 + chunk >= len(prompt), samp, matcher)
            if t is not None:
                tok = t
        return tok

    def round(self, s, anchor: int, generated: List[int], remaining: int, samp: dict, matcher=None) -> List[int]:
        """Advance by one speculative round; returns the tokens emitted (1 .. K+1).  ``matcher``: a grammar matcher
        (runtime/constraints.py) that has accepted everything up to and including ``anchor``; every verify row is then
        sampled under the mask of its own prefix, and the matcher is advanced over the emitted tokens."""
        eng = self.eng
        room = eng.sc.max_seq_len - s.position
        k = max(0, min(self.k, remaining - 1, room - 1))
        pos0 = s.position
        if k == 0:
            kw = {}
            if matcher is not None:
                _, kw["mask"], kw["mask_active"] = self._masks(matcher, [])
            toks, out = eng.step([SeqRows(s.slot, pos0, [anchor], (0,), sample_index=len(generated) + 1, **samp)], [s],
                                 tap_layers=self.taps, **kw)
            self._append_taps(out, 1, pos0, [anchor])
            self.stats["plain_steps"] += 1
            if matcher is not None:
                matcher.accept(toks[0])
            return [toks[0]]
        on_device = (hasattr(self.drafter, "propose_device") and not (self.ngram_tail and self.ngram_n)
                     and matcher is None)
        if on_device:
            # the drafts never visit the host before verification: the verify step reads them from the device and
            # brings them back together with its samples -- one host synchronisation per round
            d_dev = self.drafter.propose_device(anchor, k, pos0)
            toks, out = eng.step([SeqRows(s.slot, pos0, [anchor] + [0] * k, tuple(range(k + 1)),
                                          sample_index=len(generated) + 1, **samp)], [s], commit=False, tap_layers=self.taps,
                                 gdn_log=self.logs, gdn_to_alt=True, exact=self.verify_exact, device_ids=(1, d_dev),
                                 read_back=d_dev)
            drafts = list(out.read_back)
            rows = [anchor] + drafts
        else:
            drafts = self.drafter.propose(anchor, k, self._embed, self._lm_head, pos0)
            if self.ngram_tail and self.ngram_n:
                drafts = drafts + self.rt.ngram_tail(generated + [anchor] + drafts, self.ngram_n,
                                                     min(self.ngram_tail, max(0, remaining - 1 - len(drafts))))
            kw = {}
            if matcher is not None:
                drafts, kw["mask"], kw["mask_active"] = self._masks(matcher, drafts)
            rows = [anchor] + drafts
            n = len(rows)
            toks, out = eng.step([SeqRows(s.slot, pos0, rows, tuple(range(n)), sample_index=len(generated) + 1, **samp)], [s],
                                 commit=False, tap_layers=self.taps, gdn_log=self.logs, gdn_to_alt=True,
                                 exact=self.verify_exact, **kw)
        accepted, nxt, full = self.rt.spec_greedy_accept(drafts, toks)
        keep = accepted + 1                                  # anchor + accepted drafts are now part of the sequence
        st = eng.state
        if on_device and getattr(out, "taps_cat", None) is not None and self.commit_graphs:
            self._commit_captured(out, len(rows), keep, s.slot, pos0)
        else:
            desc = torch.tensor([[0, keep, s.slot, pos0]], dtype=torch.int32, device=eng.device)
            for li, g in enumerate(st.gdn):
                if g is not None:
                    eng.ops.gdn_replay(g, st.hv, desc, 1, self.logs[li])
            self._append_taps(out, keep, pos0, rows)
        s.position = pos0 + keep
        eng.trim_pages(s)
        self.stats["rounds"] += 1
        self.stats["accepted"] += accepted
        self.stats["proposed"] += len(drafts)
        emitted = drafts[:accepted] + [nxt]
        if matcher is not None:
            for t in emitted:
                matcher.accept(t)
        return emitted

    # ------------------------------------------------------------------ one request
    def generate(self, prompt: Sequence[int], max_new_tokens: int, stop_tokens: Sequence[int] = (), prefill_chunk: int = 2048,
                 temperature: float = 0.0, top_p: float = 1.0, top_k: int = 0, seed: int = 0) -> Tuple[List[int], dict]:
        samp = dict(temperature=temperature, top_p=top_p, top_k=top_k, seed=seed)
        self.drafter.reset()
        s = self.eng.open_sequence()
        out: List[int] = []
        try:
            tok = self.prefill(s, prompt, prefill_chunk, samp)
            out.append(tok)
            while len(out) < max_new_tokens and out[-1] not in stop_tokens:
                emitted = self.round(s, out[-1], out[:-1], max_new_tokens - len(out), samp)
                for t in emitted:
                    out.append(t)
                    if t in stop_tokens or len(out) >= max_new_tokens:
                        break
        finally:
            self.eng.close_sequence(s)
        self.stats["emitted"] = len(out)
        r = max(1, self.stats["rounds"])
        stats = dict(self.stats, tokens_per_round=round((self.stats["accepted"] + self.stats["rounds"]) / r, 3),
                     mean_accepted=round(self.stats["accepted"] / r, 3))
        return out, stats
