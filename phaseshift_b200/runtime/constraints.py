"""Grammar-constrained decoding: a thin binding over the XGrammar matcher.

Same contract as the reference's TokenConstraintCompiler / TokenConstraintState
(include/phaseshift/models/qwen35/runtime/token_constraint.h:15-94): one compiler per model with a
bounded compiled-grammar cache, one matcher per request; GBNF or Structural-Tag JSON; ``fill_next_mask``
writes a bitmask of 32 tokens per int32 word (bit set = allowed) that the sampling kernel consumes;
``accept`` advances the matcher and fails closed on a token the grammar does not allow.
"""
from __future__ import annotations

from collections import OrderedDict
from typing import List, Optional, Sequence

import torch


class ConstraintError(ValueError):
    pass


class TokenConstraintState:
    def __init__(self, xgr, compiled, vocab_size: int):
        self.xgr = xgr
        self.matcher = xgr.GrammarMatcher(compiled)
        self.words = (vocab_size + 31) // 32
        self._bitmask = xgr.allocate_token_bitmask(1, vocab_size)

    def fill_next_mask(self, out_row: torch.Tensor) -> bool:
        """Fill one [ceil(vocab/32)] int32 row; returns False when every token is allowed."""
        need = self.matcher.fill_next_token_bitmask(self._bitmask, 0)
        out_row.copy_(self._bitmask[0, :out_row.numel()])
        return bool(need)

    def accept(self, token: int) -> bool:
        return bool(self.matcher.accept_token(int(token)))

    def terminated(self) -> bool:
        return bool(self.matcher.is_terminated())

    def rollback(self, n: int) -> None:
        self.matcher.rollback(n)

    def fill_draft_masks(self, drafts: Sequence[int], out: torch.Tensor) -> int:
        """Masks for verify rows 0..len(drafts): row i is the mask after accepting drafts[:i].  The matcher is
        rolled back afterwards.  Returns how many leading drafts the grammar accepts."""
        ok = 0
        self.fill_next_mask(out[0])
        for i, t in enumerate(drafts):
            if not self.accept(t):
                break
            if self.terminated():
                # a draft that completes the grammar has no successor row to mask: leave it for the target to sample
                self.rollback(1)
                break
            ok += 1
            self.fill_next_mask(out[i + 1])
        if ok:
            self.rollback(ok)
        return ok


class TokenConstraintCompiler:
    def __init__(self, vocab: List[str], vocab_size: int, stop_token_ids: Sequence[int] = (), cache_entries: int = 64,
                 vocab_type: str = "byte_level"):
        try:
            import xgrammar as xgr
        except Exception as e:  # pragma: no cover
            raise ConstraintError(f"xgrammar is not available: {e}")
        self.xgr = xgr
        vt = {"raw": xgr.VocabType.RAW, "byte_fallback": xgr.VocabType.BYTE_FALLBACK,
              "byte_level": xgr.VocabType.BYTE_LEVEL}[vocab_type]
        self.info = xgr.TokenizerInfo(vocab, vocab_type=vt, vocab_size=vocab_size,
                                      stop_token_ids=list(stop_token_ids) or None)
        self.compiler = xgr.GrammarCompiler(self.info)
        self.vocab_size = vocab_size
        self.cache: "OrderedDict[str, object]" = OrderedDict()
        self.cache_entries = cache_entries

    @staticmethod
    def from_tokenizer(tok, vocab_size: Optional[int] = None, stop_token_ids: Sequence[int] = ()):
        import xgrammar as xgr
        c = TokenConstraintCompiler.__new__(TokenConstraintCompiler)
        c.xgr = xgr
        c.info = xgr.TokenizerInfo.from_huggingface(tok, vocab_size=vocab_size, stop_token_ids=list(stop_token_ids) or None)
        c.compiler = xgr.GrammarCompiler(c.info)
        c.vocab_size = vocab_size or c.info.vocab_size
        c.cache, c.cache_entries = OrderedDict(), 64
        return c

    def _compiled(self, key: str, build):
        if key in self.cache:
            self.cache.move_to_end(key)
            return self.cache[key]
        try:
            g = build()
        except Exception as e:
            raise ConstraintError(f"grammar rejected: {e}")      # fail closed before generation starts
        self.cache[key] = g
        while len(self.cache) > self.cache_entries:
            self.cache.popitem(last=False)
        return g

    def matcher(self, grammar: Optional[str] = None, structural_tag: Optional[str] = None,
                json_schema: Optional[str] = None) -> TokenConstraintState:
        if sum(x is not None for x in (grammar, structural_tag, json_schema)) != 1:
            raise ConstraintError("exactly one of grammar / structural_tag / json_schema must be given")
        if grammar is not None:
            comp = self._compiled("g:" + grammar, lambda: self.compiler.compile_grammar(grammar))
        elif json_schema is not None:
            comp = self._compiled("j:" + json_schema, lambda: self.compiler.compile_json_schema(json_schema))
        else:
            comp = self._compiled("s:" + structural_tag, lambda: self.compiler.compile_structural_tag(structural_tag))
        return TokenConstraintState(self.xgr, comp, self.vocab_size)
