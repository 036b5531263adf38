"""Grammar constraints end to end on CPU: the sampled stream must be a sentence of the grammar."""
import pytest
import torch

from phaseshift_b200.models.qwen35.config import tiny_config
from phaseshift_b200.models.qwen35.weights import build_engine_weights, random_hf_weights
from phaseshift_b200.runtime.engine import Engine
from phaseshift_b200.runtime.serving import ServingEngine
from phaseshift_b200.runtime.state import StateConfig

xgr = pytest.importorskip("xgrammar")


def _vocab(n):
    base = [chr(ord("a") + i) for i in range(26)] + [str(i) for i in range(10)] + ["yes", "no", " ", "{", "}", '"', ":", ","]
    return base + [f"<t{i}>" for i in range(n - len(base))]


def test_gbnf_constrained_generation():
    from phaseshift_b200.runtime.constraints import ConstraintError, TokenConstraintCompiler
    cfg = tiny_config(vocab_size=256)
    hf = random_hf_weights(cfg, seed=1)
    ew = build_engine_weights(cfg, lambda n: hf[n], "bf16", "cpu")
    vocab = _vocab(cfg.vocab_size)
    eos = cfg.vocab_size - 1
    comp = TokenConstraintCompiler(vocab, cfg.vocab_size, stop_token_ids=[eos], vocab_type="raw")
    eng = Engine(ew, "cpu", StateConfig(max_slots=2, max_seq_len=64))
    srv = ServingEngine(eng, constraint_compiler=comp)
    rid = srv.submit([1, 2, 3, 4], 12, stop_tokens=[eos], grammar='root ::= ("yes" | "no") " " [0-9] [0-9]')
    free = srv.submit([5, 6, 7], 4)                      # unconstrained neighbour in the same batch
    ev = srv.run_until_idle()
    toks = [e.token_id for e in ev if e.kind == "token" and e.request_id == rid]
    text = "".join(vocab[t] for t in toks if t != eos)
    assert text[:-3] in ("yes", "no") and text[-3] == " " and text[-2:].isdigit(), text
    assert toks[-1] == eos                               # grammar exhausted -> only the stop token remains
    assert len([e for e in ev if e.kind == "token" and e.request_id == free]) == 4
    with pytest.raises(ConstraintError):
        comp.matcher(grammar="root ::= (")                # malformed grammar is rejected before generation


def _compiler(n=256, **kw):
    from phaseshift_b200.runtime.constraints import TokenConstraintCompiler
    vocab = _vocab(n)
    return vocab, TokenConstraintCompiler(vocab, n, stop_token_ids=[n - 1], vocab_type="raw", **kw)


def _allowed(row, n):
    bits = row.to(torch.int64) & 0xFFFFFFFF
    return {t for t in range(n) if (int(bits[t // 32]) >> (t % 32)) & 1}


def test_draft_masks_follow_the_drafts_and_leave_the_matcher_where_it_was():
    """Speculative verification needs one mask per verified row: row i is the mask after the first i drafts.  The matcher
    is rolled back afterwards, and drafts the grammar refuses end the accepted run."""
    vocab, comp = _compiler()
    tid = {s: i for i, s in enumerate(vocab)}
    st = comp.matcher(grammar='root ::= "yes" " " [0-9] [0-9]')
    words = (256 + 31) // 32
    out = torch.zeros(5, words, dtype=torch.int32)
    first = torch.zeros(words, dtype=torch.int32)
    st.fill_next_mask(first)
    before = _allowed(first, 256)
    assert tid["yes"] in before and tid["no"] not in before and tid["y"] in before          # "yes" as one token or letter by letter
    drafts = [tid["yes"], tid[" "], tid["7"], tid["x"]]                                       # the fourth breaks the grammar
    ok = st.fill_draft_masks(drafts, out)
    assert ok == 3
    assert _allowed(out[0], 256) == before
    assert _allowed(out[1], 256) == {tid[" "]}
    assert _allowed(out[2], 256) == {tid[str(d)] for d in range(10)} == _allowed(out[3], 256)
    again = torch.zeros(words, dtype=torch.int32)
    st.fill_next_mask(again)
    assert _allowed(again, 256) == before                                                      # rolled back
    # a draft that completes the grammar is left for the target to sample: it has no successor row to mask
    for t in (tid["yes"], tid[" "], tid["1"]):
        assert st.accept(t)
    assert st.fill_draft_masks([tid["2"]], out) == 1 and _allowed(out[1], 256) == {255}      # only the stop token may follow
    assert st.fill_draft_masks([tid["2"], 255], out) == 1 and not st.terminated()            # the stop token itself is not pre-accepted
    assert st.accept(tid["2"]) and not st.accept(tid["3"]) and st.accept(255) and st.terminated()


def test_json_schema_structural_arguments_and_the_compile_cache():
    from phaseshift_b200.runtime.constraints import ConstraintError
    vocab, comp = _compiler(cache_entries=2)
    tid = {s: i for i, s in enumerate(vocab)}
    with pytest.raises(ConstraintError):
        comp.matcher()
    with pytest.raises(ConstraintError):
        comp.matcher(grammar='root ::= "a"', json_schema="{}")
    st = comp.matcher(json_schema='{"type": "object", "properties": {"a": {"type": "integer"}}, "required": ["a"], "additionalProperties": false}')
    row = torch.zeros((256 + 31) // 32, dtype=torch.int32)
    assert st.fill_next_mask(row) and _allowed(row, 256) == {tid["{"]}                      # an object must open
    for g in ('root ::= "a"', 'root ::= "b"', 'root ::= "c"'):
        comp.matcher(grammar=g)
    assert len(comp.cache) == 2 and 'g:root ::= "a"' not in comp.cache                     # least recently used entry evicted
    a1 = comp.matcher(grammar='root ::= "b"')
    assert list(comp.cache)[-1] == 'g:root ::= "b"'                                           # a hit moves the entry to the front
    assert a1.accept(tid["b"]) and not a1.accept(tid["b"])
