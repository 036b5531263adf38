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
