"""DFlash2 speculative decoding on CPU: the defining invariant (greedy spec == greedy target-only) for a
random drafter, an oracle drafter (full acceptance) and a half-right drafter (partial acceptance + rollback)."""
import pytest
import torch

from phaseshift_b200.models.dflash2.decoder import DFlash2SpecDecoder
from phaseshift_b200.models.dflash2.model import DFlash2Config, DFlash2Drafter, random_weights, tiny_drafter_config
from phaseshift_b200.models.qwen35.config import tiny_config
from phaseshift_b200.models.qwen35.reference import reference_greedy
from phaseshift_b200.models.qwen35.weights import build_engine_weights, random_hf_weights
from phaseshift_b200.runtime.engine import Engine
from phaseshift_b200.runtime.state import StateConfig


@pytest.fixture(scope="module")
def setup():
    cfg = tiny_config()
    hf = random_hf_weights(cfg, seed=0)
    ew = build_engine_weights(cfg, lambda n: hf[n], "bf16", "cpu")
    prompt = torch.randint(0, cfg.vocab_size, (21,), generator=torch.Generator().manual_seed(8)).tolist()
    ref = reference_greedy(cfg, hf, prompt, 24)
    return cfg, ew, prompt, ref


def _decoder(cfg, ew, k=5):
    eng = Engine(ew, "cpu", StateConfig(max_slots=1, max_seq_len=96, conv_ring=16, spec_rows=8))
    dcfg = tiny_drafter_config(cfg)
    dr = DFlash2Drafter(dcfg, random_weights(dcfg, seed=1), "cpu")
    return DFlash2SpecDecoder(eng, dr, num_drafts=k)


def test_random_drafter_keeps_greedy_output(setup):
    cfg, ew, prompt, ref = setup
    dec = _decoder(cfg, ew)
    out, stats = dec.generate(prompt, 24, prefill_chunk=8)
    assert out == ref
    assert stats["rounds"] > 0 and stats["proposed"] >= stats["accepted"]


def test_oracle_drafter_full_acceptance(setup):
    cfg, ew, prompt, ref = setup
    dec = _decoder(cfg, ew, k=5)
    full = prompt + ref

    def oracle(anchor, k, embed, lm_head, pos_start, allowed=None):
        # the token fed at position p is full[p]; the correct drafts are the next k tokens
        return full[pos_start + 1: pos_start + 1 + k]
    dec.drafter.propose = oracle
    out, stats = dec.generate(prompt, 24)
    assert out == ref
    assert stats["accepted"] == stats["proposed"] and stats["tokens_per_round"] > 3


def test_half_right_drafter_partial_acceptance_and_rollback(setup):
    cfg, ew, prompt, ref = setup
    dec = _decoder(cfg, ew, k=4)
    full = prompt + ref

    def half(anchor, k, embed, lm_head, pos_start, allowed=None):
        d = list(full[pos_start + 1: pos_start + 1 + k])
        if len(d) >= 3:
            d[2] = (d[2] + 1) % cfg.vocab_size            # third draft is wrong -> accept exactly 2, roll back the rest
        return d
    dec.drafter.propose = half
    out, stats = dec.generate(prompt, 24)
    assert out == ref
    assert 0 < stats["accepted"] < stats["proposed"]


def test_drafter_config_validation_and_save_load(tmp_path):
    cfg = tiny_config()
    dcfg = tiny_drafter_config(cfg)
    dr = DFlash2Drafter(dcfg, random_weights(dcfg, seed=2), "cpu")
    dr.save(tmp_path / "d")
    dr2 = DFlash2Drafter.from_dir(tmp_path / "d", "cpu")
    assert dr2.cfg.target_layer_ids == dcfg.target_layer_ids
    assert torch.equal(dr2.w["fc.weight"], dr.w["fc.weight"].to(torch.bfloat16).float())
    with pytest.raises(ValueError):
        DFlash2Config(is_causal=True)
    with pytest.raises(ValueError):
        DFlash2Config(target_layer_ids=[3, 3])


def test_sampled_stream_with_always_accepting_drafter_equals_plain_sampling(setup):
    """temperature > 0: verification compares drafts with the target's own samples, each row drawing with
    sample_index = tokens generated so far + row, so an oracle drafter reproduces Engine.generate token for token."""
    cfg, ew, prompt, _ = setup
    samp = dict(temperature=0.9, top_p=0.95, top_k=40, seed=1234)
    plain = Engine(ew, "cpu", StateConfig(max_slots=1, max_seq_len=96)).generate(prompt, 20, prefill_chunk=8, **samp)
    assert len(set(plain)) > 4                                   # really sampled, not a constant stream
    dec = _decoder(cfg, ew, k=5)
    full = prompt + plain
    dec.drafter.propose = lambda anchor, k, embed, lm_head, pos_start, allowed=None: full[pos_start + 1: pos_start + 1 + k]
    out, stats = dec.generate(prompt, 20, prefill_chunk=8, **samp)
    assert out == plain
    assert stats["accepted"] == stats["proposed"]
    # and with the random drafter (rejections, corrections): still the same stream
    out2, _ = _decoder(cfg, ew, k=4).generate(prompt, 20, prefill_chunk=8, **samp)
    assert out2 == plain


def test_speculative_serving_loop_matches_plain_generation(setup):
    """The serve path on speculative rounds: queued requests are served one after the other, chunked prefill feeds the
    drafter's ring per chunk, events carry every token, and the streams equal plain greedy decoding."""
    from phaseshift_b200.runtime.spec_serving import SpecServingEngine
    cfg, ew, prompt, ref = setup
    dec = _decoder(cfg, ew, k=4)
    srv = SpecServingEngine(dec, prefill_chunk=8)
    a = srv.submit(prompt, 24)
    b = srv.submit(prompt[:9], 6)
    c = srv.submit(prompt[3:], 50)
    assert srv.cancel(c) and not srv.cancel(c)
    ev = srv.run_until_idle()
    assert [e.token_id for e in ev if e.kind == "token" and e.request_id == a] == ref
    ref_b = Engine(ew, "cpu", StateConfig(max_slots=1, max_seq_len=96)).generate(prompt[:9], 6)
    assert [e.token_id for e in ev if e.kind == "token" and e.request_id == b] == ref_b
    done = {e.request_id: e.info for e in ev if e.kind == "done"}
    assert done[a]["finish_reason"] == "length" and done[a]["generated_ids"] == ref and done[a]["prefill_tokens"] == len(prompt)
    assert srv.idle() and srv.stats["rounds"] > 0 and not [e for e in ev if e.request_id == c]
    # a stop token ends the request in the middle of a round
    d = srv.submit(prompt, 24, stop_tokens=[ref[5]])
    ev = srv.run_until_idle()
    toks = [e.token_id for e in ev if e.kind == "token" and e.request_id == d]
    assert toks == ref[:ref.index(ref[5]) + 1]
    assert [e.info["finish_reason"] for e in ev if e.kind == "done"] == ["stop"]


def test_constrained_speculative_decoding_stays_in_the_grammar():
    """Grammar masks on every verify row: the emitted stream is a sentence of the grammar and equals what the plain
    constrained serving loop emits, also when the drafter proposes tokens the grammar forbids."""
    pytest.importorskip("xgrammar")
    from phaseshift_b200.runtime.constraints import TokenConstraintCompiler
    from phaseshift_b200.runtime.serving import ServingEngine
    from phaseshift_b200.runtime.spec_serving import SpecServingEngine
    cfg = tiny_config(vocab_size=256)
    hf = random_hf_weights(cfg, seed=1)
    ew = build_engine_weights(cfg, lambda n: hf[n], "bf16", "cpu")
    base = [chr(ord("a") + i) for i in range(26)] + [str(i) for i in range(10)] + ["yes", "no", " ", "{", "}", '"', ":", ","]
    vocab = base + [f"<t{i}>" for i in range(cfg.vocab_size - len(base))]
    eos = cfg.vocab_size - 1
    comp = TokenConstraintCompiler(vocab, cfg.vocab_size, stop_token_ids=[eos], vocab_type="raw")
    grammar = 'root ::= ("yes" | "no") " " [0-9] [0-9] [a-f] [a-f] [a-f]'
    plain = ServingEngine(Engine(ew, "cpu", StateConfig(max_slots=1, max_seq_len=64)), constraint_compiler=comp)
    rid = plain.submit([1, 2, 3, 4], 16, stop_tokens=[eos], grammar=grammar)
    want = [e.token_id for e in plain.run_until_idle() if e.kind == "token" and e.request_id == rid]
    eng = Engine(ew, "cpu", StateConfig(max_slots=1, max_seq_len=64, conv_ring=16, spec_rows=8))
    dcfg = tiny_drafter_config(cfg)
    for mode in ("random", "oracle"):
        dr = DFlash2Drafter(dcfg, random_weights(dcfg, seed=1), "cpu")
        dec = DFlash2SpecDecoder(eng, dr, num_drafts=4)
        if mode == "oracle":
            full = [1, 2, 3, 4] + want
            dr.propose = lambda anchor, k, embed, lm_head, pos_start, allowed=None: full[pos_start + 1: pos_start + 1 + k]
        srv = SpecServingEngine(dec, constraint_compiler=comp)
        rid = srv.submit([1, 2, 3, 4], 16, stop_tokens=[eos], grammar=grammar)
        ev = srv.run_until_idle()
        got = [e.token_id for e in ev if e.kind == "token" and e.request_id == rid]
        assert got == want, (mode, got, want)
        text = "".join(vocab[t] for t in got if t != eos)
        assert text.split(" ")[0] in ("yes", "no") and len(text.split(" ")[1]) == 5
        if mode == "oracle":
            assert dec.stats["accepted"] > 0


def test_speculative_serving_restores_prefixes_with_the_drafter_ring(setup):
    """Prefix cache under speculative serving: a prompt-boundary checkpoint and a terminal checkpoint both keep the
    drafter's context ring; requests that hit them skip the prefill, draft from the restored ring, and still emit the
    plain greedy stream."""
    from phaseshift_b200.runtime.spec_serving import SpecServingEngine
    cfg, ew, prompt, ref = setup
    dec = _decoder(cfg, ew, k=4)
    srv = SpecServingEngine(dec, prefill_chunk=8, prefix_cache_tokens=512, prefix_cache_entries=4, prefix_min_tokens=8)
    a = srv.submit(prompt, 10, checkpoint_position=16)
    ev = srv.run_until_idle()
    done = {e.request_id: e.info for e in ev if e.kind == "done"}
    assert done[a]["generated_ids"] == ref[:10] and done[a]["cache_checkpoint_tokens"] == 16
    other = prompt[:16] + [7, 8, 9, 10, 11]
    b = srv.submit(other, 6)
    ev = srv.run_until_idle()
    done = {e.request_id: e.info for e in ev if e.kind == "done"}
    assert done[b]["restored_tokens"] == 16 and done[b]["prefill_tokens"] == len(other) - 16
    assert done[b]["generated_ids"] == Engine(ew, "cpu", StateConfig(max_slots=1, max_seq_len=96)).generate(other, 6)
    turn2 = prompt + ref[:10] + [3, 4, 5]                   # continues the first conversation: terminal checkpoint
    c = srv.submit(turn2, 5)
    ev = srv.run_until_idle()
    done = {e.request_id: e.info for e in ev if e.kind == "done"}
    assert done[c]["restored_tokens"] >= len(prompt) + 8
    assert done[c]["generated_ids"] == Engine(ew, "cpu", StateConfig(max_slots=1, max_seq_len=96)).generate(turn2, 5)


def test_random_draft_counts_chunks_and_prompts_keep_the_greedy_stream(setup):
    """Speculative rounds under random draft counts, prefill chunk sizes, prompt cuts and output lengths: the stream is
    always the plain greedy one (whatever the drafter proposes, whatever gets rolled back)."""
    from hypothesis import HealthCheck, given, settings, strategies as st
    from phaseshift_b200.runtime.spec_serving import SpecServingEngine
    cfg, ew, prompt, ref = setup
    plain = Engine(ew, "cpu", StateConfig(max_slots=1, max_seq_len=96))
    memo = {}

    def greedy(p, n):
        if (tuple(p), n) not in memo:
            memo[(tuple(p), n)] = plain.generate(list(p), n)
        return memo[(tuple(p), n)]

    @settings(max_examples=10, deadline=None, derandomize=True, suppress_health_check=list(HealthCheck))
    @given(k=st.integers(1, 7), chunk=st.sampled_from([4, 8, 32]), seed=st.integers(0, 3), cache=st.booleans(),
           reqs=st.lists(st.tuples(st.integers(0, 6), st.integers(5, 21), st.integers(1, 14), st.booleans()), min_size=1, max_size=3))
    def run(k, chunk, seed, cache, reqs):
        eng = Engine(ew, "cpu", StateConfig(max_slots=1, max_seq_len=96, conv_ring=16, spec_rows=8))
        dcfg = tiny_drafter_config(cfg)
        dec = DFlash2SpecDecoder(eng, DFlash2Drafter(dcfg, random_weights(dcfg, seed=seed), "cpu"), num_drafts=k)
        kw = dict(prefix_cache_tokens=256, prefix_cache_entries=3, prefix_min_tokens=8) if cache else {}
        srv = SpecServingEngine(dec, prefill_chunk=chunk, **kw)
        last = None
        for lo, hi, n, follow in reqs:
            p = prompt[lo:max(hi, lo + 2)]
            if follow and last is not None and len(last) + 3 + n < 90:
                p = last + [5, 6, 7]                     # a next turn of the previous conversation (terminal checkpoint)
            rid = srv.submit(p, n, checkpoint_position=8 if cache and len(p) > 8 else 0)
            ev = srv.run_until_idle()
            got = [e.token_id for e in ev if e.kind == "token" and e.request_id == rid]
            assert got == greedy(p, n), (k, chunk, seed, cache, len(p), n)
            last = p + got
        assert srv.idle()
    run()
