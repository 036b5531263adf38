"""Continuous batching + prefix cache through the public serving loop on CPU (reference ops, fp32)."""
import pytest
import torch

from phaseshift_b200.models.qwen35.config import tiny_config
from phaseshift_b200.models.qwen35.reference import reference_greedy
from phaseshift_b200.models.qwen35.weights import build_engine_weights, random_hf_weights
from phaseshift_b200.runtime.engine import Engine
from phaseshift_b200.runtime.serving import ServingEngine
from phaseshift_b200.runtime.state import StateConfig


@pytest.fixture(scope="module")
def tiny():
    cfg = tiny_config()
    hf = random_hf_weights(cfg, seed=0)
    return cfg, hf, build_engine_weights(cfg, lambda n: hf[n], "bf16", "cpu")


def _prompt(cfg, n, seed):
    return torch.randint(0, cfg.vocab_size, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def _collect(events):
    toks, done = {}, {}
    for e in events:
        if e.kind == "token":
            toks.setdefault(e.request_id, []).append(e.token_id)
        else:
            done[e.request_id] = e
    return toks, done


def test_concurrent_requests_match_oracle(tiny):
    cfg, hf, ew = tiny
    eng = Engine(ew, "cpu", StateConfig(max_slots=3, max_seq_len=96, page_tokens=16))
    srv = ServingEngine(eng, max_step_tokens=24)
    prompts = [_prompt(cfg, n, s) for n, s in [(20, 1), (33, 2), (9, 3), (17, 4)]]
    ids = [srv.submit(p, 6) for p in prompts]          # 4 requests, 3 slots: the last one queues
    toks, done = _collect(srv.run_until_idle())
    for rid, p in zip(ids, prompts):
        assert toks[rid] == reference_greedy(cfg, hf, p, 6)
        assert done[rid].info["generated_ids"] == toks[rid] and done[rid].info["finish_reason"] == "length"
    assert eng.state.block_table.max().item() == -1      # every page returned


def test_prefix_cache_hit_gives_identical_tokens(tiny):
    cfg, hf, ew = tiny
    eng = Engine(ew, "cpu", StateConfig(max_slots=2, max_seq_len=160, page_tokens=16))
    srv = ServingEngine(eng, max_step_tokens=64, prefix_cache_tokens=512, prefix_cache_entries=4, prefix_min_tokens=16)
    shared = _prompt(cfg, 70, 9)
    p1, p2 = shared + _prompt(cfg, 11, 10), shared + _prompt(cfg, 8, 11)
    r1 = srv.submit(p1, 5, checkpoint_position=70)
    toks, done = _collect(srv.run_until_idle())
    assert toks[r1] == reference_greedy(cfg, hf, p1, 5)
    assert done[r1].info["cache_checkpoint_tokens"] == 70 and done[r1].info["restored_tokens"] == 0
    r2 = srv.submit(p2, 5, checkpoint_position=70)
    toks, done = _collect(srv.run_until_idle())
    assert done[r2].info["restored_tokens"] == 70 and done[r2].info["prefill_tokens"] == len(p2) - 70
    assert toks[r2] == reference_greedy(cfg, hf, p2, 5)
    assert srv.prefix.summary()["hits"] == 1


def test_cancel_and_stop_token(tiny):
    cfg, hf, ew = tiny
    eng = Engine(ew, "cpu", StateConfig(max_slots=2, max_seq_len=64))
    srv = ServingEngine(eng)
    p = _prompt(cfg, 12, 5)
    ref = reference_greedy(cfg, hf, p, 6)
    r1 = srv.submit(p, 6, stop_tokens=[ref[2]])
    r2 = srv.submit(_prompt(cfg, 10, 6), 50)
    ev = srv.step()
    assert srv.cancel(r2) and srv.request(r2)["finish_reason"] == "cancelled"
    toks, done = _collect(ev + srv.run_until_idle())
    assert toks[r1] == ref[:3] and done[r1].info["finish_reason"] == "stop"


def test_terminal_checkpoint_serves_the_next_turn_and_pool_is_bounded(tiny):
    """A finished request leaves a checkpoint of everything it fed to the model; the next turn of the conversation
    (old prompt + old answer + new text) restores it and only prefills the new part.  The cache's storage is a pool
    allocated once: saving more than fits evicts, never grows."""
    cfg, hf, ew = tiny
    eng = Engine(ew, "cpu", StateConfig(max_slots=2, max_seq_len=200, page_tokens=16))
    srv = ServingEngine(eng, max_step_tokens=64, prefix_cache_tokens=256, prefix_cache_entries=3, prefix_min_tokens=16,
                        terminal_checkpoints=True)
    pool0 = srv.prefix.pool_bytes()
    p1 = _prompt(cfg, 40, 21)
    r1 = srv.submit(p1, 9)
    toks, done = _collect(srv.run_until_idle())
    a1 = toks[r1]
    assert a1 == reference_greedy(cfg, hf, p1, 9) and srv.stats["terminal_checkpoints"] == 1
    p2 = p1 + a1 + _prompt(cfg, 6, 22)                      # second turn
    r2 = srv.submit(p2, 5)
    toks, done = _collect(srv.run_until_idle())
    assert done[r2].info["restored_tokens"] == len(p1) + len(a1) - 1          # the last token was sampled, never fed
    assert done[r2].info["prefill_tokens"] == len(p2) - done[r2].info["restored_tokens"]
    assert toks[r2] == reference_greedy(cfg, hf, p2, 5)
    for seed in range(30, 36):                              # more conversations than the pool holds
        srv.submit(_prompt(cfg, 50 + seed, seed), 3)
    srv.run_until_idle()
    s = srv.prefix.summary()
    assert srv.prefix.pool_bytes() == pool0 and s["entries"] <= 3 and s["evictions"] > 0
    assert s["pool_pages_free"] + sum(len(x.pages) for x in srv.prefix.snaps.values()) == srv.prefix.pool_pages


def test_random_arrivals_budgets_and_shared_prefixes_stay_token_exact(tiny):
    """Whatever the arrival order, step budget, slot count and prefix-cache state, every request's tokens are those of the
    whole-sequence oracle run on its prompt alone (scheduling must never leak into the arithmetic of a sequence)."""
    from hypothesis import HealthCheck, given, settings, strategies as st
    cfg, hf, ew = tiny
    oracle = {}

    def ref(p, n):
        key = (tuple(p), n)
        if key not in oracle:
            oracle[key] = reference_greedy(cfg, hf, p, n)
        return oracle[key]

    bases = [_prompt(cfg, 40, 100 + i) for i in range(2)]

    @settings(max_examples=15, deadline=None, derandomize=True, suppress_health_check=list(HealthCheck))
    @given(slots=st.integers(1, 3), budget=st.sampled_from([8, 24, 64]), cache=st.booleans(),
           reqs=st.lists(st.tuples(st.integers(0, 1), st.integers(17, 40), st.integers(0, 9), st.integers(1, 5), st.integers(0, 3)),
                         min_size=2, max_size=5))
    def run(slots, budget, cache, reqs):
        eng = Engine(ew, "cpu", StateConfig(max_slots=slots, max_seq_len=96, page_tokens=16))
        kw = dict(prefix_cache_tokens=256, prefix_cache_entries=3, prefix_min_tokens=16) if cache else {}
        srv = ServingEngine(eng, max_step_tokens=budget, **kw)
        want, events = {}, []
        for base, keep, tail, new, delay in reqs:
            p = bases[base][:keep] + _prompt(cfg, tail, 200 + tail)
            rid = srv.submit(p, new, checkpoint_position=16 if cache else 0)
            want[rid] = ref(p, new)
            for _ in range(delay):                       # later requests arrive while earlier ones are running
                events += srv.step()
        events += srv.run_until_idle()
        toks, done = _collect(events)
        for rid, w in want.items():
            assert toks[rid] == w, (slots, budget, cache, rid)
            assert done[rid].info["finish_reason"] == "length"
        assert eng.state.block_table.max().item() == -1
    run()
