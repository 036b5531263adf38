"""Randomised workloads against the C++ batcher: whatever the mix of prompt lengths, budgets, cancellations and failed
steps, the scheduler must respect its budgets, never wedge, finish every request with a reason, and return every page."""
from hypothesis import HealthCheck, event, given, settings, strategies as st

from phaseshift_b200.core.native import runtime

rt = runtime()

request = st.tuples(st.integers(1, 120), st.integers(1, 40))                  # (prompt tokens, max new tokens)
action = st.one_of(st.tuples(st.just("step"), st.integers(0, 0)), st.tuples(st.just("cancel"), st.integers(0, 63)),
                   st.tuples(st.just("fail"), st.integers(0, 0)), st.tuples(st.just("submit"), st.integers(0, 63)))


@settings(max_examples=300, deadline=None, derandomize=True, suppress_health_check=[HealthCheck.too_slow])
@given(reqs=st.lists(request, min_size=1, max_size=12), slots=st.integers(1, 4), pages=st.integers(12, 40),
       budget=st.sampled_from([16, 48, 200]), script=st.lists(action, max_size=40), stop_tok=st.integers(0, 3))
def test_random_workloads_finish_within_budgets_and_leak_nothing(reqs, slots, pages, budget, script, stop_tok):
    c = rt.BatcherConfig()
    c.max_slots, c.num_pages, c.page_tokens, c.max_seq_len, c.max_step_tokens = slots, pages, 16, 160, budget
    b = rt.Batcher(c)
    free0 = b.free_pages()
    pending = list(reqs)
    ids, finished = [], {}
    # requests that can never fit the context window are refused at submit; everything else must finish

    def submit_one():
        if not pending:
            return
        n, m = pending.pop()
        try:
            ids.append(b.submit(list(range(n)), m, rt.Sampling(), [stop_tok]))
        except Exception:
            assert n + m > c.max_seq_len or n >= c.max_seq_len

    submit_one()
    sampled_counter = [0]

    def one_step(fail=False):
        b.admit()
        p = b.plan()
        if p.empty():
            return False
        d = p.to_dict()
        assert p.num_tokens() <= budget and p.num_seqs() <= slots
        rows = sum(s[4] for s in d["seqs"])
        assert rows == p.num_tokens()
        assert len({s[0] for s in d["seqs"]}) == len(d["seqs"])                      # a request appears once per step
        if fail:
            ev = b.fail(p, "injected")
        else:
            toks = []
            for _ in range(p.n_sampled):
                sampled_counter[0] += 1
                toks.append(4 + sampled_counter[0] % 7 if sampled_counter[0] % 11 else stop_tok)
            ev = b.commit(p, toks)
        for kind, rid, _ in ev:
            if kind in (1, 2):
                finished[rid] = b.request(rid)["finish_reason"]
        return True

    for what, arg in script:
        if what == "submit":
            submit_one()
        elif what == "cancel" and ids:
            rid = ids[arg % len(ids)]
            if b.cancel(rid):
                finished[rid] = "cancelled"
        else:
            one_step(fail=(what == "fail"))
    while pending:
        submit_one()
    idle_steps = 0
    for _ in range(5000):
        if b.idle():
            break
        if not one_step():
            idle_steps += 1
            assert b.active_count() > 0 or b.queued_count() > 0
            assert idle_steps < 3, "work is queued or active but nothing can be planned"
        else:
            idle_steps = 0
    assert b.idle()
    for rid in ids:
        r = b.request(rid)
        assert r is not None and r["finish_reason"] in ("stop", "length", "cancelled", "error"), (rid, r)
        if r["finish_reason"] == "length":
            assert len(r["generated"]) == r["max_new_tokens"] if "max_new_tokens" in r else True
        if r["finish_reason"] == "stop":
            assert r["generated"][-1] == stop_tok
        event("finish=" + r["finish_reason"])
        b.retire(rid)
    assert b.free_pages() == free0, "pages leaked"
    assert b.active_count() == 0 and b.queued_count() == 0
