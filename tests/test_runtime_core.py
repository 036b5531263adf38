"""CPU contract tests of the C++ host runtime: pools, KV banker, scheduler/batcher, prefix index,
speculative helpers, safetensors IO, codecs."""
import numpy as np
import pytest
import torch

from phaseshift_b200.core.native import runtime

rt = runtime()


def test_checked_arithmetic():
    assert rt.align_up(13, 8) == 16 and rt.checked_mul(1 << 20, 1 << 20) == 1 << 40
    with pytest.raises(rt.RuntimeCoreError):
        rt.checked_mul(1 << 40, 1 << 40)
    assert rt.pages_for(17, 16) == 2 and rt.additional_pages(16, 1, 1, 16) == 1 and rt.additional_pages(15, 1, 1, 16) == 0


def test_slot_generations_and_pages():
    sp = rt.SlotPool(2)
    a, b = sp.acquire(), sp.acquire()
    assert sp.acquire().slot == -1
    sp.release(a)
    with pytest.raises(rt.RuntimeCoreError):
        sp.release(a)                       # stale
    c = sp.acquire()
    assert c.slot == a.slot and c.generation == a.generation + 1 and not sp.valid(a) and sp.valid(c)
    pp = rt.PagePool(4)
    got = [pp.acquire() for _ in range(4)]
    assert sorted(got[:3]) == [1, 2, 3] and got[3] == -1       # page 0 is never handed out
    pp.release(2)
    assert pp.acquire() == 2


def test_banker_safety():
    b = rt.KvBanker()
    b.available = 3
    b.add(5, 10); b.add(2, 4); b.add(2, 9)
    assert b.is_safe()                      # P1 (needs 2) can finish first, then P0, then P2
    assert b.max_safe_grant(0, 3) < 3       # giving everything to P0 would strand the others
    assert b.max_safe_grant(1, 2) == 2
    assert b.can_admit(3) and not b.can_admit(40)
    u = rt.KvBanker(); u.available = 1; u.add(4, 10); u.add(4, 10)
    assert not u.is_safe()


def _cfg(**kw):
    c = rt.BatcherConfig()
    c.max_slots, c.num_pages, c.page_tokens, c.max_seq_len, c.max_step_tokens = 4, 64, 16, 256, 48
    for k, v in kw.items():
        setattr(c, k, v)
    return c


def test_batcher_decodes_first_then_prefill_chunks():
    b = rt.Batcher(_cfg())
    r1 = b.submit(list(range(100)), 4)
    r2 = b.submit(list(range(30)), 3)
    assert b.admit() == [r1, r2]
    p = b.plan().to_dict() if False else b.plan()
    d = p.to_dict()
    # token budget 48: r1 gets a 48-token chunk, r2 waits
    assert [(s[0], s[4]) for s in d["seqs"]] == [(r1, 48)] and p.n_sampled == 0
    assert b.commit(p, []) == []
    p = b.plan(); d = p.to_dict()
    assert [(s[0], s[2], s[4]) for s in d["seqs"]] == [(r1, 48, 48)]
    b.commit(p, [])
    p = b.plan(); d = p.to_dict()           # r1 finishes its prompt (4 tokens, sampled), r2 prefills 30 and samples
    assert [(s[0], s[4], s[5]) for s in d["seqs"]] == [(r1, 4, True), (r2, 30, True)]
    ev = b.commit(p, [7, 9])
    assert ev == [(0, r1, 7), (0, r2, 9)]
    p = b.plan(); d = p.to_dict()           # both decode, decodes are planned before any prefill
    assert all(s[6] for s in d["seqs"]) and d["tokens"] == [7, 9]
    ev = b.commit(p, [8, 9])
    assert b.request(r1)["generated"] == [7, 8]


def test_batcher_finish_reasons_and_page_release():
    b = rt.Batcher(_cfg())
    free0 = b.free_pages()
    r = b.submit([1, 2, 3], 5, rt.Sampling(), [42])
    b.admit()
    p = b.plan(); b.commit(p, [10])
    p = b.plan(); ev = b.commit(p, [42])
    assert ev[-1] == (1, r, -1) and b.request(r)["finish_reason"] == "stop" and b.free_pages() == free0
    assert b.take_release_updates() == [(b.request(r)["slot"], 0, -1)]
    r2 = b.submit([1, 2, 3], 2); b.admit()
    b.commit(b.plan(), [5]); ev = b.commit(b.plan(), [6])
    assert b.request(r2)["finish_reason"] == "length"
    r3 = b.submit([1] * 10, 4); b.admit()
    assert b.cancel(r3) and b.request(r3)["finish_reason"] == "cancelled" and not b.cancel(r3)
    b.retire(r3)
    assert b.request(r3) is None


def test_batcher_checkpoint_cut_and_failure_poisoning():
    b = rt.Batcher(_cfg(max_step_tokens=2048))
    r = b.submit(list(range(100)), 2, rt.Sampling(), [], 64)
    b.admit()
    p = b.plan()
    assert p.to_dict()["seqs"][0][4] == 64                  # cut exactly at the prefix-cache boundary
    b.commit(p, [])
    assert b.request(r)["checkpoint_saved"]
    p = b.plan()
    assert p.to_dict()["seqs"][0][4] == 36
    free_before = b.free_pages()
    ev = b.fail(p, "device status 2")
    assert ev == [(2, r, -1)] and b.request(r)["finish_reason"] == "error" and b.request(r)["poisoned"]
    assert b.free_pages() > free_before


def test_batcher_admission_is_deadlock_free_under_page_pressure():
    # 3 requests that each need 4 pages at the end, only 8 usable pages: the banker never admits a set that can wedge
    b = rt.Batcher(_cfg(num_pages=9, max_slots=3, max_step_tokens=64))
    ids = [b.submit(list(range(40)), 24) for _ in range(3)]
    done = set()
    for _ in range(400):
        b.admit()
        p = b.plan()
        if p.empty():
            assert b.idle() or b.queued_count() > 0
            if b.idle():
                break
            assert b.active_count() > 0, "queued work but nothing runnable: deadlock"
            continue
        ev = b.commit(p, [1] * p.n_sampled)
        done |= {e[1] for e in ev if e[0] == 1}
    assert done == set(ids)


def test_prefix_index():
    px = rt.PrefixIndex(2, 1000, 4)
    a = list(range(10)); bb = list(range(20))
    ida, ev = px.insert(a); idb, ev = px.insert(bb)
    assert px.lookup(list(range(30))).tokens == 20 and px.lookup(bb).tokens == 10    # strictly shorter only
    assert px.lookup([9, 9, 9, 9, 9]).entry == -1
    assert px.insert([1, 2])[0] == -1                                              # below min length: benign skip
    px.lookup(list(range(11)))                                                     # touch `a` -> `bb` becomes LRU
    idc, ev = px.insert(list(range(100, 140)))
    assert ev == [idb] and px.entries() == 2


def test_spec_helpers():
    assert rt.spec_greedy_accept([5, 6, 7], [5, 6, 9, 1]) == (2, 9, False)
    assert rt.spec_greedy_accept([5, 6, 7], [5, 6, 7, 3]) == (3, 3, True)
    assert rt.spec_greedy_accept([5], [4, 8]) == (0, 4, False)
    t = rt.SpecTransaction()
    t.begin(100, 4); t.verified(2)
    assert t.commit() == 103
    with pytest.raises(rt.RuntimeCoreError):
        t.begin(1, 1)
    t.reset(); t.begin(5, 3); t.rollback()
    assert rt.ngram_tail([1, 2, 3, 9, 9, 1, 2, 3], 3, 2) == [9, 9]
    assert rt.ngram_tail([1, 2, 3], 3, 2) == []


def test_safetensors_roundtrip(tmp_path):
    p = str(tmp_path / "m.safetensors")
    w = rt.SafetensorsWriter(p)
    a = np.arange(24, dtype=np.float32).reshape(4, 6)
    bdat = (np.arange(10) % 255).astype(np.uint8)
    w.set_metadata("format", "pt")
    w.plan_tensor("a.weight", "F32", [4, 6]); w.plan_tensor("b", "U8", [10])
    w.write_chunk("a.weight", a[:2].tobytes()); w.write_chunk("a.weight", a[2:].tobytes()); w.write_chunk("b", bdat.tobytes())
    w.finish()
    r = rt.SafetensorsReader(p)
    assert r.names() == ["a.weight", "b"] and r.metadata()["format"] == "pt"
    assert r.spec("a.weight") == ("F32", [4, 6], 96)
    assert np.array_equal(r.data("a.weight").view(np.float32).reshape(4, 6), a)
    assert r.crc32("b") == w.tensor_crc("b") == rt.crc32(bdat.tobytes())
    # the file is a valid safetensors file for the reference python reader too
    from safetensors.numpy import load_file
    assert np.array_equal(load_file(p)["b"], bdat)


def test_codecs_match_torch():
    xs = torch.cat([torch.randn(4000) * 3, torch.tensor([0.0, 448.0, 500.0, -1e-4, 2 ** -10, 2 ** -9, 0.4375])])
    ref = xs.clamp(-448, 448).to(torch.float8_e4m3fn)
    got = torch.tensor([rt.e4m3_encode(float(v)) for v in xs], dtype=torch.uint8)
    assert torch.equal(got, ref.view(torch.uint8))
    back = torch.tensor([rt.e4m3_decode(int(b)) for b in got])
    assert torch.equal(back, ref.float())
    assert [rt.e2m1_decode(i) for i in range(8)] == [0, .5, 1, 1.5, 2, 3, 4, 6]
    assert rt.e2m1_encode(2.5) == 4 and rt.e2m1_encode(-0.25) == 0 and rt.e2m1_encode(-7.0) == 15 and rt.e2m1_encode(0.75) == 2


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp8"])
def test_cpp_row_quantiser_matches_torch(fmt):
    from phaseshift_b200.quant import formats
    g = torch.Generator().manual_seed(0)
    w = (torch.randn(24, 200, generator=g) * 0.05).contiguous()
    kp = formats.align_up(200, 32)
    if fmt == "nvfp4":
        q = formats.quantize_nvfp4(w, search=2)
        codes = torch.zeros(24, kp // 2, dtype=torch.uint8); scales = torch.zeros(24, kp // 16, dtype=torch.uint8)
        rt.quantize_rows_nvfp4(w.data_ptr(), 24, 200, kp, q.tensor_scale, 2, 0, codes.data_ptr(), scales.data_ptr())
    else:
        q = formats.quantize_mxfp8(w, search=1)
        codes = torch.zeros(24, kp, dtype=torch.uint8); scales = torch.zeros(24, kp // 32, dtype=torch.uint8)
        rt.quantize_rows_mxfp8(w.data_ptr(), 24, 200, kp, 1, 0, codes.data_ptr(), scales.data_ptr())
    same_scales = (scales == q.scales).float().mean().item()
    assert same_scales > 0.99, same_scales
    cq = formats.QuantizedTensor(fmt, (24, 200), kp, codes, scales, q.tensor_scale)
    # identical reconstruction error (ties in the scale search may pick a different, equally good scale)
    e_t = (formats.dequantize(q) - w).pow(2).sum().item()
    e_c = (formats.dequantize(cq) - w).pow(2).sum().item()
    assert abs(e_t - e_c) <= 1e-3 * e_t


def test_sampling_rng_host_bindings_match_python():
    from phaseshift_b200.utils.sampling import sampling_bits, sampling_uniform
    ids = np.array([0, 1, 77, 151935])
    for seed, idx, att in [(0, 0, 0), (123456789, 7, 3), (2 ** 63 + 5, 2 ** 40, 4095)]:
        bits = sampling_bits(seed, idx, att, ids)
        uni = sampling_uniform(seed, idx, att, ids)
        for j, t in enumerate(ids):
            assert rt.sampling_bits(seed, idx, att, int(t)) == int(bits[j])
            assert rt.sampling_uniform(seed, idx, att, int(t)) == pytest.approx(float(uni[j]), rel=0, abs=0)
            assert 0.0 < float(uni[j]) < 1.0


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp8", "mxfp4", "fp8_block128"])
def test_payload_round_trip_at_awkward_widths(fmt):
    """Every format packs, pads and unpacks at widths around its block boundaries: the logical shape comes back, the
    padding carries zeros, and the error stays that of the format."""
    from phaseshift_b200.quant import formats
    g = torch.Generator().manual_seed(3)
    bound = {"nvfp4": 0.14, "mxfp8": 0.04, "mxfp4": 0.16, "fp8_block128": 0.05}[fmt]
    for K in (1, 15, 16, 17, 31, 32, 33, 63, 64, 65, 127, 128, 129):
        w = torch.randn(5, K, generator=g) * 0.1
        q = formats.quantize(w, fmt)
        assert q.shape == (5, K) and q.k_padded % 32 == 0 and q.k_padded >= K
        d = formats.dequantize(q)
        assert d.shape == (5, K)
        # a handful of values is a noisy sample: the statistical bound applies from one full block on
        assert float((d - w).norm() / w.norm()) < (bound if K >= 32 else 2.5 * bound), (fmt, K)
        full = formats.dequantize(formats.QuantizedTensor(q.fmt, (5, q.k_padded), q.k_padded, q.codes, q.scales, q.tensor_scale))
        assert float(full[:, K:].abs().sum()) == 0.0, (fmt, K)                         # the padded tail decodes to zero
        kq = formats.to_kernel_format(q)
        assert kq.fmt in ("nvfp4", "mxfp8") and formats.dequantize(kq).shape == (5, K)


def test_prefix_index_random_operations_keep_its_invariants():
    """Random inserts, lookups and erasures: the stored token count never exceeds the capacity, a hit is always the longest
    stored strict prefix of the query, and evicted ids disappear."""
    import random
    rnd = random.Random(5)
    cap, max_entries, min_tokens = 200, 4, 8
    ix = rt.PrefixIndex(max_entries, cap, min_tokens)
    stored = {}
    stems = [[rnd.randrange(50) for _ in range(40)] for _ in range(3)]
    for step in range(400):
        seq = list(stems[rnd.randrange(3)][:rnd.randrange(4, 40)]) + [rnd.randrange(50) for _ in range(rnd.randrange(0, 6))]
        op = rnd.random()
        if op < 0.5:
            eid, evicted = ix.insert(seq)
            for e in evicted:
                stored.pop(e, None)
            if eid >= 0:
                stored[eid] = seq
            else:
                assert len(seq) < min_tokens or len(seq) > cap or any(v == seq for v in stored.values())
        elif op < 0.9:
            hit = ix.lookup(seq)
            best = max((len(v) for v in stored.values() if len(v) < len(seq) and seq[:len(v)] == v), default=0)
            if hit is None or hit.entry < 0:
                assert best == 0
            else:
                assert hit.tokens == best and stored[hit.entry] == seq[:hit.tokens]
        elif stored:
            e = rnd.choice(list(stored))
            ix.erase(e); stored.pop(e)
        assert ix.used_tokens() == sum(len(v) for v in stored.values()) <= cap
        assert ix.entries() == len(stored) <= max_entries
