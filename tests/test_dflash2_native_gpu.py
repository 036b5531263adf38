"""DFlash2 drafter kernels and the native executor against the torch drafter (plain PyTorch restatement of the
same mathematics), and the speculative round with device-side drafts and graph-captured verification."""
import ctypes

import pytest
import torch

from phaseshift_b200.models.qwen35.config import tiny_config
from phaseshift_b200.models.qwen35.weights import build_engine_weights, random_hf_weights
from phaseshift_b200.runtime.state import StateConfig

pytestmark = pytest.mark.gpu


def _rel_err(a, b):
    a, b = a.float(), b.float()
    return float((a - b).norm() / (b.norm() + 1e-12))


def _lib():
    from phaseshift_b200.ops import _lib
    return _lib


def _gen(seed):
    return torch.Generator(device="cuda").manual_seed(seed)


def test_rmsnorm_direct_matches_torch():
    from phaseshift_b200.models.dflash2.model import _rms
    L = _lib()
    g = _gen(1)
    for rows, H in ((1, 256), (7, 5120), (16, 1024)):
        x = (torch.randn(rows, H, device="cuda", generator=g) * 3).to(torch.bfloat16)
        w = (1 + 0.1 * torch.randn(H, device="cuda", generator=g)).to(torch.bfloat16)
        out = torch.empty_like(x)
        L.call("ps_dfl_rmsnorm", L.ptr(x), L.c_int(H), L.ptr(w), L.c_float(1e-6), L.c_int(rows), L.c_int(H), L.ptr(out), L.c_int(H))
        ref = _rms(x, w, 1e-6)
        assert _rel_err(out, ref) < 4e-3
        assert float((out.float() - ref.float()).abs().max()) <= 0.04 * float(ref.float().abs().max())


@pytest.mark.parametrize("phase", [0, 1])
def test_conv_apply_matches_torch(phase):
    L = _lib()
    g = _gen(2 + phase)
    T, H, gs = 9, 512, 64
    groups = H // gs
    x = torch.randn(T, H, device="cuda", generator=g).to(torch.bfloat16)
    dyn = (0.3 * torch.randn(T, 4 * groups, device="cuda", generator=g)).to(torch.bfloat16)
    base = torch.randn(2, 2, H, device="cuda", generator=g).to(torch.bfloat16)
    res = torch.randn(T, H, device="cuda", generator=g).to(torch.bfloat16)
    out = torch.empty_like(x)
    for residual in (None, res):
        L.call("ps_dfl_conv_apply", L.ptr(x), L.c_int(H), L.ptr(dyn), L.c_int(4 * groups), L.ptr(base), L.c_int(phase), L.c_int(T),
               L.c_int(H), L.c_int(groups), L.ptr(residual), L.c_int(H if residual is not None else 0), L.ptr(out), L.c_int(H))
        d = dyn.float().reshape(T, 2, 2, groups)
        k = base.float()[phase][None] + d[:, phase].repeat_interleave(gs, -1)
        prev = torch.cat([torch.zeros_like(x[:1]), x[:-1]], 0).float()
        ref = k[:, 0] * x.float() + k[:, 1] * prev
        if residual is not None:
            ref = ref + residual.float()
        assert _rel_err(out, ref) < 6e-3


@pytest.mark.parametrize("T,H,C", [(1, 256, 8), (8, 5120, 40), (16, 1024, 16)])
def test_fused_norm_projection_conv_matches_torch(T, H, C):
    """norm -> 4C-output projection -> conv prepare (mode 1) / normalised rows (mode 0) in one launch."""
    from phaseshift_b200.models.dflash2.model import _rms
    L = _lib()
    g = _gen(20 + T)
    x = (torch.randn(T, H, device="cuda", generator=g) * 2).to(torch.bfloat16)
    nw = (1 + 0.1 * torch.randn(H, device="cuda", generator=g)).to(torch.bfloat16)
    wp = (0.05 * torch.randn(4 * C, H, device="cuda", generator=g)).to(torch.bfloat16)
    base = torch.randn(2, 2, H, device="cuda", generator=g).to(torch.bfloat16)
    n = _rms(x, nw, 1e-6)
    proj_ref = n.float() @ wp.float().T
    for mode in (0, 1):
        y = torch.empty_like(x)
        proj = torch.empty(T, 4 * C, device="cuda", dtype=torch.bfloat16 if mode else torch.float32)
        L.call("ps_dfl_norm_proj4", L.ptr(x), L.c_int(H), L.ptr(nw), L.c_float(1e-6), L.ptr(wp), L.c_int(C), L.c_int(T), L.c_int(H),
               L.c_int(mode), L.ptr(base if mode else None), L.ptr(proj), L.c_int(4 * C), L.ptr(y), L.c_int(H))
        assert _rel_err(proj, proj_ref) < (1e-2 if mode else 2e-3)
        if mode == 0:
            assert _rel_err(y, n) < 4e-3
        else:
            gs = H // C
            d = proj.float().reshape(T, 2, 2, C)
            k = base.float()[0][None] + d[:, 0].repeat_interleave(gs, -1)
            prev = torch.cat([torch.zeros_like(n[:1]), n[:-1]], 0).float()
            assert _rel_err(y, k[:, 0] * n.float() + k[:, 1] * prev) < 8e-3


def test_headnorm_rope_matches_torch():
    from phaseshift_b200.models.dflash2.model import _rms, _rope
    L = _lib()
    g = _gen(4)
    T, hq, hkv, D = 6, 8, 2, 128
    x = torch.randn(T, (hq + 2 * hkv) * D, device="cuda", generator=g).to(torch.bfloat16)
    wq = (1 + 0.1 * torch.randn(D, device="cuda", generator=g)).to(torch.bfloat16)
    wk = (1 + 0.1 * torch.randn(D, device="cuda", generator=g)).to(torch.bfloat16)
    pos = torch.arange(1000, 1000 + T, device="cuda", dtype=torch.int32)
    ref_q = _rope(_rms(x[:, :hq * D].reshape(T, hq, D), wq, 1e-6), pos, 1e7).reshape(T, -1)
    ref_k = _rope(_rms(x[:, hq * D:(hq + hkv) * D].reshape(T, hkv, D), wk, 1e-6), pos, 1e7).reshape(T, -1)
    v_before = x[:, (hq + hkv) * D:].clone()
    L.call("ps_dfl_headnorm_rope", L.ptr(x), L.c_int(x.stride(0)), L.c_int(hq + hkv), L.c_int(D), L.ptr(wq), L.c_int(hq), L.ptr(wk),
           L.c_float(1e-6), L.ptr(pos), L.c_float(1e7), L.c_int(T), L.ptr(x), L.c_int(x.stride(0)))
    assert _rel_err(x[:, :hq * D], ref_q) < 8e-3
    assert _rel_err(x[:, hq * D:(hq + hkv) * D], ref_k) < 8e-3
    assert torch.equal(x[:, (hq + hkv) * D:], v_before)


def _attention_ref(q, kb, vb, k_ring, v_ring, ring_pos, pos, window, hq, hkv, D):
    T = q.shape[0]
    G = hq // hkv
    K = torch.cat([k_ring, kb], 0).reshape(-1, hkv, D).repeat_interleave(G, 1).float()
    V = torch.cat([v_ring, vb], 0).reshape(-1, hkv, D).repeat_interleave(G, 1).float()
    kpos = torch.cat([ring_pos.long(), pos.long()], 0)
    s = torch.einsum("thd,shd->hts", q.reshape(T, hq, D).float(), K) * (D ** -0.5)
    ok = ((pos.long()[:, None] - kpos[None, :]).abs() < window) & (kpos >= 0)[None, :]
    s = s.masked_fill(~ok[None], float("-inf"))
    return torch.einsum("hts,shd->thd", torch.softmax(s, -1), V).reshape(T, -1)


@pytest.mark.parametrize("T", [1, 8, 16])
@pytest.mark.parametrize("fill", [0, 17, 200])
def test_ring_attention_matches_torch(fill, T):
    L = _lib()
    g = _gen(5 + fill)
    hq, hkv, D, W = 8, 2, 128, 128
    qd, kvd = hq * D, hkv * D
    qkv = torch.randn(T, qd + 2 * kvd, device="cuda", generator=g).to(torch.bfloat16)
    k_ring = torch.randn(W, kvd, device="cuda", generator=g).to(torch.bfloat16)
    v_ring = torch.randn(W, kvd, device="cuda", generator=g).to(torch.bfloat16)
    ring_pos = torch.full((W,), -1, dtype=torch.int32, device="cuda")
    for p in range(max(0, fill - W), fill):         # the ring holds the last W committed positions
        ring_pos[p % W] = p
    pos = torch.arange(fill, fill + T, device="cuda", dtype=torch.int32)
    out = torch.empty(T, qd, device="cuda", dtype=torch.bfloat16)
    L.lib().ps_dfl_ring_attention_workspace_floats.restype = ctypes.c_longlong
    n_ws = int(L.lib().ps_dfl_ring_attention_workspace_floats(L.c_int(T), L.c_int(W), L.c_int(hkv)))
    ws = torch.full((n_ws,), float("nan"), device="cuda")
    L.call("ps_dfl_ring_attention", L.ptr(qkv), L.c_int(qkv.stride(0)), L.ptr(qkv[:, qd:]), L.ptr(qkv[:, qd + kvd:]),
           L.c_int(qkv.stride(0)), L.ptr(k_ring), L.ptr(v_ring), L.ptr(ring_pos), L.ptr(pos), L.c_int(T), L.c_int(W), L.c_int(hq),
           L.c_int(hkv), L.c_int(D), L.c_float(D ** -0.5), L.ptr(out), L.c_int(qd), L.ptr(ws))
    ref = _attention_ref(qkv[:, :qd], qkv[:, qd:qd + kvd], qkv[:, qd + kvd:], k_ring, v_ring, ring_pos, pos, W, hq, hkv, D)
    assert _rel_err(out, ref) < 6e-3


def test_kv_ring_append_matches_torch():
    from phaseshift_b200.models.dflash2.model import _rms, _rope
    L = _lib()
    g = _gen(9)
    n, layers, hkv, D, W = 37, 3, 2, 128, 32
    kvd = hkv * D
    kv = torch.randn(n, layers * 2 * kvd, device="cuda", generator=g).to(torch.bfloat16)
    kw = (1 + 0.1 * torch.randn(layers, D, device="cuda", generator=g)).to(torch.bfloat16)
    k_ring = torch.zeros(layers, W, kvd, device="cuda", dtype=torch.bfloat16)
    v_ring = torch.zeros_like(k_ring)
    ring_pos = torch.full((W,), -1, dtype=torch.int32, device="cuda")
    pos0 = 50
    # a call never holds two rows of one slot: append in pieces of at most W rows, like the executor does
    for c0 in range(0, n, W):
        m = min(W, n - c0)
        L.call("ps_dfl_kv_ring_append", L.ptr(kv[c0:]), L.c_int(kv.stride(0)), L.c_int(layers), L.c_int(hkv), L.c_int(D), L.ptr(kw),
               L.c_float(1e-6), L.c_int(pos0 + c0), L.c_int(W), L.c_float(1e7), L.c_int(m), L.ptr(k_ring), L.ptr(v_ring),
               L.ptr(ring_pos), L.ptr(None))
    pos = torch.arange(pos0, pos0 + n, device="cuda")
    for l in range(layers):
        k = kv[:, l * 2 * kvd:l * 2 * kvd + kvd].reshape(n, hkv, D)
        v = kv[:, l * 2 * kvd + kvd:(l + 1) * 2 * kvd]
        kr = _rope(_rms(k, kw[l], 1e-6), pos, 1e7).reshape(n, -1)
        for r in range(n - W, n):                    # the survivors
            slot = (pos0 + r) % W
            assert int(ring_pos[slot]) == pos0 + r
            assert _rel_err(k_ring[l, slot], kr[r]) < 8e-3
            assert torch.equal(v_ring[l, slot], v[r])
    # device-side control: keep 3 of 8 offered rows, starting at position 200
    before_k, before_pos = k_ring.clone(), ring_pos.clone()
    ctl = torch.tensor([0, 3, 0, 200], dtype=torch.int32, device="cuda")
    L.call("ps_dfl_kv_ring_append", L.ptr(kv), L.c_int(kv.stride(0)), L.c_int(layers), L.c_int(hkv), L.c_int(D), L.ptr(kw),
           L.c_float(1e-6), L.c_int(0), L.c_int(W), L.c_float(1e7), L.c_int(8), L.ptr(k_ring), L.ptr(v_ring), L.ptr(ring_pos), L.ptr(ctl))
    touched = {(200 + r) % W for r in range(3)}
    for slot in range(W):
        if slot in touched:
            assert int(ring_pos[slot]) == 200 + [r for r in range(3) if (200 + r) % W == slot][0]
        else:
            assert int(ring_pos[slot]) == int(before_pos[slot]) and torch.equal(k_ring[:, slot], before_k[:, slot])


def test_feature_concat_and_noise_ids():
    L = _lib()
    g = _gen(10)
    rows, H = 5, 256
    big = torch.randn(rows, 3 * H + 64, device="cuda", generator=g).to(torch.bfloat16)
    taps = [big[:, :H], torch.randn(rows, H, device="cuda", generator=g).to(torch.bfloat16), big[:, H + 64:2 * H + 64]]
    out = torch.empty(rows, 3 * H, device="cuda", dtype=torch.bfloat16)
    srcs = (ctypes.c_void_p * 3)(*[t.data_ptr() for t in taps])
    lds = (ctypes.c_int * 3)(*[t.stride(0) for t in taps])
    L.call("ps_dfl_feature_concat", srcs, lds, L.c_int(3), L.c_int(rows), L.c_int(H), L.ptr(out))
    assert torch.equal(out, torch.cat(taps, 1))
    ctl = torch.tensor([77, 1234], dtype=torch.int32, device="cuda")
    ids = torch.zeros(16, dtype=torch.int32, device="cuda")
    pos = torch.zeros(16, dtype=torch.int32, device="cuda")
    L.call("ps_dfl_noise_ids", L.ptr(ctl), L.c_int(3), L.c_int(7), L.ptr(ids), L.ptr(pos))
    assert ids[:8].tolist() == [77] + [3] * 7 and pos[:8].tolist() == list(range(1234, 1242))


def test_candidate_selector_matches_torch():
    L = _lib()
    g = _gen(11)
    K, kk, rank, V = 7, 16, 64, 4096
    top_ids = torch.stack([torch.randperm(V, device="cuda", generator=g)[:kk] for _ in range(K)]).to(torch.int32)
    top_l = torch.sort(torch.randn(K, kk, device="cuda", generator=g), descending=True).values.contiguous()
    hproj = torch.randn(K, rank, device="cuda", generator=g)
    pred = torch.randn(V, rank, device="cuda", generator=g).to(torch.bfloat16)
    succ = torch.randn(V, rank, device="cuda", generator=g).to(torch.bfloat16)
    anchor = torch.tensor([123], dtype=torch.int32, device="cuda")
    out = torch.zeros(K, dtype=torch.int32, device="cuda")
    L.call("ps_dfl_select", L.ptr(top_ids), L.ptr(top_l), L.c_int(kk), L.ptr(hproj), L.c_int(rank), L.ptr(pred), L.ptr(succ),
           L.ptr(anchor), L.c_int(0), L.c_int(K), L.c_int(V), L.ptr(out))
    prev, ref = 123, []
    for r in range(K):
        score = top_l[r].double() + (pred[prev].double() * hproj[r].double()) @ succ[top_ids[r].long()].double().T
        prev = int(top_ids[r][int(torch.argmax(score))])
        ref.append(prev)
    assert out.tolist() == ref


def _tiny_pair(fmt, preset="bf16", seed=1):
    from phaseshift_b200.models.dflash2.model import DFlash2Drafter, random_weights, tiny_drafter_config
    from phaseshift_b200.models.dflash2.native import DFlash2NativeDrafter
    from phaseshift_b200.runtime.engine import Engine
    cfg = tiny_config()
    hf = random_hf_weights(cfg, seed=0)
    ew = build_engine_weights(cfg, lambda n: hf[n], preset, "cuda")
    eng = Engine(ew, "cuda", StateConfig(max_slots=1, max_seq_len=128, conv_ring=16, spec_rows=8))
    dcfg = tiny_drafter_config(cfg, head_dim=128, num_attention_heads=4, num_key_value_heads=2)
    w = random_weights(dcfg, seed)
    return cfg, ew, eng, dcfg, DFlash2Drafter(dcfg, w, "cuda", torch.bfloat16), DFlash2NativeDrafter(dcfg, w, eng, fmt)


def test_native_drafter_matches_torch_drafter_bf16():
    """Unquantised weights: ring contents, final hidden rows and target-head logits of the kernels against the torch
    drafter, through the same context appends and two proposals (the second replays the captured graph)."""
    from phaseshift_b200.models.dflash2.decoder import DFlash2SpecDecoder
    cfg, ew, eng, dcfg, tdr, ndr = _tiny_pair("bf16")
    dec = DFlash2SpecDecoder(eng, tdr, num_drafts=5)
    tdr.use_graph = False
    g = _gen(3)
    taps = [torch.randn(40, cfg.hidden_size, device="cuda", generator=g).to(torch.bfloat16) for _ in dcfg.target_layer_ids]
    tdr.append_context(taps, 0)
    ndr.append_context(taps, 0)
    live = ndr.ring_pos >= 0
    assert torch.equal(ndr.ring_pos.long(), tdr.ring_pos)
    for l in range(dcfg.num_hidden_layers):
        assert _rel_err(ndr.k_ring[l][live], tdr.k_ring[l][live]) < 2e-2
        assert _rel_err(ndr.v_ring[l][live], tdr.v_ring[l][live]) < 2e-2
    for rep, (anchor, pos0) in enumerate(((7, 40), (9, 40), (11, 40))):
        got = ndr.propose(anchor, 5, pos_start=pos0)
        ids = torch.tensor([anchor] + [dcfg.mask_token_id] * 5, device="cuda")
        h = tdr.backbone(dec._embed(ids).to(torch.bfloat16), torch.arange(pos0, pos0 + 6, device="cuda"))[1:]
        assert _rel_err(ndr.last_hidden, h) < 3e-2, rep
        logits = dec._lm_head(h)
        assert _rel_err(ndr.last_logits, logits) < 3e-2, rep
        ref = tdr.select(h, logits.float(), anchor)
        assert len(got) == 5 and sum(a == b for a, b in zip(got, ref)) >= 3, (got, ref)
    assert 5 in ndr._graphs and int(eng.ops.status[0]) == 0


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp8"])
def test_native_drafter_quantised_tracks_torch(fmt):
    """Quantised backbone (tensor-core projections with quantised activations): hidden rows stay close to the
    unquantised torch drafter; proposals are deterministic across graph replays."""
    from phaseshift_b200.models.dflash2.decoder import DFlash2SpecDecoder
    cfg, ew, eng, dcfg, tdr, ndr = _tiny_pair(fmt)
    dec = DFlash2SpecDecoder(eng, tdr, num_drafts=5)
    g = _gen(4)
    taps = [torch.randn(33, cfg.hidden_size, device="cuda", generator=g).to(torch.bfloat16) for _ in dcfg.target_layer_ids]
    tdr.append_context(taps, 0)
    ndr.append_context(taps, 0)
    a = ndr.propose(5, 5, pos_start=33)
    b = ndr.propose(5, 5, pos_start=33)
    c = ndr.propose(5, 5, pos_start=33)
    assert a == b == c
    ids = torch.tensor([5] + [dcfg.mask_token_id] * 5, device="cuda")
    h = tdr.backbone(dec._embed(ids).to(torch.bfloat16), torch.arange(33, 39, device="cuda"))[1:]
    # 4-bit weights AND 4-bit activations through ~20 chained projections of random weights
    assert _rel_err(ndr.last_hidden, h) < (0.4 if fmt == "nvfp4" else 0.15)
    assert int(eng.ops.status[0]) == 0


@pytest.mark.parametrize("preset,fmt", [("bf16", "bf16"), ("nvfp4", "nvfp4")])
def test_speculative_round_with_native_drafter_is_exact(preset, fmt):
    """Device-side drafts + graph-captured verification: the emitted stream equals plain greedy decoding, a drafter
    that proposes the true continuation is fully accepted, and every round makes its proposal without a read-back."""
    from phaseshift_b200.models.dflash2.decoder import DFlash2SpecDecoder
    from phaseshift_b200.runtime.engine import Engine
    cfg, ew, eng, dcfg, tdr, ndr = _tiny_pair(fmt, preset)
    prompt = torch.randint(0, cfg.vocab_size, (21,), generator=torch.Generator().manual_seed(8)).tolist()
    dec = DFlash2SpecDecoder(eng, ndr, num_drafts=5)
    ref_eng = Engine(ew, "cuda", StateConfig(max_slots=1, max_seq_len=128))
    ref_eng.set_uniform_arithmetic(True)
    plain = ref_eng.generate(prompt, 24, prefill_chunk=8)
    out, stats = dec.generate(prompt, 24, prefill_chunk=8)
    assert out == plain
    assert stats["rounds"] > 0 and any(isinstance(k, tuple) for k in eng.graphs)        # verification replayed a graph
    assert dec._commit_graphs                                                           # ... and so did the commit
    # the same with graphs off (eager verification): same stream
    eng.graph_variants = False
    ndr.use_graph = False
    dec.commit_graphs = False
    out2, _ = dec.generate(prompt, 24, prefill_chunk=8)
    assert out2 == plain
    dec.commit_graphs = True
    # oracle drafts on the device
    eng.graph_variants = True
    full = prompt + plain
    ndr.propose_device = lambda a, k, pos: torch.tensor(full[pos + 1: pos + 1 + k], dtype=torch.int32, device="cuda")
    dec.stats = {k: 0 for k in dec.stats}
    out3, stats3 = dec.generate(prompt, 24, prefill_chunk=8)
    assert out3 == plain and stats3["accepted"] == stats3["proposed"], stats3
    assert int(eng.ops.status[0]) == 0


@pytest.mark.parametrize("preset", ["nvfp4", "bf16"])
def test_draft_vocabulary_head(preset):
    """The drafter's head restricted to a subset of the target vocabulary: with the identity subset the proposals equal
    the full head's; with a real subset every proposal lies inside it; speculative decoding stays exact either way."""
    from phaseshift_b200.models.dflash2.decoder import DFlash2SpecDecoder
    cfg, ew, eng, dcfg, tdr, ndr = _tiny_pair("nvfp4" if preset == "nvfp4" else "bf16", preset)
    g = _gen(6)
    taps = [torch.randn(20, cfg.hidden_size, device="cuda", generator=g).to(torch.bfloat16) for _ in dcfg.target_layer_ids]
    ndr.append_context(taps, 0)
    full = ndr.propose(9, 5, pos_start=20)
    ndr.set_draft_vocab(list(range(cfg.vocab_size)))
    assert ndr.propose(9, 5, pos_start=20) == full
    subset = list(range(3, cfg.vocab_size, 7))
    subset = subset[:len(subset) // 16 * 16]
    ndr.set_draft_vocab(subset)
    got = ndr.propose(9, 5, pos_start=20)
    assert len(got) == 5 and all(t in set(subset) for t in got)
    prompt = torch.randint(0, cfg.vocab_size, (21,), generator=torch.Generator().manual_seed(8)).tolist()
    from phaseshift_b200.runtime.engine import Engine
    ref_eng = Engine(ew, "cuda", StateConfig(max_slots=1, max_seq_len=128))
    ref_eng.set_uniform_arithmetic(True)
    out, _ = DFlash2SpecDecoder(eng, ndr, num_drafts=5).generate(prompt, 16, prefill_chunk=8)
    assert out == ref_eng.generate(prompt, 16, prefill_chunk=8)
    ndr.set_draft_vocab(None)
    assert ndr.sub_head is None
