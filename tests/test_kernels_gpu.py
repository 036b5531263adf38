"""CUDA kernels vs plain PyTorch fp32 references of the same op (all marked gpu)."""
import numpy as np
import pytest
import torch

from phaseshift_b200.models.qwen35.config import tiny_config, Qwen35Config
from phaseshift_b200.models.qwen35.weights import (LinearW, build_engine_weights, random_hf_weights, TpGeometry)
from phaseshift_b200.quant.formats import quantize, dequantize
from phaseshift_b200.runtime.batch import SeqRows, StepBatch
from phaseshift_b200.runtime.state import ModelState, StateConfig

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device("cuda:0")


def _ops(cfg, max_seq_len=512):
    from phaseshift_b200.ops.cuda_ops import CudaOps
    from phaseshift_b200.ops.ref_ops import RefOps
    return CudaOps(cfg, _dev(), max_seq_len=max_seq_len), RefOps(cfg, _dev())


def _rel_err(a, b):
    a, b = a.float(), b.float()
    return float((a - b).norm() / (b.norm() + 1e-12))


@pytest.mark.parametrize("fmt", ["bf16", "nvfp4", "mxfp8"])
@pytest.mark.parametrize("M", [1, 2, 3, 8, 11])
@pytest.mark.parametrize("shape", [(96, 256), (1024, 5120), (530, 17408)])
def test_linear_small_plain(fmt, M, shape):
    N, K = shape
    cfg = tiny_config()
    cu, ref = _ops(cfg)
    g = torch.Generator(device="cuda").manual_seed(N + K + M)
    w = torch.randn(N, K, device="cuda", generator=g) * 0.02
    x = (torch.randn(M, K, device="cuda", generator=g) * 1.5).to(torch.bfloat16)
    W = LinearW(quantize(w, fmt))
    y = cu.linear(x, W, name="t", out_f32=True)
    y_ref = x.float() @ W.dense().T
    torch.cuda.synchronize()
    # M > 8 goes through the tensor-core path whose weights are rounded to bf16 once
    tol = (2e-3 if fmt != "bf16" else 1e-5) if M <= 8 else 8e-3
    assert _rel_err(y, y_ref) < tol, _rel_err(y, y_ref)


@pytest.mark.parametrize("fmt", ["bf16", "nvfp4"])
def test_linear_small_fused_prologue_epilogue(fmt):
    cfg = tiny_config()
    cu, ref = _ops(cfg)
    g = torch.Generator(device="cuda").manual_seed(5)
    K, N, M = 1024, 512, 4
    w = torch.randn(N, K, device="cuda", generator=g) * 0.03
    x = (torch.randn(M, K, device="cuda", generator=g) * 3).to(torch.bfloat16)
    nw = (torch.randn(K, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
    res = torch.randn(M, N, device="cuda", generator=g).to(torch.bfloat16)
    W = LinearW(quantize(w, fmt))
    tol = 1e-2
    y = cu.linear(x, W, name="a", norm_w=nw, eps=1e-6, residual=res)
    y_ref = ref.linear(x, W, name="a", norm_w=nw, eps=1e-6, residual=res)
    assert _rel_err(y, y_ref) < tol
    y = cu.linear(x, W, name="b", norm_w=nw, eps=1e-6, swiglu=True)
    y_ref = ref.linear(x, W, name="b", norm_w=nw, eps=1e-6, swiglu=True)
    assert _rel_err(y, y_ref) < 2e-2


def test_linear_small_rows_are_batch_invariant():
    """Row r of an M=8 launch is bit-identical to the same row in an M=1 launch (Exact verify property)."""
    cfg = tiny_config()
    cu, _ = _ops(cfg)
    cu.exact_rows = True        # Exact mode: bf16 weights stay on the streaming kernel for every row count
    g = torch.Generator(device="cuda").manual_seed(9)
    for fmt in ("bf16", "nvfp4", "mxfp8"):
        w = torch.randn(640, 5120, device="cuda", generator=g) * 0.02
        x = torch.randn(8, 5120, device="cuda", generator=g).to(torch.bfloat16)
        W = LinearW(quantize(w, fmt))
        y8 = cu.linear(x, W, name="i8", out_f32=True).clone()
        for r in (0, 3, 7):
            y1 = cu.linear(x[r:r + 1], W, name="i1", out_f32=True)
            assert torch.equal(y1[0], y8[r]), fmt


def _mk_state(cfg, kv_dtype="bf16", slots=2, max_seq=256, ring=4):
    sc = StateConfig(max_slots=slots, max_seq_len=max_seq, page_tokens=16, kv_dtype=kv_dtype, conv_ring=ring)
    st_c = ModelState(cfg, sc, _dev(), torch.bfloat16)
    st_r = ModelState(cfg, sc, _dev(), torch.float32)
    for st in (st_c, st_r):
        for s in range(slots):
            nb = st.max_blocks
            st.block_table[s, :nb] = torch.arange(1 + s * nb, 1 + (s + 1) * nb, dtype=torch.int32, device=_dev()) % st.num_pages
    return sc, st_c, st_r


@pytest.mark.parametrize("kv_dtype", ["bf16", "fp8_e4m3"])
@pytest.mark.parametrize("geom", ["tiny", "big"])
def test_attention_prefill_then_decode(kv_dtype, geom):
    if geom == "tiny":
        cfg = tiny_config()
    else:
        cfg = Qwen35Config(vocab_size=1024, hidden_size=512, intermediate_size=512, num_hidden_layers=4,
                           num_attention_heads=12, num_key_value_heads=2, head_dim=256)
    cu, ref = _ops(cfg, 512)
    sc = StateConfig(max_slots=2, max_seq_len=512, page_tokens=16, kv_dtype=kv_dtype, kv_capacity_tokens=2048)
    st_c = ModelState(cfg, sc, _dev(), torch.bfloat16)
    st_r = ModelState(cfg, sc, _dev(), torch.float32)
    nb = st_c.max_blocks
    for st in (st_c, st_r):
        perm = torch.randperm(st.num_pages - 1, generator=torch.Generator().manual_seed(1))[:2 * nb] + 1
        st.block_table[0, :nb] = perm[:nb].int().to(_dev())
        st.block_table[1, :nb] = perm[nb:2 * nb].int().to(_dev())
    li = cfg.attn_layers[0]
    hf = random_hf_weights(cfg, seed=3, device="cuda")
    ew = build_engine_weights(cfg, lambda n: hf[n], "bf16", "cuda")
    aw = ew.layers[li].mixer
    Hq, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    g = torch.Generator(device="cuda").manual_seed(2)
    width = 2 * Hq * D + 2 * Hkv * D
    T = 300
    tol = 2e-2 if kv_dtype == "bf16" else 6e-2
    b = StepBatch(512, 2, _dev())
    # prefill 300 rows of sequence 0 (multi-row causal), then 3 decode steps for both sequences
    qkv = torch.randn(T, width, device="cuda", generator=g).to(torch.bfloat16)
    b.fill([SeqRows(0, 0, [0] * T, ())]); b.upload()
    q_c = cu.attn_prep(qkv, aw, Hq, Hkv, b, st_c.kv[li], st_c)
    q_r = ref.attn_prep(qkv.float(), aw, Hq, Hkv, b, st_r.kv[li], st_r)
    assert _rel_err(q_c, q_r) < 1e-2
    o_c = cu.paged_attention(q_c, qkv, Hq, Hkv, b, st_c.kv[li], st_c, b.max_visible)
    o_r = ref.paged_attention(q_r, qkv.float(), Hq, Hkv, b, st_r.kv[li], st_r, b.max_visible)
    torch.cuda.synchronize()
    assert _rel_err(o_c[:T], o_r[:T]) < tol
    assert int(st_c.status[0]) == 0
    for step in range(3):
        qkv = torch.randn(2, width, device="cuda", generator=g).to(torch.bfloat16)
        b2 = StepBatch(2, 2, _dev())
        b2.fill([SeqRows(0, T + step, [0], ()), SeqRows(1, step, [0], ())]); b2.upload()
        q_c = cu.attn_prep(qkv, aw, Hq, Hkv, b2, st_c.kv[li], st_c)
        q_r = ref.attn_prep(qkv.float(), aw, Hq, Hkv, b2, st_r.kv[li], st_r)
        o_c = cu.paged_attention(q_c, qkv, Hq, Hkv, b2, st_c.kv[li], st_c, b2.max_visible)
        o_r = ref.paged_attention(q_r, qkv.float(), Hq, Hkv, b2, st_r.kv[li], st_r, b2.max_visible)
        assert _rel_err(o_c, o_r) < tol
    assert int(st_c.status[0]) == 0


@pytest.mark.parametrize("kv_dtype", ["bf16", "fp8_e4m3"])
def test_attention_prefill_chunks_two_sequences(kv_dtype):
    """Tiled prefill attention: a second chunk that starts at an unaligned position next to a fresh sequence,
    with gate, against the fp32 reference."""
    cfg = Qwen35Config(vocab_size=1024, hidden_size=512, intermediate_size=512, num_hidden_layers=4,
                       num_attention_heads=12, num_key_value_heads=2, head_dim=256)
    cu, ref = _ops(cfg, 512)
    sc = StateConfig(max_slots=2, max_seq_len=512, page_tokens=16, kv_dtype=kv_dtype, kv_capacity_tokens=2048)
    st_c = ModelState(cfg, sc, _dev(), torch.bfloat16)
    st_r = ModelState(cfg, sc, _dev(), torch.float32)
    nb = st_c.max_blocks
    for st in (st_c, st_r):
        perm = torch.randperm(st.num_pages - 1, generator=torch.Generator().manual_seed(5))[:2 * nb] + 1
        st.block_table[0, :nb] = perm[:nb].int().to(_dev())
        st.block_table[1, :nb] = perm[nb:2 * nb].int().to(_dev())
    li = cfg.attn_layers[0]
    hf = random_hf_weights(cfg, seed=3, device="cuda")
    ew = build_engine_weights(cfg, lambda n: hf[n], "bf16", "cuda")
    aw = ew.layers[li].mixer
    Hq, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    g = torch.Generator(device="cuda").manual_seed(9)
    width = 2 * Hq * D + 2 * Hkv * D
    tol = 2e-2 if kv_dtype == "bf16" else 6e-2
    for seqs in ([SeqRows(0, 0, [0] * 100, ())], [SeqRows(0, 100, [0] * 77, ()), SeqRows(1, 0, [0] * 130, ())]):
        n = sum(len(s.token_ids) for s in seqs)
        qkv = torch.randn(n, width, device="cuda", generator=g).to(torch.bfloat16)
        b = StepBatch(512, 2, _dev())
        b.fill(seqs); b.upload()
        q_c = cu.attn_prep(qkv, aw, Hq, Hkv, b, st_c.kv[li], st_c)
        q_r = ref.attn_prep(qkv.float(), aw, Hq, Hkv, b, st_r.kv[li], st_r)
        o_c = cu.paged_attention(q_c, qkv, Hq, Hkv, b, st_c.kv[li], st_c, b.max_visible)
        o_r = ref.paged_attention(q_r, qkv.float(), Hq, Hkv, b, st_r.kv[li], st_r, b.max_visible)
        cu.ATTN_PREFILL_MIN_ROWS = 1 << 30           # split-KV kernel on the same inputs
        try:
            o_s = cu.paged_attention(q_c, qkv, Hq, Hkv, b, st_c.kv[li], st_c, b.max_visible).clone()
        finally:
            del cu.ATTN_PREFILL_MIN_ROWS
        torch.cuda.synchronize()
        assert _rel_err(o_c[:n], o_r[:n]) < tol
        assert _rel_err(o_c[:n].float(), o_s[:n].float()) < 1.5e-2
    assert int(st_c.status[0]) == 0


@pytest.mark.parametrize("geom", ["tiny", "big"])
def test_gdn_rows_and_decode(geom):
    if geom == "tiny":
        cfg = tiny_config()
    else:
        cfg = Qwen35Config(vocab_size=1024, hidden_size=512, intermediate_size=512, num_hidden_layers=4,
                           linear_num_key_heads=2, linear_num_value_heads=6)
    cu, ref = _ops(cfg)
    sc = StateConfig(max_slots=2, max_seq_len=256, page_tokens=16, conv_ring=8, spec_rows=8)
    st_c = ModelState(cfg, sc, _dev(), torch.bfloat16)
    st_r = ModelState(cfg, sc, _dev(), torch.float32)
    hf = random_hf_weights(cfg, seed=4, device="cuda")
    ew = build_engine_weights(cfg, lambda n: hf[n], "bf16", "cuda")
    li = cfg.gdn_layers[0]
    gw = ew.layers[li].mixer
    Hk, Hv = cfg.linear_num_key_heads, cfg.linear_num_value_heads
    width = gw.in_proj.N + gw.ba_proj.N
    g = torch.Generator(device="cuda").manual_seed(7)
    T = 37
    proj = (torch.randn(T + 5, width, device="cuda", generator=g) * 0.7).to(torch.bfloat16)
    b = StepBatch(64, 2, _dev())
    b.fill([SeqRows(1, 0, [0] * T, ())]); b.upload()
    o_c = cu.gdn(proj[:T], gw, Hk, Hv, b, st_c.gdn[li], st_c)
    o_r = ref.gdn(proj[:T].float(), gw, Hk, Hv, b, st_r.gdn[li], st_r)
    torch.cuda.synchronize()
    assert _rel_err(o_c[:T], o_r[:T]) < 2e-2
    assert _rel_err(st_c.gdn[li].rec[1], st_r.gdn[li].rec[1]) < 1e-3
    # single-row decode continues from the stored state and conv ring
    for i in range(5):
        b1 = StepBatch(1, 1, _dev())
        b1.fill([SeqRows(1, T + i, [0], ())]); b1.upload()
        o_c = cu.gdn(proj[T + i:T + i + 1], gw, Hk, Hv, b1, st_c.gdn[li], st_c)
        o_r = ref.gdn(proj[T + i:T + i + 1].float(), gw, Hk, Hv, b1, st_r.gdn[li], st_r)
        assert _rel_err(o_c, o_r) < 2e-2
    assert _rel_err(st_c.gdn[li].rec[1], st_r.gdn[li].rec[1]) < 1e-3


def test_gdn_chunked_matches_reference_and_row_kernel():
    """Prefill-sized steps take the chunked kernels: two sequences, several chunks with a ragged tail, a
    non-zero incoming state and a second step that continues from the stored state and conv history."""
    cfg = Qwen35Config(vocab_size=1024, hidden_size=512, intermediate_size=512, num_hidden_layers=4,
                       linear_num_key_heads=2, linear_num_value_heads=6)
    cu, ref = _ops(cfg)
    sc = StateConfig(max_slots=3, max_seq_len=512, page_tokens=16, conv_ring=8, spec_rows=8)
    st_c = ModelState(cfg, sc, _dev(), torch.bfloat16)
    st_w = ModelState(cfg, sc, _dev(), torch.bfloat16)
    st_r = ModelState(cfg, sc, _dev(), torch.float32)
    hf = random_hf_weights(cfg, seed=4, device="cuda")
    ew = build_engine_weights(cfg, lambda n: hf[n], "bf16", "cuda")
    li = cfg.gdn_layers[0]
    gw = ew.layers[li].mixer
    Hk, Hv = cfg.linear_num_key_heads, cfg.linear_num_value_heads
    width = gw.in_proj.N + gw.ba_proj.N
    g = torch.Generator(device="cuda").manual_seed(11)
    init = torch.randn(st_c.gdn[li].rec.shape, device="cuda", generator=g) * 0.1
    for st in (st_c, st_w, st_r):
        st.gdn[li].rec.copy_(init)
    pos = {2: 0, 0: 0}
    for (n2, n0) in ((150, 70), (64, 129)):
        proj = (torch.randn(n2 + n0, width, device="cuda", generator=g) * 0.7).to(torch.bfloat16)
        b = StepBatch(512, 2, _dev())
        b.fill([SeqRows(2, pos[2], [0] * n2, ()), SeqRows(0, pos[0], [0] * n0, ())]); b.upload()
        pos[2] += n2; pos[0] += n0
        o_c = cu.gdn(proj, gw, Hk, Hv, b, st_c.gdn[li], st_c)
        cu.GDN_CHUNKED_MIN_ROWS = 1 << 30            # row-sequential kernel on the same inputs
        try:
            o_w = cu.gdn(proj, gw, Hk, Hv, b, st_w.gdn[li], st_w).clone()
        finally:
            del cu.GDN_CHUNKED_MIN_ROWS
        o_r = ref.gdn(proj.float(), gw, Hk, Hv, b, st_r.gdn[li], st_r)
        torch.cuda.synchronize()
        assert _rel_err(o_c, o_r) < 2e-2
        assert _rel_err(o_c.float(), o_w.float()) < 1e-2
        for slot in (0, 2):
            assert _rel_err(st_c.gdn[li].rec[slot], st_r.gdn[li].rec[slot]) < 1e-3
        assert torch.equal(st_c.gdn[li].conv, st_w.gdn[li].conv)
    assert torch.equal(st_c.gdn[li].rec[1], init[1])      # untouched slot


def test_gdn_multirow_bit_equals_single_rows_and_replay():
    """Verify-rows launch == sequential decodes bit for bit; log replay of an accepted prefix rebuilds
    exactly the state sequential decoding reaches."""
    cfg = tiny_config()
    cu, _ = _ops(cfg)
    sc = StateConfig(max_slots=2, max_seq_len=64, conv_ring=16, spec_rows=8)
    hf = random_hf_weights(cfg, seed=5, device="cuda")
    ew = build_engine_weights(cfg, lambda n: hf[n], "bf16", "cuda")
    li = cfg.gdn_layers[0]
    gw = ew.layers[li].mixer
    Hk, Hv, Dk, Dv = cfg.linear_num_key_heads, cfg.linear_num_value_heads, cfg.linear_key_head_dim, cfg.linear_value_head_dim
    width = gw.in_proj.N + gw.ba_proj.N
    g = torch.Generator(device="cuda").manual_seed(8)
    proj = (torch.randn(6, width, device="cuda", generator=g) * 0.7).to(torch.bfloat16)
    st_a = ModelState(cfg, sc, _dev(), torch.bfloat16)
    st_b = ModelState(cfg, sc, _dev(), torch.bfloat16)
    init = torch.randn_like(st_a.gdn[li].rec) * 0.1
    st_a.gdn[li].rec.copy_(init); st_b.gdn[li].rec.copy_(init)
    # A: one launch with 6 rows, writing the new state to the alternate buffer and logging updates
    b = StepBatch(8, 1, _dev())
    b.fill([SeqRows(0, 0, [0] * 6, ())]); b.upload()
    log = (torch.zeros(8, Hv, Dk, device="cuda"), torch.zeros(8, Hv, Dv, device="cuda"), torch.zeros(8, Hv, device="cuda"))
    o_multi = cu.gdn(proj, gw, Hk, Hv, b, st_a.gdn[li], st_a, log=log, to_alt=True).clone()
    assert torch.equal(st_a.gdn[li].rec, init)          # old state untouched
    # B: six single-row launches
    outs = []
    states = []
    for i in range(6):
        b1 = StepBatch(1, 1, _dev())
        b1.fill([SeqRows(0, i, [0], ())]); b1.upload()
        outs.append(cu.gdn(proj[i:i + 1], gw, Hk, Hv, b1, st_b.gdn[li], st_b).clone())
        states.append(st_b.gdn[li].rec[0].clone())
    assert torch.equal(o_multi[:6], torch.cat(outs, 0))
    assert torch.equal(st_a.gdn[li].rec_alt[0], states[5])
    # accept 4 of the 6 rows: replay the log on the old state
    desc = torch.tensor([[0, 4, 0, 0]], dtype=torch.int32, device="cuda")
    cu.gdn_replay(st_a.gdn[li], Hv, desc, 1, log)
    torch.cuda.synchronize()
    assert torch.equal(st_a.gdn[li].rec[0], states[3])


def test_sampling_greedy_and_stochastic_match_host():
    from phaseshift_b200.utils.sampling import sample_row_host, sampling_uniform
    cfg = tiny_config()
    cu, _ = _ops(cfg)
    V = 5000
    g = torch.Generator(device="cuda").manual_seed(11)
    logits = torch.randn(6, V, device="cuda", generator=g) * 3
    logits[0, 77] = logits[0, 4000] = 50.0       # tie -> lower id
    b = StepBatch(8, 8, _dev())
    rows = [SeqRows(0, 0, [0], (0,)),
            SeqRows(0, 0, [0], (0,), temperature=1.0, seed=5, sample_index=3),
            SeqRows(0, 0, [0], (0,), temperature=0.7, top_k=20, seed=6, sample_index=1),
            SeqRows(0, 0, [0], (0,), temperature=1.3, top_p=0.8, seed=7, sample_index=9),
            SeqRows(0, 0, [0], (0,), temperature=1.0, top_p=0.9, top_k=50, seed=8),
            SeqRows(0, 0, [0], (0,))]
    b.fill(rows); b.upload()
    mask = torch.full((6, (V + 31) // 32), 0xFFFFFFFF, dtype=torch.int64).to(torch.int32).cuda()
    mask[5].zero_(); mask[5, 3] = 1 << 4        # only token 100 allowed
    active = torch.ones(6, dtype=torch.uint8, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = cu.sample(logits, b, 6, mask=mask, mask_active=active, status=status).cpu().tolist()
    assert out[0] == 77 and out[5] == 100
    lg = logits.cpu()
    for r in range(1, 5):
        assert out[r] == sample_row_host(lg[r], b._np_samp[r], None), r
    assert int(status[0]) == 0
    # NaN row fails closed
    logits[1, 5] = float("nan")
    out = cu.sample(logits, b, 6, status=status).cpu().tolist()
    assert out[1] == -1 and int(status[0]) == 4


def test_e2e_tiny_model_matches_oracle_tokens():
    from phaseshift_b200.models.qwen35.reference import reference_forward
    from phaseshift_b200.runtime.engine import Engine
    cfg = tiny_config()
    hf = random_hf_weights(cfg, seed=0)
    prompt = torch.randint(0, cfg.vocab_size, (32,), generator=torch.Generator().manual_seed(0)).tolist()
    ew = build_engine_weights(cfg, lambda n: hf[n], "bf16", "cuda")
    for kvd in ("bf16", "fp8_e4m3"):
        eng = Engine(ew, "cuda", StateConfig(max_slots=1, max_seq_len=128, page_tokens=16, kv_dtype=kvd))
        out = eng.generate(prompt, 24, prefill_chunk=16)
        # teacher-forced check: each generated token must be (near-)argmax of the fp32 oracle
        logits = reference_forward(cfg, hf, prompt + out[:-1])[len(prompt) - 1:]
        top = logits.max(-1).values
        chosen = logits[torch.arange(len(out)), torch.tensor(out)]
        assert float((top - chosen).max()) < (0.05 if kvd == "bf16" else 0.15), (kvd, (top - chosen).max())
        # graph replay and eager must agree exactly
        eng2 = Engine(ew, "cuda", StateConfig(max_slots=1, max_seq_len=128, page_tokens=16, kv_dtype=kvd), use_graphs=False)
        assert eng2.generate(prompt, 24, prefill_chunk=16) == out


def test_e2e_bf16_tokens_equal_the_oracle_on_bf16_rounded_weights():
    """bf16 weights, bf16 KV: the GPU engine's greedy stream equals, token for token, the fp32 oracle run on the same
    bf16-rounded weights wherever the oracle's decision is not a numerical tie (top-2 margin above the bf16 activation
    noise); at least 12 of the 24 steps must be that decisive, so the check cannot pass vacuously."""
    from phaseshift_b200.models.qwen35.reference import reference_forward
    from phaseshift_b200.runtime.engine import Engine
    cfg = tiny_config()
    hf = {k: v.to(torch.bfloat16).float() for k, v in random_hf_weights(cfg, seed=0).items()}
    prompt = torch.randint(0, cfg.vocab_size, (32,), generator=torch.Generator().manual_seed(0)).tolist()
    ew = build_engine_weights(cfg, lambda n: hf[n], "bf16", "cuda")
    eng = Engine(ew, "cuda", StateConfig(max_slots=1, max_seq_len=128, page_tokens=16, kv_dtype="bf16"))
    out = eng.generate(prompt, 24, prefill_chunk=16)
    logits = reference_forward(cfg, hf, prompt + out[:-1])[len(prompt) - 1:]
    top2 = logits.topk(2, -1)
    decisive = (top2.values[:, 0] - top2.values[:, 1]) > 0.02
    assert int(decisive.sum()) >= 12
    want = top2.indices[:, 0]
    got = torch.tensor(out)
    assert torch.equal(got[decisive], want[decisive]), (got.tolist(), want.tolist())


@pytest.mark.parametrize("fmt", ["bf16", "nvfp4", "mxfp8"])
def test_stream_gemv_shapes_and_row_invariance(fmt):
    """Odd N / K tails, K larger than one staging pass allows for M=8, and row invariance across M."""
    cfg = tiny_config()
    cu, _ = _ops(cfg)
    cu.exact_rows = True        # keep bf16 weights on the streaming kernel (Fast mode batches them on the tensor cores)
    g = torch.Generator(device="cuda").manual_seed(21)
    for (N, K) in [(1030, 5120), (510, 17408), (98, 2560), (7, 96)]:
        w = torch.randn(N, K, device="cuda", generator=g) * 0.02
        x = torch.randn(8, K, device="cuda", generator=g).to(torch.bfloat16)
        nw = (torch.randn(K, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
        W = LinearW(quantize(w, fmt))
        y8 = cu.linear(x, W, name="s8", norm_w=nw, eps=1e-6, out_f32=True).clone()
        y1 = cu.linear(x[5:6], W, name="s1", norm_w=nw, eps=1e-6, out_f32=True).clone()
        assert torch.equal(y1[0], y8[5])
        ref = (x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-6) * (1 + nw.float())) @ W.dense().T
        assert _rel_err(y8, ref) < 1e-2
        assert int(cu.status[0]) == 0


@pytest.mark.parametrize("fmt", ["bf16", "nvfp4", "mxfp8"])
def test_tiled_layout_roundtrip(fmt):
    from phaseshift_b200.quant.tiling import tile_weight, untile_weight, tiled_nbytes
    g = torch.Generator(device="cuda").manual_seed(3)
    for (N, K) in [(10, 96), (33, 2560), (8, 1024)]:
        q = quantize(torch.randn(N, K, device="cuda", generator=g), fmt)
        t = tile_weight(q)
        assert t.numel() == tiled_nbytes(fmt, N, q.k_padded)
        u = untile_weight(t, fmt, N, q.k_padded)
        assert torch.equal(u.codes.view(torch.uint8), q.codes.view(torch.uint8))
        if q.scales is not None:
            assert torch.equal(u.scales, q.scales)


@pytest.mark.parametrize("shape", [(128, 128, 64), (200, 384, 512), (2048, 5120, 5120), (77, 96, 2560), (1024, 1000, 17408)])
def test_tcgen05_gemm_matches_matmul(shape):
    M, N, K = shape
    cfg = tiny_config()
    cu, _ = _ops(cfg)
    g = torch.Generator(device="cuda").manual_seed(M + N)
    x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    W = LinearW(quantize(w.float(), "bf16"))
    y = cu.linear(x, W, name="g", out_f32=True)
    ref = x.float() @ w.float().T
    torch.cuda.synchronize()
    assert int(cu.status[0]) == 0
    assert _rel_err(y, ref) < 2e-3, _rel_err(y, ref)


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp8"])
def test_large_m_linear_fused_epilogues(fmt):
    cfg = tiny_config()
    cu, ref = _ops(cfg)
    g = torch.Generator(device="cuda").manual_seed(31)
    M, K, N = 300, 2560, 1536
    w = torch.randn(N, K, device="cuda", generator=g) * 0.03
    x = (torch.randn(M, K, device="cuda", generator=g) * 2).to(torch.bfloat16)
    nw = (torch.randn(K, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
    res = torch.randn(M, N, device="cuda", generator=g).to(torch.bfloat16)
    W = LinearW(quantize(w, fmt))
    y = cu.linear(x, W, name="a", norm_w=nw, eps=1e-6, residual=res)
    assert _rel_err(y, ref.linear(x, W, name="a", norm_w=nw, eps=1e-6, residual=res)) < 1e-2
    y = cu.linear(x, W, name="b", norm_w=nw, eps=1e-6, swiglu=True)
    assert _rel_err(y, ref.linear(x, W, name="b", norm_w=nw, eps=1e-6, swiglu=True)) < 2e-2
    assert int(cu.status[0]) == 0


def test_dflash2_exact_verify_on_gpu():
    """On the GPU the verify forward (8 rows, Exact mode) must reproduce single-row decoding bit for bit, so a
    perfect drafter is fully accepted and any drafter leaves the greedy stream unchanged."""
    from phaseshift_b200.models.dflash2.decoder import DFlash2SpecDecoder
    from phaseshift_b200.models.dflash2.model import DFlash2Drafter, random_weights, tiny_drafter_config
    from phaseshift_b200.runtime.engine import Engine
    cfg = tiny_config()
    hf = random_hf_weights(cfg, seed=0)
    prompt = torch.randint(0, cfg.vocab_size, (21,), generator=torch.Generator().manual_seed(8)).tolist()
    for preset in ("bf16", "nvfp4"):
        ew = build_engine_weights(cfg, lambda n: hf[n], preset, "cuda")
        plain = Engine(ew, "cuda", StateConfig(max_slots=1, max_seq_len=96)).generate(prompt, 24, prefill_chunk=8)
        eng = Engine(ew, "cuda", StateConfig(max_slots=1, max_seq_len=96, conv_ring=16, spec_rows=8))
        dcfg = tiny_drafter_config(cfg)
        dec = DFlash2SpecDecoder(eng, DFlash2Drafter(dcfg, random_weights(dcfg, 1), "cuda"), num_drafts=5)
        out, stats = dec.generate(prompt, 24, prefill_chunk=8)
        assert out == plain, preset
        full = prompt + plain
        dec2 = DFlash2SpecDecoder(Engine(ew, "cuda", StateConfig(max_slots=1, max_seq_len=96, conv_ring=16, spec_rows=8)),
                                  DFlash2Drafter(dcfg, random_weights(dcfg, 1), "cuda"), num_drafts=5)
        dec2.drafter.propose = lambda a, k, e, l, pos, allowed=None: full[pos + 1: pos + 1 + k]
        out2, stats2 = dec2.generate(prompt, 24, prefill_chunk=8)
        assert out2 == plain and stats2["accepted"] == stats2["proposed"], (preset, stats2)


def test_mtp_head_speculative_decoding_on_gpu():
    """The MTP head as drafter on the CUDA engine: Exact verification keeps the greedy stream for both chaining modes."""
    from phaseshift_b200.models.dflash2.decoder import DFlash2SpecDecoder
    from phaseshift_b200.models.qwen35.mtp import MTPDrafter, random_mtp_weights
    from phaseshift_b200.runtime.engine import Engine
    cfg = tiny_config()
    hf = random_hf_weights(cfg, seed=0)
    prompt = torch.randint(0, cfg.vocab_size, (19,), generator=torch.Generator().manual_seed(9)).tolist()
    ew = build_engine_weights(cfg, lambda n: hf[n], "nvfp4", "cuda")
    plain = Engine(ew, "cuda", StateConfig(max_slots=1, max_seq_len=96)).generate(prompt, 20, prefill_chunk=8)
    for chain in ("pre", "post"):
        eng = Engine(ew, "cuda", StateConfig(max_slots=1, max_seq_len=96, conv_ring=16, spec_rows=8))
        head = MTPDrafter(cfg, random_mtp_weights(cfg, 3, "cuda"), "cuda", torch.bfloat16, chain=chain)
        out, stats = DFlash2SpecDecoder(eng, head, num_drafts=3).generate(prompt, 20, prefill_chunk=8)
        assert out == plain, chain
        assert stats["rounds"] > 0 and int(eng.ops.status[0]) == 0


def test_dflash2_captured_proposal_matches_eager():
    """The drafter's proposal replayed from its CUDA graph (attention over the whole ring with empty slots masked)
    against the eager path (live slots compacted): same backbone output, and replays follow the ring and the anchor."""
    from phaseshift_b200.models.dflash2.decoder import DFlash2SpecDecoder
    from phaseshift_b200.models.dflash2.model import DFlash2Drafter, random_weights, tiny_drafter_config
    from phaseshift_b200.runtime.engine import Engine
    cfg = tiny_config()
    hf = random_hf_weights(cfg, seed=0)
    ew = build_engine_weights(cfg, lambda n: hf[n], "bf16", "cuda")
    eng = Engine(ew, "cuda", StateConfig(max_slots=1, max_seq_len=96, conv_ring=16, spec_rows=8))
    dcfg = tiny_drafter_config(cfg)
    dr = DFlash2Drafter(dcfg, random_weights(dcfg, 1), "cuda")
    dec = DFlash2SpecDecoder(eng, dr, num_drafts=5)
    g = torch.Generator(device="cuda").manual_seed(3)
    taps = [torch.randn(30, cfg.hidden_size, device="cuda", generator=g) for _ in dcfg.target_layer_ids]
    dr.append_context(taps, 0)
    x = torch.randn(6, cfg.hidden_size, device="cuda", generator=g)
    pos = torch.arange(30, 36, device="cuda")
    assert _rel_err(dr.backbone(x, pos, static=True), dr.backbone(x, pos)) < 1e-4
    dr.use_graph = False
    eager = dr.propose(7, 5, dec._embed, dec._lm_head, 30)
    dr.use_graph = True
    first = dr.propose(7, 5, dec._embed, dec._lm_head, 30)             # captures
    again = dr.propose(7, 5, dec._embed, dec._lm_head, 30)             # replays
    assert len(first) == 5 and first == again
    assert dr.graph_error is None and 5 in dr._graphs                  # the graph path really ran
    assert sum(a == b for a, b in zip(first, eager)) >= 4               # same mathematics (ties aside)
    dr.append_context([t[:4] for t in taps], 30)                       # the ring moved: replays must see it
    dr.use_graph = False
    eager2 = dr.propose(9, 5, dec._embed, dec._lm_head, 34)
    dr.use_graph = True
    assert sum(a == b for a, b in zip(dr.propose(9, 5, dec._embed, dec._lm_head, 34), eager2)) >= 4
    assert int(eng.ops.status[0]) == 0


def test_radix_topk_matches_sort_and_breaks_ties_by_id():
    cfg = tiny_config()
    cu, _ = _ops(cfg)
    g = torch.Generator(device="cuda").manual_seed(21)
    logits = torch.randn(5, 151936, device="cuda", generator=g) * 4
    logits[1, 777] = float("inf")
    logits[2, :] = logits[2, :].round()                     # heavy ties, also at the threshold
    logits[3, 100:200] = 50.0                               # 100 equal maxima: ids 100..131 must win for k = 32
    for k in (1, 16, 32, 128):
        ids, vals = cu.topk(logits, k)
        torch.cuda.synchronize()
        order = torch.sort(logits.double() * 1e6 - torch.arange(logits.shape[1], device="cuda").double() * 1e-3, dim=1,
                           descending=True).indices[:, :k] if False else None
        for r in range(5):
            row = logits[r]
            ref_v = torch.sort(row, descending=True).values[:k]
            assert torch.equal(vals[r], ref_v), (k, r)
            assert torch.equal(row[ids[r].long()], ref_v)                    # ids point at those values
            # ties: among equal values the ids ascend, and no lower id with the same value was skipped
            v, i = vals[r].tolist(), ids[r].tolist()
            assert all(not (v[j] == v[j + 1] and i[j] > i[j + 1]) for j in range(k - 1))
            thr = v[-1]
            eq_ids = (row == thr).nonzero().flatten().tolist()
            taken = [x for x, vv in zip(i, v) if vv == thr]
            assert taken == eq_ids[:len(taken)]
    # constrained: only the allowed tokens compete; fewer allowed than k pads with -1
    mask = torch.zeros(5, (151936 + 31) // 32, dtype=torch.int32, device="cuda")
    allowed = [5, 64, 1000, 150000]
    for a in allowed:
        mask[:, a // 32] |= (1 << (a % 32))
    ids, vals = cu.topk(logits, 8, mask=mask)
    torch.cuda.synchronize()
    for r in range(5):
        got = [x for x in ids[r].tolist() if x >= 0]
        assert sorted(got) == allowed and ids[r, 4:].tolist() == [-1] * 4
        assert got == sorted(allowed, key=lambda a: (-float(logits[r, a]), a))


def test_batched_steps_agree_with_single_row_arithmetic():
    """A 3-row decode batch (tensor-core kernels: block-scaled for nvfp4, swap-AB bf16 GEMM for bf16 weights) gives
    logits close to what three single-row steps give, and engines over one weight set decode identically."""
    from phaseshift_b200.runtime.engine import Engine
    cfg = tiny_config()
    hf = random_hf_weights(cfg, seed=0)
    prompt = torch.randint(0, cfg.vocab_size, (19,), generator=torch.Generator().manual_seed(3)).tolist()
    for preset in ("nvfp4", "bf16"):
        ew = build_engine_weights(cfg, lambda n: hf[n], preset, "cuda")
        eng = Engine(ew, "cuda", StateConfig(max_slots=8, max_seq_len=96))
        single = eng.generate(prompt, 6, prefill_chunk=64)
        assert Engine(ew, "cuda", StateConfig(max_slots=4, max_seq_len=96)).generate(prompt, 6, prefill_chunk=64) == single
        # a step advances the recurrent state even when the position is not committed: the batched step and the
        # single-row steps get sequences of their own over the same prompts
        seqs = [eng.open_sequence() for _ in range(6)]
        for i, s in enumerate(seqs):
            eng.prefill(s, prompt[i % 3:], 64)
        rows = [SeqRows(s.slot, s.position, [5 + i % 3], (0,)) for i, s in enumerate(seqs)]
        _, out = eng.step(rows[:3], seqs[:3], want_logits=True, commit=False)
        batch = out.logits[:3].float().clone()
        one = []
        for i in range(3, 6):
            _, o1 = eng.step([rows[i]], [seqs[i]], want_logits=True, commit=False)
            one.append(o1.logits[0].float().clone())
        for s in seqs:
            eng.close_sequence(s)
        assert _rel_err(batch, torch.stack(one)) < 3e-2, preset


@pytest.mark.parametrize("shape", [(3, 5120, 5120), (8, 1024, 17408), (64, 34816, 512), (128, 600, 256)])
def test_tcgen05_gemm_small_m_weight_streaming(shape):
    M, N, K = shape
    cfg = tiny_config()
    cu, _ = _ops(cfg)
    g = torch.Generator(device="cuda").manual_seed(M + N)
    a = (torch.randn(M, K, device="cuda", generator=g)).to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    res = torch.randn(M, N, device="cuda", generator=g).to(torch.bfloat16)
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    import ctypes
    from phaseshift_b200.ops import _lib
    vp = lambda t: ctypes.c_void_p(t.data_ptr())
    _lib.call("ps_gemm_bf16_tc", vp(a), ctypes.c_int(K), vp(w), ctypes.c_int(K), ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(K),
              ctypes.c_int(1), vp(res), ctypes.c_int(N), vp(out), ctypes.c_int(N), ctypes.c_int(0), vp(cu.status))
    torch.cuda.synchronize()
    ref = (a.float() @ w.float().T).to(torch.bfloat16).float() + res.float()
    assert _rel_err(out.float(), ref) < 4e-3
    assert int(cu.status[0]) == 0


def test_gdn_and_attention_mixed_step_long_and_short_sequences():
    """Continuous batching: one step carries a prefill chunk of one request and single decode rows of others.  The
    long sequence goes through the chunked / tiled kernels, the short ones through the row kernels, in one call."""
    cfg = Qwen35Config(vocab_size=1024, hidden_size=512, intermediate_size=512, num_hidden_layers=4,
                       linear_num_key_heads=2, linear_num_value_heads=6, num_attention_heads=12, num_key_value_heads=2,
                       head_dim=256)
    cu, ref = _ops(cfg, 512)
    sc = StateConfig(max_slots=4, max_seq_len=512, page_tokens=16, conv_ring=8, spec_rows=8, kv_capacity_tokens=4096)
    st_c = ModelState(cfg, sc, _dev(), torch.bfloat16)
    st_r = ModelState(cfg, sc, _dev(), torch.float32)
    nb = st_c.max_blocks
    for st in (st_c, st_r):
        perm = torch.randperm(st.num_pages - 1, generator=torch.Generator().manual_seed(5))[:4 * nb] + 1
        for s in range(4):
            st.block_table[s, :nb] = perm[s * nb:(s + 1) * nb].int().to(_dev())
    hf = random_hf_weights(cfg, seed=4, device="cuda")
    ew = build_engine_weights(cfg, lambda n: hf[n], "bf16", "cuda")
    lg, la = cfg.gdn_layers[0], cfg.attn_layers[0]
    gw, aw = ew.layers[lg].mixer, ew.layers[la].mixer
    Hk, Hv = cfg.linear_num_key_heads, cfg.linear_num_value_heads
    Hq, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    g = torch.Generator(device="cuda").manual_seed(13)
    gwidth, awidth = gw.in_proj.N + gw.ba_proj.N, 2 * Hq * D + 2 * Hkv * D
    # step 1: give the three "decode" sequences some history; step 2: mixed step
    steps = [[SeqRows(1, 0, [0] * 20, ()), SeqRows(2, 0, [0] * 33, ()), SeqRows(3, 0, [0] * 5, ())],
             [SeqRows(0, 0, [0] * 100, ()), SeqRows(1, 20, [0], ()), SeqRows(2, 33, [0, 0], ()), SeqRows(3, 5, [0], ())]]
    for seqs in steps:
        n = sum(len(s.token_ids) for s in seqs)
        b = StepBatch(256, 4, _dev())
        b.fill(seqs); b.upload()
        proj = (torch.randn(n, gwidth, device="cuda", generator=g) * 0.7).to(torch.bfloat16)
        o_c = cu.gdn(proj, gw, Hk, Hv, b, st_c.gdn[lg], st_c)
        o_r = ref.gdn(proj.float(), gw, Hk, Hv, b, st_r.gdn[lg], st_r)
        qkv = torch.randn(n, awidth, device="cuda", generator=g).to(torch.bfloat16)
        q_c = cu.attn_prep(qkv, aw, Hq, Hkv, b, st_c.kv[la], st_c)
        q_r = ref.attn_prep(qkv.float(), aw, Hq, Hkv, b, st_r.kv[la], st_r)
        a_c = cu.paged_attention(q_c, qkv, Hq, Hkv, b, st_c.kv[la], st_c, b.max_visible)
        a_r = ref.paged_attention(q_r, qkv.float(), Hq, Hkv, b, st_r.kv[la], st_r, b.max_visible)
        torch.cuda.synchronize()
        assert _rel_err(o_c[:n], o_r[:n]) < 2e-2
        assert _rel_err(a_c[:n], a_r[:n]) < 2e-2
        for slot in range(4):
            assert _rel_err(st_c.gdn[lg].rec[slot], st_r.gdn[lg].rec[slot]) < 1e-3 or float(st_r.gdn[lg].rec[slot].abs().max()) == 0
    assert int(st_c.status[0]) == 0


def test_decode_batches_beyond_eight_rows_replay_from_graphs():
    """Pure decode batches (one row per sequence) up to 64 rows are captured per bucket; replays must produce the
    tokens of the eager path."""
    from phaseshift_b200.runtime.engine import Engine
    cfg = tiny_config()
    hf = random_hf_weights(cfg, seed=0)
    ew = build_engine_weights(cfg, lambda n: hf[n], "nvfp4", "cuda")
    outs = []
    for graphs in (True, False):
        eng = Engine(ew, "cuda", StateConfig(max_slots=12, max_seq_len=64), use_graphs=graphs)
        seqs = [eng.open_sequence() for _ in range(12)]
        toks = [eng.prefill(s, list(range(3 + i, 12 + i)), 64) for i, s in enumerate(seqs)]
        hist = []
        for _ in range(4):
            rows = [SeqRows(s.slot, s.position, [t], (0,)) for s, t in zip(seqs, toks)]
            toks, _ = eng.step(rows, seqs)
            hist.append(list(toks))
        outs.append(hist)
        if graphs:
            assert any(eng.graph_key_bucket(k) == 16 for k in eng.graphs), "the 12-row decode batch must have been captured (bucket 16)"
    assert outs[0] == outs[1]


@pytest.mark.parametrize("kvd", ["bf16", "fp8_e4m3"])
def test_long_context_prefill_and_decode_paths_agree_at_32k(kvd):
    """2048-token prefill chunks (the largest step) up to a 32 K context, then decoding: the logits of the last position computed by the
    prefill path (tiled attention over 32 K keys, chunked GDN) and by the decode path (split-KV attention with the
    split length doubled to stay within 512 splits, row-sequential GDN) must agree -- two independent kernel families
    over the same paged cache, block table and positions."""
    from phaseshift_b200.runtime.engine import Engine
    cfg = tiny_config()
    hf = random_hf_weights(cfg, seed=0)
    ew = build_engine_weights(cfg, lambda n: hf[n], "bf16", "cuda")
    N = 32768
    ids = torch.randint(0, cfg.vocab_size, (N,), generator=torch.Generator().manual_seed(2)).tolist()
    sc = StateConfig(max_slots=2, max_seq_len=N + 16, page_tokens=16, kv_dtype=kvd)
    eng = Engine(ew, "cuda", sc)
    assert eng.ops.split_tokens * 512 >= N                      # the split length grew with the context
    a, b = eng.open_sequence(), eng.open_sequence()
    C = 2048
    for c0 in range(0, N, C):
        last = c0 + C >= N
        _, out_a = eng.step([SeqRows(a.slot, c0, ids[c0:c0 + C], (C - 1,) if last else ())], [a], want_logits=True)
    for c0 in range(0, N - 1, C):
        chunk = ids[c0:min(c0 + C, N - 1)]
        eng.step([SeqRows(b.slot, c0, chunk, ())], [b])
    _, out_b = eng.step([SeqRows(b.slot, N - 1, [ids[N - 1]], (0,))], [b], want_logits=True)
    la, lb = out_a.logits[0].float(), out_b.logits[0].float()
    assert torch.isfinite(la).all() and torch.isfinite(lb).all()
    assert _rel_err(lb, la) < (3e-2 if kvd == "bf16" else 8e-2)
    # and decoding simply continues from there
    toks = []
    t = int(la.argmax())
    for i in range(4):
        tk, _ = eng.step([SeqRows(a.slot, N + i, [t], (0,))], [a])
        t = tk[0]
        toks.append(t)
    assert len(toks) == 4 and int(eng.ops.status[0]) == 0 and int(eng.state.status[0]) == 0


@pytest.mark.parametrize("kv_dtype", ["bf16", "fp8_e4m3"])
def test_attention_mixed_step_long_rows_tiled_short_rows_per_row(kv_dtype):
    """A serving-shaped step: one prefill chunk of 150 rows at position 200 next to two decode rows of sequences with 300
    and 37 tokens of context.  The chunk runs on the tiled tensor-core kernel (FP8 pages through the bf16 scratch pool),
    the decode rows on the per-row kernel; all rows against the fp32 reference and against the per-row kernel alone."""
    cfg = Qwen35Config(vocab_size=1024, hidden_size=512, intermediate_size=512, num_hidden_layers=4,
                       num_attention_heads=12, num_key_value_heads=2, head_dim=256)
    cu, ref = _ops(cfg, 512)
    sc = StateConfig(max_slots=3, max_seq_len=512, page_tokens=16, kv_dtype=kv_dtype, kv_capacity_tokens=2048)
    st_c = ModelState(cfg, sc, _dev(), torch.bfloat16)
    st_r = ModelState(cfg, sc, _dev(), torch.float32)
    nb = st_c.max_blocks
    for st in (st_c, st_r):
        perm = torch.randperm(st.num_pages - 1, generator=torch.Generator().manual_seed(7))[:3 * nb] + 1
        for s in range(3):
            st.block_table[s, :nb] = perm[s * nb:(s + 1) * nb].int().to(_dev())
    li = cfg.attn_layers[0]
    hf = random_hf_weights(cfg, seed=3, device="cuda")
    aw = build_engine_weights(cfg, lambda n: hf[n], "bf16", "cuda").layers[li].mixer
    Hq, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    g = torch.Generator(device="cuda").manual_seed(11)
    width = 2 * Hq * D + 2 * Hkv * D
    tol = 2e-2 if kv_dtype == "bf16" else 6e-2

    def run(seqs):
        n = sum(len(s.token_ids) for s in seqs)
        qkv = torch.randn(n, width, device="cuda", generator=g).to(torch.bfloat16)
        b = StepBatch(512, 3, _dev())
        b.fill(seqs); b.upload()
        q_c = cu.attn_prep(qkv, aw, Hq, Hkv, b, st_c.kv[li], st_c)
        q_r = ref.attn_prep(qkv.float(), aw, Hq, Hkv, b, st_r.kv[li], st_r)
        o_c = cu.paged_attention(q_c, qkv, Hq, Hkv, b, st_c.kv[li], st_c, b.max_visible).clone()
        o_r = ref.paged_attention(q_r, qkv.float(), Hq, Hkv, b, st_r.kv[li], st_r, b.max_visible)
        cu.ATTN_PREFILL_MIN_ROWS = 1 << 30
        try:
            o_s = cu.paged_attention(q_c, qkv, Hq, Hkv, b, st_c.kv[li], st_c, b.max_visible).clone()
        finally:
            del cu.ATTN_PREFILL_MIN_ROWS
        return n, o_c, o_r, o_s
    # contexts: sequence 0 gets 200 tokens, sequence 1 300, sequence 2 37
    for seqs in ([SeqRows(0, 0, [0] * 200, ())], [SeqRows(1, 0, [0] * 300, ())], [SeqRows(2, 0, [0] * 37, ())]):
        run(seqs)
    launches = cu.launches
    n, o_c, o_r, o_s = run([SeqRows(1, 300, [0], ()), SeqRows(0, 200, [0] * 150, ()), SeqRows(2, 37, [0], ())])
    torch.cuda.synchronize()
    assert n == 152 and int(st_c.status[0]) == 0
    assert _rel_err(o_c[:n], o_r[:n]) < tol
    assert _rel_err(o_c[:n].float(), o_s[:n].float()) < (1.5e-2 if kv_dtype == "bf16" else 3e-2)
    for r in (0, 151):                                   # FP8 pages: the decode rows came from the per-row kernel both times
        if kv_dtype == "bf16":
            assert _rel_err(o_c[r].float(), o_s[r].float()) < 1.5e-2        # tensor-core decode kernel against the per-row one
        else:
            assert torch.equal(o_c[r], o_s[r])
    # prep + (dequantise +) tiled + split + merge for the mixed call, prep excluded: 3 or 4 launches, then 2 for the per-row run
    assert cu.launches - launches == 1 + (4 if kv_dtype != "bf16" else 3) + 2


@pytest.mark.parametrize("preset", ["nvfp4", "mxfp8", "bf16"])
def test_lm_head_fused_argmax_matches_projection_then_sample(preset):
    """The streaming projection with greedy sampling in its epilogue against the same projection followed by the sampling
    kernel: identical token ids for 1, 3 and 8 rows (same values, same tie rule), over a 27B-sized vocabulary, the state
    re-armed between launches; a non-finite activation fails closed (-1 and the status word)."""
    from phaseshift_b200.models.qwen35.weights import LinearW
    from phaseshift_b200.quant import formats
    cfg = tiny_config()
    cu, _ = _ops(cfg, 16)
    N, K = 151936, 1024
    g = torch.Generator(device="cuda").manual_seed(5)
    w = torch.randn(N, K, device="cuda", generator=g) * 0.02
    W = LinearW(formats.quantize(w, preset)) if preset != "bf16" else LinearW(formats.quantize(w, "bf16"))
    W.make_tiled()
    norm_w = (torch.randn(K, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
    for M in (1, 3, 8, 1):
        x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
        if not cu.can_fuse_argmax(W, M):
            assert preset == "bf16" and M > 1          # batched bf16 rows prefer the tensor-core GEMM of the row-major weights
            continue
        logits = cu.linear(x, W, name="t_logits", norm_w=norm_w, eps=1e-6, out_f32=True)
        want = logits[:M].argmax(-1).to(torch.int32)
        n0 = cu.launches
        got = cu.linear_argmax(x, W, norm_w=norm_w, eps=1e-6).clone()
        assert cu.launches - n0 == 1
        torch.cuda.synchronize()
        assert torch.equal(got, want), (M, got.tolist(), want.tolist())
    assert int(cu.status[0]) == 0 and int(cu._amax_state.abs().sum()) == 0
    # ties go to the lower index: two identical weight rows that win
    w2 = w.clone(); w2[777] = w2[123] = 3.0 * x[0].float() / x[0].float().norm()
    W2 = LinearW(formats.quantize(w2, "bf16")); W2.make_tiled()
    got = cu.linear_argmax(x[:1], W2)
    torch.cuda.synchronize()
    assert int(got[0]) == 123
    xb = x.clone(); xb[0, 5] = float("inf")
    got = cu.linear_argmax(xb, W, norm_w=norm_w, eps=1e-6)
    torch.cuda.synchronize()
    assert int(got[0]) == -1 and int(cu.status[0]) != 0
    cu.reset_after_error()


def test_engine_greedy_steps_use_the_fused_argmax_and_match_the_sampling_kernel():
    """Decode through the engine with the fused arg-max (its own CUDA graph, one launch fewer) and with it switched off:
    the same tokens; a step that asks for logits keeps the sampling kernel."""
    from phaseshift_b200.runtime.engine import Engine
    cfg = Qwen35Config(vocab_size=4096, hidden_size=512, intermediate_size=1024, num_hidden_layers=4,
                       num_attention_heads=4, num_key_value_heads=2, head_dim=128)
    hf = random_hf_weights(cfg, seed=4, device="cuda")
    ew = build_engine_weights(cfg, lambda n: hf[n], "nvfp4", "cuda", layout="both")
    prompt = torch.randint(0, cfg.vocab_size, (40,), generator=torch.Generator().manual_seed(1)).tolist()
    outs, launches = [], []
    for fused in (True, False):
        eng = Engine(ew, _dev(), StateConfig(max_slots=2, max_seq_len=128))
        eng.fused_argmax = fused
        outs.append(eng.generate(prompt, 24))
        launches.append(max(eng.launches_per_graph.values()))
        if fused:
            s = eng.open_sequence()
            _, o = eng.step([SeqRows(s.slot, 0, prompt, (len(prompt) - 1,))], [s], want_logits=True)
            assert o.logits is not None
            _, o = eng.step([SeqRows(s.slot, s.position, [1], (0,))], [s])
            assert o.logits is None
    assert outs[0] == outs[1]
    assert launches[0] == launches[1] - 1


def test_steps_of_17_to_32_rows_match_smaller_steps_on_27b_shaped_layers():
    """27B-sized projections, 17..32 rows: the down projection no longer fits the resident-activation path and runs the
    streamed kernel, whose staged epilogue leaves no row statistics for the next layer's fused RMSNorm; the next layer must
    then compute them itself.  (It once consumed whatever the statistics buffer held: activations of every fourth layer off
    by an order of magnitude, laundered into finite values by the activation quantiser.)  Checked on the hidden states
    after the second and the sixth layer (MXFP8, whose rounding noise stays small over a few layers): prefilling 20 and 31
    tokens in one step against two steps of at most 16 rows, and finite recurrent state after prefill steps and a batched
    decode step of 20 sequences."""
    from phaseshift_b200.models.qwen35.config import PRESETS
    from phaseshift_b200.models.qwen35.weights import random_getter
    from phaseshift_b200.runtime.engine import Engine
    base = PRESETS["27b"]()
    cfg = type(base)(**{**base.__dict__, "num_hidden_layers": 8, "layer_types": None, "vocab_size": 8192})
    ew = build_engine_weights(cfg, random_getter(cfg, 0, _dev()), "mxfp8", _dev(), layout="both")
    eng = Engine(ew, _dev(), StateConfig(max_slots=24, max_seq_len=128), use_graphs=False)
    g = torch.Generator().manual_seed(3)
    taps = [1, 5]

    def rel(x, y):
        return float((x.float() - y.float()).norm() / y.float().norm())
    for n in (20, 31):
        ids = torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist()
        a, b = eng.open_sequence(), eng.open_sequence()
        _, oa = eng.step([SeqRows(a.slot, 0, ids, (n - 1,))], [a], tap_layers=taps)
        ta = {li: oa.taps[li][n - 1].clone() for li in taps}
        eng.step([SeqRows(b.slot, 0, ids[:16], ())], [b])
        _, ob = eng.step([SeqRows(b.slot, 16, ids[16:], (n - 17,))], [b], tap_layers=taps)
        errs = {li: rel(ta[li], ob.taps[li][n - 17]) for li in taps}
        assert errs[1] < 0.2 and errs[5] < 0.4, (n, errs)          # 0.08 / 0.15 measured; an order of magnitude with wrong statistics
        for li in cfg.gdn_layers:
            assert bool(torch.isfinite(eng.state.gdn[li].rec[a.slot]).all()), (n, li)
        eng.close_sequence(a); eng.close_sequence(b)
    # a batched decode step of 20 sequences (one row each) leaves every recurrent state finite and samples valid tokens
    seqs = [eng.open_sequence() for _ in range(20)]
    toks = [eng.prefill(s, torch.randint(0, cfg.vocab_size, (18 + i,), generator=g).tolist(), 64) for i, s in enumerate(seqs)]
    toks, _ = eng.step([SeqRows(s.slot, s.position, [t], (0,)) for s, t in zip(seqs, toks)], seqs)
    assert all(t >= 0 for t in toks)
    for li in cfg.gdn_layers:
        assert bool(torch.isfinite(eng.state.gdn[li].rec).all()) and bool(torch.isfinite(eng.state.gdn[li].conv.float()).all()), li


def test_tensor_core_decode_attention_rows_do_not_depend_on_their_tile_neighbours():
    """bf16 pages, head dim 256, six query heads per KV head: a block of 8 new rows of one sequence (speculative
    verification) through the grouped-query tensor-core decode kernel against the fp32 reference, and bit for bit against
    the same rows computed one per step (what Exact-mode verification relies on); also two sequences with different
    contexts in one step."""
    cfg = Qwen35Config(vocab_size=1024, hidden_size=512, intermediate_size=512, num_hidden_layers=4,
                       num_attention_heads=12, num_key_value_heads=2, head_dim=256)
    cu, ref = _ops(cfg, 512)
    assert cu.attn_decode_tc
    sc = StateConfig(max_slots=2, max_seq_len=512, page_tokens=16, kv_dtype="bf16", kv_capacity_tokens=2048)
    st_c = ModelState(cfg, sc, _dev(), torch.bfloat16)
    st_r = ModelState(cfg, sc, _dev(), torch.float32)
    nb = st_c.max_blocks
    for st in (st_c, st_r):
        perm = torch.randperm(st.num_pages - 1, generator=torch.Generator().manual_seed(3))[:2 * nb] + 1
        st.block_table[0, :nb] = perm[:nb].int().to(_dev())
        st.block_table[1, :nb] = perm[nb:2 * nb].int().to(_dev())
    li = cfg.attn_layers[0]
    hf = random_hf_weights(cfg, seed=3, device="cuda")
    aw = build_engine_weights(cfg, lambda n: hf[n], "bf16", "cuda").layers[li].mixer
    Hq, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    g = torch.Generator(device="cuda").manual_seed(21)
    width = 2 * Hq * D + 2 * Hkv * D

    def run(seqs, qkv):
        n = qkv.shape[0]
        b = StepBatch(16, 2, _dev())
        b.fill(seqs); b.upload()
        q_c = cu.attn_prep(qkv, aw, Hq, Hkv, b, st_c.kv[li], st_c)
        q_r = ref.attn_prep(qkv.float(), aw, Hq, Hkv, b, st_r.kv[li], st_r)
        o_c = cu.paged_attention(q_c, qkv, Hq, Hkv, b, st_c.kv[li], st_c, b.max_visible)[:n].clone()
        o_r = ref.paged_attention(q_r, qkv.float(), Hq, Hkv, b, st_r.kv[li], st_r, b.max_visible)[:n]
        return o_c, o_r
    # contexts of 203 and 70 tokens through the tiled prefill kernel
    for slot, n in ((0, 203), (1, 70)):
        run_pre = torch.randn(n, width, device="cuda", generator=g).to(torch.bfloat16)
        b = StepBatch(512, 2, _dev())
        b.fill([SeqRows(slot, 0, [0] * n, ())]); b.upload()
        cu.attn_prep(run_pre, aw, Hq, Hkv, b, st_c.kv[li], st_c)
        ref.attn_prep(run_pre.float(), aw, Hq, Hkv, b, st_r.kv[li], st_r)
    qkv8 = torch.randn(8, width, device="cuda", generator=g).to(torch.bfloat16)
    o8, r8 = run([SeqRows(0, 203, [0] * 8, ())], qkv8)
    torch.cuda.synchronize()
    assert int(st_c.status[0]) == 0 and _rel_err(o8, r8) < 2e-2
    for i in range(8):
        o1, _ = run([SeqRows(0, 203 + i, [0], ())], qkv8[i:i + 1])
        assert torch.equal(o1[0], o8[i]), i
    # two sequences, one row each, in one step
    qkv2 = torch.randn(2, width, device="cuda", generator=g).to(torch.bfloat16)
    o2, r2 = run([SeqRows(1, 70, [0], ()), SeqRows(0, 211, [0], ())], qkv2)
    assert _rel_err(o2, r2) < 2e-2 and int(st_c.status[0]) == 0
