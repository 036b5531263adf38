"""MTP head on CPU: forward math against an independent restatement built from the reference-model helpers,
KV bookkeeping of chained proposals, and the speculative-decoding invariant (greedy spec == greedy target-only)."""
import pytest
import torch

from phaseshift_b200.models.dflash2.decoder import DFlash2SpecDecoder
from phaseshift_b200.models.qwen35 import reference as R
from phaseshift_b200.models.qwen35.config import tiny_config
from phaseshift_b200.models.qwen35.mtp import (LP, MP, MTPDrafter, mtp_reference_rows, mtp_tensor_shapes, random_mtp_weights,
                                               validate_mtp_geometry)
from phaseshift_b200.models.qwen35.weights import build_engine_weights, random_hf_weights
from phaseshift_b200.runtime.engine import Engine
from phaseshift_b200.runtime.state import StateConfig


@pytest.fixture(scope="module")
def setup():
    cfg = tiny_config()
    hf = random_hf_weights(cfg, seed=0)
    mw = random_mtp_weights(cfg, seed=3)
    return cfg, hf, mw


def _independent_logits(cfg, hf, mw, tokens, hidden):
    w = {k: v.float() for k, v in mw.items()}
    emb = hf[R.P + "embed_tokens.weight"].float()
    eps = cfg.rms_norm_eps
    e = R.rms_norm_one_plus(emb[torch.tensor(tokens[1:])], w[MP + "pre_fc_norm_embedding.weight"], eps)
    h = R.rms_norm_one_plus(hidden.float(), w[MP + "pre_fc_norm_hidden.weight"], eps)
    x = torch.cat([e, h], -1) @ w[MP + "fc.weight"].T
    a = R.rms_norm_one_plus(x, w[LP + "input_layernorm.weight"], eps)
    r = R.attention_mixer(cfg, w, LP + "self_attn.", a, torch.arange(x.shape[0])) + x
    m = R.rms_norm_one_plus(r, w[LP + "post_attention_layernorm.weight"], eps)
    out = (torch.nn.functional.silu(m @ w[LP + "mlp.gate_proj.weight"].T) * (m @ w[LP + "mlp.up_proj.weight"].T)) \
        @ w[LP + "mlp.down_proj.weight"].T + r
    return R.rms_norm_one_plus(out, w[MP + "norm.weight"], eps) @ emb.T


def test_mtp_forward_and_chained_proposals(setup):
    cfg, hf, mw = setup
    T = 11
    tokens = torch.randint(0, cfg.vocab_size, (T + 1,), generator=torch.Generator().manual_seed(5)).tolist()
    _, taps = R.reference_forward(cfg, hf, tokens[:T], return_hidden_layers=[cfg.num_hidden_layers - 1])
    hidden = taps[cfg.num_hidden_layers - 1]
    emb = hf[R.P + "embed_tokens.weight"]
    want = _independent_logits(cfg, hf, mw, tokens, hidden)
    got = mtp_reference_rows(cfg, mw, tokens, hidden, emb, emb)
    assert torch.allclose(got, want, rtol=1e-4, atol=1e-4)

    d = MTPDrafter(cfg, mw, "cpu")
    d.bind(lambda ids: emb.float()[ids], lambda h: h.float() @ emb.float().T)
    # committed rows arrive in two pieces, as prefill chunks do
    d.append_context([hidden[:4]], 0, tokens=tokens[:4])
    d.append_context([hidden[4:]], 4, tokens=tokens[4:T])
    assert d.kv_len == T - 1
    with pytest.raises(ValueError):
        d.append_context([hidden[:2]], 3, tokens=tokens[3:5])          # rows must continue the committed prefix
    drafts = d.propose(tokens[T], 3, pos_start=T)
    assert len(drafts) == 3 and drafts[0] == int(torch.argmax(want[T - 1]))
    assert d.kv_len == T - 1 and d.propose(tokens[T], 3, pos_start=T) == drafts       # speculative rows left no trace
    # the chained rows really are the head run on its own output: replay the second draft by hand
    d2 = MTPDrafter(cfg, mw, "cpu")
    d2.bind(d.embed, d.lm_head_logits)
    ids = torch.tensor(tokens[1:T + 1])
    out = d2.forward(emb.float()[ids], hidden, 0)
    nxt = d2.forward(emb.float()[torch.tensor([drafts[0]])], out[-1:], T)
    assert int(torch.argmax(d2.logits(nxt))) == drafts[1]
    post = MTPDrafter(cfg, mw, "cpu", chain="post")
    post.bind(d.embed, d.lm_head_logits)
    post.append_context([hidden], 0, tokens=tokens[:T])
    assert post.propose(tokens[T], 2, pos_start=T)[0] == drafts[0]


def test_mtp_geometry_contract(setup):
    cfg, hf, mw = setup
    shapes = {k: tuple(v.shape) for k, v in mw.items()}
    validate_mtp_geometry(cfg, shapes)
    bad = dict(shapes); bad[MP + "fc.weight"] = (cfg.hidden_size, cfg.hidden_size)
    with pytest.raises(ValueError):
        validate_mtp_geometry(cfg, bad)
    missing = dict(shapes); missing.pop(LP + "self_attn.q_norm.weight")
    with pytest.raises(ValueError):
        validate_mtp_geometry(cfg, missing)
    assert set(mtp_tensor_shapes(cfg)) == set(shapes)


@pytest.mark.parametrize("chain", ["pre", "post"])
def test_mtp_speculative_decoding_equals_greedy(setup, chain):
    cfg, hf, mw = setup
    ew = build_engine_weights(cfg, lambda n: hf[n], "bf16", "cpu")
    prompt = torch.randint(0, cfg.vocab_size, (19,), generator=torch.Generator().manual_seed(9)).tolist()
    ref = R.reference_greedy(cfg, hf, prompt, 20)
    eng = Engine(ew, "cpu", StateConfig(max_slots=1, max_seq_len=96, conv_ring=16, spec_rows=8))
    dec = DFlash2SpecDecoder(eng, MTPDrafter(cfg, mw, "cpu", chain=chain), num_drafts=3)
    out, stats = dec.generate(prompt, 20, prefill_chunk=8)
    assert out == ref
    assert stats["rounds"] > 0 and stats["proposed"] >= stats["accepted"]
