"""End-to-end token exactness of the engine (paged KV, chunked prefill, ring conv state) against the
whole-sequence PyTorch oracle on the tiny hybrid model, on CPU in fp32."""
import pytest
import torch

from phaseshift_b200.models.qwen35.config import tiny_config
from phaseshift_b200.models.qwen35.reference import reference_forward, reference_greedy
from phaseshift_b200.models.qwen35.weights import build_engine_weights, random_hf_weights
from phaseshift_b200.runtime.batch import SeqRows
from phaseshift_b200.runtime.engine import Engine, SequenceError
from phaseshift_b200.runtime.state import StateConfig


@pytest.fixture(scope="module")
def tiny():
    cfg = tiny_config()
    hf = random_hf_weights(cfg, seed=0)
    ew = build_engine_weights(cfg, lambda n: hf[n], "bf16", "cpu")
    return cfg, hf, ew


def _prompt(cfg, n, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist()


def test_greedy_64_tokens_token_exact(tiny):
    cfg, hf, ew = tiny
    prompt = _prompt(cfg, 32)
    ref = reference_greedy(cfg, hf, prompt, 64)
    eng = Engine(ew, "cpu", StateConfig(max_slots=1, max_seq_len=128, page_tokens=16))
    out = eng.generate(prompt, 64, prefill_chunk=2048)
    assert out == ref


@pytest.mark.parametrize("chunk", [1, 5, 16, 31])
def test_chunked_prefill_matches(tiny, chunk):
    cfg, hf, ew = tiny
    prompt = _prompt(cfg, 32, seed=1)
    ref = reference_greedy(cfg, hf, prompt, 8)
    eng = Engine(ew, "cpu", StateConfig(max_slots=1, max_seq_len=64, page_tokens=16))
    assert eng.generate(prompt, 8, prefill_chunk=chunk) == ref


def test_mixed_batch_two_sequences(tiny):
    """A decode row of one request and a prefill chunk of another in the same step."""
    cfg, hf, ew = tiny
    pa, pb = _prompt(cfg, 20, seed=2), _prompt(cfg, 24, seed=3)
    ra, rb = reference_greedy(cfg, hf, pa, 6), reference_greedy(cfg, hf, pb, 6)
    eng = Engine(ew, "cpu", StateConfig(max_slots=2, max_seq_len=64, page_tokens=16))
    sa, sb = eng.open_sequence(), eng.open_sequence()
    ta = eng.prefill(sa, pa)
    outs_a, outs_b = [ta], []
    # step 1: A decodes, B prefills its first 10 tokens
    toks, _ = eng.step([SeqRows(sa.slot, sa.position, [ta], (0,)), SeqRows(sb.slot, 0, pb[:10], ())], [sa, sb])
    outs_a.append(toks[0])
    # step 2: A decodes, B finishes prefill and samples
    toks, _ = eng.step([SeqRows(sa.slot, sa.position, [outs_a[-1]], (0,)),
                        SeqRows(sb.slot, sb.position, pb[10:], (len(pb) - 11,))], [sa, sb])
    outs_a.append(toks[0]); outs_b.append(toks[1])
    while len(outs_b) < 6:
        rows = [SeqRows(sb.slot, sb.position, [outs_b[-1]], (0,))]
        objs = [sb]
        if len(outs_a) < 6:
            rows.insert(0, SeqRows(sa.slot, sa.position, [outs_a[-1]], (0,)))
            objs.insert(0, sa)
        toks, _ = eng.step(rows, objs)
        if len(objs) == 2:
            outs_a.append(toks[0]); outs_b.append(toks[1])
        else:
            outs_b.append(toks[0])
    assert outs_a == ra and outs_b == rb


def test_logits_close_to_oracle(tiny):
    cfg, hf, ew = tiny
    prompt = _prompt(cfg, 17, seed=4)
    ref = reference_forward(cfg, hf, prompt)
    eng = Engine(ew, "cpu", StateConfig(max_slots=1, max_seq_len=32, page_tokens=16))
    s = eng.open_sequence()
    _, out = eng.step([SeqRows(s.slot, 0, prompt, tuple(range(len(prompt))))], [s])
    assert torch.allclose(out.logits, ref, atol=2e-4, rtol=1e-4)


def test_out_of_pages_rolls_back(tiny):
    cfg, hf, ew = tiny
    eng = Engine(ew, "cpu", StateConfig(max_slots=2, max_seq_len=64, page_tokens=16, kv_capacity_tokens=32))
    free0 = eng.alloc.pages_free
    s = eng.open_sequence()
    with pytest.raises(SequenceError):
        eng.step([SeqRows(s.slot, 0, _prompt(cfg, 16 * (free0 + 1)), ())], [s])
    assert eng.alloc.pages_free == free0 and s.position == 0


def test_stale_handle_detected(tiny):
    cfg, hf, ew = tiny
    eng = Engine(ew, "cpu", StateConfig(max_slots=1, max_seq_len=32))
    s = eng.open_sequence()
    eng.close_sequence(s)
    s2 = eng.open_sequence()
    assert s2.slot == s.slot and s2.generation != s.generation
    with pytest.raises(SequenceError):
        eng.close_sequence(s)
