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
