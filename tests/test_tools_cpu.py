"""phaseshift-tools and the draft-vocabulary profile on CPU."""
import json

import numpy as np
import pytest

from phaseshift_b200.apps import tools
from phaseshift_b200.models.dflash2 import draft_vocab as dv


def test_draft_vocab_profile_roundtrip_and_validation(tmp_path):
    ids = list(range(0, 640, 2))                     # 320 ids, multiple of 16
    out = dv.pack(ids[::-1], tmp_path / "p", "test-v1", 4096, 256)
    prof = dv.load_profile(out, 4096, 256)
    assert prof.count == 320 and prof.profile_id == "test-v1" and prof.ids[0] == 0 and prof.ids[-1] == 638
    assert dv.load_profile(tmp_path, 4096, 256) is None                       # nothing installed: no profile
    with pytest.raises(dv.DraftVocabError):
        dv.load_profile(out, 4096, 512)                                       # other model shape
    (out / dv.PAYLOAD_NAME).write_bytes((out / dv.PAYLOAD_NAME).read_bytes()[:-4] + b"\\x00\\x00\\x00\\x00")
    with pytest.raises(dv.DraftVocabError):
        dv.load_profile(out, 4096, 256)                                       # damaged payload
    (out / dv.PAYLOAD_NAME).unlink()
    with pytest.raises(dv.DraftVocabError):
        dv.load_profile(out, 4096, 256)                                       # partly installed
    for bad in ([1, 2, 3], list(range(16)) + [15] * 16, [5000] + list(range(15))):
        with pytest.raises(dv.DraftVocabError):
            dv.validate_ids(np.asarray(sorted(bad)), 4096)


def test_resolution_is_opt_in(tmp_path):
    out = dv.pack(range(64), tmp_path, "p", 4096, 256)
    assert dv.resolve(out, 4096, 256, env={}) is None                          # installed but not asked for
    assert dv.resolve(out, 4096, 256, env={"PS_DFLASH2_DRAFT_VOCAB": "0"}) is None
    assert dv.resolve(out, 4096, 256, env={"PS_DFLASH2_DRAFT_VOCAB": "1"}).count == 64
    raw = tmp_path / "raw.u32"
    np.arange(0, 96, 3, dtype="<u4").tofile(raw)
    assert dv.resolve(None, 4096, 256, env={"PS_DFLASH2_DRAFT_VOCAB_FILE": str(raw)}).count == 32
    with pytest.raises(dv.DraftVocabError):
        dv.resolve(None, 4096, 256, env={"PS_DFLASH2_DRAFT_VOCAB_FILE": str(raw), "PS_DFLASH2_DRAFT_VOCAB": "0"})


def test_tools_cli_corpus_select_pack_check_and_oracle(tmp_path, capsys):
    from phaseshift_b200.models.qwen35.config import tiny_config
    from phaseshift_b200.models.qwen35.reference import reference_greedy
    from phaseshift_b200.models.qwen35.weights import random_hf_weights
    from phaseshift_b200.quant.offline import read_tokens
    corpus = tmp_path / "c.bin"
    assert tools.main(["token-corpus", "--byte-tokenizer", "512", "--text", "hello hello world", "--output", str(corpus)]) == 0
    toks = read_tokens(corpus)
    assert len(toks) == 17 and toks[0] == ord("h") + 3
    assert tools.main(["token-corpus", "--byte-tokenizer", "512", "--base", str(corpus), "--text", "!", "--output", str(corpus)]) == 0
    assert len(read_tokens(corpus)) == 18
    ids = tmp_path / "ids.u32"
    assert tools.main(["draft-vocab", "select", "--tokens", str(corpus), "--count", "20", "--model-vocab-size", "512",
                       "--always", "1 2", "--output", str(ids)]) == 0
    sel = np.fromfile(ids, dtype="<u4")
    assert sel.size == 32 and ord("l") + 3 in sel and 1 in sel and 2 in sel          # rounded up to 32, frequent + forced ids
    # a model directory to install the profile into
    from phaseshift_b200.io.model_dir import ShardWriter
    cfg = tiny_config(vocab_size=512)
    hf = random_hf_weights(cfg, seed=0)
    md = tmp_path / "model"
    cfg.save(md)
    wr = ShardWriter(md)
    for n, t in hf.items():
        wr.add(n, t.dtype, t.shape)
    wr.begin()
    for n, t in hf.items():
        wr.write(n, t)
    wr.finish()
    assert tools.main(["draft-vocab", "pack", "--vocab-file", str(ids), "--profile-id", "tiny-v1", "--model-vocab-size", "512",
                       "--hidden-size", str(cfg.hidden_size), "--output-dir", str(md)]) == 0
    capsys.readouterr()
    assert tools.main(["draft-vocab", "check", "--model-dir", str(md)]) == 0
    assert "DRAFT_VOCAB=ok" in capsys.readouterr().out
    prompt = tmp_path / "p.txt"
    prompt.write_text("5 6 7 8 9 10 11")
    assert tools.main(["oracle-tokens", "--model-dir", str(md), "--input-ids-file", str(prompt), "--max-new-tokens", "4",
                       "--dump-logits", str(tmp_path / "lg.bin")]) == 0
    out = capsys.readouterr().out
    want = reference_greedy(cfg, {k: v.to(hf[k].dtype).float() for k, v in hf.items()}, [5, 6, 7, 8, 9, 10, 11], 4)
    assert "GENERATED_IDS=" + ",".join(map(str, want)) in out
    assert np.fromfile(tmp_path / "lg.bin", dtype="<f4").size == 4 * 512
