"""Offline quantiser round trip on a tiny model (CPU): quantize -> verify -> load -> kld / ppl / imatrix."""
import json

import pytest
import torch

from phaseshift_b200.io.model_dir import ShardCollection, save_hf_model
from phaseshift_b200.models.qwen35.config import tiny_config
from phaseshift_b200.models.qwen35.weights import build_engine_weights, load_engine_weights, random_hf_weights
from phaseshift_b200.quant import offline
from phaseshift_b200.quant.manifest import Manifest


@pytest.fixture(scope="module")
def model_dirs(tmp_path_factory):
    d = tmp_path_factory.mktemp("m")
    cfg = tiny_config()
    hf = random_hf_weights(cfg, seed=0)
    src = d / "bf16"
    save_hf_model(src, cfg, hf, max_shard_size=1 << 20)      # force several shards
    return cfg, hf, src, d


def test_sharded_hf_dir_roundtrip(model_dirs):
    cfg, hf, src, _ = model_dirs
    assert (src / "model.safetensors.index.json").exists()
    col = ShardCollection(src)
    for n, t in hf.items():
        assert torch.equal(col.tensor(n), t)
    ew = load_engine_weights(src, "cpu")
    assert ew.layers[0].mixer.in_proj.N == cfg.gdn_conv_dim + cfg.gdn_v_dim


def test_quantize_verify_load_and_eval(model_dirs):
    cfg, hf, src, d = model_dirs
    out = d / "nvfp4"
    man = offline.quantize_model(src, out, preset="nvfp4", backend="cpu", max_shard_size=1 << 20, log=lambda *_: None)
    assert offline.validate_model_dir(out) == []
    m2 = Manifest.load(out)
    enc = {t.name: t.encoding for t in m2.tensors}
    assert enc["model.language_model.embed_tokens.weight"] == "mxfp8"
    assert enc["model.language_model.layers.0.mlp.down_proj.weight"] == "mxfp8"      # layer % 4 == 0
    assert enc["model.language_model.layers.1.mlp.down_proj.weight"] == "nvfp4"
    assert enc["model.language_model.layers.0.linear_attn.in_proj_a.weight"] == "bf16"
    assert enc["model.language_model.layers.3.self_attn.q_proj.weight"] == "nvfp4"
    # q/k/v share one NVFP4 tensor scale so they can be fused into one projection without requantising
    byn = m2.by_name()
    a = "model.language_model.layers.3.self_attn."
    assert byn[a + "q_proj.weight"].metadata2 == byn[a + "k_proj.weight"].metadata2 == byn[a + "v_proj.weight"].metadata2
    # quantised directory loads into the engine and agrees with on-the-fly quantisation of the same weights
    ew_dir = load_engine_weights(out, "cpu")
    ew_fly = build_engine_weights(cfg, lambda n: hf[n], "nvfp4", "cpu")
    for ld, lf in zip(ew_dir.layers, ew_fly.layers):
        rel = (ld.gate_up.dense() - lf.gate_up.dense()).norm() / lf.gate_up.dense().norm()
        assert rel < 0.05
    toks = torch.randint(0, cfg.vocab_size, (80,), generator=torch.Generator().manual_seed(3)).tolist()
    rep = offline.evaluate_kld(src, out, toks, window=32, stride=32)
    assert rep["positions"] > 60 and 0 <= rep["mean"] < 0.05 and rep["max"] >= rep["p99"] >= rep["p50"] >= 0
    selfrep = offline.evaluate_kld(src, out, toks, window=32, stride=32, self_check=True)
    # baseline-logit cache: the second run reads every window from disk and reports the same numbers
    cdir = d / "kld_cache"
    r1 = offline.evaluate_kld(src, out, toks, window=32, stride=32, baseline_cache=cdir)
    r2 = offline.evaluate_kld(src, out, toks, window=32, stride=32, baseline_cache=cdir)
    assert r1["baseline_cache_misses"] > 0 and r1["baseline_cache_hits"] == 0
    assert r2["baseline_cache_misses"] == 0 and r2["baseline_cache_hits"] == r1["baseline_cache_misses"]
    assert abs(r1["mean"] - rep["mean"]) < 1e-12 and abs(r2["mean"] - rep["mean"]) < 1e-9
    assert selfrep["max"] < 1e-9 and selfrep["top1_agreement"] == 1.0
    ppl = offline.evaluate_ppl(out, toks, max_tokens=48)
    assert ppl["ppl"] > 1.0
    # corrupt one byte -> verify must notice
    victim = next(out.glob("model-00001*.safetensors"))
    b = bytearray(victim.read_bytes()); b[-5] ^= 0xFF; victim.write_bytes(bytes(b))
    assert any("CRC" in p for p in offline.validate_model_dir(out))


def test_imatrix_collect_and_weighted_quantize(model_dirs):
    cfg, hf, src, d = model_dirs
    toks = torch.randint(0, cfg.vocab_size, (70,), generator=torch.Generator().manual_seed(4)).tolist()
    im = d / "im.safetensors"
    rep = offline.collect_imatrix(src, toks, im, window=32, stride=32)
    assert rep["sites"] == 4 * cfg.num_hidden_layers + 1      # 4 projection inputs per layer + lm_head
    assert rep["windows"] == 3 and rep["flushes"] == 0
    loaded = offline.load_imatrix(im)
    # periodic flushes leave the same final file, and the command line carries the upstream flag names
    from phaseshift_b200.apps import quantizer as qapp
    tf = d / "cal.tokens"
    tf.write_text(" ".join(map(str, toks)))
    im2 = d / "im2.safetensors"
    assert qapp.main(["imatrix", "--model-dir", str(src), "--tokens", str(tf), "--output", str(im2), "--window", "32",
                      "--stride", "32", "--flush-windows", "1", "--arena-gib", "1", "--device", "cpu"]) == 0
    loaded2 = offline.load_imatrix(im2)
    assert set(loaded2) == set(loaded) and all(torch.equal(loaded2[k_], loaded[k_]) for k_ in loaded)
    assert qapp.main(["kld", "--input", str(src), "--bundle", str(src), "--tokens", str(tf), "--window", "32", "--stride", "32",
                      "--batch-positions", "8", "--cache-dir", str(d / "cd"), "--keep-logit-cache", "--keep-shadow",
                      "--device", "cpu"]) == 0
    assert any((d / "cd").iterdir())
    k = "model.language_model.layers.0.mlp.gate_proj.weight"
    assert loaded[k].shape == (cfg.hidden_size,) and float(loaded[k].min()) >= 0
    out = d / "nvfp4_im"
    offline.quantize_model(src, out, preset="nvfp4", backend="cpu", imatrix=str(im), imatrix_policy="best-effort",
                           log=lambda *_: None)
    assert offline.validate_model_dir(out) == [] and Manifest.load(out).imatrix["file"] == str(im)


def test_interchange_formats_roundtrip_and_kernel_conversion():
    """MXFP4 and FP8-block128 (interchange formats): quantise/dequantise, and re-expression in the formats the
    kernels execute -- lossless for MXFP4 -> NVFP4, one e4m3 re-rounding for FP8-block128 -> MXFP8."""
    import torch
    from phaseshift_b200.quant import formats as F
    g = torch.Generator().manual_seed(0)
    w = torch.randn(40, 200, generator=g) * 0.05
    w[3, :64] = 0
    w[7] *= 30
    q4 = F.quantize(w, "mxfp4")
    d4 = F.dequantize(q4)
    assert q4.codes.shape == (40, 112) and q4.scales.shape == (40, 7)
    assert float((d4 - w).norm() / w.norm()) < 0.13
    k4 = F.to_kernel_format(q4)
    assert k4.fmt == "nvfp4" and torch.equal(F.dequantize(k4), d4)
    q8 = F.quantize(w, "fp8_block128")
    d8 = F.dequantize(q8)
    assert q8.scales.dtype == torch.float32 and q8.scales.shape == (1, 2)
    assert float((d8 - w).norm() / w.norm()) < 0.04
    k8 = F.to_kernel_format(q8)
    assert k8.fmt == "mxfp8" and float((F.dequantize(k8) - d8).norm() / d8.norm()) < 0.04
    assert F.to_kernel_format(F.quantize(w, "nvfp4")).fmt == "nvfp4"


def test_mxfp4_bundle_loads_and_runs_as_nvfp4(tmp_path):
    """An OCP-MXFP4 model directory written by the quantizer loads through the NVFP4 path without re-quantisation
    loss: the engine built from the bundle and the engine built from the dequantised MXFP4 weights emit the same
    tokens; the in-memory interchange presets build too."""
    import torch
    from phaseshift_b200.io.model_dir import save_hf_model
    from phaseshift_b200.models.qwen35.config import tiny_config
    from phaseshift_b200.models.qwen35.weights import build_engine_weights, load_engine_weights, random_hf_weights
    from phaseshift_b200.quant import offline
    from phaseshift_b200.runtime.engine import Engine
    from phaseshift_b200.runtime.state import StateConfig
    cfg = tiny_config()
    hf = random_hf_weights(cfg, seed=2)
    src = tmp_path / "bf16"
    save_hf_model(src, cfg, hf)
    out = tmp_path / "mxfp4"
    man = offline.quantize_model(src, out, "mxfp4", "cpu")
    assert any(t.encoding == "mxfp4" for t in man.tensors)
    assert offline.validate_model_dir(out) == []
    ew = load_engine_weights(out, "cpu")
    assert ew.layers[0].gate_up.fmt == "nvfp4"
    prompt = list(range(5, 25))
    toks = Engine(ew, "cpu", StateConfig(max_slots=1, max_seq_len=64)).generate(prompt, 8, prefill_chunk=16)
    ew2 = build_engine_weights(cfg, lambda n: hf[n], "mxfp4", "cpu")
    toks2 = Engine(ew2, "cpu", StateConfig(max_slots=1, max_seq_len=64)).generate(prompt, 8, prefill_chunk=16)
    assert toks == toks2
    ew3 = build_engine_weights(cfg, lambda n: hf[n], "fp8_block128", "cpu")
    assert ew3.layers[0].gate_up.fmt == "mxfp8"
    assert len(Engine(ew3, "cpu", StateConfig(max_slots=1, max_seq_len=64)).generate(prompt, 4, prefill_chunk=16)) == 4


def test_dflash2_adapter_quantizes_and_loads_a_drafter(tmp_path):
    """The quantizer's DFlash2 adapter: backbone projections of a drafter directory become NVFP4, norms /
    dynamic-conv kernels / selector tables stay BF16, the bundle verifies (and notices corruption), and the
    drafter loaded from it carries the dequantised weights."""
    import torch
    from phaseshift_b200.models.dflash2.model import DFlash2Drafter, random_weights, tiny_drafter_config
    from phaseshift_b200.models.qwen35.config import tiny_config
    from phaseshift_b200.quant import formats as F, offline
    from phaseshift_b200.quant.manifest import Manifest
    dc = tiny_drafter_config(tiny_config())
    w = random_weights(dc, seed=5)
    src = tmp_path / "drafter_bf16"
    DFlash2Drafter(dc, w, "cpu").save(src)
    assert offline.is_drafter_dir(src)
    out = tmp_path / "drafter_nvfp4"
    man = offline.quantize_model(src, out, "nvfp4", "cpu", log=lambda *_: None)
    enc = {t.name: t.encoding for t in man.tensors}
    assert enc["layers.0.self_attn.q_proj.weight"] == "nvfp4" and enc["layers.1.mlp.down_proj.weight"] == "nvfp4"
    assert enc["fc.weight"] == "nvfp4"
    assert enc["layers.0.attn_conv.kernel_projection.weight"] == "bf16" and enc["selector.pred_codebook"] == "bf16"
    assert enc["norm.weight"] == "bf16" and enc["layers.0.attn_conv.base_kernel"] == "bf16"
    assert offline.validate_model_dir(out) == []
    d2 = DFlash2Drafter.from_dir(out, "cpu")
    n = "layers.0.mlp.gate_proj.weight"
    ref = w[n].to(torch.bfloat16).float()
    assert torch.equal(d2.w[n], F.dequantize(F.quantize(ref, "nvfp4")).reshape(ref.shape))
    assert float((d2.w[n] - ref).norm() / ref.norm()) < 0.12
    assert torch.equal(d2.w["norm.weight"], w["norm.weight"].to(torch.bfloat16).float())
    assert Manifest.load(out).preset == "nvfp4"
    victim = next(out.glob("model*.safetensors"))
    b = bytearray(victim.read_bytes()); b[-3] ^= 0xFF; victim.write_bytes(bytes(b))
    assert any("CRC" in p for p in offline.validate_model_dir(out))


def test_fingerprint_separates_checkpoints_of_one_architecture(tmp_path):
    """The baseline-logit cache is keyed by the fingerprint: two checkpoints with identical shapes must not share it."""
    from phaseshift_b200.io.model_dir import save_hf_model
    from phaseshift_b200.models.qwen35.config import tiny_config
    from phaseshift_b200.models.qwen35.weights import random_hf_weights
    from phaseshift_b200.quant import offline
    cfg = tiny_config()
    a, b, c = tmp_path / "a", tmp_path / "b", tmp_path / "c"
    save_hf_model(a, cfg, random_hf_weights(cfg, seed=1))
    save_hf_model(b, cfg, random_hf_weights(cfg, seed=2))
    save_hf_model(c, cfg, random_hf_weights(cfg, seed=1))
    fa, fb, fc = offline.model_fingerprint(a), offline.model_fingerprint(b), offline.model_fingerprint(c)
    assert fa == fc and fa != fb and len(fa) == 64
