"""Entry points on CPU: compute single-shot / serve-stdio contract, quantizer CLI, argument validation."""
import io
import json
import os
import subprocess
import sys

import pytest
import torch

from phaseshift_b200.apps import compute, quantizer
from phaseshift_b200.io.model_dir import save_hf_model
from phaseshift_b200.models.qwen35.config import tiny_config
from phaseshift_b200.models.qwen35.reference import reference_greedy
from phaseshift_b200.models.qwen35.weights import random_hf_weights

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def model_dir(tmp_path_factory):
    d = tmp_path_factory.mktemp("app") / "tiny"
    cfg = tiny_config(eos_token_ids=[4095])
    hf = random_hf_weights(cfg, seed=0)
    save_hf_model(d, cfg, hf)
    return cfg, hf, d


def test_invalid_flags_exit_2_before_load():
    assert compute.main(["--random-model", "tiny", "--decode-backend", "gpu-mcu"]) == 2
    assert compute.main(["--max-new-tokens", "4"]) == 2
    assert compute.main(["--random-model", "tiny", "--dflash2-ngram-tail", "2"]) == 2
    with pytest.raises(SystemExit):
        compute.main(["--help"])


def test_single_shot_contract(model_dir, tmp_path, capsys):
    cfg, hf, d = model_dir
    ids = torch.randint(0, 4000, (12,), generator=torch.Generator().manual_seed(2)).tolist()
    f = tmp_path / "p.ids"
    f.write_text(" ".join(map(str, ids)))
    assert compute.main(["--model-dir", str(d), "--input-ids-file", str(f), "--max-new-tokens", "6", "--device", "cpu"]) == 0
    out = dict(l.split("=", 1) for l in capsys.readouterr().out.strip().splitlines())
    assert out["PROMPT_TOKENS"] == "12" and out["GENERATED_TOKENS"] == "6" and out["KV_CACHE_DTYPE"] == "bf16"
    assert [int(t) for t in out["GENERATED_IDS"].split(",")] == reference_greedy(cfg, hf, ids, 6)
    # the upstream names of the block-coded caches select the 4-bit / 8-bit pools (the fp32 CPU oracle keeps full precision)
    assert compute.main(["--model-dir", str(d), "--input-ids-file", str(f), "--max-new-tokens", "2", "--device", "cpu",
                         "--kv-cache-dtype", "psq4"]) == 0
    assert "KV_CACHE_DTYPE=nvfp4" in capsys.readouterr().out
    lg = tmp_path / "l.bin"
    assert compute.main(["--model-dir", str(d), "--input-ids-file", str(f), "--max-new-tokens", "3", "--device", "cpu",
                         "--dump-logits", str(lg)]) == 0
    out2 = dict(l.split("=", 1) for l in capsys.readouterr().out.strip().splitlines())
    assert out2["LOGITS_VOCAB"] == "4096" and out2["LOGITS_TOTAL_ROWS"] == "3" and lg.stat().st_size == 3 * 4096 * 4
    assert out2["GENERATED_IDS"].split(",") == out["GENERATED_IDS"].split(",")[:3]


@pytest.mark.timeout(180)
def test_serve_stdio_protocol(model_dir):
    cfg, hf, d = model_dir
    p = subprocess.Popen([sys.executable, "-m", "phaseshift_b200.apps.compute", "--model-dir", str(d), "--device", "cpu",
                          "--serve-stdio", "--max-concurrent-requests", "2", "--max-seq-len", "128"],
                         stdin=subprocess.PIPE, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, cwd=ROOT,
                         env=dict(os.environ, PYTHONPATH=ROOT))
    try:
        assert "PHASESHIFT_SERVE_READY" in p.stderr.readline()
        ids = list(range(5, 25))

        def send(o):
            p.stdin.write(json.dumps(o) + "\n"); p.stdin.flush()
        send({"op": "ping"})
        assert json.loads(p.stdout.readline()) == {"event": "pong"}
        send({"op": "generate", "request_id": 7, "input_ids": ids, "max_new_tokens": 5})
        send({"op": "generate", "request_id": 8, "input_ids": ids[:9], "max_new_tokens": 100})
        toks, done = {7: [], 8: []}, {}
        while 7 not in done:
            e = json.loads(p.stdout.readline())
            if e["event"] == "token":
                toks[e["request_id"]].append(e["token_id"])
            elif e["event"] == "done":
                done[e["request_id"]] = e
        assert toks[7] == done[7]["generated_ids"] == reference_greedy(cfg, hf, ids, 5)
        assert done[7]["finish_reason"] == "length" and done[7]["prompt_tokens"] == 20
        send({"op": "cancel", "request_id": 8})
        while 8 not in done:
            e = json.loads(p.stdout.readline())
            if e["event"] == "done":
                done[e["request_id"]] = e
        assert done[8]["finish_reason"] == "cancelled"
        send({"op": "bogus", "request_id": 9})
        assert json.loads(p.stdout.readline())["event"] == "error"
        send({"op": "shutdown"})
        assert json.loads(p.stdout.readline()) == {"event": "shutdown"}
        assert p.wait(timeout=30) == 0
    finally:
        if p.poll() is None:
            p.kill()


def test_serve_stdio_with_speculative_decoding(model_dir, tmp_path):
    """--dflash2-model-dir under --serve-stdio: requests are served through speculative rounds and emit exactly the
    plain greedy stream."""
    from phaseshift_b200.models.dflash2.model import DFlash2Drafter, random_weights, tiny_drafter_config
    cfg, hf, d = model_dir
    dcfg = tiny_drafter_config(cfg)
    ddir = tmp_path / "drafter"
    DFlash2Drafter(dcfg, random_weights(dcfg, seed=1), "cpu").save(ddir)
    p = subprocess.Popen([sys.executable, "-m", "phaseshift_b200.apps.compute", "--model-dir", str(d), "--device", "cpu",
                          "--serve-stdio", "--max-seq-len", "128", "--dflash2-model-dir", str(ddir), "--dflash2-drafts", "4",
                          "--max-scheduled-tokens", "8"],
                         stdin=subprocess.PIPE, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, cwd=ROOT,
                         env=dict(os.environ, PYTHONPATH=ROOT))
    try:
        assert "PHASESHIFT_SERVE_READY" in p.stderr.readline()
        ids = list(range(5, 25))
        for rid, n in ((1, 12), (2, 7)):
            p.stdin.write(json.dumps({"op": "generate", "request_id": rid, "input_ids": ids[:20 - rid], "max_new_tokens": n}) + "\n")
        p.stdin.flush()
        toks, done = {1: [], 2: []}, {}
        while len(done) < 2:
            e = json.loads(p.stdout.readline())
            if e["event"] == "token":
                toks[e["request_id"]].append(e["token_id"])
            elif e["event"] == "done":
                done[e["request_id"]] = e
            else:
                raise AssertionError(e)
        assert toks[1] == done[1]["generated_ids"] == reference_greedy(cfg, hf, ids[:19], 12)
        assert toks[2] == done[2]["generated_ids"] == reference_greedy(cfg, hf, ids[:18], 7)
        assert done[1]["prefill_tokens"] == 19
        p.stdin.write(json.dumps({"op": "shutdown"}) + "\n"); p.stdin.flush()
        assert json.loads(p.stdout.readline()) == {"event": "shutdown"}
        assert p.wait(timeout=30) == 0
    finally:
        if p.poll() is None:
            p.kill()


def test_tensor_parallel_apps_on_cpu(model_dir, tmp_path):
    """--tp 2 on the compute app (gloo ranks on CPU): the process becomes rank 0 and starts rank 1 itself; single shot
    prints the single-rank stream, and under --serve-stdio rank 1 replays rank 0's commands step for step."""
    cfg, hf, d = model_dir
    ids = list(range(5, 25))
    idf = tmp_path / "ids.txt"
    idf.write_text(" ".join(map(str, ids)))
    stats = tmp_path / "perf.json"
    env = dict(os.environ, PYTHONPATH=ROOT)
    env.pop("RANK", None); env.pop("WORLD_SIZE", None)
    r = subprocess.run([sys.executable, "-m", "phaseshift_b200.apps.compute", "--model-dir", str(d), "--device", "cpu", "--tp", "2",
                        "--input-ids-file", str(idf), "--max-new-tokens", "6", "--max-seq-len", "64",
                        "--perf-stats-output", str(stats)], capture_output=True, text=True, cwd=ROOT, env=env, timeout=240)
    assert r.returncode == 0, r.stderr[-2000:]
    want = reference_greedy(cfg, hf, ids, 6)
    assert "GENERATED_IDS=" + ",".join(map(str, want)) in r.stdout
    ps = json.loads(stats.read_text())
    assert ps["tp"]["size"] == 2 and ps["steps"] > 0 and "serving" in ps
    p = subprocess.Popen([sys.executable, "-m", "phaseshift_b200.apps.compute", "--model-dir", str(d), "--device", "cpu", "--tp", "2",
                          "--serve-stdio", "--max-concurrent-requests", "2", "--max-seq-len", "64"],
                         stdin=subprocess.PIPE, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, cwd=ROOT, env=env)
    try:
        assert "PHASESHIFT_SERVE_READY" in p.stderr.readline()
        for rid, n in ((1, 6), (2, 4)):
            p.stdin.write(json.dumps({"op": "generate", "request_id": rid, "input_ids": ids[:20 - rid], "max_new_tokens": n}) + "\n")
        p.stdin.flush()
        done = {}
        while len(done) < 2:
            e = json.loads(p.stdout.readline())
            if e["event"] == "done":
                done[e["request_id"]] = e
            assert e["event"] != "error", e
        assert done[1]["generated_ids"] == reference_greedy(cfg, hf, ids[:19], 6)
        assert done[2]["generated_ids"] == reference_greedy(cfg, hf, ids[:18], 4)
        p.stdin.write(json.dumps({"op": "shutdown"}) + "\n"); p.stdin.flush()
        assert json.loads(p.stdout.readline()) == {"event": "shutdown"}
        assert p.wait(timeout=60) == 0
    finally:
        if p.poll() is None:
            p.kill()


def test_quantizer_cli(model_dir, tmp_path, capsys):
    cfg, hf, d = model_dir
    out = tmp_path / "q"
    assert quantizer.main(["quantize", "--input", str(d), "--output", str(out), "--preset", "nvfp4"]) == 0
    assert quantizer.main(["quantize", "--input", str(d), "--output", str(out)]) == 2          # not empty, no --overwrite
    assert quantizer.main(["verify", str(out)]) == 0
    tk = tmp_path / "t.txt"
    tk.write_text(" ".join(str(i % 4000) for i in range(3, 70)))
    capsys.readouterr()
    assert quantizer.main(["kld", "--input", str(d), "--bundle", str(out), "--tokens", str(tk), "--window", "32",
                           "--stride", "32", "--device", "cpu"]) == 0
    rep = dict(l.split("=", 1) for l in capsys.readouterr().out.strip().splitlines())
    assert float(rep["KLD_MEAN"]) >= 0 and float(rep["KLD_MAX"]) >= float(rep["KLD_P50"])
    assert quantizer.main(["ppl", "--model-dir", str(out), "--tokens", str(tk), "--max-tokens", "40", "--device", "cpu"]) == 0
    # quantised directory runs through compute with the exact-match contract against itself
    assert compute.main(["--model-dir", str(out), "--max-new-tokens", "4", "--device", "cpu", "--verify-weights", "1"]) == 0


def test_bench_subcommands_help_and_cpu_runs(capsys):
    from phaseshift_b200.apps import bench
    for sub in bench.SUBCOMMANDS:
        with pytest.raises(SystemExit) as e:
            bench.main([sub, "--help"])
        assert e.value.code == 0
    with pytest.raises(SystemExit) as e:
        bench.main(["rmsnorm", "--variant", "bogus"])            # invalid variant must fail
    assert e.value.code == 2
    capsys.readouterr()
    assert bench.main(["tg", "--random-model", "tiny", "--device", "cpu", "--context", "12", "--tokens", "4", "--runs", "2"]) == 0
    out = dict(l.split("=", 1) for l in capsys.readouterr().out.strip().splitlines())
    assert out["deterministic"] == "1" and float(out["gpu_tokens_per_sec"]) > 0 and "GREEDY_TOKEN_SUM" in out
    assert bench.main(["pp", "--random-model", "tiny", "--device", "cpu", "--prompt-tokens", "24", "--runs", "1", "--warmup", "0"]) == 0
    assert bench.main(["batch", "--random-model", "tiny", "--device", "cpu", "--requests", "3", "--prompt-tokens", "20",
                       "--tokens", "3"]) == 0
    assert "aggregate_tokens_per_sec" in capsys.readouterr().out
    # MTP speculative decoding with a random head: exact verification reproduces plain greedy decoding
    assert bench.main(["mtp", "--random-model", "tiny", "--device", "cpu", "--context", "20", "--tokens", "10", "--draft-k", "3",
                       "--runs", "1", "--warmup", "0", "--replay-check"]) == 0
    out = dict(l.split("=", 1) for l in capsys.readouterr().out.strip().splitlines())
    assert out["replay_match"] == "1" and int(out["proposed"]) >= int(out["accepted"]) and out["mtp_head"] == "random-init"
    assert bench.main(["tg", "--mtp", "--draft-k", "2", "--random-model", "tiny", "--device", "cpu", "--context", "16", "--tokens", "6",
                       "--runs", "1", "--warmup", "0"]) == 0                               # the upstream spelling of the same run
    assert "proposed" in capsys.readouterr().out
    # quantised preset against the bf16 model of the same random weights: small divergence on a 4-layer model, and the
    # 8-bit preset closer than the 4-bit one
    kld = {}
    for preset in ("nvfp4", "mxfp8"):
        assert bench.main(["kld", "--random-model", "tiny", "--device", "cpu", "--tokens", "16", "--streams", "1", "--preset", preset]) == 0
        kld[preset] = dict(l.split("=", 1) for l in capsys.readouterr().out.strip().splitlines())
    assert 0 <= float(kld["mxfp8"]["kld_mean"]) < float(kld["nvfp4"]["kld_mean"]) < 0.05
    assert float(kld["nvfp4"]["kld_over_decorrelated"]) < 0.3


def test_cli_single_turn_prints_the_decoded_continuation(model_dir, capsys):
    """phaseshift-cli spawns the compute program for a turn; a directory without tokenizer assets gets the byte tokenizer."""
    from phaseshift_b200.apps import cli
    from phaseshift_b200.serving.chat import ByteTokenizer
    cfg, hf, d = model_dir
    assert cli.main(["--model-dir", str(d), "--prompt", "hi", "--max-new-tokens", "4", "--max-seq-len", "128", "--device", "cpu"]) == 0
    printed = capsys.readouterr().out
    tok = ByteTokenizer(cfg.vocab_size)
    ids = tok.apply_chat_template([{"role": "user", "content": "hi"}], add_generation_prompt=True, tokenize=True)
    want = tok.decode(reference_greedy(cfg, hf, ids, 4))
    assert printed == want + "\n"
