"""phaseshift-cli: minimal chat front end.  Tokenises with the model directory's HF tokenizer, spawns
``phaseshift-compute`` per turn and prints the decoded continuation (reference: src/apps/cli/
phaseshift_cli.py:57-121)."""
from __future__ import annotations

import argparse
import subprocess
import sys
import tempfile
from typing import List, Optional


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="phaseshift-cli")
    ap.add_argument("--model-dir", required=True); ap.add_argument("--binary", default=None)
    ap.add_argument("--prompt"); ap.add_argument("--max-new-tokens", type=int, default=128)
    ap.add_argument("--max-seq-len", type=int, default=4096); ap.add_argument("--arena-gib", type=float, default=16)
    ap.add_argument("--device", default=None); ap.add_argument("--dflash2-model-dir")
    ap.add_argument("--dflash2-drafts", type=int, default=7); ap.add_argument("--dflash2-stats", type=int, default=0)
    return ap


def main(argv: Optional[List[str]] = None) -> int:
    a = build_parser().parse_args(argv)
    import json
    import os
    from .server import load_tokenizer
    try:
        vocab = int(json.load(open(os.path.join(a.model_dir, "config.json"))).get("vocab_size", 0)) or 259
    except (OSError, ValueError):
        vocab = 259
    # the directory's own tokenizer and chat template; directories without tokenizer assets (random test models) get the
    # byte tokenizer the server uses for them
    tok = load_tokenizer(a.model_dir, vocab)
    history = []

    def turn(text: str) -> str:
        history.append({"role": "user", "content": text})
        ids = tok.apply_chat_template(history, add_generation_prompt=True, tokenize=True)
        with tempfile.NamedTemporaryFile("w", suffix=".ids", delete=False) as f:
            f.write(" ".join(map(str, ids)))
        cmd = ([a.binary] if a.binary else [sys.executable, "-m", "phaseshift_b200.apps.compute"]) + [
            "--model-dir", a.model_dir, "--input-ids-file", f.name, "--max-new-tokens", str(a.max_new_tokens),
            "--max-seq-len", str(a.max_seq_len), "--arena-gib", str(a.arena_gib)]
        if a.device:
            cmd += ["--device", a.device]
        if a.dflash2_model_dir:
            cmd += ["--dflash2-model-dir", a.dflash2_model_dir, "--dflash2-drafts", str(a.dflash2_drafts),
                    "--dflash2-stats", str(a.dflash2_stats)]
        out = subprocess.run(cmd, capture_output=True, text=True)
        if out.returncode != 0:
            raise RuntimeError(out.stderr[-2000:])
        line = [l for l in out.stdout.splitlines() if l.startswith("GENERATED_IDS=")][0]
        gen = [int(t) for t in line.split("=", 1)[1].split(",") if t]
        reply = tok.decode(gen, skip_special_tokens=True)
        history.append({"role": "assistant", "content": reply})
        return reply

    if a.prompt:
        print(turn(a.prompt))
        return 0
    try:
        while True:
            line = input("> ")
            if line.strip() in ("/exit", "/quit"):
                break
            print(turn(line))
    except EOFError:
        pass
    return 0


if __name__ == "__main__":
    sys.exit(main())
