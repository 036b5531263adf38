"""phaseshift-quantizer {quantize, verify, kld, imatrix, ppl} (reference: src/apps/quantizer/main.cpp:35-39,
docs/user/quantizer.md:5-96)."""
from __future__ import annotations

import argparse
import json
import sys
from typing import List, Optional


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="phaseshift-quantizer")
    sub = ap.add_subparsers(dest="cmd", required=True)
    q = sub.add_parser("quantize", help="BF16 model directory -> self-contained quantised directory")
    q.add_argument("--input", required=True); q.add_argument("--output", required=True)
    q.add_argument("--preset", default="nvfp4", choices=["nvfp4", "mxfp8", "bf16", "mxfp4"])
    q.add_argument("--backend", default="cpu", choices=["cpu", "cuda"])
    q.add_argument("--scope", default="text-only", choices=["text-only"])
    q.add_argument("--imatrix"); q.add_argument("--imatrix-policy", default="strict", choices=["strict", "best-effort"])
    q.add_argument("--max-shard-size", default="4GiB"); q.add_argument("--overwrite", action="store_true")
    q.add_argument("--no-verify", action="store_true"); q.add_argument("--search", type=int, default=2)
    v = sub.add_parser("verify", help="check manifest, shapes and CRCs of a quantised directory")
    v.add_argument("dir")
    k = sub.add_parser("kld", help="KL divergence of a quantised bundle against its BF16 source")
    k.add_argument("--input", required=True); k.add_argument("--bundle", required=True); k.add_argument("--tokens", required=True)
    k.add_argument("--report"); k.add_argument("--window", type=int, default=512); k.add_argument("--stride", type=int, default=512)
    k.add_argument("--max-eval-tokens", type=int, default=0); k.add_argument("--self", dest="self_check", action="store_true")
    k.add_argument("--device", default=None)
    k.add_argument("--baseline-cache", "--cache-dir", dest="baseline_cache", default=None,
                   help="directory that keeps the baseline model's logits between runs")
    k.add_argument("--keep-logit-cache", action="store_true", help="accepted for compatibility: the logits cached in --cache-dir are always kept")
    k.add_argument("--keep-shadow", action="store_true", help="accepted for compatibility: the bundle is evaluated directly, no shadow model is written")
    k.add_argument("--batch-positions", type=int, default=512, help="rows per evaluation step")
    k.add_argument("--arena-gib", type=float, default=0, help="accepted for compatibility: the evaluation engines size their own pools")
    i = sub.add_parser("imatrix", help="collect per-channel activation importance")
    i.add_argument("--input", help="unused alias of --model-dir"); i.add_argument("--model-dir", required=True)
    i.add_argument("--tokens", required=True); i.add_argument("--output", required=True)
    i.add_argument("--window", type=int, default=512); i.add_argument("--stride", type=int, default=512)
    i.add_argument("--max-calibration-tokens", type=int, default=0); i.add_argument("--device", default=None)
    i.add_argument("--flush-windows", type=int, default=16, help="rewrite the output file every N windows (0: only at the end)")
    i.add_argument("--arena-gib", type=float, default=0, help="accepted for compatibility")
    p = sub.add_parser("ppl", help="teacher-forced perplexity")
    p.add_argument("--model-dir", required=True); p.add_argument("--tokens", required=True)
    p.add_argument("--max-tokens", type=int, default=2048); p.add_argument("--device", default=None)
    return ap


def _device(d):
    import torch
    return d or ("cuda:0" if torch.cuda.is_available() else "cpu")


def main(argv: Optional[List[str]] = None) -> int:
    a = build_parser().parse_args(argv)
    from ..io.model_dir import parse_size
    from ..quant import offline
    try:
        if a.cmd == "quantize":
            man = offline.quantize_model(a.input, a.output, a.preset, a.backend, a.imatrix, a.imatrix_policy,
                                         parse_size(a.max_shard_size), a.overwrite, not a.no_verify, a.search)
            print(f"QUANTIZED_TENSORS={len(man.tensors)}")
            print(f"OUTPUT={a.output}")
        elif a.cmd == "verify":
            problems = offline.validate_model_dir(a.dir)
            for p in problems:
                print("PROBLEM=" + p)
            print("VERIFY=" + ("ok" if not problems else "failed"))
            return 0 if not problems else 1
        elif a.cmd == "kld":
            rep = offline.evaluate_kld(a.input, a.bundle, offline.read_tokens(a.tokens), a.window, a.stride,
                                       a.max_eval_tokens, _device(a.device), a.self_check, a.baseline_cache, a.batch_positions)
            if a.report:
                open(a.report, "w").write(json.dumps(rep, indent=1))
            for k in ("positions", "mean", "p50", "p90", "p99", "p99_9", "max", "top1_agreement"):
                print(f"KLD_{k.upper()}={rep[k]}")
            if a.baseline_cache:
                print(f"KLD_BASELINE_CACHE_HITS={rep['baseline_cache_hits']}"); print(f"KLD_BASELINE_CACHE_MISSES={rep['baseline_cache_misses']}")
        elif a.cmd == "imatrix":
            rep = offline.collect_imatrix(a.model_dir, offline.read_tokens(a.tokens), a.output, a.window, a.stride,
                                          a.max_calibration_tokens, _device(a.device), a.flush_windows)
            print(f"IMATRIX_SITES={rep['sites']}"); print(f"IMATRIX_WINDOWS={rep['windows']}"); print(f"IMATRIX_FLUSHES={rep['flushes']}")
        elif a.cmd == "ppl":
            rep = offline.evaluate_ppl(a.model_dir, offline.read_tokens(a.tokens), a.max_tokens, _device(a.device))
            print(f"PPL_TOKENS={rep['tokens']}"); print(f"NLL={rep['nll']}"); print(f"PPL={rep['ppl']}")
    except (ValueError, FileExistsError, FileNotFoundError) as e:
        print(f"phaseshift-quantizer: {e}", file=sys.stderr)
        return 2
    return 0


if __name__ == "__main__":
    sys.exit(main())
