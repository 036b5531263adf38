"""phaseshift-tools: corpus, draft-vocabulary and oracle helpers around the engine.

Counterparts of the reference's tools/ scripts (tools/gen_token_corpus.py, tools/quantization/prepare_draft_vocab.py,
tools/quantization/prepare_kld_corpus.py, tools/qwen35_oracle_tokens.py):

  token-corpus        text -> token id file (little-endian int32 ``.bin``; what `phaseshift-quantizer kld / imatrix / ppl
                      --tokens` read), with the model's tokenizer or the built-in byte tokenizer; can extend a base corpus
  draft-vocab select  the N most frequent ids of a corpus -> raw ``.u32`` id list (the aggregation recipe)
  draft-vocab pack    raw id list -> profile directory (payload + metadata with hashes) to drop beside a target model
  draft-vocab check   validate the profile of a model directory against the model's shape
  oracle-tokens       greedy continuation (and optionally the logits) of a prompt from the fp32 whole-sequence oracle,
                      for comparison with what an engine build emits
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path
from typing import List, Optional

import numpy as np


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="phaseshift-tools")
    sub = ap.add_subparsers(dest="cmd", required=True)
    tc = sub.add_parser("token-corpus")
    tc.add_argument("--model-dir"); tc.add_argument("--byte-tokenizer", type=int, default=0, help="vocab size of the built-in byte tokenizer")
    tc.add_argument("--text", action="append", default=[]); tc.add_argument("--text-file", action="append", default=[])
    tc.add_argument("--base"); tc.add_argument("--output", required=True)
    dv = sub.add_parser("draft-vocab")
    dsub = dv.add_subparsers(dest="dv_cmd", required=True)
    s = dsub.add_parser("select")
    s.add_argument("--tokens", required=True); s.add_argument("--count", type=int, required=True)
    s.add_argument("--model-vocab-size", type=int, required=True); s.add_argument("--always", default="")
    s.add_argument("--output", required=True)
    p = dsub.add_parser("pack")
    p.add_argument("--vocab-file", required=True); p.add_argument("--profile-id", required=True)
    p.add_argument("--model-vocab-size", type=int, required=True); p.add_argument("--hidden-size", type=int, required=True)
    p.add_argument("--tokenizer"); p.add_argument("--output-dir", required=True); p.add_argument("--min-count", type=int, default=16)
    c = dsub.add_parser("check")
    c.add_argument("--model-dir", required=True)
    o = sub.add_parser("oracle-tokens")
    o.add_argument("--model-dir", required=True); o.add_argument("--input-ids-file", required=True)
    o.add_argument("--max-new-tokens", type=int, default=16); o.add_argument("--dump-logits")
    return ap


def _tokenizer(a):
    if a.model_dir and (Path(a.model_dir) / "tokenizer.json").exists():
        from transformers import AutoTokenizer
        return AutoTokenizer.from_pretrained(a.model_dir)
    from ..serving.chat import ByteTokenizer
    return ByteTokenizer(a.byte_tokenizer or 512)


def cmd_token_corpus(a) -> int:
    from ..quant.offline import read_tokens
    tok = _tokenizer(a)
    ids: List[int] = list(read_tokens(a.base)) if a.base else []
    texts = list(a.text) + [Path(f).read_text(encoding="utf-8") for f in a.text_file]
    if not texts and not ids:
        print("phaseshift-tools: nothing to tokenise", file=sys.stderr)
        return 2
    for t in texts:
        enc = tok.encode(t)
        ids.extend(int(i) for i in (enc if isinstance(enc, list) else enc["input_ids"]))
    np.asarray(ids, dtype="<i4").tofile(a.output)
    print(f"TOKENS={len(ids)}"); print(f"OUTPUT={a.output}")
    return 0


def cmd_draft_vocab(a) -> int:
    from ..models.dflash2 import draft_vocab as dv
    if a.dv_cmd == "select":
        from ..quant.offline import read_tokens
        always = [int(t) for t in a.always.replace(",", " ").split()]
        ids = dv.select_by_frequency(read_tokens(a.tokens), a.count, a.model_vocab_size, always)
        ids.astype("<u4").tofile(a.output)
        print(f"VOCAB_COUNT={ids.size}"); print(f"OUTPUT={a.output}")
        return 0
    if a.dv_cmd == "pack":
        ids = np.fromfile(a.vocab_file, dtype="<u4")
        try:
            out = dv.pack(ids, a.output_dir, a.profile_id, a.model_vocab_size, a.hidden_size, a.tokenizer, a.min_count)
        except dv.DraftVocabError as e:
            print(f"phaseshift-tools: {e}", file=sys.stderr)
            return 2
        meta = json.loads((out / dv.META_NAME).read_text())
        print(f"PROFILE_ID={meta['profile_id']}"); print(f"VOCAB_COUNT={meta['vocab_count']}"); print(f"VOCAB_SHA256={meta['vocab_sha256']}")
        return 0
    from ..models.qwen35.config import Qwen35Config
    cfg = Qwen35Config.from_dir(a.model_dir)
    try:
        prof = dv.load_profile(a.model_dir, cfg.vocab_size, cfg.hidden_size)
    except dv.DraftVocabError as e:
        print(f"DRAFT_VOCAB=invalid"); print(f"REASON={e}")
        return 1
    if prof is None:
        print("DRAFT_VOCAB=absent")
        return 0
    print("DRAFT_VOCAB=ok"); print(f"PROFILE_ID={prof.profile_id}"); print(f"VOCAB_COUNT={prof.count}")
    return 0


def cmd_oracle_tokens(a) -> int:
    import torch
    from ..io.model_dir import ShardCollection
    from ..models.qwen35.config import Qwen35Config
    from ..models.qwen35.reference import reference_forward
    from ..models.qwen35.weights import hf_tensor_shapes
    cfg = Qwen35Config.from_dir(a.model_dir)
    col = ShardCollection(a.model_dir)
    hf = {n: col.tensor(n).float() for n in hf_tensor_shapes(cfg) if col.has(n)}
    ids = [int(t) for t in Path(a.input_ids_file).read_text().replace(",", " ").split()]
    gen, rows = [], []
    for _ in range(a.max_new_tokens):
        lg = reference_forward(cfg, hf, ids + gen)[-1]
        rows.append(lg.numpy())
        gen.append(int(torch.argmax(lg)))
    if a.dump_logits:
        np.stack(rows).astype("<f4").tofile(a.dump_logits)
        print(f"LOGITS_VOCAB={cfg.vocab_size}"); print(f"LOGITS_TOTAL_ROWS={len(rows)}")
    print(f"PROMPT_TOKENS={len(ids)}"); print("GENERATED_IDS=" + ",".join(map(str, gen)))
    return 0


def main(argv: Optional[List[str]] = None) -> int:
    a = build_parser().parse_args(argv)
    return {"token-corpus": cmd_token_corpus, "draft-vocab": cmd_draft_vocab, "oracle-tokens": cmd_oracle_tokens}[a.cmd](a)


if __name__ == "__main__":
    sys.exit(main())
