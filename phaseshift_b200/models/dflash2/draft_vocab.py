"""Fixed draft-vocabulary profile: the drafter scores only a subset of the target vocabulary.

Behaviour follows the reference (src/phaseshift/models/qwen35/dflash2/draft_vocab_profile.cpp:134-269,
docs/developer/dflash2.md "fixed vocabulary profile"): a profile lives beside the target model as
``dflash2-draft-vocab.json`` (metadata) + ``dflash2-draft-vocab.u32`` (little-endian uint32 token ids, ascending,
unique, count a multiple of 16, every id inside the target vocabulary, at least as many ids as the selector's
candidate pool).  It is OFF unless asked for: ``PS_DFLASH2_DRAFT_VOCAB=1`` enables the profile found in the model
directory (silently ignored when absent, refused loudly when present but damaged or not matching the model),
``PS_DFLASH2_DRAFT_VOCAB_FILE`` names a raw id file explicitly.  Proposals made under a profile are still verified
by the full target, so a profile can only change acceptance, never the emitted tokens.  Constrained requests do not
use it (a grammar may need tokens outside the subset).

The drafter's head pass then streams ``vocab_count`` rows of the target's lm_head instead of all of them
(``DFlash2NativeDrafter.set_draft_vocab``); top-k runs on local ids and is mapped back to global ids before the
candidate selector, which works on global ids (the reference maps back right after its top-N, executor.hip:210).
"""
from __future__ import annotations

import hashlib
import json
import os
from dataclasses import dataclass
from pathlib import Path
from typing import Optional, Sequence

import numpy as np

SCHEMA = "phaseshift-dflash2-vocab-v1"
META_NAME, PAYLOAD_NAME = "dflash2-draft-vocab.json", "dflash2-draft-vocab.u32"


class DraftVocabError(ValueError):
    pass


@dataclass
class DraftVocab:
    ids: np.ndarray            # uint32, ascending, unique
    profile_id: str = ""
    source: str = ""

    @property
    def count(self) -> int:
        return int(self.ids.shape[0])


def _sha256_file(p: Path) -> str:
    h = hashlib.sha256()
    with open(p, "rb") as f:
        for blk in iter(lambda: f.read(1 << 20), b""):
            h.update(blk)
    return h.hexdigest()


def validate_ids(ids: np.ndarray, target_vocab_size: int, min_count: int = 16) -> np.ndarray:
    ids = np.asarray(ids)
    if ids.ndim != 1 or ids.size == 0:
        raise DraftVocabError("draft vocabulary must be a non-empty id list")
    ids = ids.astype(np.uint32)
    if ids.size % 16:
        raise DraftVocabError("draft vocabulary count must be a multiple of 16")
    if ids.size < min_count:
        raise DraftVocabError(f"draft vocabulary has {ids.size} ids, fewer than the candidate pool ({min_count})")
    if not np.all(ids[1:] > ids[:-1]):
        raise DraftVocabError("draft vocabulary ids must be strictly ascending (sorted, no duplicates)")
    if int(ids[-1]) >= target_vocab_size:
        raise DraftVocabError("draft vocabulary contains ids outside the target vocabulary")
    return ids


def pack(ids: Sequence[int], out_dir, profile_id: str, target_vocab_size: int, target_hidden_size: int,
         tokenizer_path: Optional[str] = None, min_count: int = 16) -> Path:
    """Write a profile directory (payload + metadata).  ``ids`` need not be sorted; duplicates are an error."""
    arr = np.asarray(sorted(int(i) for i in ids), dtype=np.uint32)
    arr = validate_ids(arr, target_vocab_size, min_count)
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    arr.astype("<u4").tofile(out / PAYLOAD_NAME)
    meta = {"schema_version": SCHEMA, "profile_id": profile_id, "vocab_file": PAYLOAD_NAME, "vocab_count": int(arr.size),
            "target_vocab_size": int(target_vocab_size), "target_hidden_size": int(target_hidden_size),
            "vocab_sha256": _sha256_file(out / PAYLOAD_NAME),
            "tokenizer_sha256": _sha256_file(Path(tokenizer_path)) if tokenizer_path else ""}
    (out / META_NAME).write_text(json.dumps(meta, indent=1))
    return out


def load_profile(model_dir, target_vocab_size: int, target_hidden_size: int, min_count: int = 16) -> Optional[DraftVocab]:
    """The standard profile of a model directory: None when there is none; DraftVocabError when one is present but
    unknown, damaged, partial or made for another model (never used silently)."""
    d = Path(model_dir)
    mp, pp = d / META_NAME, d / PAYLOAD_NAME
    if not mp.exists() and not pp.exists():
        return None
    if not mp.exists() or not pp.exists():
        raise DraftVocabError("draft vocabulary profile is only partly installed")
    try:
        meta = json.loads(mp.read_text())
    except Exception as e:
        raise DraftVocabError(f"draft vocabulary metadata is not valid JSON: {e}")
    if meta.get("schema_version") != SCHEMA:
        raise DraftVocabError(f"unknown draft vocabulary schema {meta.get('schema_version')!r}")
    if meta.get("vocab_file") != PAYLOAD_NAME:
        raise DraftVocabError("draft vocabulary metadata names another payload file")
    if int(meta.get("target_vocab_size", -1)) != target_vocab_size or int(meta.get("target_hidden_size", -1)) != target_hidden_size:
        raise DraftVocabError("draft vocabulary profile was made for another model shape")
    if _sha256_file(pp) != meta.get("vocab_sha256"):
        raise DraftVocabError("draft vocabulary payload does not match its recorded hash")
    tok = d / "tokenizer.json"
    if meta.get("tokenizer_sha256") and tok.exists() and _sha256_file(tok) != meta["tokenizer_sha256"]:
        raise DraftVocabError("draft vocabulary profile was made for another tokenizer")
    raw = np.fromfile(pp, dtype="<u4")
    if raw.size != int(meta.get("vocab_count", -1)):
        raise DraftVocabError("draft vocabulary payload length differs from the metadata")
    return DraftVocab(validate_ids(raw, target_vocab_size, min_count), meta.get("profile_id", ""), str(pp))


def resolve(model_dir, target_vocab_size: int, target_hidden_size: int, min_count: int = 16, env=None) -> Optional[DraftVocab]:
    """What the environment asks for: the explicit file, the standard profile (only with PS_DFLASH2_DRAFT_VOCAB=1), or
    nothing.  An explicit file together with PS_DFLASH2_DRAFT_VOCAB=0 is a contradiction and is refused."""
    env = os.environ if env is None else env
    flag = (env.get("PS_DFLASH2_DRAFT_VOCAB") or "").strip()
    explicit = (env.get("PS_DFLASH2_DRAFT_VOCAB_FILE") or "").strip()
    if explicit:
        if flag == "0":
            raise DraftVocabError("PS_DFLASH2_DRAFT_VOCAB_FILE conflicts with PS_DFLASH2_DRAFT_VOCAB=0")
        raw = np.fromfile(explicit, dtype="<u4")
        return DraftVocab(validate_ids(raw, target_vocab_size, min_count), "explicit", explicit)
    if flag in ("", "0") or model_dir is None:
        return None
    return load_profile(model_dir, target_vocab_size, target_hidden_size, min_count)


def select_by_frequency(tokens: Sequence[int], count: int, target_vocab_size: int, always: Sequence[int] = ()) -> np.ndarray:
    """The ``count`` most frequent token ids of a corpus (ties to the lower id), plus the ids in ``always`` (stop /
    mask tokens); ``count`` is rounded up to a multiple of 16.  This is the aggregation recipe; `pack` only wraps."""
    count = -(-count // 16) * 16
    if count > target_vocab_size:
        raise DraftVocabError("asked for more ids than the vocabulary has")
    freq = np.bincount(np.asarray(tokens, dtype=np.int64), minlength=target_vocab_size)[:target_vocab_size]
    order = np.lexsort((np.arange(target_vocab_size), -freq))
    chosen = set(int(i) for i in always)
    for i in order:
        if len(chosen) >= count:
            break
        chosen.add(int(i))
    return np.asarray(sorted(chosen), dtype=np.uint32)
