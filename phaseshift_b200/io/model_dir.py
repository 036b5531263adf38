"""Model directories: HF-style BF16 checkpoints and the self-contained quantised format.

A directory holds ``config.json`` (+ optional ``generation_config.json`` / tokenizer assets), one or
more ``model*.safetensors`` shards (+ ``model.safetensors.index.json`` when sharded) and, for quantised
models, the manifest ``phaseshift_quantization.json`` (quant/manifest.py).  Reading goes through the
C++ mmap reader (zero-copy views into the mapping); writing through the C++ streaming writer.
Reference: SafetensorsCollection / weight loader (include/phaseshift/weights/weight_loader.h:20-93).
"""
from __future__ import annotations

import json
import os
from pathlib import Path
from typing import Callable, Dict, Iterable, List, Optional

import numpy as np
import torch

from ..core.native import runtime

_ST2TORCH = {"F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16, "U8": torch.uint8, "I8": torch.int8,
             "I32": torch.int32, "I64": torch.int64, "F64": torch.float64, "F8_E4M3": torch.float8_e4m3fn, "BOOL": torch.bool}
_TORCH2ST = {v: k for k, v in _ST2TORCH.items()}


def parse_size(s) -> int:
    """'4GiB', '512MiB', '1000000' -> bytes."""
    if isinstance(s, int):
        return s
    s = s.strip()
    for suf, mul in (("GiB", 1 << 30), ("MiB", 1 << 20), ("KiB", 1 << 10), ("GB", 10 ** 9), ("MB", 10 ** 6)):
        if s.endswith(suf):
            return int(float(s[:-len(suf)]) * mul)
    return int(s)


class ShardCollection:
    """All tensors of a model directory, resolved across shards through the index file when present."""

    def __init__(self, model_dir):
        self.dir = Path(model_dir)
        rt = runtime()
        idx = self.dir / "model.safetensors.index.json"
        files: List[str]
        if idx.exists():
            wm = json.loads(idx.read_text())["weight_map"]
            files = sorted(set(wm.values()))
        else:
            files = sorted(p.name for p in self.dir.glob("*.safetensors"))
        if not files:
            raise FileNotFoundError(f"no .safetensors files in {self.dir}")
        self.readers = {f: rt.SafetensorsReader(str(self.dir / f)) for f in files}
        self.where: Dict[str, str] = {}
        for f, r in self.readers.items():
            for n in r.names():
                self.where[n] = f

    def names(self) -> List[str]:
        return list(self.where)

    def has(self, name: str) -> bool:
        return name in self.where

    def spec(self, name: str):
        return self.readers[self.where[name]].spec(name)

    def tensor(self, name: str) -> torch.Tensor:
        """Zero-copy CPU tensor backed by the file mapping (read-only: clone before writing)."""
        r = self.readers[self.where[name]]
        dtype, shape, nbytes = r.spec(name)
        if nbytes == 0:
            return torch.empty(shape, dtype=_ST2TORCH[dtype])
        buf = r.data(name)                      # numpy uint8 view whose base keeps the mapping alive
        buf.flags.writeable = False
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            t = torch.from_numpy(buf)
        return t.view(_ST2TORCH[dtype]).reshape(shape)

    def crc32(self, name: str) -> int:
        return self.readers[self.where[name]].crc32(name)

    def close(self) -> None:
        for r in self.readers.values():
            r.close()


class ShardWriter:
    """Streams tensors into ``model-0000k-of-0000n.safetensors`` shards bounded by ``max_shard_size`` and
    writes the index.  Tensors are planned first (sizes known), then written in plan order."""

    def __init__(self, out_dir, max_shard_size: int = 4 << 30, metadata: Optional[Dict[str, str]] = None):
        self.dir = Path(out_dir)
        self.dir.mkdir(parents=True, exist_ok=True)
        self.max = max_shard_size
        self.meta = metadata or {"format": "pt"}
        self.plan: List[tuple] = []      # (name, dtype, shape, nbytes)

    def add(self, name: str, dtype: torch.dtype, shape: Iterable[int]) -> None:
        shape = [int(s) for s in shape]
        n = int(np.prod(shape)) if shape else 1
        self.plan.append((name, _TORCH2ST[dtype], shape, n * torch.empty((), dtype=dtype).element_size()))

    def begin(self) -> None:
        shards, cur, size = [], [], 0
        for item in self.plan:
            if cur and size + item[3] > self.max:
                shards.append(cur)
                cur, size = [], 0
            cur.append(item)
            size += item[3]
        if cur:
            shards.append(cur)
        rt = runtime()
        self.writers, self.where, self.files = [], {}, []
        n = len(shards)
        for i, sh in enumerate(shards):
            fname = "model.safetensors" if n == 1 else f"model-{i + 1:05d}-of-{n:05d}.safetensors"
            w = rt.SafetensorsWriter(str(self.dir / fname))
            for k, v in self.meta.items():
                w.set_metadata(k, v)
            for (name, dt, shape, _) in sh:
                w.plan_tensor(name, dt, shape)
                self.where[name] = (w, fname)
            w.write_header()
            self.writers.append(w)
            self.files.append(fname)

    def write(self, name: str, t: torch.Tensor) -> int:
        """Write a whole tensor (or the next row chunk of it); returns the running CRC32 of the tensor."""
        w, _ = self.where[name]
        t = t.detach().contiguous().cpu()
        w.write_chunk_ptr(name, t.data_ptr(), t.numel() * t.element_size())
        return w.tensor_crc(name)

    def finish(self) -> None:
        for w in self.writers:
            w.finish()
        if len(self.files) > 1:
            total = sum(p[3] for p in self.plan)
            idx = {"metadata": {"total_size": total}, "weight_map": {n: f for n, (_, f) in self.where.items()}}
            (self.dir / "model.safetensors.index.json").write_text(json.dumps(idx, indent=1))


def save_hf_model(model_dir, cfg, tensors: Dict[str, torch.Tensor], max_shard_size: int = 4 << 30) -> None:
    cfg.save(model_dir)
    if cfg.eos_token_ids:
        (Path(model_dir) / "generation_config.json").write_text(json.dumps({"eos_token_id": cfg.eos_token_ids}))
    w = ShardWriter(model_dir, max_shard_size)
    for n, t in tensors.items():
        w.add(n, t.dtype, t.shape)
    w.begin()
    for n, t in tensors.items():
        w.write(n, t)
    w.finish()


def is_quantized_dir(model_dir) -> bool:
    return (Path(model_dir) / "phaseshift_quantization.json").exists()
