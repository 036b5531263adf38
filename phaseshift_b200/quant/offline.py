"""Offline quantiser core: quantize / verify / kld / imatrix / ppl.

Counterpart of the reference's ``phaseshift_quantizer_core`` (src/phaseshift/quantization/offline/
quantizer.cpp:98-989, kld.cpp, imatrix_collect.cpp, ppl.cpp).  ``quantize_model`` streams one HF tensor
at a time: classify the name into a role, pick the encoding from the preset, quantise rows on the CPU
reference quantiser (C++) or on the GPU, write structure-of-arrays tensors into size-bounded shards,
record per-tensor CRC32 in the manifest, copy tokenizer / config assets and (unless disabled) verify the
result.  ``evaluate_kld`` runs the BF16 model and the quantised bundle teacher-forced over token windows
and reports the distribution of KL(p_bf16 || p_quant); ``collect_imatrix`` accumulates per-input-channel
activation energy at every projection input; ``evaluate_ppl`` reports teacher-forced perplexity.
"""
from __future__ import annotations

import os

import hashlib
import json
import shutil
from pathlib import Path
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..core.native import runtime
from ..io.model_dir import ShardCollection, ShardWriter, is_quantized_dir
from ..models.qwen35.config import Qwen35Config
from ..models.qwen35.weights import format_for, scale_groups
from . import formats
from .manifest import CODES, META1, Manifest, TensorEntry, classify_qwen35, layer_of

ASSETS = ("config.json", "generation_config.json", "tokenizer.json", "tokenizer_config.json", "vocab.json",
          "merges.txt", "special_tokens_map.json", "chat_template.jinja", "added_tokens.json")


def model_fingerprint(model_dir) -> str:
    """sha256 over config.json and, per tensor, its name, dtype, shape, byte count and the CRC32 of its first and last
    64 KiB (cheap: a 27B directory costs a few hundred MB of reads; two checkpoints of one architecture still differ)."""
    from ..core.native import runtime
    rt = runtime()
    h = hashlib.sha256()
    h.update((Path(model_dir) / "config.json").read_bytes())
    col = ShardCollection(model_dir)
    edge = 64 * 1024
    for n in sorted(col.names()):
        dt, shape, nbytes = col.spec(n)
        h.update(f"{n}:{dt}:{shape}:{nbytes}".encode())
        if nbytes:
            buf = col.readers[col.where[n]].data(n)                  # uint8 view of the file mapping
            head = rt.crc32_ptr(buf.ctypes.data, min(edge, nbytes), 0)
            tail = rt.crc32_ptr(buf.ctypes.data + max(0, nbytes - edge), min(edge, nbytes), 0)
            h.update(f":{head}:{tail}".encode())
    col.close()
    return h.hexdigest()


def read_tokens(path) -> List[int]:
    p = Path(path)
    if p.suffix == ".npy":
        return np.load(p).astype(np.int64).reshape(-1).tolist()
    if p.suffix == ".bin":
        return np.fromfile(p, dtype=np.int32).astype(np.int64).tolist()
    return [int(t) for t in p.read_text().replace(",", " ").split()]


# ------------------------------------------------------------------------------------------------ imatrix file
def save_imatrix(path, sums: Dict[str, torch.Tensor], counts: Dict[str, int], meta: Optional[dict] = None) -> None:
    from safetensors.torch import save_file
    md = {"format": "phaseshift-imatrix", "counts": json.dumps(counts)}
    md.update({k: str(v) for k, v in (meta or {}).items()})
    save_file({k: v.float().contiguous().cpu() for k, v in sums.items()}, str(path), metadata=md)


def load_imatrix(path):
    rt = runtime()
    r = rt.SafetensorsReader(str(path))
    md = r.metadata()
    if md.get("format") != "phaseshift-imatrix":
        raise ValueError("not an imatrix file")
    counts = json.loads(md["counts"])
    out = {}
    for n in r.names():
        out[n] = torch.from_numpy(np.array(r.data(n)).view(np.float32).copy()) / max(1, counts.get(n, 1))
    return out


# ------------------------------------------------------------------------------------------------ quantize
def imatrix_key(name: str) -> str:
    """Projections that read the same activations share one importance vector (collected under the first)."""
    for a, b in (("k_proj", "q_proj"), ("v_proj", "q_proj"), ("up_proj", "gate_proj"), ("in_proj_z", "in_proj_qkv")):
        name = name.replace(a + ".weight", b + ".weight")
    return name


def is_drafter_dir(model_dir) -> bool:
    """True for a DFlash2 drafter directory (config.json names the DFlash2DraftModel architecture)."""
    try:
        raw = json.loads((Path(model_dir) / "config.json").read_text())
    except Exception:
        return False
    return (raw.get("architectures") or [""])[0] == "DFlash2DraftModel"


def classify_drafter(name: str) -> str:
    """Role of a DFlash2 drafter tensor.  The backbone projections (q/k/v/o, gate/up/down and the tap
    projection ``fc``) are the drafter's weight traffic and follow the preset's 4-bit role (reference:
    src/phaseshift/quantization/fpx/profile.cpp:96-128, "DFlash backbone linears"); norms, the dynamic-conv
    kernels and the selector tables stay BF16."""
    if name == "fc.weight" or (name.startswith("layers.") and name.endswith("_proj.weight")):
        return "dflash_backbone"
    return "other"


def _quantize_tensor(w: torch.Tensor, fmt: str, backend: str, tensor_scale: Optional[float], importance, search: int):
    if fmt == "bf16":
        return formats.quantize(w, "bf16")
    if fmt == "mxfp4":
        return formats.quantize_mxfp4(w.to("cuda") if backend == "cuda" else w).to("cpu")
    if fmt not in ("nvfp4", "mxfp8"):
        raise ValueError(f"the quantizer cannot write {fmt!r} bundles")
    if backend == "cuda":
        wd = w.to("cuda").float()
        imp = None if importance is None else importance.to("cuda")
        q = formats.quantize_nvfp4(wd, imp, search, tensor_scale) if fmt == "nvfp4" else formats.quantize_mxfp8(wd, imp, min(search, 1))
        return q.to("cpu")
    rt = runtime()
    wf = w.float().contiguous()
    n, k = wf.shape
    kp = formats.align_up(k, formats.K_ALIGN)
    imp_ptr = 0
    if importance is not None:
        importance = importance.float().contiguous()
        imp_ptr = importance.data_ptr()
    if fmt == "nvfp4":
        ts = tensor_scale if tensor_scale is not None else (float(wf.abs().max()) / (6.0 * 448.0) or 1.0)
        codes = torch.zeros(n, kp // 2, dtype=torch.uint8)
        scales = torch.zeros(n, kp // 16, dtype=torch.uint8)
        rt.quantize_rows_nvfp4(wf.data_ptr(), n, k, kp, ts, search, imp_ptr, codes.data_ptr(), scales.data_ptr())
        return formats.QuantizedTensor("nvfp4", (n, k), kp, codes, scales, ts)
    codes = torch.zeros(n, kp, dtype=torch.uint8)
    scales = torch.zeros(n, kp // 32, dtype=torch.uint8)
    rt.quantize_rows_mxfp8(wf.data_ptr(), n, k, kp, min(search, 1), imp_ptr, codes.data_ptr(), scales.data_ptr())
    return formats.QuantizedTensor("mxfp8", (n, k), kp, codes, scales, 1.0)


def quantize_model(input_dir, output_dir, preset: str = "nvfp4", backend: str = "cpu", imatrix: Optional[str] = None,
                   imatrix_policy: str = "strict", max_shard_size: int = 4 << 30, overwrite: bool = False,
                   verify: bool = True, search: int = 2, log=print) -> Manifest:
    inp, out = Path(input_dir), Path(output_dir)
    if is_quantized_dir(inp):
        raise ValueError("input is already a quantised directory")
    if out.exists() and any(out.iterdir()):
        if not overwrite:
            raise FileExistsError(f"{out} is not empty (use --overwrite)")
        shutil.rmtree(out)
    out.mkdir(parents=True, exist_ok=True)
    if backend == "cuda" and not torch.cuda.is_available():
        raise RuntimeError("--backend cuda requested but no CUDA device is available")
    drafter = is_drafter_dir(inp)
    col = ShardCollection(inp)
    imat = load_imatrix(imatrix) if imatrix else None
    group_of = {}
    if drafter:
        # DFlash2 adapter: same bundle format, drafter tensor names and roles
        from ..models.dflash2.model import DFlash2Config, tensor_shapes
        cfg = DFlash2Config.from_dir(inp)
        names = [n for n in tensor_shapes(cfg) if col.has(n)]
        classify = classify_drafter
    else:
        cfg = Qwen35Config.from_dir(inp)
        names = [n for n in col.names() if n.startswith("model.language_model.") or n.startswith("lm_head")]
        classify = classify_qwen35
        for g in scale_groups(cfg):
            for n in g:
                group_of[n] = g
    man = Manifest(preset=preset, source_fingerprint=model_fingerprint(inp),
                   imatrix={"file": str(imatrix), "policy": imatrix_policy} if imatrix else None)
    plan = []
    for n in names:
        dt, shape, _ = col.spec(n)
        role = classify(n)
        is_matrix = len(shape) == 2 and role not in ("norm", "other")
        fmt = format_for(preset, role, layer_of(n)) if is_matrix else "bf16"
        if imat is not None and is_matrix and fmt != "bf16" and imatrix_key(n) not in imat and role not in ("embed",):
            if imatrix_policy == "strict":
                raise ValueError(f"imatrix has no entry for {n} (policy strict)")
        plan.append((n, role, fmt, shape))
    writer = ShardWriter(out, max_shard_size)
    for (n, role, fmt, shape) in plan:
        if fmt == "bf16":
            writer.add(n, torch.bfloat16 if len(shape) else torch.bfloat16, shape)
        else:
            kp = formats.align_up(shape[1], formats.K_ALIGN)
            writer.add(n + CODES, torch.uint8, [shape[0], kp // 2 if fmt in ("nvfp4", "mxfp4") else kp])
            writer.add(n + META1, torch.uint8, [shape[0], kp // (16 if fmt == "nvfp4" else 32)])
    writer.begin()
    tscale_cache: Dict[str, float] = {}
    for (n, role, fmt, shape) in plan:
        w = col.tensor(n)
        if fmt == "bf16":
            crc = writer.write(n, w.to(torch.bfloat16))
            man.tensors.append(TensorEntry(n, role, "bf16", "row_major_k_contiguous", list(shape),
                                           shape[-1] if shape else 1, data=n, crc32={n: crc}))
            continue
        ts = None
        if fmt == "nvfp4":
            grp = group_of.get(n, [n])
            key = grp[0]
            if key not in tscale_cache:
                amax = max(float(col.tensor(m).float().abs().max()) for m in grp)
                tscale_cache[key] = amax / (6.0 * 448.0) if amax > 0 else 1.0
            ts = tscale_cache[key]
        q = _quantize_tensor(w, fmt, backend, ts, None if imat is None else imat.get(imatrix_key(n)), search)
        c1 = writer.write(n + CODES, q.codes)
        c2 = writer.write(n + META1, q.scales)
        man.tensors.append(TensorEntry(n, role, fmt, "row_major_k_contiguous", list(shape), q.k_padded,
                                       codes=n + CODES, metadata1=n + META1,
                                       metadata2=q.tensor_scale if fmt == "nvfp4" else None,
                                       crc32={n + CODES: c1, n + META1: c2}))
        log(f"quantized {n} {tuple(shape)} -> {fmt}")
    writer.finish()
    if not drafter and cfg.tie_word_embeddings:
        man.aliases["model.language_model.lm_head.weight"] = "model.language_model.embed_tokens.weight"
    man.save(out)
    for a in ASSETS:
        if (inp / a).exists():
            shutil.copy2(inp / a, out / a)
    col.close()
    if verify:
        problems = validate_model_dir(out)
        if problems:
            raise RuntimeError("self-verification failed: " + "; ".join(problems[:5]))
    return man


def verify_crc(col: ShardCollection, man: Manifest) -> None:
    for t in man.tensors:
        for stored, crc in t.crc32.items():
            if col.crc32(stored) != crc:
                raise ValueError(f"CRC mismatch in {stored}")


def validate_model_dir(model_dir) -> List[str]:
    """Returns a list of problems (empty = valid)."""
    problems: List[str] = []
    d = Path(model_dir)
    try:
        man = Manifest.load(d)
        if is_drafter_dir(d):
            from ..models.dflash2.model import DFlash2Config, tensor_shapes
            expected = tensor_shapes(DFlash2Config.from_dir(d))
        else:
            from ..models.qwen35.weights import hf_tensor_shapes
            expected = hf_tensor_shapes(Qwen35Config.from_dir(d))
        col = ShardCollection(d)
    except Exception as e:
        return [f"cannot open: {e}"]
    have = man.by_name()
    for n, shape in expected.items():
        n2 = man.aliases.get(n, n)
        if n2 not in have:
            problems.append(f"missing tensor {n}")
            continue
        e = have[n2]
        if list(e.logical_shape) != list(shape):
            problems.append(f"{n}: logical shape {e.logical_shape} != {list(shape)}")
        for stored in ([e.data] if e.encoding == "bf16" else [e.codes, e.metadata1]):
            if not col.has(stored):
                problems.append(f"{n}: stored tensor {stored} missing")
                continue
            if col.crc32(stored) != e.crc32.get(stored):
                problems.append(f"{n}: CRC mismatch in {stored}")
        if e.encoding != "bf16":
            kp = formats.align_up(e.logical_shape[1], formats.K_ALIGN)
            if e.k_padded != kp:
                problems.append(f"{n}: k_padded {e.k_padded} != {kp}")
            _, cs, _ = col.spec(e.codes)
            want = [e.logical_shape[0], kp // 2 if e.encoding in ("nvfp4", "mxfp4") else kp]
            if list(cs) != want:
                problems.append(f"{n}: codes shape {cs} != {want}")
    col.close()
    return problems


# ------------------------------------------------------------------------------------------------ evaluation
def _engine_for(model_dir, device, max_seq_len: int, preset: Optional[str] = None):
    from ..models.qwen35.weights import load_engine_weights
    from ..runtime.engine import Engine
    from ..runtime.state import StateConfig
    ew = load_engine_weights(model_dir, device, preset)
    return Engine(ew, device, StateConfig(max_slots=1, max_seq_len=max_seq_len, page_tokens=16), use_graphs=False)


def _window_logits(eng, ids: Sequence[int], chunk: int = 512) -> torch.Tensor:
    """Teacher-forced logits [len(ids), vocab] (fp32, on CPU) for one window starting at position 0."""
    from ..runtime.batch import SeqRows
    s = eng.open_sequence()
    outs = []
    try:
        for c0 in range(0, len(ids), chunk):
            part = list(ids[c0:c0 + chunk])
            _, out = eng.step([SeqRows(s.slot, s.position, part, tuple(range(len(part))))], [s], sample=False)
            outs.append(out.logits[:len(part)].float().clone())
    finally:
        eng.close_sequence(s)
    return torch.cat(outs, 0)


def _vp(t: torch.Tensor):
    import ctypes
    return ctypes.c_void_p(t.data_ptr())


def kl_divergence(base_logits: torch.Tensor, test_logits: torch.Tensor) -> torch.Tensor:
    """Per-position KL(p_base || p_test) in nats: the reduction kernel on CUDA tensors
    (csrc/kernels/quant_kernels.cu), fp64 torch math otherwise."""
    if base_logits.is_cuda and base_logits.dtype == torch.float32 and test_logits.dtype == torch.float32:
        import ctypes
        from ..ops import _lib
        b, t = base_logits.contiguous(), test_logits.contiguous()
        rows, vocab = b.shape
        kl = torch.empty(rows, dtype=torch.float32, device=b.device)
        agree = torch.empty(rows, dtype=torch.int32, device=b.device)
        with torch.cuda.device(b.device):
            _lib.call("ps_kld_rows", _vp(b), _vp(t), ctypes.c_int(rows), ctypes.c_int(vocab), ctypes.c_longlong(vocab), _vp(kl), _vp(agree))
        return kl.double().cpu()
    lp = torch.log_softmax(base_logits.double(), -1)
    lq = torch.log_softmax(test_logits.double(), -1)
    return (lp.exp() * (lp - lq)).sum(-1).cpu()


def nll_rows(logits: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    """-log softmax(logits)[target] per row (kernel on CUDA fp32 logits, fp64 torch math otherwise)."""
    if logits.is_cuda and logits.dtype == torch.float32:
        import ctypes
        from ..ops import _lib
        lg = logits.contiguous()
        tg = targets.to(lg.device, torch.int32).contiguous()
        out = torch.empty(lg.shape[0], dtype=torch.float32, device=lg.device)
        with torch.cuda.device(lg.device):
            _lib.call("ps_nll_rows", _vp(lg), _vp(tg), ctypes.c_int(lg.shape[0]), ctypes.c_int(lg.shape[1]), ctypes.c_longlong(lg.shape[1]), _vp(out))
        return out.double().cpu()
    lp = torch.log_softmax(logits.double(), -1)
    return (-lp[torch.arange(logits.shape[0]), targets.long().to(lp.device)]).cpu()


def kld_report(kl: torch.Tensor, top1_agree: float) -> dict:
    q = lambda p: float(torch.quantile(kl, p))
    return {"positions": int(kl.numel()), "mean": float(kl.mean()), "p50": q(0.5), "p90": q(0.9), "p99": q(0.99),
            "p99_9": q(0.999), "max": float(kl.max()), "top1_agreement": top1_agree}


class BaselineLogitCache:
    """On-disk cache of the baseline model's logits, one file per evaluation window, keyed by the source model's
    fingerprint, the window's token ids and its position: repeated `kld` runs against different bundles of the same
    source (the usual sweep over presets) run the BF16 baseline only once.  Logits are kept in fp32 (half precision
    would lose range or mantissa that the divergence needs); a 512-token window of a 152 k vocabulary is ~300 MB, hence
    the cache is opt-in (`--baseline-cache DIR`) and bounded by `max_bytes` (oldest files are evicted)."""

    def __init__(self, directory, fingerprint: str, max_bytes: int = 64 << 30):
        self.dir = Path(directory)
        self.dir.mkdir(parents=True, exist_ok=True)
        self.fp, self.max_bytes = fingerprint, max_bytes
        self.hits = self.misses = 0

    def _path(self, w0: int, ids: Sequence[int]) -> Path:
        import hashlib
        h = hashlib.sha256()
        h.update(self.fp.encode()); h.update(str(w0).encode()); h.update(torch.tensor(list(ids), dtype=torch.int32).numpy().tobytes())
        return self.dir / (h.hexdigest()[:32] + ".pt")

    def get(self, w0: int, ids: Sequence[int]) -> Optional[torch.Tensor]:
        p = self._path(w0, ids)
        if p.exists():
            try:
                t = torch.load(p, map_location="cpu")
                if t.shape[0] == len(ids):
                    self.hits += 1
                    os.utime(p)
                    return t
            except Exception:
                p.unlink(missing_ok=True)
        self.misses += 1
        return None

    def put(self, w0: int, ids: Sequence[int], logits: torch.Tensor) -> None:
        p = self._path(w0, ids)
        tmp = p.with_suffix(".tmp")
        torch.save(logits.float().cpu(), tmp)
        os.replace(tmp, p)
        files = sorted(self.dir.glob("*.pt"), key=lambda f: f.stat().st_mtime)
        total = sum(f.stat().st_size for f in files)
        while total > self.max_bytes and len(files) > 1:
            f = files.pop(0)
            total -= f.stat().st_size
            f.unlink(missing_ok=True)


def evaluate_kld(input_dir, bundle_dir, tokens: Sequence[int], window: int = 512, stride: int = 512,
                 max_eval_tokens: int = 0, device="cpu", self_check: bool = False, baseline_cache=None,
                 batch_positions: int = 512) -> dict:
    """``batch_positions``: rows per engine step while a window is evaluated (the reference's ``--batch-positions``,
    docs/user/quantizer.md:5-96; here it bounds the logits held on the device at once)."""
    cache = BaselineLogitCache(baseline_cache, model_fingerprint(input_dir)) if baseline_cache else None
    batch_positions = max(1, min(int(batch_positions), 2048))
    base = None                                   # built lazily: a fully cached run never loads the baseline model
    test = None if self_check else _engine_for(bundle_dir, device, window + 1)
    kls, agree, total = [], 0, 0
    n = len(tokens) if max_eval_tokens <= 0 else min(len(tokens), max_eval_tokens)
    for w0 in range(0, max(1, n - 1), stride):
        ids = tokens[w0:w0 + window]
        if len(ids) < 2:
            break
        lb = cache.get(w0, ids) if cache is not None else None
        if lb is None:
            if base is None:
                base = _engine_for(input_dir, device, window + 1)
            lb = _window_logits(base, ids, batch_positions)
            if cache is not None:
                cache.put(w0, ids, lb)
        lt = lb if self_check else _window_logits(test, ids, batch_positions)
        lb = lb.to(lt.device)
        kls.append(kl_divergence(lb, lt))
        agree += int((lb.argmax(-1) == lt.argmax(-1)).sum())
        total += lb.shape[0]
    kl = torch.cat(kls)
    rep = kld_report(kl, agree / max(1, total))
    rep.update(window=window, stride=stride, baseline=str(input_dir), bundle=str(bundle_dir))
    if cache is not None:
        rep.update(baseline_cache_hits=cache.hits, baseline_cache_misses=cache.misses)
    return rep


def evaluate_ppl(model_dir, tokens: Sequence[int], max_tokens: int = 2048, device="cpu") -> dict:
    ids = list(tokens[:max_tokens])
    eng = _engine_for(model_dir, device, len(ids) + 1)
    lg = _window_logits(eng, ids)
    nll = nll_rows(lg[:-1], torch.tensor(ids[1:]))
    return {"tokens": len(ids) - 1, "nll": float(nll.mean()), "ppl": float(nll.mean().exp())}


def collect_imatrix(model_dir, tokens: Sequence[int], output, window: int = 512, stride: int = 512,
                    max_calibration_tokens: int = 0, device="cpu", flush_windows: int = 0) -> dict:
    """Accumulate sum(x^2) per input channel for every projection input (7 sites per layer + lm_head, the
    tags the reference places in its lowering, src/phaseshift/models/qwen35/model/lower_to_primitives.cpp:
    717-719,819-821,899-901,928-930,940-942,979-980)."""
    eng = _engine_for(model_dir, device, window + 1)
    sums: Dict[str, torch.Tensor] = {}
    counts: Dict[str, int] = {}

    def collector(tag: str, x: torch.Tensor) -> None:
        if x.is_cuda and x.dtype == torch.bfloat16 and x.stride(1) == 1:
            import ctypes
            from ..ops import _lib
            if tag not in sums:
                sums[tag] = torch.zeros(x.shape[1], dtype=torch.float32, device=x.device)
                counts[tag] = 0
            with torch.cuda.device(x.device):
                _lib.call("ps_imatrix_accumulate", _vp(x), ctypes.c_longlong(x.stride(0)), ctypes.c_int(x.shape[0]),
                          ctypes.c_int(x.shape[1]), _vp(sums[tag]))
            counts[tag] += x.shape[0]
            return
        v = x.float().pow(2).sum(0).cpu()
        if tag in sums:
            sums[tag] += v
            counts[tag] += x.shape[0]
        else:
            sums[tag] = v
            counts[tag] = x.shape[0]
    eng.runner.imatrix_collector = collector
    n = len(tokens) if max_calibration_tokens <= 0 else min(len(tokens), max_calibration_tokens)
    windows = flushes = 0
    for w0 in range(0, max(1, n - 1), stride):
        ids = tokens[w0:w0 + window]
        if len(ids) < 2:
            break
        _window_logits(eng, ids)
        windows += 1
        if flush_windows > 0 and windows % flush_windows == 0:
            # a long calibration run leaves a usable file behind every `flush_windows` windows
            save_imatrix(output, sums, counts, {"model": str(model_dir), "tokens": min(n, w0 + len(ids)), "partial": True})
            flushes += 1
    save_imatrix(output, sums, counts, {"model": str(model_dir), "tokens": n})
    return {"sites": len(sums), "tokens": n, "output": str(output), "windows": windows, "flushes": flushes}
