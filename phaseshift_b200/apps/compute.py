"""phaseshift-compute: token ids in, token ids out.  Single-shot mode and a JSON-Lines stdio server.

Flag set, stdout ``KEY=VALUE`` contract and the ``--serve-stdio`` protocol follow the reference
(src/apps/compute/main.hip:47-81,1322-1683; docs/user/compute.md:6-31,133-220): requests
``generate / cancel / ping / shutdown``, events ``token / done / error / pong / shutdown``, ready marker
``PHASESHIFT_SERVE_READY`` on stderr, invalid flag combinations exit 2 before the model is loaded.
"""
from __future__ import annotations

import argparse
import json
import os
import select
import sys
from typing import List, Optional

DEFAULT_PROMPT = [248041, 77091]


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="phaseshift-compute", description=__doc__.split("\n")[0])
    ap.add_argument("--model-dir")
    ap.add_argument("--random-model", choices=["tiny", "4b", "27b"], help="random-init weights instead of --model-dir")
    ap.add_argument("--preset", default=None, choices=["bf16", "nvfp4", "mxfp8"], help="quantise a BF16 model on load")
    ap.add_argument("--input-ids-file")
    ap.add_argument("--max-new-tokens", type=int, default=32)
    ap.add_argument("--max-seq-len", type=int, default=512)
    ap.add_argument("--arena-gib", type=float, default=0,
                    help="byte budget (GiB) of the device arenas holding the KV pages and the recurrent state; the engine "
                         "refuses to start when the configuration needs more (0 = framework allocator, no budget)")
    ap.add_argument("--page-tokens", type=int, default=16)
    ap.add_argument("--max-concurrent-requests", type=int, default=1)
    ap.add_argument("--kv-cache-capacity-tokens", type=int, default=0)
    ap.add_argument("--prefix-cache-capacity-tokens", type=int, default=0)
    ap.add_argument("--prefix-cache-max-entries", type=int, default=16)
    ap.add_argument("--constraint-tokenizer-info")
    ap.add_argument("--device", default=None)
    ap.add_argument("--kv-cache-dtype", default="bf16", choices=["bf16", "fp8_e4m3", "nvfp4", "psq4", "psq8"],
                    help="storage of the paged key/value cache; psq4 / psq8 are the upstream names of the 4-bit (nvfp4) and 8-bit (fp8_e4m3) block formats")
    ap.add_argument("--decode-backend", default="host", choices=["host", "gpu-mcu"])
    ap.add_argument("--verify-weights", type=int, default=0, choices=[0, 1])
    ap.add_argument("--dump-logits")
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--top-k", type=int, default=0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--dflash2-model-dir")
    ap.add_argument("--dflash2-drafts", type=int, default=7)
    ap.add_argument("--dflash2-ngram-tail", type=int, default=0)
    ap.add_argument("--dflash2-ngram-n", type=int, default=0)
    ap.add_argument("--dflash2-stats", type=int, default=0, choices=[0, 1])
    ap.add_argument("--serve-stdio", action="store_true")
    ap.add_argument("--tp", type=int, default=1, choices=[1, 2, 4, 8],
                    help="tensor-parallel ranks (one process per GPU; this process becomes rank 0 and starts the others)")
    ap.add_argument("--perf-stats-output", help="write launch / timing / fallback counters of the run as JSON")
    ap.add_argument("--max-scheduled-tokens", type=int, default=2048)
    return ap


def validate_args(a) -> Optional[str]:
    """Everything that can be rejected without touching the model (exit code 2)."""
    if not a.model_dir and not a.random_model:
        return "--model-dir is required"
    if a.decode_backend == "gpu-mcu":
        return "--decode-backend gpu-mcu is not implemented"
    if a.max_new_tokens < 0 or a.max_seq_len <= 0 or a.page_tokens <= 0:
        return "token counts must be positive"
    if a.temperature < 0 or not (0 < a.top_p <= 1) or a.top_k < 0:
        return "bad sampling parameters"
    if a.dflash2_model_dir and a.serve_stdio and a.max_concurrent_requests > 1:
        return "speculative serving advances one request at a time: use --max-concurrent-requests 1"
    if a.dflash2_model_dir and not (1 <= a.dflash2_drafts <= 15):
        return "--dflash2-drafts must be in [1, 15]"
    if a.dflash2_ngram_tail and not a.dflash2_model_dir:
        return "--dflash2-ngram-tail needs --dflash2-model-dir"
    if getattr(a, "tp", 1) > 1 and a.dflash2_model_dir:
        return "--tp with --dflash2-model-dir is not supported (the drafter is not tensor parallel)"
    return None


class ComputeRuntime:
    """Model + state + serving loop for one process (reference: Qwen35ComputeRuntime,
    src/apps/compute/compute_runtime.hip:51-224)."""

    def __init__(self, a):
        import torch
        from ..models.qwen35.config import PRESETS
        from ..models.qwen35.weights import build_engine_weights, load_engine_weights, random_getter
        from ..runtime.engine import Engine
        from ..runtime.serving import ServingEngine
        from ..runtime.state import StateConfig
        dev = a.device or ("cuda:0" if torch.cuda.is_available() else "cpu")
        self.device = torch.device(dev)
        self.tp, self.host_group, self.rank = None, None, 0
        tp_kw = {}
        if getattr(a, "tp", 1) > 1:
            from ..parallel.launch import init_tensor_parallel
            self.tp, self.device, self.host_group = init_tensor_parallel(self.device.type)
            self.rank = self.tp.rank
            tp_kw = dict(tp_rank=self.tp.rank, tp_size=self.tp.size)
        if a.random_model:
            cfg = PRESETS[a.random_model]()
            ew = build_engine_weights(cfg, random_getter(cfg, 0, self.device), a.preset or "bf16", self.device,
                                      keep_canonical=self.device.type != "cuda", **tp_kw)
        else:
            ew = load_engine_weights(a.model_dir, self.device, a.preset, verify_weights=bool(a.verify_weights),
                                     keep_canonical=self.device.type != "cuda", **tp_kw)
        self.cfg = ew.cfg
        spec = bool(a.dflash2_model_dir)
        from ..runtime.state import KV_DTYPE_ALIASES
        a.kv_cache_dtype = KV_DTYPE_ALIASES.get(a.kv_cache_dtype, a.kv_cache_dtype)
        sc = StateConfig(max_slots=a.max_concurrent_requests, max_seq_len=a.max_seq_len, page_tokens=a.page_tokens,
                         kv_capacity_tokens=a.kv_cache_capacity_tokens, kv_dtype=a.kv_cache_dtype,
                         conv_ring=32 if spec else 4, spec_rows=a.dflash2_drafts + 1 if spec else 0)
        try:
            self.engine = Engine(ew, self.device, sc, tp=self.tp, arena_gib=getattr(a, "arena_gib", 0) or 0)
        except MemoryError as e:
            raise SystemExit(f"phaseshift-compute: {e} (raise --arena-gib or lower --max-seq-len / --max-concurrent-requests)")
        compiler = None
        if a.constraint_tokenizer_info:
            from ..runtime.constraints import TokenConstraintCompiler
            info = json.load(open(a.constraint_tokenizer_info))
            compiler = TokenConstraintCompiler(info["vocab"], info.get("vocab_size", self.cfg.vocab_size),
                                               info.get("stop_token_ids", self.cfg.eos_token_ids),
                                               vocab_type=info.get("vocab_type", "byte_level"))
        self.serving = ServingEngine(self.engine, max_step_tokens=a.max_scheduled_tokens,
                                     prefix_cache_tokens=a.prefix_cache_capacity_tokens,
                                     prefix_cache_entries=a.prefix_cache_max_entries, constraint_compiler=compiler,
                                     terminal_checkpoints=a.prefix_cache_capacity_tokens > 0)
        self.spec = None
        if spec:
            from ..models.dflash2.decoder import DFlash2SpecDecoder
            from ..runtime.spec_serving import SpecServingEngine
            self.spec = DFlash2SpecDecoder.from_dir(self.engine, a.dflash2_model_dir, a.dflash2_drafts,
                                                    ngram_tail=a.dflash2_ngram_tail, ngram_n=a.dflash2_ngram_n,
                                                    target_model_dir=a.model_dir)
            # served requests go through speculative rounds too (one request at a time, like the reference's
            # serve_step_dflash, src/apps/compute/main.hip:1077-1124); the plain loop stays available as `plain_serving`
            self.plain_serving = self.serving
            self.serving = SpecServingEngine(self.spec, prefill_chunk=a.max_scheduled_tokens, constraint_compiler=compiler,
                                             prefix_cache_tokens=a.prefix_cache_capacity_tokens,
                                             prefix_cache_entries=a.prefix_cache_max_entries)


def run_single_shot(a, rt: ComputeRuntime, out=None) -> int:
    out = out or sys.stdout
    if a.input_ids_file:
        ids = [int(t) for t in open(a.input_ids_file).read().replace(",", " ").split()]
    else:
        ids = [t % rt.cfg.vocab_size for t in DEFAULT_PROMPT]
    stop = rt.cfg.eos_token_ids
    stats = {}
    if rt.spec is not None:
        gen, stats = rt.spec.generate(ids, a.max_new_tokens, stop_tokens=stop, temperature=a.temperature, top_p=a.top_p,
                                      top_k=a.top_k, seed=a.seed)
    elif a.dump_logits:
        import numpy as np
        from ..runtime.batch import SeqRows
        s = rt.engine.open_sequence()
        rows, gen = [], []
        toks, o = rt.engine.step([SeqRows(s.slot, 0, ids, (len(ids) - 1,), temperature=a.temperature, top_p=a.top_p,
                                          top_k=a.top_k, seed=a.seed)], [s], want_logits=True)
        rows.append(o.logits[:1].float().cpu().numpy())
        gen.append(toks[0])
        while len(gen) < a.max_new_tokens and gen[-1] not in stop:
            toks, o = rt.engine.step([SeqRows(s.slot, s.position, [gen[-1]], (0,), temperature=a.temperature,
                                              top_p=a.top_p, top_k=a.top_k, seed=a.seed, sample_index=len(gen))], [s], want_logits=True)
            rows.append(o.logits[:1].float().cpu().numpy())
            gen.append(toks[0])
        np.concatenate(rows, 0).astype("<f4").tofile(a.dump_logits)
        print(f"LOGITS_VOCAB={rt.cfg.vocab_size}", file=out)
        print("LOGITS_STEP_ROWS=1", file=out)
        print(f"LOGITS_TOTAL_ROWS={len(rows)}", file=out)
    else:
        rid = rt.serving.submit(ids, a.max_new_tokens, a.temperature, a.top_p, a.top_k, a.seed, stop)
        ev = rt.serving.run_until_idle()
        gen = [e.token_id for e in ev if e.kind == "token" and e.request_id == rid]
        err = [e for e in ev if e.kind == "error"]
        if err:
            print("ERROR=" + str(err[0].info.get("message")), file=out)
            return 1
    print(f"PROMPT_TOKENS={len(ids)}", file=out)
    print(f"GENERATED_TOKENS={len(gen)}", file=out)
    print(f"KV_CACHE_DTYPE={a.kv_cache_dtype}", file=out)
    print(f"KV_POOL_RESERVED_BYTES={rt.engine.state.kv_bytes()}", file=out)
    for k, v in stats.items():
        print(f"DFLASH2_{k.upper()}={v}", file=out)
    print("GENERATED_IDS=" + ",".join(str(t) for t in gen), file=out)
    return 0


def run_serve_stdio(a, rt: ComputeRuntime, fin=None, fout=None) -> int:
    """Single-threaded loop: poll stdin without blocking while work is pending, step the engine, emit events."""
    fin = fin or sys.stdin
    fout = fout or sys.stdout
    srv = rt.serving
    ids_of = {}            # engine request id -> client request id

    def emit(obj):
        fout.write(json.dumps(obj, separators=(",", ":")) + "\n")
        fout.flush()

    def handle(line: str) -> bool:
        try:
            req = json.loads(line)
            op = req.get("op")
        except Exception as e:
            emit({"event": "error", "request_id": None, "message": f"bad json: {e}"})
            return True
        if op == "ping":
            emit({"event": "pong"})
        elif op == "shutdown":
            srv.batcher.cancel_all()
            emit({"event": "shutdown"})
            return False
        elif op == "cancel":
            for eid, cid in list(ids_of.items()):
                if cid == req.get("request_id") and srv.cancel(eid):
                    r = srv.request(eid)
                    emit({"event": "done", "request_id": cid, "generated_ids": r["generated"], "finish_reason": "cancelled",
                          "prompt_tokens": r["prompt_tokens"], "restored_tokens": r["restored_tokens"],
                          "prefill_tokens": r["prefill_tokens"], "cache_checkpoint_tokens": 0})
                    ids_of.pop(eid)
        elif op == "generate":
            cid = req.get("request_id")
            try:
                eid = srv.submit(req["input_ids"], int(req.get("max_new_tokens", 32)), float(req.get("temperature", 0.0)),
                                 float(req.get("top_p", 1.0)), int(req.get("top_k", 0)), int(req.get("seed", 0)),
                                 req.get("stop_token_ids", rt.cfg.eos_token_ids),
                                 int(req.get("prefix_cache_checkpoint_position", 0)), grammar=req.get("grammar"),
                                 structural_tag=req.get("structural_tag"))
                ids_of[eid] = cid
            except Exception as e:
                emit({"event": "error", "request_id": cid, "message": str(e)})
        else:
            emit({"event": "error", "request_id": req.get("request_id"), "message": f"unknown op {op!r}"})
        return True

    print("PHASESHIFT_SERVE_READY", file=sys.stderr, flush=True)
    # Read the pipe through its file descriptor with our own line buffer: select() only knows about the
    # descriptor, so lines parked in a Python-level read buffer would otherwise never wake the loop.
    fd = fin.fileno()
    pending = b""
    alive, eof = True, False
    while alive:
        busy = not srv.idle()
        if not eof:
            ready, _, _ = select.select([fd], [], [], 0 if (busy or b"\n" in pending) else None)
            if ready:
                chunk = os.read(fd, 1 << 16)
                if not chunk:
                    eof = True
                pending += chunk
        while alive and b"\n" in pending:
            line, pending = pending.split(b"\n", 1)
            if line.strip():
                alive = handle(line.decode("utf-8", "replace"))
        if not alive:
            break
        if eof and srv.idle():
            break
        if srv.idle():
            continue
        for e in srv.step():
            cid = ids_of.get(e.request_id)
            if e.kind == "token":
                emit({"event": "token", "request_id": cid, "token_id": e.token_id})
            elif e.kind == "done":
                emit(dict({"event": "done", "request_id": cid}, **{k: v for k, v in e.info.items() if k != "message"}))
                srv.batcher.retire(e.request_id)
                ids_of.pop(e.request_id, None)
            else:
                emit({"event": "error", "request_id": cid, "message": e.info.get("message", "error")})
                ids_of.pop(e.request_id, None)
    return 0


def main(argv: Optional[List[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    a = build_parser().parse_args(argv)
    err = validate_args(a)
    if err:
        print(f"phaseshift-compute: {err}", file=sys.stderr)
        return 2
    if a.tp > 1:
        from ..parallel.launch import spawn_ranks
        spawn_ranks(a.tp, "phaseshift_b200.apps.compute", argv)
    rt = ComputeRuntime(a)
    rc = 0
    if a.tp > 1 and a.serve_stdio:
        # rank 0 owns stdin / stdout; the other ranks replay its commands (runtime/tp_serving.py)
        from ..runtime.tp_serving import TpServingLeader, follow
        if rt.rank == 0:
            rt.serving = TpServingLeader(rt.serving, rt.host_group)
            try:
                rc = run_serve_stdio(a, rt)
            finally:
                rt.serving.shutdown()
        else:
            follow(rt.serving, rt.host_group)
    elif a.serve_stdio:
        rc = run_serve_stdio(a, rt)
    elif rt.rank == 0:
        rc = run_single_shot(a, rt)
    else:
        rc = run_single_shot(a, rt, out=open(os.devnull, "w"))     # every rank runs the same request; rank 0 reports
    if a.perf_stats_output and rt.rank == 0:
        from ..utils.perf_stats import collect
        with open(a.perf_stats_output, "w") as f:
            json.dump(collect(rt.engine, rt.serving), f, indent=1)
    if rt.tp is not None:
        import torch.distributed as dist
        m = getattr(rt.tp, "monitor", None)
        if m is not None:
            m.stop()
        dist.destroy_process_group()
    return rc


if __name__ == "__main__":
    sys.exit(main())
