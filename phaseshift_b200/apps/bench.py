"""phaseshift-bench: end-to-end and per-kernel micro-benchmarks (reference: src/apps/bench/main.cpp:46-99,
docs/user/bench.md).  Every sub-command times on the device with CUDA events after warm-up, flushes L2
between samples for kernel benches and prints ``key=value`` lines (``gpu_tokens_per_sec``,
``GREEDY_TOKEN_SUM`` determinism checksum for pp / tg) or CSV rows for kernel sweeps.
"""
from __future__ import annotations

import argparse
import statistics
import sys
from typing import List, Optional

SUBCOMMANDS = ("pp", "tg", "batch", "gemm", "activation-quantize", "rmsnorm", "l2-normalize", "kv-append",
               "paged-attention", "rope", "gdn-recurrence", "gdn-conv1d", "elementwise", "embedding", "sampling", "mtp",
               "gpu-memory", "tp-reduce", "dflash2", "kld")
# Reference sub-commands whose op has no stand-alone launch here: each times the kernel the op is fused into.
FUSED_INTO = {"l2-normalize": "gdn-recurrence",      # q/k L2 normalisation happens inside the GDN mixer kernel
              "gdn-conv1d": "gdn-recurrence",        # so does the short causal conv
              "rope": "kv-append"}                   # partial RoPE is fused with q/k norm and the paged KV append


def _model_args(p):
    p.add_argument("--model-dir"); p.add_argument("--random-model", default=None, choices=["tiny", "4b", "27b"])
    p.add_argument("--preset", default=None); p.add_argument("--device", default=None)
    p.add_argument("--kv-cache-dtype", default="bf16", choices=["bf16", "fp8_e4m3", "nvfp4"])
    p.add_argument("--runs", type=int, default=3); p.add_argument("--warmup", type=int, default=1); p.add_argument("--output")
    p.add_argument("--tp", type=int, default=1, choices=[1, 2, 4, 8], help="tensor-parallel ranks, one process per GPU")


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="phaseshift-bench")
    sub = ap.add_subparsers(dest="cmd", required=True)
    pp = sub.add_parser("pp", help="prefill throughput"); _model_args(pp)
    pp.add_argument("--prompt-tokens", type=int, default=128); pp.add_argument("--mode", default="forward", choices=["forward", "greedy"])
    pp.add_argument("--prefill-chunk", type=int, default=2048)
    tg = sub.add_parser("tg", help="decode throughput"); _model_args(tg)
    tg.add_argument("--mode", default="greedy", choices=["forward", "greedy"]); tg.add_argument("--context", type=int, default=128)
    tg.add_argument("--tokens", type=int, default=8); tg.add_argument("--prefill-chunk", type=int, default=2048)
    tg.add_argument("--compute-logits", type=int, default=1)
    # upstream spells MTP speculative decoding as a mode of `tg` (docs/user/bench.md:5-216); `mtp` is the same measurement
    tg.add_argument("--mtp", action="store_true", help="decode with the MTP head as a drafter (the `mtp` command)")
    tg.add_argument("--draft-k", type=int, default=4); tg.add_argument("--mtp-chain", default="pre", choices=["pre", "post"])
    ba = sub.add_parser("batch", help="concurrent serving throughput"); _model_args(ba)
    ba.add_argument("--requests", type=int, default=8); ba.add_argument("--prompt-tokens", type=int, default=512)
    ba.add_argument("--tokens", type=int, default=64); ba.add_argument("--shared-prefix", type=int, default=0)
    mt = sub.add_parser("mtp", help="speculative decoding with the built-in MTP head (random-init head unless the "
                                    "model directory carries mtp.* tensors)"); _model_args(mt)
    mt.add_argument("--context", type=int, default=128); mt.add_argument("--tokens", type=int, default=32)
    mt.add_argument("--draft-k", type=int, default=4); mt.add_argument("--mtp-chain", default="pre", choices=["pre", "post"])
    mt.add_argument("--verify-mode", default="exact", choices=["exact", "fast"])
    mt.add_argument("--replay-check", action="store_true", help="compare the emitted tokens with plain greedy decoding")
    mt.add_argument("--prefill-chunk", type=int, default=2048)
    ge = sub.add_parser("gemm", help="projection kernels")
    ge.add_argument("--dtype", default="nvfp4", choices=["bf16", "nvfp4", "mxfp8"])
    ge.add_argument("--variant", default="auto", choices=["gemv", "gemm", "tc", "auto"]); ge.add_argument("--rows", default="1,4,8,256,2048")
    ge.add_argument("--n", type=int, default=5120); ge.add_argument("--k", type=int, default=5120)
    ge.add_argument("--actual-qwen-shapes", action="store_true"); ge.add_argument("--warmup", type=int, default=5)
    ge.add_argument("--samples", type=int, default=10); ge.add_argument("--check", action="store_true"); ge.add_argument("--out")
    ge.add_argument("--launches", type=int, default=1, help="launches per timed sample (1: every launch starts from a flushed L2)")
    for name in ("rmsnorm", "kv-append", "paged-attention", "gdn-recurrence", "embedding", "sampling", "gpu-memory", "dflash2",
                 "activation-quantize", "elementwise") + tuple(FUSED_INTO):
        p = sub.add_parser(name); p.add_argument("--rows", type=int, default=1); p.add_argument("--context", type=int, default=4096)
        p.add_argument("--page-tokens", type=int, default=16)
        p.add_argument("--samples", type=int, default=20); p.add_argument("--model", default="27b", choices=["tiny", "4b", "27b"])
        p.add_argument("--kv-cache-dtype", default="bf16", choices=["bf16", "fp8_e4m3", "nvfp4"]); p.add_argument("--variant", default="optimized", choices=["optimized"])
    kl = sub.add_parser("kld", help="KL divergence of a quantised preset against the bf16 model of the same random weights"); _model_args(kl)
    kl.add_argument("--tokens", type=int, default=512); kl.add_argument("--streams", type=int, default=2)
    kl.add_argument("--layout", default="both", choices=["both", "tc", "stream"])
    tr = sub.add_parser("tp-reduce", help="row-parallel combine latency (run under torchrun for > 1 GPU)")
    tr.add_argument("--rows", default="1,8"); tr.add_argument("--hidden", type=int, default=5120); tr.add_argument("--samples", type=int, default=50)
    return ap


def _engine(a, max_seq_len: int, slots: int = 1, spec_rows: int = 0):
    import torch
    from ..models.qwen35.config import PRESETS
    from ..models.qwen35.weights import build_engine_weights, load_engine_weights, random_getter
    from ..runtime.engine import Engine
    from ..runtime.state import StateConfig
    dev = torch.device(a.device or ("cuda:0" if torch.cuda.is_available() else "cpu"))
    tp, tp_kw = None, {}
    if getattr(a, "tp", 1) > 1:
        # every rank runs the same deterministic script (same requests, same scheduler decisions); rank 0 reports
        import os
        from ..parallel.launch import init_tensor_parallel, spawn_ranks
        spawn_ranks(a.tp, "phaseshift_b200.apps.bench", sys.argv[1:])
        tp, dev, _ = init_tensor_parallel(dev.type)
        tp_kw = dict(tp_rank=tp.rank, tp_size=tp.size)
        if tp.rank != 0:
            sys.stdout = open(os.devnull, "w")
    if a.model_dir:
        ew = load_engine_weights(a.model_dir, dev, a.preset, keep_canonical=dev.type != "cuda", **tp_kw)
    else:
        cfg = PRESETS[a.random_model or "tiny"]()
        ew = build_engine_weights(cfg, random_getter(cfg, 0, dev), a.preset or "bf16", dev, keep_canonical=dev.type != "cuda", **tp_kw)
    extra = dict(conv_ring=max(16, 3 + spec_rows), spec_rows=spec_rows) if spec_rows else {}
    return Engine(ew, dev, StateConfig(max_slots=slots, max_seq_len=max_seq_len, kv_dtype=a.kv_cache_dtype, **extra), tp=tp), dev


def _timed(dev, fn):
    import time
    import torch
    if dev.type == "cuda":
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize(); e0.record(); r = fn(); e1.record(); torch.cuda.synchronize()
        return e0.elapsed_time(e1), r
    t0 = time.perf_counter(); r = fn()
    return (time.perf_counter() - t0) * 1e3, r


def cmd_pp(a) -> int:
    import torch
    eng, dev = _engine(a, a.prompt_tokens + 8)
    ids = torch.randint(0, eng.cfg.vocab_size, (a.prompt_tokens,), generator=torch.Generator().manual_seed(0)).tolist()
    times, tok = [], 0
    for i in range(a.warmup + a.runs):
        s = eng.open_sequence()
        ms, tok = _timed(dev, lambda: eng.prefill(s, ids, a.prefill_chunk, sample_last=a.mode == "greedy"))
        eng.close_sequence(s)
        if i >= a.warmup:
            times.append(ms)
    ms = statistics.median(times)
    print(f"prompt_tokens={a.prompt_tokens}"); print(f"prefill_ms={ms:.3f}")
    print(f"gpu_tokens_per_sec={a.prompt_tokens / ms * 1e3:.2f}"); print(f"GREEDY_TOKEN_SUM={tok or 0}")
    return 0


def cmd_tg(a) -> int:
    if getattr(a, "mtp", False):
        a.verify_mode, a.replay_check = "exact", False
        return cmd_mtp(a)
    import torch
    eng, dev = _engine(a, a.context + a.tokens + 8)
    ids = torch.randint(0, eng.cfg.vocab_size, (a.context,), generator=torch.Generator().manual_seed(0)).tolist()
    times, sums = [], []
    for i in range(a.warmup + a.runs):
        s = eng.open_sequence()
        tok = eng.prefill(s, ids, a.prefill_chunk)
        out = [tok]

        def run():
            for _ in range(a.tokens):
                out.append(eng.decode(s, out[-1], sample_index=len(out)))
        ms, _ = _timed(dev, run)
        eng.close_sequence(s)
        if i >= a.warmup:
            times.append(ms); sums.append(sum(out))
    ms = statistics.median(times)
    print(f"context={a.context}"); print(f"tokens={a.tokens}"); print(f"decode_ms_per_token={ms / a.tokens:.4f}")
    print(f"gpu_tokens_per_sec={a.tokens / ms * 1e3:.2f}"); print(f"GREEDY_TOKEN_SUM={sums[-1]}")
    print(f"deterministic={int(len(set(sums)) == 1)}")
    return 0


def cmd_mtp(a) -> int:
    """Speculative decoding with the MTP head (reference bench: src/apps/bench/main.cpp `mtp`, --spec / --verify-mode /
    --replay-check).  Prints acceptance statistics and the decode rate; the head is random-init unless the model
    directory has mtp.* tensors, so the acceptance of a random head is the chance level."""
    import torch
    from ..models.dflash2.decoder import DFlash2SpecDecoder
    from ..models.qwen35.mtp import MTPDrafter, random_mtp_weights
    if not 1 <= a.draft_k <= 7:
        print("error: --draft-k must be in 1..7", file=sys.stderr)
        return 2
    eng, dev = _engine(a, a.context + a.tokens + 16, spec_rows=8)
    dt = torch.float32 if dev.type == "cpu" else torch.bfloat16
    head = None
    if a.model_dir:
        try:
            head = MTPDrafter.from_dir(a.model_dir, eng.cfg, dev, dt, a.mtp_chain)
        except ValueError:
            head = None
    source = "model-dir" if head is not None else "random-init"
    if head is None:
        head = MTPDrafter(eng.cfg, random_mtp_weights(eng.cfg, 0, dev), dev, dt, a.mtp_chain)
    dec = DFlash2SpecDecoder(eng, head, num_drafts=a.draft_k)
    dec.verify_exact = a.verify_mode == "exact"
    ids = torch.randint(0, eng.cfg.vocab_size, (a.context,), generator=torch.Generator().manual_seed(0)).tolist()
    times, out, stats = [], [], {}
    for i in range(a.warmup + a.runs):
        for k in dec.stats:
            dec.stats[k] = 0
        ms, (out, stats) = _timed(dev, lambda: dec.generate(ids, a.tokens, prefill_chunk=a.prefill_chunk))
        if i >= a.warmup:
            times.append(ms)
    ms = statistics.median(times)
    print(f"context={a.context}"); print(f"tokens={len(out)}"); print(f"draft_k={a.draft_k}"); print(f"mtp_head={source}")
    print(f"verify_mode={a.verify_mode}"); print(f"rounds={stats['rounds']}"); print(f"accepted={stats['accepted']}")
    print(f"proposed={stats['proposed']}"); print(f"tokens_per_round={stats['tokens_per_round']}")
    print(f"request_ms={ms:.3f}"); print(f"gpu_tokens_per_sec={len(out) / ms * 1e3:.2f}   # prefill included")
    print(f"GREEDY_TOKEN_SUM={sum(out)}")
    if a.replay_check:
        plain = eng.generate(ids, a.tokens, prefill_chunk=a.prefill_chunk)
        print(f"replay_match={int(plain == out)}")
        return 0 if plain == out or a.verify_mode == "fast" else 1
    return 0


def cmd_batch(a) -> int:
    import torch
    from ..runtime.serving import ServingEngine
    eng, dev = _engine(a, a.prompt_tokens + a.tokens + 8, slots=a.requests)
    srv = ServingEngine(eng, prefix_cache_tokens=4 * a.shared_prefix if a.shared_prefix else 0, prefix_min_tokens=16)
    g = torch.Generator().manual_seed(0)
    shared = torch.randint(0, eng.cfg.vocab_size, (a.shared_prefix,), generator=g).tolist()

    def run():
        for _ in range(a.requests):
            rest = torch.randint(0, eng.cfg.vocab_size, (a.prompt_tokens - a.shared_prefix,), generator=g).tolist()
            srv.submit(shared + rest, a.tokens, checkpoint_position=a.shared_prefix)
        return srv.run_until_idle()
    ms, ev = _timed(dev, run)
    n = sum(1 for e in ev if e.kind == "token")
    print(f"requests={a.requests}"); print(f"generated_tokens={n}"); print(f"wall_ms={ms:.2f}")
    print(f"aggregate_tokens_per_sec={n / ms * 1e3:.2f}"); print(f"steps={srv.stats['steps']}")
    return 0


QWEN27B_SHAPES = [("gdn_in_proj", 16384, 5120), ("gdn_out_proj", 5120, 6144), ("attn_qkv", 14336, 5120), ("attn_o", 5120, 6144),
                  ("mlp_gate_up", 34816, 5120), ("mlp_down", 5120, 17408), ("lm_head", 151936, 5120)]


def cmd_gemm(a) -> int:
    import torch
    from ..models.qwen35.config import tiny_config
    from ..models.qwen35.weights import LinearW
    from ..ops.cuda_ops import CudaOps
    from ..quant import formats
    dev = torch.device("cuda:0")
    ops = CudaOps(tiny_config(), dev)
    shapes = QWEN27B_SHAPES if a.actual_qwen_shapes else [("custom", a.n, a.k)]
    flush = torch.empty(64 * 1024 * 1024, device=dev)
    rows = [int(r) for r in a.rows.split(",")]
    lines = ["dtype,requested_variant,selected_variant,shape_name,rows,n,k,warmup,samples,min_us,p50_us,p95_us,mean_us,GBps,TFLOPs"]
    formats.DEFAULT_SEARCH = 0
    for (name, n, k) in shapes:
        # variants: gemv = streaming CUDA-core kernel (<= 8 rows), gemm = bf16 tcgen05 GEMM after a weight expansion,
        # tc = block-scaled tcgen05 kernel on the quantised codes (any rows), auto = what the engine's selector picks
        # with both layouts resident
        W = LinearW(formats.quantize(torch.randn(n, k, device=dev) * 0.02, a.dtype))
        block = a.dtype in ("nvfp4", "mxfp8")
        if a.variant in ("gemv", "gemm", "auto") or not block:
            W.make_tiled(True)
        if a.variant in ("tc", "auto") and block:
            W.make_umma(True)
        for m in rows:
            if a.variant == "gemv" and m > 8 or a.variant == "gemm" and m <= 8 or a.variant == "tc" and not block:
                continue
            x = torch.randn(m, k, device=dev).to(torch.bfloat16)
            sel = {"stream": "gemv"}.get(ops.select_linear(W, m), ops.select_linear(W, m))
            for _ in range(a.warmup):
                ops.linear(x, W, name="b")
            ts = []
            for _ in range(a.samples):
                flush.zero_()
                if a.launches <= 1:
                    ms, y = _timed(dev, lambda: ops.linear(x, W, name="b"))
                else:
                    ms, ys = _timed(dev, lambda: [ops.linear(x, W, name="b") for _ in range(a.launches)])
                    ms, y = ms / a.launches, ys[-1]
                ts.append(ms * 1e3)
            ts.sort()
            p50 = ts[len(ts) // 2]
            if a.check:
                from ..quant.act_quant import fake_quant
                xr = fake_quant(x.float(), W.fmt, W.act_scale) if sel == "tc" else x.float()
                ref = xr @ W.dense().T
                err = float((y.float() - ref).norm() / ref.norm())
                assert err < 2e-2, f"numerics check failed: rel err {err}"
            lines.append(f"{a.dtype},{a.variant},{sel},{name},{m},{n},{k},{a.warmup},{a.samples},{ts[0]:.2f},{p50:.2f},"
                         f"{ts[int(len(ts) * 0.95) - 1]:.2f},{sum(ts) / len(ts):.2f},{W.nbytes / p50 / 1e3:.1f},{2 * m * n * k / p50 / 1e6:.2f}")
        del W
    text = "\n".join(lines)
    print(text)
    if a.out:
        open(a.out, "w").write(text + "\n")
    return 0


def cmd_dflash2(a, cfg, dev) -> int:
    """The drafter on its own: one proposal (captured graph, `--rows` = draft count, ring filled to `--context` rows),
    the context append of one verified block, and the weights it streams.  The target is cut to 4 layers (the drafter
    only borrows its embedding and lm_head); the drafter keeps the full shape of the named model's DFlash2 companion."""
    import torch
    from ..models.dflash2.model import DFlash2Config, random_weights, tiny_drafter_config
    from ..models.dflash2.native import DFlash2NativeDrafter
    from ..models.qwen35.weights import build_engine_weights, random_getter
    from ..runtime.engine import Engine
    from ..runtime.state import StateConfig
    small = type(cfg)(**{**cfg.__dict__, "num_hidden_layers": 4, "layer_types": None})
    ew = build_engine_weights(small, random_getter(small, 0, dev), "nvfp4", dev, layout="both")
    eng = Engine(ew, dev, StateConfig(max_slots=1, max_seq_len=a.context + 64, conv_ring=16, spec_rows=16))
    if a.model == "tiny":
        dcfg = tiny_drafter_config(small, head_dim=128, num_attention_heads=4, num_key_value_heads=2)
    else:
        dcfg = DFlash2Config(vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, intermediate_size=cfg.intermediate_size,
                             target_layer_ids=[0, 1, 2, 3], num_target_layers=4)
    dr = DFlash2NativeDrafter(dcfg, random_weights(dcfg, 1, dev), eng, "nvfp4")
    k = max(1, min(15, a.rows if a.rows > 1 else 7))
    n_ctx = min(a.context, dcfg.sliding_window)
    g = torch.Generator(device=dev).manual_seed(0)
    taps = [torch.randn(n_ctx, cfg.hidden_size, device=dev, generator=g).to(torch.bfloat16) for _ in dcfg.target_layer_ids]
    dr.append_context(taps, 0)
    for _ in range(3):
        dr.propose_device(5, k, n_ctx)
    rep = 20
    ts = sorted(_timed(dev, lambda: [dr.propose_device(5, k, n_ctx) for _ in range(rep)])[0] * 1e3 / rep for _ in range(max(3, a.samples // 4)))
    blk = [t[:k + 1] for t in taps]
    for _ in range(2):
        dr.append_context(blk, n_ctx)
    ta = sorted(_timed(dev, lambda: [dr.append_context(blk, n_ctx) for _ in range(rep)])[0] * 1e3 / rep for _ in range(3))
    wb = dr.weight_bytes() + eng.runner.w.lm_head.nbytes
    print("kernel=dflash2"); print(f"model={a.model}"); print(f"drafts={k}"); print(f"context_rows={n_ctx}")
    print(f"proposal_p50_us={ts[len(ts) // 2]:.1f}"); print(f"append_block_p50_us={ta[len(ta) // 2]:.1f}")
    print(f"launches_per_proposal={dr.graph_launches.get(k, 0)}"); print(f"weight_bytes_per_proposal={wb}")
    print(f"hbm_GBps={wb / ts[len(ts) // 2] / 1e3:.0f}")
    return 0


def cmd_kernel(a) -> int:
    """Single-kernel latency on a synthetic decode-shaped problem of the named model."""
    import torch
    from ..models.qwen35.config import PRESETS
    from ..models.qwen35.weights import build_engine_weights, random_getter
    from ..runtime.batch import SeqRows, StepBatch
    from ..runtime.engine import Engine
    from ..runtime.state import StateConfig
    dev = torch.device("cuda:0")
    cfg = PRESETS[a.model]()
    if a.cmd == "gpu-memory":
        free, total = torch.cuda.mem_get_info()
        print(f"gpu_total_bytes={total}"); print(f"gpu_free_bytes={free}")
        print(f"model_params={cfg.param_count()}"); return 0
    if a.cmd == "dflash2":
        return cmd_dflash2(a, cfg, dev)
    small = type(cfg)(**{**cfg.__dict__, "num_hidden_layers": 4, "layer_types": None, "vocab_size": min(cfg.vocab_size, 32768)})
    ew = build_engine_weights(small, random_getter(small, 0, dev), "bf16", dev)
    eng = Engine(ew, dev, StateConfig(max_slots=1, max_seq_len=a.context + a.rows + 64, kv_dtype=a.kv_cache_dtype, page_tokens=a.page_tokens), use_graphs=False)
    ops, st = eng.ops, eng.state
    s = eng.open_sequence()
    eng._reserve(s, a.context + a.rows + 1)
    b = StepBatch(max(a.rows, 1), 1, dev)
    b.fill([SeqRows(s.slot, a.context, [1] * a.rows, tuple(range(a.rows)))]); b.upload()
    L_attn = next(l for l in ew.layers if l.kind == 1); L_gdn = next(l for l in ew.layers if l.kind == 0)
    li_a, li_g = small.attn_layers[0], small.gdn_layers[0]
    g = torch.Generator(device=dev).manual_seed(0)
    x = torch.randn(a.rows, small.hidden_size, device=dev, generator=g).to(torch.bfloat16)
    qkv = torch.randn(a.rows, L_attn.mixer.qkv_proj.N, device=dev, generator=g).to(torch.bfloat16)
    proj = torch.randn(a.rows, L_gdn.mixer.in_proj.N + L_gdn.mixer.ba_proj.N, device=dev, generator=g).to(torch.bfloat16)
    logits = torch.randn(a.rows, cfg.vocab_size, device=dev, generator=g)
    q = ops.attn_prep(qkv, L_attn.mixer, eng.runner.hq, eng.runner.hkv, b, st.kv[li_a], st)
    from ..models.qwen35.weights import LinearW
    from ..ops import _lib
    from ..ops._lib import c_int, ptr
    from ..quant import formats
    wq = LinearW(formats.quantize(torch.randn(256, small.hidden_size, device=dev) * 0.02, "nvfp4")).make_umma()
    gu = torch.randn(a.rows, 2 * small.intermediate_size, device=dev, generator=g).to(torch.bfloat16)
    gu_out = torch.empty(a.rows, small.intermediate_size, dtype=torch.bfloat16, device=dev)

    def elementwise():          # the two stand-alone elementwise kernels that exist: residual add and interleaved SwiGLU
        _lib.call("ps_add", ptr(x), c_int(x.stride(0)), ptr(x), c_int(x.stride(0)), ptr(x), c_int(x.stride(0)), c_int(a.rows),
                  c_int(small.hidden_size))
        _lib.call("ps_swiglu_interleaved", ptr(gu), c_int(gu.stride(0)), ptr(gu_out), c_int(gu_out.stride(0)), c_int(a.rows),
                  c_int(small.intermediate_size))
    fused_into = FUSED_INTO.get(a.cmd)
    if fused_into:
        print(f"fused_into={fused_into}")
        a.cmd = fused_into
    fns = {"activation-quantize": lambda: ops.act_quant(x, wq, L_attn.input_norm, 1e-6),
           "elementwise": elementwise,
           "rmsnorm": lambda: ops.rmsnorm(x, L_attn.input_norm, 1e-6, "bn"),
           "kv-append": lambda: ops.attn_prep(qkv, L_attn.mixer, eng.runner.hq, eng.runner.hkv, b, st.kv[li_a], st),
           "paged-attention": lambda: ops.paged_attention(q, qkv, eng.runner.hq, eng.runner.hkv, b, st.kv[li_a], st, a.context + a.rows),
           "gdn-recurrence": lambda: ops.gdn(proj, L_gdn.mixer, eng.runner.hk, eng.runner.hv, b, st.gdn[li_g], st),
           "embedding": lambda: ops.embed(b, a.rows, ew.embed, st.status),
           "sampling": lambda: ops.sample(logits, b, a.rows, status=st.status)}
    fn = fns[a.cmd]
    for _ in range(5):
        fn()
    ts = sorted(_timed(dev, fn)[0] * 1e3 for _ in range(a.samples))
    print(f"kernel={a.cmd}"); print(f"model={a.model}"); print(f"rows={a.rows}"); print(f"context={a.context}")
    print(f"min_us={ts[0]:.2f}"); print(f"p50_us={ts[len(ts) // 2]:.2f}"); print(f"p95_us={ts[int(len(ts) * 0.95) - 1]:.2f}")
    return 0


def cmd_tp_reduce(a) -> int:
    import os
    import torch
    import torch.distributed as dist
    from ..models.qwen35.config import tiny_config
    from ..models.qwen35.weights import LinearW
    from ..ops.cuda_ops import CudaOps
    from ..parallel.tp import TensorParallel
    from ..quant.formats import quantize
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    torch.cuda.set_device(rank); dev = torch.device("cuda", rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    tp = TensorParallel(dist.group.WORLD, dev) if world > 1 else None
    ops = CudaOps(tiny_config(), dev)
    H = a.hidden
    W = LinearW(quantize(torch.randn(H, 1024, device=dev) * 0.02, "bf16")).make_tiled()
    for m in [int(r) for r in a.rows.split(",")]:
        x = torch.randn(m, 1024, device=dev).to(torch.bfloat16); res = torch.zeros(m, H, device=dev, dtype=torch.bfloat16)
        comb = tp.combine_for(H) if tp else None
        run_f = lambda: ops.linear(x, W, name="o", residual=res, tp_combine=comb)
        part = torch.empty(m, H, device=dev, dtype=torch.bfloat16)

        def run_n():
            y = ops.linear(x, W, name="p")
            if world > 1:
                dist.all_reduce(y)
            return torch.add(y, res, out=part)
        run_p = lambda: ops.linear(x, W, name="o", residual=res)          # the projection alone (no combine)
        for name, fn in (("none", run_p), ("fused", run_f), ("nccl", run_n)):
            for _ in range(5):
                fn()
            ts = sorted(_timed(dev, fn)[0] * 1e3 for _ in range(a.samples))
            t = torch.tensor([ts[len(ts) // 2]], device=dev)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            if rank == 0:
                print(f"tp_reduce transport={name} ranks={world} rows={m} hidden={H} payload_bytes={m * H * 2} p50_us={float(t):.2f}")
    # stand-alone all-reduce kernels against the library collective on prefill-sized payloads
    if tp is not None and tp.transport == "fused":
        for m in (256, 2048):
            part = (torch.randn(m, H, device=dev) * 0.1).to(torch.bfloat16)
            res = torch.zeros(m, H, device=dev, dtype=torch.bfloat16); out = torch.empty_like(part)
            cases = [("two_shot", lambda: tp.reduce_gather(m, H, res, "bench_ar_out", partial=part)),
                     ("peer", lambda: (setattr(tp, "use_multimem", False), tp.peer_all_reduce(part, res, out))),
                     ("multimem", lambda: (setattr(tp, "use_multimem", True), tp.peer_all_reduce(part, res, out))),
                     ("nccl", lambda: (dist.all_reduce(part.clone()), None))]
            for name, fn in cases:
                for _ in range(5):
                    fn()
                ts = sorted(_timed(dev, fn)[0] * 1e3 for _ in range(a.samples))
                t = torch.tensor([ts[len(ts) // 2]], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                if rank == 0:
                    nbytes = m * H * 2
                    wire = 2 * (world - 1) / world * nbytes          # what a bandwidth-optimal all-reduce sends per GPU
                    print(f"tp_allreduce kernel={name} ranks={world} rows={m} hidden={H} payload_bytes={nbytes} p50_us={float(t):.2f} "
                          f"bus_GBps={wire / float(t) / 1e3:.1f} frac_of_nvlink_770GBps={wire / 770e9 * 1e6 / float(t):.3f}")
        tp.use_multimem = False
    # block-scaled tensor-core projection fused with its collective: a 27B down_proj (5120 x 17408 / ranks, NVFP4)
    #  * rows <= 32 : partial sums combined inside the projection kernel
    #  * more rows  : epilogue pushes rows to their owners (reduce-scatter), then reduce + residual + all-gather
    # roofline target = max(FLOPs / measured bf16 GEMM peak, bytes each GPU must send / measured peer-copy bandwidth)
    import json
    from pathlib import Path
    peaks = {"bf16_tflops": 1590.0}
    for cand in (Path.cwd() / "MEASURED_PEAKS.json", Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"):
        if cand.exists():
            peaks.update(json.loads(cand.read_text()))
            break
    link_gbs = 770.0
    Kfull, N = 17408, 5120
    Wd = LinearW(quantize(torch.randn(N, Kfull // world, device=dev) * 0.02, "nvfp4")).make_umma()
    for m in (1, 8, 32, 256, 2048):
        x = (torch.randn(m, Kfull // world, device=dev)).to(torch.bfloat16)
        res = torch.zeros(m, N, device=dev, dtype=torch.bfloat16)
        cases = [("projection_only", lambda: ops.linear(x, Wd, name="tpb_o", residual=res))]
        if tp is not None and tp.transport == "fused":
            if m <= 32:
                comb = tp.combine_for(N)
                cases.append(("fused_combine", lambda: ops.linear(x, Wd, name="tpb_f", residual=res, tp_combine=comb)))
            else:
                def run_scatter():
                    ops.linear(x, Wd, name="tpb_p", tp_scatter=tp.scatter_for(m, N))
                    return tp.reduce_gather(m, N, res, "tpb_out")
                cases.append(("fused_scatter_gather", run_scatter))
            outn = torch.empty(m, N, device=dev, dtype=torch.bfloat16)

            def run_nccl():
                y = ops.linear(x, Wd, name="tpb_n")
                dist.all_reduce(y)
                return torch.add(y, res, out=outn)
            cases.append(("nccl", run_nccl))
        for name, fn in cases:
            for _ in range(5):
                fn()
            rep = 10                                     # back-to-back calls: device time, not host launch gaps
            ts = sorted(_timed(dev, lambda: [fn() for _ in range(rep)])[0] * 1e3 / rep for _ in range(max(5, a.samples // rep)))
            t = torch.tensor([ts[len(ts) // 2]], device=dev)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            if rank == 0:
                us = float(t)
                flops = 2.0 * m * N * (Kfull // world)
                wire = 0.0 if name == "projection_only" else 2.0 * (world - 1) / world * m * N * (4 if m <= 32 else 2)
                target_us = max(flops / (peaks["bf16_tflops"] * 1e12), wire / (link_gbs * 1e9)) * 1e6
                print(f"tp_fused path={name} ranks={world} rows={m} n={N} k_local={Kfull // world} p50_us={us:.2f} "
                      f"wire_bytes_per_gpu={int(wire)} roofline_target_us={target_us:.2f} frac_of_roofline={target_us / us:.3f}")
    if world > 1:
        dist.destroy_process_group()
    return 0


def cmd_kld(a) -> int:
    """Random-init model, random token streams: logits of every position from the bf16 engine and from the quantised
    preset (same underlying weights, the engine's own kernels on both sides); KL(bf16 || preset), top-1 agreement."""
    import torch
    from ..models.qwen35.config import PRESETS
    from ..models.qwen35.weights import build_engine_weights, random_getter
    from ..runtime.batch import SeqRows
    from ..runtime.engine import Engine
    from ..runtime.state import StateConfig
    dev = torch.device(a.device or "cuda:0")
    cfg = PRESETS[a.random_model or "tiny"]()
    preset = a.preset or "nvfp4"
    n = a.tokens
    g = torch.Generator().manual_seed(0)
    streams = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for _ in range(a.streams)]

    def logits_of(p, layout):
        ew = build_engine_weights(cfg, random_getter(cfg, 0, dev), p, dev, keep_canonical=False, **({"layout": layout} if p != "bf16" else {}))
        eng = Engine(ew, dev, StateConfig(max_slots=1, max_seq_len=n + 8, kv_dtype=a.kv_cache_dtype), use_graphs=False)
        out = []
        for ids in streams:
            s = eng.open_sequence()
            _, o = eng.step([SeqRows(s.slot, 0, ids, tuple(range(n)))], [s], want_logits=True)
            out.append(torch.log_softmax(o.logits[:n].float(), -1).to(torch.bfloat16 if cfg.vocab_size > 65536 else torch.float32).cpu())
            eng.close_sequence(s)
        del eng, ew
        torch.cuda.empty_cache()
        return out
    ref = logits_of("bf16", None)
    got = logits_of(preset, a.layout)
    kls, agree = [], 0
    for r, q in zip(ref, got):
        r, q = r.float(), q.float()
        kls.append((r.exp() * (r - q)).sum(-1))
        agree += int((r.argmax(-1) == q.argmax(-1)).sum())
    kl = torch.cat(kls)
    # two models whose logits are independent Gaussians of standard deviation s are about s^2 nats apart: the ceiling that
    # a random-init model, which amplifies any perturbation layer after layer, approaches as it gets deeper
    sd = float(torch.cat([r.float().std(-1) for r in ref]).mean())
    qs = torch.quantile(kl, torch.tensor([0.5, 0.9, 0.99]))
    print(f"model={a.random_model or 'tiny'}"); print(f"preset={preset}"); print(f"layout={a.layout}"); print(f"positions={kl.numel()}")
    print(f"kld_mean={float(kl.mean()):.6f}"); print(f"kld_p50={float(qs[0]):.6f}"); print(f"kld_p90={float(qs[1]):.6f}")
    print(f"kld_p99={float(qs[2]):.6f}"); print(f"kld_max={float(kl.max()):.6f}"); print(f"top1_agreement={agree / kl.numel():.4f}")
    print(f"logit_std={sd:.4f}"); print(f"kld_over_decorrelated={float(kl.mean()) / max(sd * sd, 1e-12):.3f}")
    return 0


def main(argv: Optional[List[str]] = None) -> int:
    a = build_parser().parse_args(argv)
    if a.cmd == "kld":
        return cmd_kld(a)
    return {"pp": cmd_pp, "tg": cmd_tg, "batch": cmd_batch, "gemm": cmd_gemm, "tp-reduce": cmd_tp_reduce,
            "mtp": cmd_mtp}.get(a.cmd, cmd_kernel)(a)


if __name__ == "__main__":
    sys.exit(main())
