#!/usr/bin/env python
"""Headline benchmark: batch-1 greedy decode tokens/s of the Qwen3.5-27B-shaped hybrid model with
NVFP4/MXFP8 block-quantised weights (the Blackwell counterpart of the reference's PSQ checkpoint), after a
prefill of `--context` tokens -- the reference's `tg` figure (docs/perf/current.md:48-61: 27.51 tok/s on
one R9700).  With --gpus N the same single stream is decoded tensor-parallel over N GPUs (strong scaling).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line on rank 0.  `value` is timed on the device with CUDA events around K decode steps
whose sampled token is fed back on the device; `e2e.value` is the same K steps driven through the public
`Engine.decode` call: each step copies its inputs host->device from pinned memory and reads the sampled
token back to the host.  Weights are random-init N(0, 0.02) and prompts are uniform-random token ids.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

BASELINE_TOK_S = 27.51      # docs/perf/current.md:48-61 (tg128 @ ctx 2048, batch 1, non-speculative)


def _parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="27b", choices=["27b", "4b", "tiny"])
    ap.add_argument("--preset", default="nvfp4", choices=["nvfp4", "bf16", "mxfp8"])
    ap.add_argument("--context", type=int, default=2048, help="prompt tokens prefilled before decoding")
    ap.add_argument("--kv-dtype", default="bf16", choices=["bf16", "fp8_e4m3"])
    ap.add_argument("--prefill-chunk", type=int, default=2048)
    ap.add_argument("--quant-search", type=int, default=1)
    ap.add_argument("--dflash2", type=int, default=1, help="also time DFlash2 speculative rounds (1 GPU only)")
    ap.add_argument("--dflash2-tokens", type=int, default=48)
    ap.add_argument("--dflash2-distill-steps", type=int, default=150,
                    help="distil the random-init drafter on the target's own greedy samples for this many steps and report "
                         "the acceptance it reaches on a held-out prompt (0 = skip)")
    ap.add_argument("--dflash2-distill-seqs", type=int, default=6)
    ap.add_argument("--layout", default="both", choices=["both", "tc", "stream"],
                    help="kernel-side weight layouts kept resident: tensor-core operands, streaming tiles, or both "
                         "(single-row decode streams, everything else runs on the tensor cores)")
    ap.add_argument("--config", type=int, default=0, choices=[0, 2, 3, 4, 5],
                    help="workload preset: 2 = the 4B-shaped model in bf16, prefill 2048 + 512 decode steps (pick the KV "
                         "dtype with --kv-dtype); 3 = prefill 4096 + 1024 decode steps; 4 = 8k-token prompt, 256 speculative "
                         "tokens; 5 = the full serving load (256 requests)")
    ap.add_argument("--serving-requests", type=int, default=48,
                    help="continuous-batching block: concurrent requests with prompts U(512, 8192), outputs U(128, 1024), "
                         "FP8 KV, half of them sharing a 1024-token prefix (0 = skip; the full load is 256)")
    ap.add_argument("--serving-slots", type=int, default=32,
                    help="sequence slots of the serving block (fewer than the requests, so that later admissions can hit "
                         "the prefix cache the earlier ones filled)")
    ap.add_argument("--watchdog", type=int, default=1500,
                    help="seconds after which a hung run dumps every thread's stack to stderr and exits")
    a = ap.parse_args()
    if a.config == 2:
        a.model, a.preset, a.context, a.steps, a.dflash2, a.serving_requests = "4b", "bf16", 2048, 512, 0, 0
    elif a.config == 3:
        a.context, a.steps = 4096, 1024
    elif a.config == 4:
        a.context, a.dflash2_tokens = 8192, 256
    elif a.config == 5:
        a.serving_requests, a.serving_slots = 256, 64
    return a


class ClockSampler:
    """Samples SM clocks and throttle reasons while the timed regions run.

    Reads NVML in a background thread every 10 ms (read-only queries; the handle is found by the CUDA device's
    UUID so CUDA_VISIBLE_DEVICES does not matter); only samples taken between `begin()` and `stop()` count.
    Falls back to an `nvidia-smi -lms` child process when NVML cannot be loaded."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        import threading
        self.p = None
        self.nv = None
        self.samples = []          # (sm_mhz, reasons bitmask, power W)
        self.max_mhz = None
        self.active = False
        self.done = False
        try:
            import pynvml as nv
            import torch
            nv.nvmlInit()
            try:
                uuid = str(torch.cuda.get_device_properties(gpu_index).uuid)
                self.h = nv.nvmlDeviceGetHandleByUUID(("GPU-" + uuid).encode())
            except Exception:
                self.h = nv.nvmlDeviceGetHandleByIndex(gpu_index)
            self.max_mhz = float(nv.nvmlDeviceGetMaxClockInfo(self.h, nv.NVML_CLOCK_SM))
            self.nv = nv
            self.th = threading.Thread(target=self._run, daemon=True)
            self.th.start()
        except Exception:
            self.nv = None
            try:
                self.p = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                           "-lms", "100", "-i", str(gpu_index)], stdout=subprocess.PIPE,
                                          stderr=subprocess.DEVNULL, text=True)
            except Exception:
                self.p = None

    def _run(self):
        nv = self.nv
        while not self.done:
            if self.active:
                try:
                    mhz = float(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                    rs = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.h))
                    pw = nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0
                    self.samples.append((mhz, rs, pw))
                except Exception:
                    pass
            time.sleep(0.01)

    def begin(self):
        self.active = True

    def stop(self) -> dict:
        if self.nv is not None:
            self.active = False
            self.done = True
            self.th.join(timeout=2)
            nv = self.nv
            names = (("hw_slowdown", nv.nvmlClocksEventReasonHwSlowdown),
                     ("hw_thermal_slowdown", nv.nvmlClocksEventReasonHwThermalSlowdown),
                     ("sw_thermal_slowdown", nv.nvmlClocksEventReasonSwThermalSlowdown),
                     ("sw_power_cap", nv.nvmlClocksEventReasonSwPowerCap),
                     ("hw_power_brake", nv.nvmlClocksEventReasonHwPowerBrakeSlowdown),
                     ("applications_clocks", nv.nvmlClocksEventReasonApplicationsClocksSetting))
            seen = 0
            for _, rs, _ in self.samples:
                seen |= rs
            sm = [x[0] for x in self.samples]
            pw = [x[2] for x in self.samples]
            return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": self.max_mhz,
                    "reasons": sorted(n for n, bit in names if seen & bit),
                    "power_w": round(statistics.median(pw), 1) if pw else None,
                    "samples": len(sm), "source": "nvml"}
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.p.terminate()
        try:
            out, _ = self.p.communicate(timeout=5)
        except Exception:
            self.p.kill()
            out = ""
        sm, mx, reasons = [], [], set()
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "source": "nvidia-smi"}


def reference_arm(args):
    """The reference is a HIP/RDNA4-only C++ project (its CMake rejects every other GPU architecture and
    non-clang toolchains); it has no Python package, so it cannot be installed or run on a B200."""
    print(json.dumps({"impl": "reference", "unavailable":
                      "reference is a HIP C++20 runtime that builds only for AMD gfx1201 (cmake/options.cmake:109-115); "
                      "pip install of the reference tree fails: no setup.py/pyproject.toml, no CUDA path"}))
    return 0


def dflash2_arm(eng, cfg, dev, prompt, args):
    """DFlash2 speculative decoding through the public decoder API with a random-init drafter of the
    published 27B drafter shape running on the engine's own kernels (NVFP4 backbone).  Two acceptance regimes
    bracket a trained drafter: `chance` (the random drafter's own proposals: ~0 accepted, so a round costs
    draft + 8-row verify for one token) and `oracle` (the drafter still runs, then its proposals are replaced by
    the target's own greedy continuation: every draft accepted; the cost of a round at full acceptance, not a
    throughput claim).  Both must emit exactly the plain greedy stream."""
    import torch
    from phaseshift_b200.models.dflash2.decoder import DFlash2SpecDecoder
    from phaseshift_b200.models.dflash2.model import DFlash2Config, random_weights, tiny_drafter_config
    from phaseshift_b200.models.dflash2.native import DFlash2NativeDrafter
    n = args.dflash2_tokens
    dcfg = DFlash2Config(vocab_size=cfg.vocab_size) if args.model == "27b" else \
        tiny_drafter_config(cfg, head_dim=128, num_attention_heads=4, num_key_value_heads=2)
    with torch.no_grad():
        w = random_weights(dcfg, 1, dev)
        drafter = DFlash2NativeDrafter(dcfg, w, eng, "nvfp4")
        del w
        torch.cuda.empty_cache()
        dec = DFlash2SpecDecoder(eng, drafter, num_drafts=7)      # pins every step to the tensor-core arithmetic
        plain = eng.generate(prompt, n, prefill_chunk=args.prefill_chunk)
        out = {}
        full = list(prompt) + list(plain)
        dec.generate(list(prompt[:64]), 10)                     # untimed warm-up: workspaces, calibration, graphs
        native_propose = drafter.propose_device
        for mode in ("chance", "oracle"):
            if mode == "oracle":
                def propose_device(anchor, k, pos, _p=native_propose):
                    _p(anchor, k, pos)                          # the drafter still runs, its output is replaced
                    return torch.tensor(full[pos + 1: pos + 1 + k], dtype=torch.int32).pin_memory().to(dev, non_blocking=True)
                drafter.propose_device = propose_device
            for rep in range(2):                                # the first pass captures the graphs of the short tail rounds
                drafter.reset()
                dec.stats = {k: 0 for k in dec.stats}
                samp = dict(temperature=0.0, top_p=1.0, top_k=0, seed=0)
                s = eng.open_sequence()
                toks = [dec.prefill(s, prompt, args.prefill_chunk, samp)]
                torch.cuda.synchronize(); t0 = time.perf_counter()
                while len(toks) < n:
                    toks.extend(dec.round(s, toks[-1], toks[:-1], n - len(toks), samp))
                torch.cuda.synchronize(); dt = time.perf_counter() - t0
                eng.close_sequence(s)
            r = max(1, dec.stats["rounds"])
            out[mode] = {"round_ms": round(dt * 1e3 / r, 3), "rounds": r,
                         "tokens_per_round": round((len(toks) - 1) / r, 3), "exact_match": toks[:n] == list(plain)[:n]}
            if mode == "chance":
                out[mode]["tok_s"] = round((len(toks) - 1) / dt, 2)
        drafter.propose_device = native_propose
        if args.dflash2_distill_steps > 0:
            try:
                out["distilled"] = distilled_arm(eng, cfg, dcfg, dev, prompt, plain, args)
            except Exception as e:                      # the measurement above stands on its own
                out["distilled"] = {"error": repr(e)[:300]}
        # the proposal alone, device time of graph replays
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        for _ in range(3):
            native_propose(full[len(prompt)], 7, len(prompt))
        ev[0].record()
        for _ in range(20):
            native_propose(full[len(prompt)], 7, len(prompt))
        ev[1].record(); torch.cuda.synchronize()
        out["draft_ms"] = round(ev[0].elapsed_time(ev[1]) / 20, 4)
        out["drafter_weight_bytes"] = drafter.weight_bytes()
        out["num_drafts"] = 7
        out["drafter"] = "random-init, %d layers, hidden %d, NVFP4 backbone on the block-scaled tensor-core kernel, " \
                         "one CUDA graph per proposal, drafts verified from device memory" % (dcfg.num_hidden_layers, dcfg.hidden_size)
    return out


def distilled_arm(eng, cfg, dcfg, dev, prompt, plain, args):
    """Honest acceptance: a drafter of the same shape distilled for a few hundred steps on what the engine itself
    decodes (random-init target, random prompts), then run on the engine's kernels (NVFP4 backbone) on the bench
    prompt, which the training never saw.  Reports what it accepts and the resulting tokens/s."""
    import torch
    from phaseshift_b200.models.dflash2.decoder import DFlash2SpecDecoder
    from phaseshift_b200.models.dflash2.distill import distill_on_engine, engine_samples
    from phaseshift_b200.models.dflash2.model import DFlash2Drafter, random_weights
    from phaseshift_b200.models.dflash2.native import DFlash2NativeDrafter
    n = args.dflash2_tokens
    t0 = time.time()
    samples = engine_samples(eng, dcfg.target_layer_ids, args.dflash2_distill_seqs, 96, 160, seed=7)
    t_samples = time.time() - t0
    with torch.enable_grad():
        td = DFlash2Drafter(dcfg, random_weights(dcfg, 1, dev), dev, torch.float32)
        td.use_graph = False
        t0 = time.time()
        loss = distill_on_engine(td, eng, samples, k=7, steps=args.dflash2_distill_steps, lr=3e-4, ctx=192)
        t_train = time.time() - t0
    with torch.no_grad():
        nd = DFlash2NativeDrafter(dcfg, td.w, eng, "nvfp4")
        del td
        torch.cuda.empty_cache()
        dec = DFlash2SpecDecoder(eng, nd, num_drafts=7)
        samp = dict(temperature=0.0, top_p=1.0, top_k=0, seed=0)
        for rep in range(2):
            nd.reset()
            dec.stats = {k: 0 for k in dec.stats}
            s = eng.open_sequence()
            toks = [dec.prefill(s, prompt, args.prefill_chunk, samp)]
            torch.cuda.synchronize(); t0 = time.perf_counter()
            while len(toks) < n:
                toks.extend(dec.round(s, toks[-1], toks[:-1], n - len(toks), samp))
            torch.cuda.synchronize(); dt = time.perf_counter() - t0
            eng.close_sequence(s)
    r = max(1, dec.stats["rounds"])
    distinct = len(set(plain[:n]))
    return {"tok_s": round((len(toks) - 1) / dt, 2), "round_ms": round(dt * 1e3 / r, 3), "rounds": r,
            "tokens_per_round": round((len(toks) - 1) / r, 3), "accepted_per_round": round(dec.stats["accepted"] / r, 3),
            "exact_match": toks[:n] == list(plain)[:n], "distill_steps": args.dflash2_distill_steps,
            "distill_sequences": len(samples), "final_loss": round(loss, 3), "sample_s": round(t_samples, 1),
            "train_s": round(t_train, 1), "distinct_tokens_in_target_stream": distinct,
            "note": "random-init target: its greedy stream carries no linguistic structure, so acceptance reflects how "
                    "much of that stream is predictable from the tapped states, not a trained model pair"}


def serving_block(ew, cfg, dev, tp, world, args):
    """Continuous-batching serving through the public ServingEngine API: every request is submitted at t = 0, the
    scheduler mixes prefill chunks and decode rows per step under the KV banker, half of the prompts start with one
    shared 1024-token prefix (checkpointed by the first request that reaches it, restored by the later ones).  Under
    tensor parallelism every rank runs the same deterministic scheduler.  Device time, max over ranks."""
    import torch
    import torch.distributed as dist
    from phaseshift_b200.runtime.engine import Engine
    from phaseshift_b200.runtime.serving import ServingEngine
    from phaseshift_b200.runtime.state import StateConfig
    n = args.serving_requests
    g = torch.Generator().manual_seed(99)
    small = args.model != "27b"
    lo_p, hi_p, lo_o, hi_o, pre = (64, 256, 16, 64, 32) if small else (512, 8192, 128, 1024, 1024)
    plen = torch.randint(lo_p, hi_p + 1, (n,), generator=g).tolist()
    olen = torch.randint(lo_o, hi_o + 1, (n,), generator=g).tolist()
    shared = torch.randint(0, cfg.vocab_size, (pre,), generator=g).tolist()
    slots = max(1, min(n, args.serving_slots))
    max_seq = hi_p + hi_o + 16
    eng = Engine(ew, dev, StateConfig(max_slots=slots, max_seq_len=max_seq, page_tokens=16, kv_dtype="fp8_e4m3",
                                      kv_capacity_tokens=slots * max_seq), tp=tp)
    srv = ServingEngine(eng, max_step_tokens=2048, prefix_cache_tokens=8 * pre, prefix_cache_entries=4, prefix_min_tokens=min(64, pre))
    for i in range(n):
        body = torch.randint(0, cfg.vocab_size, (plen[i],), generator=g).tolist()
        if i % 2 == 0:
            srv.submit(shared + body[pre:], olen[i], checkpoint_position=pre)
        else:
            srv.submit(body, olen[i])
    sampler = ClockSampler(dev.index or 0)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler.begin()
    ev0.record()
    t0 = time.perf_counter()
    first = {}
    n_tok = 0
    while not srv.idle():
        for e in srv.step():
            if e.kind == "token":
                n_tok += 1
                first.setdefault(e.request_id, (time.perf_counter() - t0) * 1e3)
            elif e.kind in ("done", "error"):
                srv.batcher.retire(e.request_id)
    ev1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    t = torch.tensor([ev0.elapsed_time(ev1)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t)
    prompt_tokens = sum(plen)
    return {"requests": n, "slots": slots, "prompt_len": f"U({lo_p},{hi_p})", "output_len": f"U({lo_o},{hi_o})",
            "shared_prefix_tokens": pre, "shared_prefix_fraction": 0.5, "kv_cache": "fp8_e4m3", "weight_preset": args.preset,
            "generated_tokens": n_tok, "prompt_tokens": prompt_tokens, "wall_ms": round(ms, 1),
            "aggregate_tok_s": round(n_tok / ms * 1e3, 1), "aggregate_tok_s_per_gpu": round(n_tok / ms * 1e3 / world, 1),
            "processed_tok_s": round((n_tok + srv.stats["prefill_tokens"]) / ms * 1e3, 1),
            "p50_ttft_ms": round(statistics.median(first.values()), 1) if first else None,
            "prefill_tokens_computed": srv.stats["prefill_tokens"],
            "prefix_hit_tokens": srv.prefix.stats["restored_tokens"] if srv.prefix is not None else 0,
            "steps": srv.stats["steps"], "failed_steps": srv.stats["failed_steps"], "last_status": srv.stats.get("last_status", 0),
            "tp": dict(tp.stats, transport=tp.transport) if tp is not None else None, "clocks": clocks,
            "timing": "CUDA events around the whole run, max over ranks; TTFT on the host clock of rank 0"}


def main():
    args = _parse()
    if args.impl == "reference":
        return reference_arm(args)

    import faulthandler
    if args.watchdog > 0:
        faulthandler.dump_traceback_later(args.watchdog, exit=True)
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            # relaunch under torchrun so `python bench.py --gpus N` works on its own
            cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
                   "--master-addr", "127.0.0.1", "--master-port", os.environ.get("MASTER_PORT", "29531"),
                   os.path.abspath(__file__)] + sys.argv[1:]
            return subprocess.call(cmd)
        raise SystemExit(f"WORLD_SIZE={world} does not match --gpus {args.gpus}")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    tp = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
        from phaseshift_b200.parallel.tp import TensorParallel
        tp = TensorParallel(dist.group.WORLD, dev)

    from phaseshift_b200.models.qwen35.config import PRESETS
    from phaseshift_b200.models.qwen35.weights import build_engine_weights, random_getter
    from phaseshift_b200.quant import formats
    from phaseshift_b200.runtime.batch import SeqRows
    from phaseshift_b200.runtime.engine import Engine
    from phaseshift_b200.runtime.state import StateConfig

    cfg = PRESETS[args.model]()
    t0 = time.time()
    formats.DEFAULT_SEARCH = args.quant_search
    with torch.no_grad():
        ew = build_engine_weights(cfg, random_getter(cfg, seed=0, device=dev), args.preset, dev,
                                  tp_rank=rank, tp_size=world, keep_canonical=False, layout=args.layout)
    torch.cuda.synchronize()
    build_s = time.time() - t0
    K, W = args.steps, args.warmup
    max_seq = args.context + max(2 * (K + W), (args.dflash2_tokens + 32) if args.dflash2 else 0) + 64
    eng = Engine(ew, dev, StateConfig(max_slots=1, max_seq_len=max_seq, page_tokens=16, kv_dtype=args.kv_dtype,
                                      conv_ring=16, spec_rows=8), tp=tp)
    g = torch.Generator().manual_seed(1234)
    prompt = torch.randint(0, cfg.vocab_size, (args.context,), generator=g).tolist()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    with torch.no_grad():
        s = eng.open_sequence()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier(); ev0.record()
        tok = eng.prefill(s, prompt, args.prefill_chunk)
        ev1.record(); barrier()
        prefill_ms = ev0.elapsed_time(ev1)

        # ---------------- end-to-end arm: public API, per-step H2D of inputs + D2H of the sampled token
        sampler = ClockSampler(local_rank)
        for _ in range(W):
            tok = eng.decode(s, tok)
        b1 = eng.batches[1]
        h2d = b1.h2d_bytes()
        launches0 = eng.ops.launches
        barrier()
        sampler.begin()
        t_e2e0 = time.perf_counter()
        for _ in range(K):
            tok = eng.decode(s, tok)
        torch.cuda.synchronize()
        t_e2e = time.perf_counter() - t_e2e0
        barrier()
        e2e_ms = t_e2e * 1e3 / K
        checksum = 0

        # ---------------- device-timed arm: K graph replays, token fed back on the device
        pos0 = s.position
        eng._reserve(s, pos0 + K + max(W, 3) + 1)
        graph_key = eng.graph_key(1, 1, True, greedy=eng.fused_argmax)     # bucket 1, one output row, identity output gather
        graph = eng.graphs[graph_key]
        gout = eng.graph_out[graph_key]
        b1.fill([SeqRows(s.slot, pos0, [tok], (0,))]); b1.graph_static = True; b1.upload()

        def dev_step():
            graph.replay()
            b1.ids[:1].copy_(gout.tokens[:1])
            b1.row_pos[:1].add_(1)
            b1.seq_desc[0, 3:4].add_(1)
        for _ in range(max(W, 3)):
            dev_step()
        barrier()
        ev0.record()
        for _ in range(K):
            dev_step()
        ev1.record()
        barrier()
        dev_ms = ev0.elapsed_time(ev1) / K
        clocks = sampler.stop()
        s.position = pos0 + K + max(W, 3)
        checksum = int(gout.tokens[0])
        eng.close_sequence(s)

        # ---------------- time to first token through the public API (warm): prefill + first sampled token on the host
        ttft = []
        for _ in range(3):
            s2 = eng.open_sequence()
            barrier(); t_a = time.perf_counter()
            eng.prefill(s2, prompt, args.prefill_chunk)
            torch.cuda.synchronize(); ttft.append((time.perf_counter() - t_a) * 1e3)
            eng.close_sequence(s2)
        ttft_ms = statistics.median(ttft)

        dflash = None
        if args.dflash2 and world == 1:
            dflash = dflash2_arm(eng, cfg, dev, prompt, args)
        serving = None
        if args.serving_requests > 0:
            serving = serving_block(ew, cfg, dev, tp, world, args)

    # max over ranks of the per-step time
    t = torch.tensor([dev_ms, e2e_ms, prefill_ms, ttft_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms, prefill_ms, ttft_ms = (float(x) for x in t.tolist())
    launches_per_step = eng.launches_per_graph.get(graph_key, 0)
    rd_bytes = ew.decode_read_bytes()
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")))
    except Exception:
        pass
    hbm = peaks.get("hbm_gbs", 6650.0)
    value = 1000.0 / dev_ms
    res = {
        "metric": "decode tok/s (bs=1) at 27B" if args.model == "27b" else f"decode tok/s (bs=1) at {args.model}",
        "value": round(value, 3), "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": round(dev_ms, 4), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": round(value / BASELINE_TOK_S, 3) if args.model == "27b" else None,
        "dtype": "bf16 activations; weights " + args.preset, "data": "synthetic (random-init weights, uniform-random prompt ids)",
        "config": {"model": f"qwen3.5-{args.model}-shaped hybrid (GDN:attn 3:1)", "global_batch": 1,
                   "seq_len": args.context, "parallelism": f"tp{world}", "kv_cache": args.kv_dtype,
                   "weight_preset": args.preset,
                   "weight_layouts": args.layout, "l2": "inputs larger than L2 (%.1f GB of weights per step)" % (rd_bytes / 1e9)},
        "clocks": clocks,
        "e2e": {"value": round(1000.0 / e2e_ms, 3), "unit": "tok/s", "ms_per_step": round(e2e_ms, 4),
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 8},
        "gpu_launches": launches_per_step * K,
        "launches_per_step": launches_per_step,
        "prefill": {"tokens": args.context, "first_call_ms": round(prefill_ms, 2), "ms": round(ttft_ms, 2),
                    "tok_s": round(args.context / ttft_ms * 1e3, 1)},
        "ttft_p50_ms": round(ttft_ms, 2),
        "dflash2": dflash,
        "serving": serving,
        "weights_gb_per_step": round(rd_bytes / 1e9, 3),
        "hbm_roofline_frac_of_measured": round(rd_bytes / (dev_ms * 1e-3) / (hbm * 1e9), 4),
        "build_s": round(build_s, 1), "token_checksum": checksum, "impl": "ours",
    }
    if rank == 0:
        print(json.dumps(res), flush=True)
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
