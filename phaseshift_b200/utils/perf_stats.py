"""Performance statistics of a run as one JSON-able dict (``--perf-stats-output``): steps, kernel launches (eager and
per captured graph), which projection kernel served how many calls, transport counters, serving counters and the
per-op-family device times of a profile step.  Counterpart of the reference's decode perf statistics
(src/phaseshift/models/qwen35/runtime/decode_perf_stats.h:12-90)."""
from __future__ import annotations

from typing import Optional


def collect(engine, serving=None, profile: Optional[dict] = None) -> dict:
    ops = engine.ops
    out = {
        "backend": engine.backend,
        "steps": engine.steps,
        "kernel_launches_eager": getattr(ops, "launches", 0),
        "graphs_captured": len(engine.graphs),
        "launches_per_graph": {str(k): v for k, v in engine.launches_per_graph.items()},
        "projection_kernel_calls": dict(getattr(ops, "sel_counts", {})),
        "fallbacks": dict(getattr(ops, "fallbacks", {})),
        "device_status_errors": getattr(engine, "status_errors", 0),
    }
    if engine.tp is not None:
        out["tp"] = {"size": engine.tp.size, "transport": engine.tp.transport, **engine.tp.stats}
    if serving is not None:
        out["serving"] = dict(getattr(serving, "stats", {}))
        pc = getattr(getattr(serving, "srv", serving), "prefix", None)
        if pc is not None:
            out["prefix_cache"] = dict(getattr(pc, "stats", {}))
    times = ops.collect_times() if hasattr(ops, "collect_times") else {}
    if times:
        out["op_family_ms"] = {k: {"calls": v[0], "ms": round(v[1], 4)} for k, v in sorted(times.items(), key=lambda kv: -kv[1][1])}
    if profile:
        out["profile_step"] = profile
    return out
