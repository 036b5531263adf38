"""Op-family ranges: NVTX markers for a timeline profiler and an optional per-family device timing.

The model forward wraps each op family (embedding, GDN / attention projections and mixers, MLP, head, sampling) in
``ops.range(name)``.  With ``PS_NVTX=1`` (or ``ops.nvtx = True``) that pushes an NVTX range -- the counterpart of the
reference's ROCTx ranges (src/apps/bench/tg.hip:245-273).  With ``ops.timing_enabled`` the range is bracketed by CUDA
events and the elapsed times accumulate in ``ops.op_times`` (name -> [calls, ms]); reading them synchronises, so the
engine only switches this on for explicit profile steps (``Engine.profile_step``), which run eagerly -- the
counterpart of the reference's per-op dump (src/phaseshift/models/qwen35/runtime/program_executor.hip:238-242,469-511)
and decode perf statistics (src/phaseshift/models/qwen35/runtime/decode_perf_stats.h:12-90).
Both switches off (the default) costs one attribute test per range.
"""
from __future__ import annotations

import contextlib
import os
import time
from typing import Dict, List

import torch

_NULL = contextlib.nullcontext()


class _Range:
    __slots__ = ("tr", "name", "e0", "t0")

    def __init__(self, tr, name):
        self.tr, self.name = tr, name

    def __enter__(self):
        tr = self.tr
        if tr.nvtx:
            torch.cuda.nvtx.range_push(self.name)
        if tr.timing_enabled:
            if torch.device(tr.device).type == "cuda":
                self.e0 = torch.cuda.Event(enable_timing=True)
                self.e0.record()
            else:
                self.t0 = time.perf_counter()
        return self

    def __exit__(self, *exc):
        tr = self.tr
        if tr.timing_enabled:
            if torch.device(tr.device).type == "cuda":
                e1 = torch.cuda.Event(enable_timing=True)
                e1.record()
                tr._pending.append((self.name, self.e0, e1))
            else:
                c = tr.op_times.setdefault(self.name, [0, 0.0])
                c[0] += 1
                c[1] += (time.perf_counter() - self.t0) * 1e3
        if tr.nvtx:
            torch.cuda.nvtx.range_pop()
        return False


class OpTrace:
    """Mixin of the op sets.  Needs ``self.device``."""
    nvtx = os.environ.get("PS_NVTX", "0") == "1"
    timing_enabled = False

    def range(self, name: str):
        if not (self.nvtx or self.timing_enabled):
            return _NULL
        if not hasattr(self, "_pending"):
            self._pending: List[tuple] = []
            self.op_times: Dict[str, list] = {}
        return _Range(self, name)

    def collect_times(self) -> Dict[str, list]:
        """Fold the recorded event pairs into ``op_times`` (synchronises the device) and return it."""
        if not hasattr(self, "_pending"):
            self._pending, self.op_times = [], {}
        if self._pending:
            torch.cuda.synchronize(self.device)
            for name, e0, e1 in self._pending:
                c = self.op_times.setdefault(name, [0, 0.0])
                c[0] += 1
                c[1] += e0.elapsed_time(e1)
            self._pending = []
        return self.op_times
