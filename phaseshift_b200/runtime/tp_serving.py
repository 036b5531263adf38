"""Serving under tensor parallelism: one request interface, N identical schedulers.

Every rank owns a full copy of the serving loop (batcher, KV banker, prefix cache, grammar matchers): the scheduler is
deterministic, so ranks that see the same commands in the same order plan the same batches, and the engine's logits are
bit-identical across ranks, so they commit the same tokens.  Only rank 0 talks to the outside world; what it hears
(submit / cancel) and when it steps is broadcast to the others over a gloo group, one small message per step.  That is
the job of the reference's coordinator fan-out (src/phaseshift/models/qwen35/runtime/tensor_parallel.cpp:396-515,
hook src/phaseshift/models/qwen35/runtime/continuous_batcher.cpp:433-435) without shipping the batch itself.

A rank that fails raises, stops beating (parallel/health.py) and leaves; the others notice before their next launch
(``assert_alive`` inside ``Engine.step`` / ``run_rows``), fail their requests and shut down.
"""
from __future__ import annotations

from typing import List, Optional

import torch.distributed as dist


class TpServingLeader:
    """Rank 0: same interface as the serving loop it wraps; records commands and replays them to the followers."""

    def __init__(self, serving, host_group):
        self.srv, self.group = serving, host_group
        self.pending: List[tuple] = []
        self.batcher = serving.batcher
        self.engine = serving.engine

    @property
    def constraints(self):
        return self.srv.constraints

    @constraints.setter
    def constraints(self, v):
        self.srv.constraints = v

    @property
    def stats(self):
        return self.srv.stats

    def submit(self, *args, **kw) -> int:
        rid = self.srv.submit(*args, **kw)            # raises here, before anything is broadcast, on a bad request
        self.pending.append(("submit", args, kw))
        return rid

    def cancel(self, rid: int) -> bool:
        ok = self.srv.cancel(rid)
        self.pending.append(("cancel", (rid,), {}))
        return ok

    def request(self, rid: int):
        return self.srv.request(rid)

    def idle(self) -> bool:
        return self.srv.idle()

    def _publish(self, step: bool, stop: bool = False) -> None:
        msg = [(self.pending, step, stop)]
        dist.broadcast_object_list(msg, src=0, group=self.group)
        self.pending = []

    def step(self):
        self._publish(True)
        return self.srv.step()

    def run_until_idle(self, max_steps: int = 1_000_000):
        ev = []
        for _ in range(max_steps):
            if self.idle():
                break
            ev += self.step()
        return ev

    def shutdown(self) -> None:
        self._publish(False, stop=True)


def follow(serving, host_group) -> int:
    """Ranks > 0: apply rank 0's commands, step when it steps, until it says stop.  Returns the number of steps."""
    steps = 0
    while True:
        msg = [None]
        dist.broadcast_object_list(msg, src=0, group=host_group)
        cmds, step, stop = msg[0]
        for (op, args, kw) in cmds:
            try:
                getattr(serving, op)(*args, **kw)
            except Exception:
                if op != "submit":          # a submit the leader accepted cannot fail here; anything else is fatal
                    raise
        if stop:
            return steps
        if step:
            for e in serving.step():
                if e.kind in ("done", "error"):
                    serving.batcher.retire(e.request_id)
            steps += 1
