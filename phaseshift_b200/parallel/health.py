"""Rank-loss detection for tensor-parallel serving, on the host.

Every rank runs a `PeerMonitor`: a daemon thread that publishes a heartbeat counter in the job's
key-value store (the process group's TCPStore, or any object with ``set``/``get``) and watches the
counters of its peers.  A peer whose counter has not moved for ``timeout_s`` is declared lost;
``assert_alive()`` -- called by the serving loop between steps, before the next launch -- then raises
``RankLostError`` so the engine can fail its requests and shut down instead of entering a collective
that can never complete.  The device side is bounded independently: every in-kernel wait on a peer flag
gives up after about a second and reports ``PS_DEV_WAIT_TIMEOUT`` through the status word.

The reference runs its ranks as threads of one process and aborts the shared barrier group when one of them
fails (src/phaseshift/runtime/tp/tp_barrier_group.cpp:60-119,
src/phaseshift/models/qwen35/runtime/tensor_parallel.cpp:396-515); here the ranks are SPMD processes, so
liveness is a store-based heartbeat.
"""
from __future__ import annotations

import threading
import time
from typing import Dict, List, Optional


class RankLostError(RuntimeError):
    def __init__(self, ranks: List[int]):
        super().__init__("tensor-parallel peer(s) lost: " + ", ".join(str(r) for r in ranks))
        self.ranks = ranks


class PeerMonitor:
    def __init__(self, store, rank: int, world: int, interval_s: float = 0.2, timeout_s: float = 2.0, prefix: str = "ps_hb"):
        self.store, self.rank, self.world = store, rank, world
        self.interval_s, self.timeout_s, self.prefix = interval_s, timeout_s, prefix
        self._stop = threading.Event()
        self._lost: List[int] = []
        self._lock = threading.Lock()
        self._beat = 0
        self._seen: Dict[int, tuple] = {}          # peer -> (last counter, time it last changed)
        self._thread: Optional[threading.Thread] = None
        self.error: Optional[BaseException] = None

    def _key(self, r: int) -> str:
        return f"{self.prefix}/{r}"

    def start(self) -> "PeerMonitor":
        self.store.set(self._key(self.rank), "0")
        self._thread = threading.Thread(target=self._run, name="ps-peer-monitor", daemon=True)
        self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval_s + 1.0)

    def _read(self, r: int) -> Optional[int]:
        try:
            return int(self.store.get(self._key(r)))
        except Exception:
            return None

    def _run(self) -> None:
        t_start = time.monotonic()
        while not self._stop.wait(self.interval_s):
            try:
                self._beat += 1
                self.store.set(self._key(self.rank), str(self._beat))
                now = time.monotonic()
                lost = []
                for r in range(self.world):
                    if r == self.rank:
                        continue
                    v = self._read(r)
                    last = self._seen.get(r)
                    if v is not None and (last is None or v != last[0]):
                        self._seen[r] = (v, now)
                    else:
                        since = last[1] if last is not None else t_start
                        if now - since > self.timeout_s:
                            lost.append(r)
                with self._lock:
                    self._lost = lost
            except BaseException as e:       # the store itself went away (rank 0 died): everyone is lost to us
                self.error = e
                with self._lock:
                    self._lost = [r for r in range(self.world) if r != self.rank]
                return

    def lost(self) -> List[int]:
        with self._lock:
            return list(self._lost)

    def assert_alive(self) -> None:
        l = self.lost()
        if l:
            raise RankLostError(l)
