"""Starting and joining a tensor-parallel job from an app (``--tp N``).

The process the user started becomes rank 0 and keeps its stdin / stdout / HTTP socket; it spawns ranks 1..N-1 as
copies of its own command line (one process per GPU) and every rank joins one NCCL process group plus a small gloo
group for host-side messages.  The reference starts its ranks as worker threads of one coordinator
(src/phaseshift/models/qwen35/runtime/tensor_parallel.cpp:241-314); with one process per GPU the coordinator's job
is this launcher plus the command channel of runtime/tp_serving.py.
"""
from __future__ import annotations

import atexit
import datetime
import os
import socket
import subprocess
import sys
from typing import List, Optional, Sequence, Tuple


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def under_launcher() -> bool:
    return "RANK" in os.environ and "WORLD_SIZE" in os.environ


def spawn_ranks(n: int, module: str, argv: Sequence[str]) -> List[subprocess.Popen]:
    """Make this process rank 0 of an n-rank job and start the other ranks.  No-op under torchrun (RANK is set)."""
    if n <= 1 or under_launcher():
        return []
    port = _free_port()
    base = dict(os.environ, WORLD_SIZE=str(n), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), PS_TP_SPAWNED="1")
    os.environ.update(RANK="0", LOCAL_RANK="0", WORLD_SIZE=str(n), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    procs = []
    for r in range(1, n):
        env = dict(base, RANK=str(r), LOCAL_RANK=str(r))
        procs.append(subprocess.Popen([sys.executable, "-m", module, *argv], env=env, stdin=subprocess.DEVNULL,
                                      stdout=subprocess.DEVNULL))

    def _reap():
        for p in procs:                       # exactly the processes started here, nothing by pattern
            if p.poll() is None:
                p.terminate()
        for p in procs:
            try:
                p.wait(timeout=10)
            except Exception:
                p.kill()
    atexit.register(_reap)
    return procs


def init_tensor_parallel(device_type: str = "cuda", transport: str = "auto", monitor: bool = True,
                         heartbeat_timeout_s: float = 5.0):
    """Join the job described by RANK / WORLD_SIZE / MASTER_*.  Returns (tp, device, host_group): the
    ``TensorParallel`` over the default group, this rank's device and a gloo group for host-side messages."""
    import torch
    import torch.distributed as dist
    from .tp import TensorParallel
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    if device_type == "cuda":
        torch.cuda.set_device(local)
        dev = torch.device("cuda", local)
        dist.init_process_group("nccl", device_id=dev)
    else:
        dev = torch.device("cpu")
        dist.init_process_group("gloo")
    host_group = dist.new_group(backend="gloo", timeout=datetime.timedelta(days=7))
    tp = TensorParallel(dist.group.WORLD, dev, transport=transport)
    if monitor:
        tp.start_monitor(timeout_s=heartbeat_timeout_s)
    return tp, dev, host_group
