"""phaseshift-gpu-test-runner: run one GPU test command under a device-memory ledger, a GPU assignment and a hard deadline.

Several test processes share the GPUs of one machine.  Each invocation

* reserves ``--vram-gib`` of device memory on ``--gpus N`` GPUs in a ledger kept under a lock file (one JSON document for the
  machine), waiting up to ``--wait`` seconds for room, and picks the least loaded GPUs that are not tainted;
* runs the command in a process group of its own with ``CUDA_VISIBLE_DEVICES`` set to the GPUs it was given;
* ends that process group (SIGTERM, then SIGKILL after a grace period) when the deadline passes, and then marks the GPUs it
  used as *tainted*: a test that had to be killed may have left its device in a bad state, so later invocations avoid those
  GPUs until ``--clear-taint`` is given by an operator who has looked at them;
* normalises the exit code: 0 pass, 1 test failure, 77 (the command's "skipped") is reported as failure 1 unless
  ``--allow-skip``, 124 deadline, 125 no GPU available within ``--wait``, 126 the command could not be started.

Only the process group started here is ever signalled.  Nothing about a GPU is changed: the ledger is advisory bookkeeping
between cooperating test processes.

Reference counterpart: ``tests/support/gpu_test_runner/main.cpp:26-34,53-118,216,239,286-349`` (file-lock VRAM ledger with a
24 GB default, assignment through the visible-devices variable, SIGKILL deadline, tainting after a timeout, exit-code
normalisation).
"""
from __future__ import annotations

import argparse
import fcntl
import json
import os
import signal
import subprocess
import sys
import time
from contextlib import contextmanager
from pathlib import Path
from typing import Dict, List, Optional

EXIT_PASS, EXIT_FAIL, EXIT_SKIP, EXIT_DEADLINE, EXIT_NO_GPU, EXIT_NO_START = 0, 1, 77, 124, 125, 126
DEFAULT_GPU_GIB = 180.0


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="phaseshift-gpu-test-runner")
    ap.add_argument("--ledger", default=os.path.join(os.environ.get("TMPDIR", "/tmp"), "phaseshift-gpu-ledger.json"))
    ap.add_argument("--gpu-count", type=int, default=0, help="GPUs of the machine (0: ask the driver)")
    ap.add_argument("--gpu-gib", type=float, default=DEFAULT_GPU_GIB, help="device memory per GPU the ledger may hand out")
    ap.add_argument("--gpus", type=int, default=1, help="GPUs this test needs")
    ap.add_argument("--vram-gib", type=float, default=24.0, help="device memory this test may use on each of its GPUs")
    ap.add_argument("--deadline", type=float, default=600.0, help="seconds before the test's process group is ended")
    ap.add_argument("--grace", type=float, default=5.0, help="seconds between SIGTERM and SIGKILL")
    ap.add_argument("--wait", type=float, default=0.0, help="seconds to wait for room in the ledger")
    ap.add_argument("--allow-skip", action="store_true", help="pass exit code 77 through instead of counting it as a failure")
    ap.add_argument("--clear-taint", action="store_true", help="forget every taint mark and exit")
    ap.add_argument("--status", action="store_true", help="print the ledger and exit")
    ap.add_argument("command", nargs=argparse.REMAINDER, help="-- program and arguments")
    return ap


def _gpu_count(requested: int) -> int:
    if requested > 0:
        return requested
    try:
        import torch
        return int(torch.cuda.device_count())
    except Exception:
        return 0


@contextmanager
def _locked(path: Path):
    """The ledger document under an exclusive file lock; written back on exit."""
    path.parent.mkdir(parents=True, exist_ok=True)
    with open(str(path) + ".lock", "a+") as lk:
        fcntl.flock(lk, fcntl.LOCK_EX)
        try:
            try:
                doc = json.loads(path.read_text())
            except (FileNotFoundError, ValueError):
                doc = {}
            doc.setdefault("reservations", [])
            doc.setdefault("tainted", {})
            yield doc
            tmp = path.with_suffix(".tmp")
            tmp.write_text(json.dumps(doc, indent=1))
            os.replace(tmp, path)
        finally:
            fcntl.flock(lk, fcntl.LOCK_UN)


def _alive(pid: int) -> bool:
    try:
        os.kill(pid, 0)
    except ProcessLookupError:
        return False
    except PermissionError:
        return True
    return True


def _prune(doc: dict) -> None:
    """Drop reservations whose runner is gone (it crashed before releasing them)."""
    doc["reservations"] = [r for r in doc["reservations"] if _alive(int(r["runner_pid"]))]


def _used(doc: dict) -> Dict[int, float]:
    used: Dict[int, float] = {}
    for r in doc["reservations"]:
        for g in r["gpus"]:
            used[g] = used.get(g, 0.0) + float(r["gib"])
    return used


def try_reserve(doc: dict, n_gpus: int, gib: float, gpu_count: int, gpu_gib: float, runner_pid: int,
                res_id: str = "") -> Optional[List[int]]:
    _prune(doc)
    used = _used(doc)
    free = [(used.get(g, 0.0), g) for g in range(gpu_count)
            if str(g) not in doc["tainted"] and used.get(g, 0.0) + gib <= gpu_gib + 1e-9]
    if len(free) < n_gpus:
        return None
    chosen = sorted(g for _, g in sorted(free)[:n_gpus])
    doc["reservations"].append({"id": res_id or str(runner_pid), "runner_pid": runner_pid, "gpus": chosen, "gib": gib,
                                "since": time.time()})
    return chosen


def release(doc: dict, res_id: str) -> None:
    doc["reservations"] = [r for r in doc["reservations"] if str(r.get("id", r["runner_pid"])) != res_id]


def normalise(returncode: int, allow_skip: bool) -> int:
    if returncode == 0:
        return EXIT_PASS
    if returncode == EXIT_SKIP:
        return EXIT_SKIP if allow_skip else EXIT_FAIL
    return EXIT_FAIL


def run(a) -> int:
    ledger = Path(a.ledger)
    if a.clear_taint:
        with _locked(ledger) as doc:
            doc["tainted"] = {}
        return 0
    if a.status:
        with _locked(ledger) as doc:
            _prune(doc)
            print(json.dumps(doc, indent=1))
        return 0
    cmd = a.command[1:] if a.command and a.command[0] == "--" else a.command
    if not cmd:
        print("phaseshift-gpu-test-runner: no command given", file=sys.stderr)
        return 2
    count = _gpu_count(a.gpu_count)
    me = os.getpid()
    res_id = f"{me}-{time.monotonic_ns()}-{id(a)}"            # one per invocation, also when several share a process
    t_end = time.monotonic() + max(0.0, a.wait)
    gpus = None
    while True:
        with _locked(ledger) as doc:
            gpus = try_reserve(doc, a.gpus, a.vram_gib, count, a.gpu_gib, me, res_id)
        if gpus is not None or time.monotonic() >= t_end:
            break
        time.sleep(0.2)
    if gpus is None:
        print(f"phaseshift-gpu-test-runner: no {a.gpus} GPU(s) with {a.vram_gib} GiB free (of {count}; tainted ones excluded)",
              file=sys.stderr)
        return EXIT_NO_GPU
    env = dict(os.environ, CUDA_VISIBLE_DEVICES=",".join(map(str, gpus)), PS_TEST_VRAM_GIB=str(a.vram_gib))
    timed_out = False
    try:
        try:
            proc = subprocess.Popen(cmd, env=env, start_new_session=True)       # a process group of its own
        except OSError as e:
            print(f"phaseshift-gpu-test-runner: cannot start {cmd[0]!r}: {e}", file=sys.stderr)
            return EXIT_NO_START
        try:
            rc = proc.wait(timeout=a.deadline)
        except subprocess.TimeoutExpired:
            timed_out = True
            pgid = proc.pid                                                      # session leader: pgid == pid
            for sig, pause in ((signal.SIGTERM, a.grace), (signal.SIGKILL, None)):
                try:
                    os.killpg(pgid, sig)
                except ProcessLookupError:
                    break
                try:
                    proc.wait(timeout=pause)
                    break
                except subprocess.TimeoutExpired:
                    continue
            rc = EXIT_DEADLINE
    finally:
        with _locked(ledger) as doc:
            release(doc, res_id)
            if timed_out:
                for g in gpus:
                    doc["tainted"][str(g)] = {"since": time.time(), "command": " ".join(cmd)[:200]}
    if timed_out:
        print(f"phaseshift-gpu-test-runner: deadline of {a.deadline:g} s passed; GPUs {gpus} marked tainted", file=sys.stderr)
        return EXIT_DEADLINE
    if rc < 0:
        print(f"phaseshift-gpu-test-runner: command ended by signal {-rc}", file=sys.stderr)
        return EXIT_FAIL
    return normalise(rc, a.allow_skip)


def main(argv: Optional[List[str]] = None) -> int:
    return run(build_parser().parse_args(argv))


if __name__ == "__main__":
    sys.exit(main())
