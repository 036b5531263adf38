"""The GPU test runner's bookkeeping with plain host commands: exit-code normalisation, GPU assignment, the memory ledger,
the deadline that ends the command's own process group, and tainting."""
import json
import os
import subprocess
import sys
import threading
import time

import pytest

from phaseshift_b200.apps import gpu_test_runner as R

PY = sys.executable


def _run(ledger, *flags, cmd):
    return R.main(["--ledger", str(ledger), "--gpu-count", "2", "--gpu-gib", "40", *flags, "--", *cmd])


def test_exit_codes_are_normalised(tmp_path):
    led = tmp_path / "l.json"
    assert _run(led, cmd=[PY, "-c", "pass"]) == 0
    assert _run(led, cmd=[PY, "-c", "import sys; sys.exit(3)"]) == 1
    assert _run(led, cmd=[PY, "-c", "import sys; sys.exit(77)"]) == 1                       # a skip counts as a failure
    assert _run(led, "--allow-skip", cmd=[PY, "-c", "import sys; sys.exit(77)"]) == 77
    assert _run(led, cmd=[PY, "-c", "import os, signal; os.kill(os.getpid(), signal.SIGKILL)"]) == 1
    assert _run(led, cmd=[str(tmp_path / "no-such-program")]) == 126
    assert R.main(["--ledger", str(led)]) == 2                                                # no command
    assert json.loads(led.read_text())["reservations"] == []


def test_gpus_are_assigned_through_the_visible_devices_variable(tmp_path):
    led, out = tmp_path / "l.json", tmp_path / "o.txt"
    code = f"import os; open({str(out)!r}, 'w').write(os.environ['CUDA_VISIBLE_DEVICES'] + ' ' + os.environ['PS_TEST_VRAM_GIB'])"
    assert _run(led, "--gpus", "2", "--vram-gib", "10", cmd=[PY, "-c", code]) == 0
    assert out.read_text() == "0,1 10.0"
    assert _run(led, "--gpus", "3", cmd=[PY, "-c", "pass"]) == 125                            # the machine has two


def test_ledger_refuses_then_admits_when_room_appears(tmp_path):
    led, gate = tmp_path / "l.json", tmp_path / "gate"
    hold = f"import os, time\nwhile not os.path.exists({str(gate)!r}): time.sleep(0.05)"
    rcs = []
    ts = [threading.Thread(target=lambda: rcs.append(_run(led, "--gpus", "1", "--vram-gib", "24", cmd=[PY, "-c", hold])))
          for _ in range(2)]
    for t in ts:
        t.start()
    deadline = time.time() + 20
    while time.time() < deadline:
        try:
            if len(json.loads(led.read_text())["reservations"]) == 2:
                break
        except (FileNotFoundError, ValueError):
            pass
        time.sleep(0.05)
    doc = json.loads(led.read_text())
    assert sorted(g for r in doc["reservations"] for g in r["gpus"]) == [0, 1]               # spread over both GPUs
    # 24 of 40 GiB are taken on each GPU: a third 24 GiB test finds no room, a 16 GiB one does
    assert _run(led, "--vram-gib", "24", cmd=[PY, "-c", "pass"]) == 125
    assert _run(led, "--vram-gib", "16", cmd=[PY, "-c", "pass"]) == 0
    waiter = []
    tw = threading.Thread(target=lambda: waiter.append(_run(led, "--vram-gib", "24", "--wait", "20", cmd=[PY, "-c", "pass"])))
    tw.start()
    time.sleep(0.5)
    gate.write_text("go")
    for t in ts + [tw]:
        t.join(30)
    assert rcs == [0, 0] and waiter == [0]
    assert json.loads(led.read_text())["reservations"] == []


def _gone(pid: int) -> bool:
    try:
        with open(f"/proc/{pid}/status") as f:
            return "State:\tZ" in f.read()
    except FileNotFoundError:
        return True


@pytest.mark.timeout(60)
def test_deadline_ends_the_whole_process_group_and_taints_the_gpu(tmp_path):
    led, pidf = tmp_path / "l.json", tmp_path / "pids"
    # the command starts a child of its own; both ignore nothing, both must be gone after the deadline
    code = (f"import os, subprocess, sys, time\n"
            f"c = subprocess.Popen([sys.executable, '-c', 'import time; time.sleep(600)'])\n"
            f"open({str(pidf)!r}, 'w').write(f'{{os.getpid()}} {{c.pid}}')\n"
            f"time.sleep(600)")
    t0 = time.time()
    assert _run(led, "--gpus", "1", "--deadline", "1.5", "--grace", "1", cmd=[PY, "-c", code]) == 124
    assert time.time() - t0 < 30
    pids = [int(p) for p in pidf.read_text().split()]
    for _ in range(100):
        if all(_gone(p) for p in pids):
            break
        time.sleep(0.05)
    assert all(_gone(p) for p in pids)
    doc = json.loads(led.read_text())
    assert list(doc["tainted"]) == ["0"] and doc["reservations"] == []
    # the tainted GPU is avoided: one GPU is left, two cannot be had
    out = tmp_path / "o.txt"
    assert _run(led, cmd=[PY, "-c", f"import os; open({str(out)!r}, 'w').write(os.environ['CUDA_VISIBLE_DEVICES'])"]) == 0
    assert out.read_text() == "1"
    assert _run(led, "--gpus", "2", cmd=[PY, "-c", "pass"]) == 125
    assert R.main(["--ledger", str(led), "--clear-taint"]) == 0
    assert _run(led, "--gpus", "2", cmd=[PY, "-c", "pass"]) == 0


def test_reservations_of_a_runner_that_died_are_dropped(tmp_path):
    led = tmp_path / "l.json"
    p = subprocess.Popen([PY, "-c", "pass"]); p.wait()
    led.write_text(json.dumps({"reservations": [{"runner_pid": p.pid, "gpus": [0, 1], "gib": 40, "since": 0}], "tainted": {}}))
    assert _run(led, "--gpus", "2", "--vram-gib", "40", cmd=[PY, "-c", "pass"]) == 0
