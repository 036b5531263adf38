"""The checked kernel library (-DPS_CHECKED): same results as the normal one, descriptor assertions that report instead
of faulting, and workspace canaries.  Runs in a child process because the library choice is made at load time."""
import os
import subprocess
import sys
import textwrap

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = textwrap.dedent('''
    import ctypes, json, sys, torch
    from phaseshift_b200.models.qwen35.config import tiny_config
    from phaseshift_b200.models.qwen35.weights import build_engine_weights, random_hf_weights
    from phaseshift_b200.ops import _lib
    from phaseshift_b200.runtime.batch import SeqRows
    from phaseshift_b200.runtime.engine import Engine
    from phaseshift_b200.runtime.state import StateConfig
    cfg = tiny_config()
    hf = random_hf_weights(cfg, seed=0)
    ew = build_engine_weights(cfg, lambda n: hf[n], "nvfp4", "cuda")
    eng = Engine(ew, "cuda", StateConfig(max_slots=2, max_seq_len=96))
    prompt = list(range(7, 40))
    out = {"checked": _lib.checked_build(), "tokens": eng.generate(prompt, 12, prefill_chunk=16)}
    if out["checked"]:
        # a descriptor that points at a slot which does not exist: the kernel must refuse it and say so
        desc = torch.tensor([[0, 1, 9999, 0]], dtype=torch.int32, device="cuda")
        st = eng.state
        li = [i for i, g in enumerate(st.gdn) if g is not None][0]
        log = (torch.zeros(8, st.hv, cfg.linear_key_head_dim, device="cuda"), torch.zeros(8, st.hv, cfg.linear_value_head_dim, device="cuda"),
               torch.zeros(8, st.hv, device="cuda"))
        eng.ops.gdn_replay(st.gdn[li], st.hv, desc, 1, log)
        torch.cuda.synchronize()
        out["bad_slot_status"] = int(st.status[0])
        st.status.zero_()
        # canaries: intact after real steps, and an overwrite next to a workspace is noticed
        out["canaries_clean"] = eng.ops.check_canaries() == []
        key = next(iter(eng.ops._guarded))
        eng.ops._guarded[key][-1] = 0
        out["canary_hit"] = eng.ops.check_canaries()
        eng.ops._guarded[key][-1] = eng.ops.CANARY
        out["guarded"] = len(eng.ops._guarded)
    print("RESULT " + json.dumps(out))
''')


def _run(checked: bool):
    env = dict(os.environ, PYTHONPATH=ROOT, PS_CHECKED="1" if checked else "0")
    p = subprocess.run([sys.executable, "-c", CHILD], capture_output=True, text=True, env=env, timeout=600, cwd=ROOT)
    assert p.returncode == 0, p.stdout[-1500:] + p.stderr[-3000:]
    import json
    return json.loads([l for l in p.stdout.splitlines() if l.startswith("RESULT ")][-1][7:])


def test_checked_library_matches_and_reports():
    normal, checked = _run(False), _run(True)
    assert normal["checked"] is False and checked["checked"] is True
    assert checked["tokens"] == normal["tokens"]
    assert checked["bad_slot_status"] == 5                  # PS_DEV_CHECK_FAILED, no fault
    assert checked["canaries_clean"] and checked["guarded"] > 10
    assert len(checked["canary_hit"]) == 1
