"""Tensor parallel on real GPUs (needs >= 2): the fused in-kernel combine against the NCCL transport and
against the single-GPU engine.  Ranks run as torchrun children with a hard timeout."""
import json
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(world, preset, transport, tmp_path, n_new=12, worker="tp_worker.py"):
    out = tmp_path / f"tp_{world}_{preset}_{transport}.json"
    env = dict(os.environ, PS_TP_TRANSPORT=transport, NCCL_NVLS_ENABLE="0")
    if world == 1:
        cmd = [sys.executable, os.path.join(HERE, worker), str(out), preset, str(n_new)]
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
               "--master-addr", "127.0.0.1", "--master-port", str(_free_port()),
               os.path.join(HERE, worker), str(out), preset, str(n_new)]
    p = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=240)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-2000:]
    res = json.loads(out.read_text())
    if worker != "tp_worker.py":
        return res, torch.load(str(out) + ".pt")
    return res


@pytest.mark.parametrize("preset", ["bf16", "nvfp4"])
def test_tp2_fused_matches_nccl_and_ranks_agree(preset, tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    fused = _run(2, preset, "fused", tmp_path)
    nccl = _run(2, preset, "nccl", tmp_path)
    assert fused[0]["tokens"] == fused[1]["tokens"], "ranks must produce identical tokens"
    assert all(r["transport"] == "fused" and r["stats"]["fused"] > 0 and r["status"] == 0 for r in fused)
    assert fused[0]["graphs"] > 0, "the fused combine must be graph-capturable"
    assert all(r["stats"]["peer_allreduce"] > 0 for r in fused), "prefill chunks must use the peer all-reduce kernel"
    for r in fused:
        for variant, ar in r["allreduce"].items():
            assert ar["status"] == 0 and ar["rank_disagreement"] == 0.0, (variant, ar)
            assert ar["max_err"] < 0.06, (variant, ar)
    assert all(r["transport"] == "nccl" for r in nccl) and nccl[0]["tokens"] == nccl[1]["tokens"]
    # same partial sums, different summation order and rounding (fp32 partials vs a bf16 all-reduce): the
    # tiny random model has nearly flat logits, so only the leading tokens are comparable
    n_same = 4 if preset == "bf16" else 1
    assert fused[0]["tokens"][:n_same] == nccl[0]["tokens"][:n_same]


@pytest.mark.parametrize("world,preset", [(2, "mxfp8"), (2, "nvfp4"), (4, "mxfp8"), (8, "mxfp8")])
def test_tp_logits_match_single_gpu_on_a_mid_size_model(world, preset, tmp_path):
    """hidden 2048, block-quantised weights on the tensor-core kernels: prefill rows go projection -> pushed
    reduce-scatter -> owner reduce + residual -> all-gather, decode rows combine inside the projection kernel.
    Checked: every rank bit-identical to rank 0 at every step; one 300-row row-parallel projection through that
    routing against fp32 partials summed by the library collective; first-layer hidden states and prefill logits
    against the single-GPU engine.  A random-weight model with quantised activations amplifies any change of the
    fp32 summation order by a few percent per layer (on one GPU a different stream-K partition alone moves the
    fourth layer's output by 3-7 % with MXFP8 and by 20 % with NVFP4), so the whole-model bounds are loose and the
    isolated collective carries the precision claim."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    one, t1 = _run(1, preset, "fused", tmp_path, n_new=8, worker="tp_logits_worker.py")
    par, tn = _run(world, preset, "fused", tmp_path, n_new=8, worker="tp_logits_worker.py")
    assert all(r["status"] == 0 and r["transport"] == "fused" for r in par)
    assert all(r["rank_disagreement"] == 0.0 for r in par), [r["rank_disagreement"] for r in par]
    assert all(r["tokens"] == par[0]["tokens"] for r in par)
    assert all(r["stats"].get("scatter", 0) > 0 and r["stats"]["fused"] > 0 for r in par), par[0]["stats"]
    assert all(r["collective_err"] < 8e-3 for r in par), [r["collective_err"] for r in par]
    rel0 = float((tn["layer0"] - t1["layer0"]).norm() / t1["layer0"].norm())
    rel = float((tn["logits"][0] - t1["logits"][0]).norm() / t1["logits"][0].norm())
    assert rel0 < (0.05 if preset == "mxfp8" else 0.08), rel0
    assert rel < (0.25 if preset == "mxfp8" else 0.7), rel
