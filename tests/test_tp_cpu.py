"""Tensor-parallel host logic on CPU ranks (gloo): rank-local weight slicing, KV-head replication,
row-parallel combine.  TP=2 and TP=4 greedy output must equal the single-rank output."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from phaseshift_b200.models.qwen35.config import tiny_config
from phaseshift_b200.models.qwen35.reference import reference_greedy
from phaseshift_b200.models.qwen35.weights import TpGeometry, build_engine_weights, random_hf_weights


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, prompt, n_new, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from phaseshift_b200.parallel.tp import TensorParallel
        from phaseshift_b200.runtime.engine import Engine
        from phaseshift_b200.runtime.state import StateConfig
        torch.set_num_threads(1)
        cfg = tiny_config()
        hf = random_hf_weights(cfg, seed=0)
        ew = build_engine_weights(cfg, lambda n: hf[n], "bf16", "cpu", tp_rank=rank, tp_size=world)
        tp = TensorParallel(dist.group.WORLD, "cpu")
        eng = Engine(ew, "cpu", StateConfig(max_slots=1, max_seq_len=64), tp=tp)
        out = eng.generate(prompt, n_new, prefill_chunk=7)
        q.put((rank, out))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_tp_greedy_equals_single_rank(world):
    cfg = tiny_config()
    hf = random_hf_weights(cfg, seed=0)
    prompt = torch.randint(0, cfg.vocab_size, (20,), generator=torch.Generator().manual_seed(5)).tolist()
    ref = reference_greedy(cfg, hf, prompt, 10)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, prompt, 10, q)) for r in range(world)]
    for p in procs:
        p.start()
    outs = dict(q.get(timeout=180) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for r in range(world):
        assert outs[r] == ref, (r, outs[r], ref)


def test_tp_geometry_kv_replication():
    from phaseshift_b200.models.qwen35.config import qwen35_27b_config
    cfg = qwen35_27b_config()
    for tp in (1, 2, 4, 8):
        seen_q = []
        for r in range(tp):
            g = TpGeometry.make(cfg, r, tp)
            seen_q += list(g.q_heads)
            group = cfg.num_attention_heads // cfg.num_key_value_heads
            # every local query head must map to a local kv head
            for h in g.q_heads:
                assert h // group in g.kv_heads
            assert len(g.gdn_v_heads) * tp == cfg.linear_num_value_heads
            assert len(g.gdn_v_heads) % len(g.gdn_k_heads) == 0
        assert seen_q == list(range(cfg.num_attention_heads))
    g = TpGeometry.make(cfg, 5, 8)
    assert list(g.kv_heads) == [2] and list(g.q_heads) == [15, 16, 17]
    with pytest.raises(ValueError):
        TpGeometry.make(cfg, 0, 3)
