"""Rank-loss detection without any GPU: gloo-less child processes share a TCPStore; one of them stops
beating (exits) and the others must notice within the timeout, between steps."""
import multiprocessing as mp
import socket
import time

import pytest


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank(rank, world, port, die_rank, q):
    from datetime import timedelta
    from torch.distributed import TCPStore
    from phaseshift_b200.parallel.health import PeerMonitor, RankLostError
    store = TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=timedelta(seconds=20), wait_for_workers=True)
    # the timeout leaves room for a loaded machine: a healthy rank whose thread is starved for a second must not be declared lost
    mon = PeerMonitor(store, rank, world, interval_s=0.05, timeout_s=1.5).start()
    t0 = time.monotonic()
    steps = 0
    try:
        while time.monotonic() - t0 < 12.0:
            mon.assert_alive()               # "before the next launch"
            steps += 1
            time.sleep(0.02)
            if rank == die_rank and steps == 20:
                mon.stop()                    # leaves between steps: no more heartbeats
                q.put((rank, "left", steps))
                time.sleep(5.0)               # keep the process (and a rank-0 store) alive while the others notice
                return
        q.put((rank, "no-detection", steps))
    except RankLostError as e:
        q.put((rank, "detected", e.ranks))
        if rank == 0:
            time.sleep(1.5)                   # the store lives in rank 0: let the others finish reading it


@pytest.mark.timeout(60)
@pytest.mark.parametrize("die_rank", [1, 2])
def test_peers_detect_a_rank_that_stops(die_rank):
    ctx = mp.get_context("spawn")
    world, port = 3, _free_port()
    q = ctx.Queue()
    ps = [ctx.Process(target=_rank, args=(r, world, port, die_rank, q)) for r in range(world)]
    for p in ps:
        p.start()
    res = {}
    for _ in range(world):
        r, what, info = q.get(timeout=40)
        res[r] = (what, info)
    for p in ps:
        p.join(timeout=20)
    assert res[die_rank][0] == "left"
    for r in range(world):
        if r != die_rank:
            assert res[r] == ("detected", [die_rank]), res


def test_monitor_with_fake_store_reports_only_stale_peers():
    from phaseshift_b200.parallel.health import PeerMonitor, RankLostError

    class Store(dict):
        def set(self, k, v): self[k] = v
        def get(self, k): return self[k].encode()

    st = Store()
    mon = PeerMonitor(st, 0, 3, interval_s=0.02, timeout_s=0.25).start()
    try:
        t0 = time.monotonic()
        i = 0
        while time.monotonic() - t0 < 0.8:
            i += 1
            st.set("ps_hb/1", str(i))          # rank 1 keeps beating, rank 2 never shows up
            time.sleep(0.02)
        assert mon.lost() == [2]
        with pytest.raises(RankLostError):
            mon.assert_alive()
    finally:
        mon.stop()


def test_nonzero_device_status_poisons_the_step_on_cpu():
    """Whatever raises the op set's status word -- a projection, the tensor-parallel all-reduce (which reports into the
    same word) -- the engine poisons the sequences of that step and clears the word."""
    import torch
    from phaseshift_b200.models.qwen35.config import tiny_config
    from phaseshift_b200.models.qwen35.weights import build_engine_weights, random_hf_weights
    from phaseshift_b200.runtime.batch import SeqRows
    from phaseshift_b200.runtime.engine import Engine, SequenceError
    from phaseshift_b200.runtime.state import StateConfig
    cfg = tiny_config()
    hf = random_hf_weights(cfg, seed=0)
    eng = Engine(build_engine_weights(cfg, lambda n: hf[n], "bf16", "cpu"), "cpu", StateConfig(max_slots=2, max_seq_len=32))
    eng.ops.status = torch.zeros(1, dtype=torch.int32)

    class Tp:                                   # the transport's kernels write into the word the engine attached
        size, rank, transport, stats = 1, 0, "nccl", {}
        status_word = eng.ops.status

        def assert_alive(self):
            pass
    eng.tp = Tp()
    s = eng.open_sequence()
    eng.step([SeqRows(s.slot, 0, [1, 2, 3], (2,))], [s])
    Tp.status_word[0] = 2                       # a bounded wait ran out somewhere in the next step
    with pytest.raises(SequenceError):
        eng.step([SeqRows(s.slot, 3, [4], (0,))], [s])
    assert s.poisoned and int(eng.ops.status[0]) == 0 and eng.status_errors == 1
    s2 = eng.open_sequence()
    assert len(eng.step([SeqRows(s2.slot, 0, [1, 2, 3], (2,))], [s2])[0]) == 1


def _tp_rank(rank, world, port, q):
    """gloo tensor-parallel engine; rank 1 raises between steps, the others must leave through RankLostError."""
    import os
    from datetime import timedelta
    import torch
    import torch.distributed as dist
    from phaseshift_b200.models.qwen35.config import tiny_config
    from phaseshift_b200.models.qwen35.weights import build_engine_weights, random_hf_weights
    from phaseshift_b200.parallel.health import RankLostError
    from phaseshift_b200.parallel.tp import TensorParallel
    from phaseshift_b200.runtime.batch import SeqRows
    from phaseshift_b200.runtime.engine import Engine
    from phaseshift_b200.runtime.state import StateConfig
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", timeout=timedelta(seconds=20))
    cfg = tiny_config()
    hf = random_hf_weights(cfg, seed=0)
    tp = TensorParallel(dist.group.WORLD, "cpu")
    eng = Engine(build_engine_weights(cfg, lambda n: hf[n], "bf16", "cpu", tp_rank=rank, tp_size=world), "cpu",
                 StateConfig(max_slots=1, max_seq_len=64), tp=tp)
    dist.barrier()                            # every rank is past its (unevenly long) set-up before heartbeats are judged
    tp.start_monitor(interval_s=0.05, timeout_s=1.5)
    s = eng.open_sequence()
    toks, _ = eng.step([SeqRows(s.slot, 0, [3, 4, 5, 6], (3,))], [s])
    try:
        for i in range(50):
            if rank == 1 and i == 3:
                tp.monitor.stop()
                q.put((rank, "raised", i))
                raise RuntimeError("rank 1 fails between steps")
            if i >= 3 and rank != 1:
                time.sleep(0.6)              # between steps (waiting for requests): the heartbeat has time to lapse
            toks, _ = eng.step([SeqRows(s.slot, s.position, [toks[0]], (0,))], [s])
        q.put((rank, "no-detection", None))
    except RankLostError as e:
        q.put((rank, "rank-lost", e.ranks))
        if rank == 0:
            time.sleep(1.5)
    except RuntimeError:
        pass                                  # rank 1's own failure: it leaves without touching the group again
    q.close()
    q.join_thread()                           # the result must be on its way before the hard exit
    os._exit(0 if rank != 1 else 3)           # no collective teardown with a dead peer


@pytest.mark.timeout(120)
def test_a_rank_that_raises_takes_the_others_out_through_rank_lost_error():
    ctx = mp.get_context("spawn")
    world, port = 4, _free_port()
    q = ctx.Queue()
    ps = [ctx.Process(target=_tp_rank, args=(r, world, port, q)) for r in range(world)]
    for p in ps:
        p.start()
    res = {}
    for _ in range(world):
        r, what, info = q.get(timeout=90)
        res[r] = (what, info)
    for p in ps:
        p.join(timeout=30)
    assert res[1][0] == "raised"
    # every survivor leaves through RankLostError naming rank 1 (a late one may also name a survivor that already left)
    assert all(res[r][0] == "rank-lost" and 1 in res[r][1] for r in (0, 2, 3)), res
    assert ps[1].exitcode == 3 and all(ps[r].exitcode == 0 for r in (0, 2, 3))
